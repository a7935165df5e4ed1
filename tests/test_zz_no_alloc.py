"""``dsb_linear_static`` - the quantised Linear for callers that cannot allocate device memory (a plugin living
inside another runtime's fixed memory plan, an FFI binding that passes only the tensors it was handed).  Its
intermediates sit in a fixed array inside the library, shared by every call, so the checks here are: same result
as the ordinary two-call path (``dsb_quant_rows`` + ``dsb_gemm`` with caller-allocated scratch), twice in a row
with different shapes so that what the first call left in the array cannot leak into the second, and a clear
refusal above the size limit.  Runs last by file name, and stands alone in a fresh process."""
import pytest
import torch

from oracle import ops as O

pytestmark = pytest.mark.gpu


def _pair(dsb, dev, M, N, K, fmt, per_channel, act, seed):
    ops = dsb.ops
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, K, generator=g) * 1.5).to(torch.bfloat16).to(dev)
    W = (torch.randn(N, K, generator=g) * 0.05).to(dev)
    bias = (torch.randn(N, generator=g) * 0.1).to(dev)
    code = ops.FMT_E4M3 if fmt == "e4m3" else ops.FMT_INT8
    Wq, ws = ops.pack_quant_weight(W, code, per_channel=per_channel)
    xq, rs = ops.quant_rows(x, code)                                   # caller-allocated scratch
    want = ops.gemm(xq, Wq, row_scale=rs, col_scale=ws, bias=bias, act=act)
    got = ops.linear_static(x, Wq, ws, bias=bias, act=act)             # scratch inside the library
    # and the CPU oracle of the same quantised Linear (same quantisation rules, fp32 accumulation)
    mode = ("fp8_channel" if per_channel else "fp8_tensor") if fmt == "e4m3" else "int8_channel"
    oq, os_ = O.quant_weight(W.cpu(), mode)
    aq, as_ = (O.quant_rows_e4m3 if fmt == "e4m3" else O.quant_rows_int8)(x.cpu())
    ref = O.linear_quant(aq, as_, oq, os_, bias.cpu())
    if act == ops.ACT_GELU_TANH:
        ref = O.gelu_tanh(ref)
    assert O.rel_l2(got.float().cpu(), ref) < 4e-3                     # bf16 output rounding only
    return got, want


def test_static_linear_matches_two_call_path_twice_in_a_row(dsb, cuda_dev):
    ops = dsb.ops
    # first call: a large-ish problem that fills a good part of the shared array
    got, want = _pair(dsb, cuda_dev, 1111, 768, 2048, "e4m3", False, ops.ACT_GELU_TANH, 1)
    assert O.rel_l2(got.float().cpu(), want.float().cpu()) < 3e-3
    assert torch.equal(got, want)  # same kernels, same operands: identical bits
    # second call right after: other shape, other format; stale bytes of call one lie beyond and between its rows
    got, want = _pair(dsb, cuda_dev, 77, 136, 512, "int8", True, ops.ACT_NONE, 2)
    assert O.rel_l2(got.float().cpu(), want.float().cpu()) < 3e-3
    assert torch.equal(got, want)
    # and once more with the first shape: results must not depend on the call history
    got2, want2 = _pair(dsb, cuda_dev, 1111, 768, 2048, "e4m3", False, ops.ACT_GELU_TANH, 1)
    assert torch.equal(got2, want2)
    ops.check_status(0)


def test_static_linear_rejects_what_does_not_fit(dsb, cuda_dev):
    ops = dsb.ops
    K = 16384
    M = (64 << 20) // K + 1  # one row more than the fixed array can take
    x = torch.zeros(M, K, dtype=torch.bfloat16, device=cuda_dev)
    Wq = torch.zeros(64, K, dtype=torch.float8_e4m3fn, device=cuda_dev)
    ws = torch.ones(1, device=cuda_dev)
    with pytest.raises(dsb.DsbError, match="TOO_LARGE"):
        ops.linear_static(x, Wq, ws)
    with pytest.raises(dsb.DsbError):  # K must be a multiple of 16
        ops.linear_static(x[:4, :40], Wq[:, :40], ws)
    assert ops.linear_static(x[:0], Wq, ws).shape == (0, 64)
