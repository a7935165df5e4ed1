"""Parity at the sizes the benchmark times: the Flux double-stream block of the CPU-runnable configuration
(hidden 3072, 24 heads, 1024 image + 512 text tokens) in all four weight formats, a single-stream block over the
full 4608-token sequence, a Wan-14B-width block over the 4095 tokens an 8-GPU rank owns, and the GEMM and attention
kernels at the sweep shapes (4096..32760 rows, K up to 15360, 24x4608 and 40x32760 attention).  The CPU oracle
evaluates whole blocks where that takes seconds and a row subsample where it does not; rows of a Linear and of an
attention are independent, so a subsample checks exactly the sampled outputs.

Tolerances: block output rel-L2 <= 1e-2 (FP8 / INT8) and <= 2e-3 (BF16) against the oracle with the same
quantisation.  The block's UPDATE (output minus input), which is not diluted by the residual stream, is reported and
held to the same bound - or, where that is physically out of reach, to 1.5 x the oracle's own reproducibility: the
disagreement of two oracle runs that differ only in fp32 summation order (``LinearEval(shuffle_k=...)``).  At these
widths a 1e-7 difference before a bf16 or e4m3 rounding moves a few values to the neighbouring code, the next
quantiser amplifies that (a flip is 2^-8 resp. 2^-4 relative), and after the three or four low-precision tensors of a
block two evaluations of the SAME formula disagree by several 1e-3 (bf16) or 1e-2 (FP8) on the update."""
import functools
import importlib

import pytest
import torch

from oracle import flux as OF
from oracle import ops as O
from oracle import wan as OW
from oracle.linear import LinearEval

pytestmark = pytest.mark.gpu
synth = importlib.import_module("diffsynth_engine_b200.synth")


def _bf(t):
    return t.to(torch.bfloat16)


def _rows(n, k=384, seed=0):
    """Sampled row indices: the first and last 130 rows (tile edges) plus k random ones."""
    g = torch.Generator().manual_seed(seed)
    idx = torch.cat([torch.arange(min(130, n)), torch.arange(max(0, n - 130), n), torch.randint(0, n, (k,), generator=g)])
    return torch.unique(idx)


# ------------------------------------------------------------------------------------ Flux blocks at width 3072
def _weights(shapes, seed):
    """Seeded weights as a bf16 checkpoint holds them, drawn on the GPU (the host generator needs ~10 s per block at
    these widths) and handed to both sides as the same fp32 tensors."""
    return {k: v.bfloat16().float().cpu() for k, v in synth.make_state_dict(shapes, seed=seed, device="cuda:0").items()}


@functools.lru_cache(maxsize=2)
def _flux_block_case(n_double, n_single, hw, S_txt, seed):
    w = _weights(synth.flux_dit_shapes(d=3072, H=24, n_double=n_double, n_single=n_single), seed)
    lat = synth.randn((1, 16, hw, hw), seed + 1).bfloat16().float()
    pe = synth.randn((1, S_txt, 4096), seed + 2).bfloat16().float()
    pooled = synth.randn((1, 768), seed + 3)
    return w, lat, pe, pooled, torch.tensor([500.0]), torch.tensor([3.5])


def _engine_hidden(dsb, dev, w, fmt, lat, pe, pooled, t, g, n_double, n_single):
    from diffsynth_engine_b200.flux import FluxDiTEngine
    eng = FluxDiTEngine(dict(w), fmt=fmt, device=dev, n_double=n_double, n_single=n_single, num_heads=24)
    eng.prepare(pe.shape[1], lat.shape[2], lat.shape[3], pe.shape[2], pooled.shape[1])
    eng.set_inputs(lat.to(dev), t.to(dev), pe.to(dev), pooled.to(dev), g.to(dev))
    eng.step()
    dsb.ops.check_status(0)
    hid = eng._bufs["x"].float().cpu()
    del eng
    torch.cuda.empty_cache()
    return hid


def _check_block(dsb, dev, fmt, n_double, n_single, hw, S_txt, seed, what):
    w, lat, pe, pooled, t, g = _flux_block_case(n_double, n_single, hw, S_txt, seed)
    kw = dict(H=24, rt=OF.round_bf16, return_hidden=True)
    with torch.no_grad():
        _, x0_ref = OF.flux_dit_forward(w, lat, t, pe, pooled, g, n_double=0, n_single=0, lin=LinearEval(fmt), **kw)
        _, y_ref = OF.flux_dit_forward(w, lat, t, pe, pooled, g, n_double=n_double, n_single=n_single,
                                       lin=LinearEval(fmt), **kw)
        # the same oracle with another fp32 summation order: how well the formula reproduces ITSELF
        _, y_alt = OF.flux_dit_forward(w, lat, t, pe, pooled, g, n_double=n_double, n_single=n_single,
                                       lin=LinearEval(fmt, shuffle_k=1), **kw)
    x0 = _engine_hidden(dsb, dev, w, fmt, lat, pe, pooled, t, g, 0, 0)
    y = _engine_hidden(dsb, dev, w, fmt, lat, pe, pooled, t, g, n_double, n_single)
    err, floor = O.rel_l2(y, y_ref), O.rel_l2(y_alt, y_ref)
    err_upd, floor_upd = O.rel_l2(y - x0, y_ref - x0_ref), O.rel_l2(y_alt - x0_ref, y_ref - x0_ref)
    print(f"{what} {fmt}: block output rel-L2 {err:.3e} (oracle vs reordered oracle {floor:.3e}), block update "
          f"{err_upd:.3e} (oracle vs reordered oracle {floor_upd:.3e}), |update|/|output| = "
          f"{float((y_ref - x0_ref).norm() / y_ref.norm()):.2f}")
    tol = 2e-3 if fmt == "bf16" else 1e-2
    assert torch.isfinite(y).all()
    assert err < max(tol, 1.5 * floor)
    assert err_upd < max(tol, 1.5 * floor_upd)


@pytest.mark.parametrize("fmt", ["fp8_tensor", "fp8_channel", "int8_channel", "bf16"])
def test_flux_double_block_1024_image_512_text_tokens(dsb, cuda_dev, fmt):
    """models/flux/flux_dit.py:219-236 at hidden 3072, 24 heads, 32x32 image tokens + 512 text tokens: 1536 rows, so
    the image-stream GEMMs run on 256x256 CTA-pair tiles and the text stream rides in the same grouped launch."""
    _check_block(dsb, cuda_dev, fmt, 1, 0, 64, 512, 40, "double block 1024+512")


@pytest.mark.parametrize("fmt", ["fp8_tensor", "bf16"])
def test_flux_single_block_full_sequence(dsb, cuda_dev, fmt):
    """models/flux/flux_dit.py:308-321 at the benchmark's sequence: 4096 image + 512 text tokens; the N = 21504
    projection with RMSNorm/RoPE/GELU epilogue and the K = 15360 output projection with the gate-residual epilogue."""
    _check_block(dsb, cuda_dev, fmt, 0, 1, 128, 512, 50, "single block 4096+512")


# ------------------------------------------------------------------------------------ Wan block at width 5120
@functools.lru_cache(maxsize=1)
def _wan_weights(d, ffn):
    return _weights(synth.wan_dit_shapes(d=d, ffn=ffn, num_layers=1), 60)


@pytest.mark.parametrize("fmt", ["fp8_channel", "bf16"])
def test_wan_block_width_5120_on_4095_tokens(dsb, cuda_dev, fmt):
    """models/wan/wan_dit.py:185-193 at dim 5120, 40 heads, FFN 13824 on a 21 x 15 x 13 token grid = 4095 tokens (what
    one of eight ranks owns of the 32760-token video), 512 context tokens."""
    from diffsynth_engine_b200.wan import WanDiTEngine
    d, ffn, H = 5120, 13824, 40
    fr, hh, ww = 21, 30, 26
    w = _wan_weights(d, ffn)
    x = synth.randn((1, 16, fr, hh, ww), 61).bfloat16().float()
    ctx = synth.randn((1, 512, 4096), 62).bfloat16().float()
    t = torch.tensor([417.0])
    with torch.no_grad():
        y_ref, h0_ref, h1_ref = OW.wan_dit_forward(w, x, ctx, t, num_layers=1, H=H, lin=LinearEval(fmt),
                                                   rt=OF.round_bf16, return_hidden=True)
        _, _, h1_alt = OW.wan_dit_forward(w, x, ctx, t, num_layers=1, H=H, lin=LinearEval(fmt, shuffle_k=1),
                                          rt=OF.round_bf16, return_hidden=True)
    eng = WanDiTEngine(dict(w), fmt=fmt, device=cuda_dev, num_layers=1, num_heads=H)
    y = eng(x.to(cuda_dev), ctx.to(cuda_dev), t.to(cuda_dev)).float().cpu()
    h1 = eng.hidden().float().cpu()
    eng0 = WanDiTEngine(dict(w), fmt=fmt, device=cuda_dev, num_layers=0, num_heads=H)
    eng0(x.to(cuda_dev), ctx.to(cuda_dev), t.to(cuda_dev))
    h0 = eng0.hidden().float().cpu()
    dsb.ops.check_status(0)
    err, err_upd, err_out = O.rel_l2(h1, h1_ref), O.rel_l2(h1 - h0, h1_ref - h0_ref), O.rel_l2(y, y_ref)
    floor, floor_upd = O.rel_l2(h1_alt, h1_ref), O.rel_l2(h1_alt - h0_ref, h1_ref - h0_ref)
    print(f"wan block d=5120 S=4095 {fmt}: block output {err:.3e} (oracle vs reordered oracle {floor:.3e}), block "
          f"update {err_upd:.3e} ({floor_upd:.3e}), model output {err_out:.3e}")
    tol = 2e-3 if fmt == "bf16" else 1e-2
    assert err < max(tol, 1.5 * floor) and err_upd < max(tol, 1.5 * floor_upd)


# ------------------------------------------------------------------------------------ GEMM at the sweep shapes
def _quant_case(M, N, K, per_channel, seed, rows):
    g = torch.Generator().manual_seed(seed)
    x = _bf(torch.randn(M, K, generator=g))
    W = torch.randn(N, K, generator=g) * 0.02
    b = torch.randn(N, generator=g) * 0.1
    wq, ws = O.quant_weight(W, "fp8_channel" if per_channel else "fp8_tensor")
    xq_s, xs_s = O.quant_rows_e4m3(x[rows])
    acc = O.linear_quant(xq_s, xs_s, wq, ws, b)       # oracle on the sampled rows only
    return x, wq, ws, b, acc


@pytest.mark.parametrize("M,K,N,per_channel", [(4096, 3072, 12288, False), (8192, 3072, 9216, True),
                                               (32760, 5120, 13824, True), (1024, 3072, 3072, False)])
def test_fp8_linear_bias_gelu_at_sweep_shapes(dsb, cuda_dev, M, K, N, per_channel):
    """FP8 Linear + bias + GELU-tanh, bf16 output and the e4m3 (unit scale) output form, sampled rows vs the oracle."""
    ops = dsb.ops
    rows = _rows(M, seed=M)
    x, wq, ws, b, acc = _quant_case(M, N, K, per_channel, 70 + (M % 7), rows)
    ref = O.gelu_tanh(acc)
    dev = cuda_dev
    xq, xs = ops.quant_rows(x.to(dev))
    out = ops.gemm(xq, wq.to(dev), row_scale=xs, col_scale=ws.to(dev), bias=b.to(dev), act=ops.ACT_GELU_TANH)
    err = O.rel_l2(out[rows.to(dev)].float().cpu(), ref)
    assert err < 4e-3, (M, K, N, err)
    out8 = torch.empty(M, N, dtype=torch.float8_e4m3fn, device=dev)
    ops.gemm_group([dict(a=xq, w=wq.to(dev), row_scale=xs, col_scale=ws.to(dev), bias=b.to(dev),
                         act=ops.ACT_GELU_TANH, out=out8)])
    got8 = out8[rows.to(dev)].float().cpu()
    assert O.rel_l2(got8, ref) < 4e-2                 # e4m3 resolution (3 mantissa bits)
    want8 = ref.clamp(-448, 448).to(torch.float8_e4m3fn).float()
    assert ((got8 - want8).abs() <= 0.0626 * ref.abs() + 2e-3).float().mean() > 0.999
    ops.check_status(0)


@pytest.mark.parametrize("M,K,N", [(4096, 12288, 3072), (4608, 15360, 3072), (8192, 12288, 3072), (4096, 3072, 3072)])
def test_fp8_linear_gate_residual_on_pair_tiles(dsb, cuda_dev, M, K, N):
    """x <- x + gate * (A W^T * scales + bias) written IN PLACE over the residual, as every residual write of the
    model does (out-proj, FF2, single-block proj_out with K = 15360): 256x256 CTA-pair tiles, residual by TMA."""
    ops = dsb.ops
    rows = _rows(M, seed=K)
    x, wq, ws, b, acc = _quant_case(M, N, K, False, 80 + (K % 5), rows)
    g = torch.Generator().manual_seed(K)
    resid = _bf(torch.randn(M, N, generator=g))
    gate = torch.randn(N, generator=g)
    ref = resid[rows].float() + gate * acc
    dev = cuda_dev
    xq, xs = ops.quant_rows(x.to(dev))
    buf = resid.to(dev).clone()
    ops.gemm(xq, wq.to(dev), row_scale=xs, col_scale=ws.to(dev), bias=b.to(dev), gate=gate.to(dev), resid=buf, out=buf)
    assert O.rel_l2(buf[rows.to(dev)].float().cpu(), ref) < 4e-3
    ops.check_status(0)


@pytest.mark.parametrize("fmt", ["e4m3", "int8", "bf16"])
def test_grouped_launch_image_and_text_rows(dsb, cuda_dev, fmt):
    """Two problems in one persistent launch - 4096 image rows and 512 text rows of one [4608, d] buffer with their
    own weights, gates and biases, residual in place - as the double-stream blocks issue them."""
    ops = dsb.ops
    dev = cuda_dev
    K, N, Mi, Mt = 3072, 3072, 4096, 512
    g = torch.Generator().manual_seed(90)
    x = _bf(torch.randn(Mt + Mi, K, generator=g))
    resid = _bf(torch.randn(Mt + Mi, N, generator=g))
    rows = _rows(Mt + Mi, seed=5)
    rng = {"t": slice(0, Mt), "i": slice(Mt, Mt + Mi)}
    W = {s: torch.randn(N, K, generator=g) * 0.02 for s in rng}
    b = {s: torch.randn(N, generator=g) * 0.1 for s in rng}
    gate = {s: torch.randn(N, generator=g) for s in rng}
    if fmt == "bf16":
        a_d, rs_d = x.to(dev), None
        wq = {s: (_bf(W[s]), None) for s in rng}
        acc = {s: x.float() @ _bf(W[s]).float().t() + b[s] for s in rng}
    else:
        mode = "fp8_tensor" if fmt == "e4m3" else "int8_channel"
        wq = {s: O.quant_weight(W[s], mode) for s in rng}
        xq, xs = (O.quant_rows_e4m3 if fmt == "e4m3" else O.quant_rows_int8)(x)
        a_d, rs_d = xq.to(dev), xs.to(dev)
        acc = {s: O.linear_quant(xq, xs, wq[s][0], wq[s][1], b[s]) for s in rng}
    ref = resid.float().clone()
    for s, sl in rng.items():
        ref[sl] = resid[sl].float() + gate[s] * acc[s][sl]
    buf = resid.to(dev).clone()
    probs = []
    for s in ("i", "t"):
        sl = rng[s]
        probs.append(dict(a=a_d[sl], w=wq[s][0].to(dev), row_scale=None if rs_d is None else rs_d[sl],
                          col_scale=None if wq[s][1] is None else wq[s][1].to(dev), bias=b[s].to(dev),
                          gate=gate[s].to(dev), resid=buf[sl], out=buf[sl]))
    ops.gemm_group(probs)
    assert O.rel_l2(buf[rows.to(dev)].float().cpu(), ref[rows]) < 4e-3
    ops.check_status(0)


# ------------------------------------------------------------------------------------ attention at the sweep shapes
def test_joint_attention_24_heads_4608_tokens(dsb, cuda_dev):
    g = torch.Generator().manual_seed(100)
    H, S = 24, 4608
    q, k, v = (_bf(torch.randn(1, S, H, 128, generator=g)) for _ in range(3))
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    out = dsb.ops.flash_attn(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev)).float().cpu()
    dsb.ops.check_status(0)
    assert O.rel_l2(out, O.attention(qh, kh, vh).transpose(1, 2)) < 4e-3          # exact softmax: bf16 P and output
    # same roundings (bf16 probabilities, bf16 output): only accumulation order and the ex2 approximation remain
    same = O.attention_bf16_probs(qh, kh, vh).transpose(1, 2).bfloat16().float()
    err = O.rel_l2(out, same)
    print(f"attention 24x4608 vs the bf16-probability restatement: {err:.3e}")
    assert err < 5e-4


@pytest.mark.parametrize("peaked", [False, True])
def test_attention_40_heads_32760_tokens_sampled_query_tiles(dsb, cuda_dev, peaked):
    """The Wan self-attention shape: 256 key tiles per query tile.  All queries run on the GPU; four query tiles
    (first, two inner, the ragged last) are checked against the oracle over all 32760 keys.  ``peaked``: a few keys
    beyond key tile 200 carry scores far above everything before them, so the reference maximum of the running
    softmax must be refreshed (and O rescaled) late in the sequence."""
    g = torch.Generator().manual_seed(101)
    H, S = 40, 32760
    q, k, v = (_bf(torch.randn(1, S, H, 128, generator=g)) for _ in range(3))
    if peaked:
        k[:, 26000:26010] *= 8.0
        k[:, 32000:32002] *= 14.0
    out = dsb.ops.flash_attn(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev))
    dsb.ops.check_status(0)
    rows = torch.cat([torch.arange(0, 128), torch.arange(12800, 12928), torch.arange(25600 + 77, 25600 + 205),
                      torch.arange(32640, 32760)])
    qh, kh, vh = q[:, rows].transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    got = out[:, rows.to(cuda_dev)].float().cpu()
    assert torch.isfinite(out).all()
    assert O.rel_l2(got, O.attention(qh, kh, vh).transpose(1, 2)) < 4e-3
    err = O.rel_l2(got, O.attention_bf16_probs(qh, kh, vh).transpose(1, 2).bfloat16().float())
    print(f"attention 40x32760 (peaked={peaked}) vs the bf16-probability restatement: {err:.3e}")
    assert err < 5e-4
