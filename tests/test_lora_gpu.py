"""Unfused LoRAs folded into the quantised GEMM (extra K columns) against the oracle's restatement of the same
arithmetic and against the reference's LoRALinear semantics."""
from collections import OrderedDict

import pytest
import torch
import torch.nn as nn

from oracle import ops as O
from oracle.linear import LinearEval, lora_linear_quant, lora_reference

pytestmark = pytest.mark.gpu
synth = __import__("importlib").import_module("diffsynth_engine_b200.synth")


def _case(M=300, K=512, N=384, seed=70):
    W, b = (synth.randn((N, K), seed) * 0.05).bfloat16().float(), synth.randn((N,), seed + 1) * 0.1
    loras = [(0.8 * 16 / 8, (synth.randn((N, 8), seed + 2) * 0.02).bfloat16().float(),
              (synth.randn((8, K), seed + 3) * 0.05).bfloat16().float()),
             (1.0, (synth.randn((N, 4), seed + 4) * 0.02).bfloat16().float(),
              (synth.randn((4, K), seed + 5) * 0.05).bfloat16().float())]
    return synth.randn((M, K), seed + 6).bfloat16().float(), W, b, loras


@pytest.mark.parametrize("fmt", [1, 2])
def test_cast_quant_is_bit_exact(dsb, cuda_dev, fmt):
    x = (synth.randn((70, 64), 5) * 90).bfloat16()
    x[0, :4] = torch.tensor([1000.0, -1000.0, 0.0, 449.0])
    out = torch.zeros(70, 256, dtype=torch.uint8, device=cuda_dev)
    if fmt == 1:
        dsb.ops.cast_quant(x.to(cuda_dev), out[:, 64:256].view(torch.float8_e4m3fn), 1, split=True)
        hi = torch.clamp(x.float(), -448, 448).to(torch.float8_e4m3fn)
        lo = (x.float() - hi.float()).clamp(-448, 448).to(torch.float8_e4m3fn)
        # the remainder of a saturated element is itself large; it is what the kernel must produce as well
        got = out.cpu()
        assert torch.equal(got[:, 64:128], hi.view(torch.uint8))
        assert torch.equal(got[:, 128:192], lo.view(torch.uint8))
        assert torch.equal(got[:, 192:256], hi.view(torch.uint8))
    else:
        dsb.ops.cast_quant(x.to(cuda_dev), out[:, 64:128].view(torch.int8), 2)
        ref = torch.clamp(torch.round(x.float()), -127, 127).to(torch.int8)
        assert torch.equal(out.cpu()[:, 64:128], ref.view(torch.uint8))
    assert int(out[:, :64].sum()) == 0


@pytest.mark.parametrize("fmt", ["fp8_tensor", "fp8_channel", "int8_channel", "bf16"])
def test_linear_lora_matches_oracle(dsb, cuda_dev, fmt):
    from diffsynth_engine_b200.lora import build_lora_extension, linear_lora
    from diffsynth_engine_b200.packed import pack_linear
    x, W, b, loras = _case()
    exact = lora_reference(x, W, b, loras)
    p = pack_linear(W, b, fmt, cuda_dev)
    ext = build_lora_extension(p.w, p.scale, fmt, loras)
    y = linear_lora(x.bfloat16().to(cuda_dev), p.w, p.scale, p.bias, ext).float().cpu()
    dsb.ops.check_status(0)
    if fmt == "bf16":
        ref = lora_reference(x, W, b, [(c, u, d) for c, u, d in loras])
        err = O.rel_l2(y, ref)
        assert err < 5e-3
    else:
        ref = lora_linear_quant(x, W, b, loras, fmt)
        err = O.rel_l2(y, ref)
        assert err < 1e-2
    # the LoRA contribution itself is resolved, not just the main product
    main = LinearEval("fp32")(x, W, b)
    base = LinearEval(fmt)(x, W, b)
    part = O.rel_l2(y - base, exact - main)
    print(f"lora linear {fmt}: vs same-arithmetic oracle {err:.3e}, vs exact {O.rel_l2(y, exact):.3e}, "
          f"LoRA part alone vs exact {part:.3e}")
    assert part < 0.15


def test_linear_lora_with_fused_epilogue(dsb, cuda_dev):
    """The extended GEMM keeps the main GEMM's epilogue: gate * (.) + residual."""
    from diffsynth_engine_b200.lora import build_lora_extension, linear_lora
    from diffsynth_engine_b200.packed import pack_linear
    x, W, b, loras = _case(M=130, K=256, N=256, seed=90)
    gate, resid = synth.randn((256,), 97), synth.randn((130, 256), 98).bfloat16()
    p = pack_linear(W, b, "fp8_tensor", cuda_dev)
    ext = build_lora_extension(p.w, p.scale, "fp8_tensor", loras)
    y = linear_lora(x.bfloat16().to(cuda_dev), p.w, p.scale, p.bias, ext, gate=gate.to(cuda_dev),
                    resid=resid.to(cuda_dev)).float().cpu()
    ref = resid.float() + gate * lora_linear_quant(x, W, b, loras, "fp8_tensor")
    assert O.rel_l2(y, ref) < 1e-2


class _Adapter:
    def __init__(self, scale, rank, alpha, up, down):
        self.scale, self.rank, self.alpha = scale, rank, alpha
        self.up, self.down = nn.Linear(up.shape[1], up.shape[0], bias=False), nn.Linear(down.shape[1], down.shape[0],
                                                                                         bias=False)
        self.up.weight.data, self.down.weight.data = up, down

    def __call__(self, x):
        return self.scale * (self.alpha / self.rank) * self.up(self.down(x))


class _LoraLinearLike(nn.Linear):
    """A Linear with the attributes the fused path reads from the reference's LoRALinear (``_lora_dict`` of adapters
    with ``scale``, ``rank``, ``alpha``, ``up``, ``down``) and its forward rule: main Linear plus every adapter."""

    def __init__(self, i, o):
        super().__init__(i, o)
        self._lora_dict = OrderedDict()

    def forward(self, x):
        y = super().forward(x)
        for lora in self._lora_dict.values():
            y = y + lora(x)
        return y


def test_fuse_lora_on_a_module(dsb, cuda_dev):
    from diffsynth_engine_b200.lora import fuse_lora, unfuse_lora
    from diffsynth_engine_b200.quant import b200_inference, enable_b200_linear
    x, W, b, loras = _case(M=96, K=256, N=128, seed=110)
    lin = _LoraLinearLike(256, 128)
    lin.weight.data, lin.bias.data = W.clone(), b.clone()
    lin = lin.to(cuda_dev).bfloat16()
    for i, (c, up, down) in enumerate(loras):
        a = _Adapter(c, up.shape[1], up.shape[1], up.to(cuda_dev).bfloat16(), down.to(cuda_dev).bfloat16())
        lin._lora_dict[f"l{i}"] = a
    enable_b200_linear(lin, "fp8_tensor")
    xb = x.bfloat16().to(cuda_dev)
    with b200_inference():
        unfused = lin(xb).float().cpu()          # quantised main GEMM, side matrices through the original F.linear
        assert fuse_lora(lin) == 1
        fused = lin(xb).float().cpu()            # first call builds the K-extension of the weight
        n0 = dsb._lib.launches
        assert torch.equal(lin(xb).float().cpu(), fused)
        assert dsb._lib.launches - n0 == 4       # quantise, down GEMM, cast, extended GEMM
        exact = lora_reference(x, W, b, loras)
        assert O.rel_l2(fused, exact) < 5e-2 and O.rel_l2(fused, unfused) < 2e-2
        lin._lora_dict["l0"].scale = 0.0         # what modify_scale does: the extension follows on the next call
        off = lin(xb).float().cpu()
        assert O.rel_l2(off, lora_reference(x, W, b, loras[1:])) < 5e-2
        assert unfuse_lora(lin) == 1 and type(lin) is _LoraLinearLike
        lin._lora_dict.clear()
        plain = lin(xb).float().cpu()
    assert O.rel_l2(plain, LinearEval("fp8_tensor")(x, W, b)) < 1e-2


@pytest.mark.parametrize("fmt", ["fp8_tensor", "int8_channel"])
def test_activation_rows_aligned_with_a_down_row_do_not_saturate(dsb, cuda_dev, fmt):
    """A trained LoRA's down-projection correlates with the activations it was trained on.  Rows that point along a
    down row make x_q.D_j several times larger than the uncorrelated estimate the range split starts from
    (here sqrt(K)/4 = 5.6 times); the headroom that split leaves on the activation side absorbs it, so the LoRA term
    of those rows is still resolved instead of being clipped at the 8-bit maximum."""
    from diffsynth_engine_b200.lora import build_lora_extension, linear_lora
    from diffsynth_engine_b200.packed import pack_linear
    x, W, b, loras = _case(M=128, K=512, N=256, seed=130)
    loras = [(c, u * 0.1, d) for c, u, d in loras]                 # a small adapter: the 8-bit range has slack to give
    d0 = loras[0][2][0]
    x[:64] = (d0 * 20.0).bfloat16().float()[None, :] * torch.linspace(0.5, 2.0, 64)[:, None]   # fully aligned rows
    x = x.bfloat16().float()
    exact = lora_reference(x, W, b, loras)
    main = LinearEval("fp32")(x, W, b)
    p = pack_linear(W, b, fmt, cuda_dev)
    ext = build_lora_extension(p.w, p.scale, fmt, loras)
    y = linear_lora(x.bfloat16().to(cuda_dev), p.w, p.scale, p.bias, ext).float().cpu()
    dsb.ops.check_status(0)
    ref = lora_linear_quant(x, W, b, loras, fmt)
    assert O.rel_l2(y, ref) < 1e-2
    base = LinearEval(fmt)(x, W, b)
    part = O.rel_l2((y - base)[:64], (exact - main)[:64])
    print(f"aligned rows {fmt}: LoRA part alone vs exact {part:.3e}")
    assert part < (0.1 if fmt == "fp8_tensor" else 0.35)
