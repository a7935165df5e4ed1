"""The drop-in seams on the GPU: patched ``F.linear`` with ``QuantLinearWeight`` parameters, and the attention
functions installed where the reference dispatches (same call shapes as models/flux/flux_dit.py:166-183,297-304 and
models/wan/wan_dit.py:18-22)."""
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from oracle import ops as O
from oracle.linear import LinearEval

pytestmark = pytest.mark.gpu
synth = __import__("importlib").import_module("diffsynth_engine_b200.synth")


class FF(nn.Module):  # the shape of FluxJointTransformerBlock.ff_a (flux_dit.py:208-210)
    def __init__(self, d):
        super().__init__()
        self.net = nn.Sequential(nn.Linear(d, 4 * d), nn.GELU(approximate="tanh"), nn.Linear(4 * d, d))

    def forward(self, x):
        return self.net(x)


@pytest.mark.parametrize("fmt", ["fp8_tensor", "fp8_channel", "int8_channel", "bf16"])
def test_patched_linear_module(dsb, cuda_dev, fmt):
    from diffsynth_engine_b200.quant import QuantLinearWeight, b200_inference, enable_b200_linear
    d = 256
    ff = FF(d)
    with torch.no_grad():
        for i, p in enumerate(ff.parameters()):
            p.copy_(synth.randn(tuple(p.shape), 40 + i) * (0.05 if p.dim() == 2 else 0.1))
    x = synth.randn((2, 75, d), 50).bfloat16()
    w = {k: v.detach().clone().bfloat16().float() for k, v in ff.state_dict().items()}
    lin = LinearEval(fmt)
    # the module rounds the first Linear's output to bf16, then nn.GELU rounds again
    h = lin(x.reshape(-1, d).float(), w["net.0.weight"], w["net.0.bias"]).bfloat16().float()
    h = O.gelu_tanh(h).bfloat16().float()
    ref = lin(h, w["net.2.weight"], w["net.2.bias"]).reshape(2, 75, d)
    ff = ff.to(cuda_dev, torch.bfloat16)
    enable_b200_linear(ff, fmt)
    assert ff.b200_linear_enabled and isinstance(ff.net[0].weight, QuantLinearWeight)
    origin = F.linear
    with torch.no_grad(), b200_inference():
        assert F.linear is not origin
        y = ff(x.to(cuda_dev))
    assert F.linear is origin
    assert y.dtype == torch.bfloat16 and y.shape == (2, 75, d)
    assert O.rel_l2(y.float().cpu(), ref) < (4e-3 if fmt == "bf16" else 1e-2)
    # M=1 conditioning vector goes through the GEMV path
    v = synth.randn((1, d), 51).bfloat16()
    with torch.no_grad(), b200_inference():
        y1 = ff.net[0](v.to(cuda_dev))
    ref1 = lin(v.float(), w["net.0.weight"], w["net.0.bias"], act_quant=False)
    assert O.rel_l2(y1.float().cpu(), ref1) < 5e-3


def test_patched_linear_restores_on_error_and_falls_through(dsb, cuda_dev):
    from diffsynth_engine_b200.quant import b200_inference
    origin = F.linear
    plain = nn.Linear(64, 32).to(cuda_dev, torch.bfloat16)
    x = torch.randn(5, 64, device=cuda_dev, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="boom"):
        with b200_inference():
            y = plain(x)          # not a QuantLinearWeight: original F.linear
            assert torch.equal(y, origin(x, plain.weight, plain.bias))
            raise RuntimeError("boom")
    assert F.linear is origin
    with b200_inference(False):
        assert F.linear is origin


def test_b200_attn_flux_call_shapes(dsb, cuda_dev):
    """q, k contiguous [B,H,S,D]; v a strided view of the fused [B,S,7d] projection (flux_dit.py:297-312)."""
    from diffsynth_engine_b200.attention import b200_attn
    B, H, S, D = 1, 4, 333, 128
    d = H * D
    fused = synth.randn((B, S, 7 * d), 60).bfloat16()
    qkv = fused[:, :, :3 * d].view(B, S, 3 * H, D).transpose(1, 2)
    q, k, v = qkv.chunk(3, dim=1)
    ref = O.attention(q, k, v)
    fd = fused.to(cuda_dev)
    qd, kd, vd = fd[:, :, :3 * d].view(B, S, 3 * H, D).transpose(1, 2).chunk(3, dim=1)
    out = b200_attn(qd.contiguous(), kd.contiguous(), vd)
    assert out.shape == (B, H, S, D)
    flat = out.transpose(1, 2).reshape(B, S, d)      # what the caller does next (flux_dit.py:304)
    assert flat.data_ptr() == out.data_ptr()         # ... and it is a view, not a copy
    assert O.rel_l2(flat.float().cpu(), ref.transpose(1, 2).reshape(B, S, d)) < 4e-3
    with pytest.raises(dsb.DsbError):
        b200_attn(q, k, v)  # CPU tensors: no fallback


def test_b200_wan_attention_call_shapes(dsb, cuda_dev):
    from diffsynth_engine_b200.attention import b200_wan_attention
    B, S, L, H = 1, 420, 77, 5
    q, k, v = (synth.randn((B, n, H * 128), 70 + i).bfloat16() for i, n in enumerate((S, L, L)))
    mh = lambda t: t.unflatten(2, (H, 128)).transpose(1, 2)
    ref = O.attention(mh(q), mh(k), mh(v)).transpose(1, 2).flatten(2)
    out = b200_wan_attention(q.to(cuda_dev), k.to(cuda_dev), v.to(cuda_dev), num_heads=H)
    assert out.shape == (B, S, H * 128)
    assert O.rel_l2(out.float().cpu(), ref) < 4e-3


def test_set_attn_implementation_names(dsb):
    import types
    from diffsynth_engine_b200 import attention as A
    fake_flux, fake_wan = types.SimpleNamespace(_attn_func=None), types.SimpleNamespace(attention=lambda *a: None)
    with pytest.raises(ValueError):
        A.set_attn_implementation("flash9", fake_flux)
    A.set_attn_implementation("b200", fake_flux, fake_wan)
    assert fake_flux._attn_func is A.b200_attn and fake_wan.attention is A.b200_wan_attention
    A.set_attn_implementation("sdpa", fake_flux, fake_wan)
    assert fake_flux._attn_func is F.scaled_dot_product_attention and fake_wan.attention is not A.b200_wan_attention


class _Q8Param(torch.nn.Parameter):
    """Stand-in for the reference's GGUFParameter: raw bytes plus a ``quant_dtype`` tag with a ``name``."""

    def __new__(cls, data, qtype="Q8_0"):
        self = torch.Tensor._make_subclass(cls, data, False)
        self.quant_dtype = type("QT", (), {"name": qtype})()
        return self

    __torch_function__ = torch._C._disabled_torch_function_impl


def test_gguf_q8_0_dequantisation_and_linear(dsb, cuda_dev):
    """Q8_0 bytes -> bf16 on the device, bit-identical to the reference's dequantisation; a Linear holding such a
    weight is prepacked once (bf16 = the reference's numbers; FP8 = re-quantised) and then runs like any other."""
    from oracle import ops as O
    from oracle.linear import LinearEval
    from diffsynth_engine_b200.quant import b200_inference, enable_b200_linear
    synth = __import__("importlib").import_module("diffsynth_engine_b200.synth")
    N, K = 200, 512
    W = synth.randn((N, K), 120) * 0.05
    raw = O.q8_0_quantize(W)
    ref_w = O.q8_0_dequantize(raw, torch.bfloat16)
    got = dsb.ops.dequant_q8_0(raw.to(cuda_dev)).cpu()
    assert torch.equal(got.view(torch.int16), ref_w.view(torch.int16))
    x = synth.randn((96, K), 121).bfloat16()
    for fmt, tol in (("bf16", 3e-3), ("fp8_channel", 1e-2)):
        lin = torch.nn.Linear(K, N).to(cuda_dev).bfloat16()
        bias = lin.bias.detach().float().cpu()
        lin.weight = _Q8Param(raw.to(cuda_dev))
        enable_b200_linear(lin, fmt)
        with b200_inference():
            y = lin(x.to(cuda_dev)).float().cpu()
        ref = LinearEval(fmt)(x.float(), ref_w.float(), bias)
        assert O.rel_l2(y, ref) < tol, fmt


def test_gguf_q4_k_dequantisation_is_bit_exact(dsb, cuda_dev):
    """Q4_K super-blocks -> bf16 on the device against the oracle's restatement of the reference's evaluation order
    (itself pinned bit-exactly by a reference-generated fixture), and the Linear seam on such a weight."""
    from oracle import ops as O
    from diffsynth_engine_b200.quant import b200_inference, enable_b200_linear
    raw = O.q4_k_random_blocks(72, 1024, 130)
    ref_w = O.q4_k_dequantize(raw, torch.bfloat16)
    got = dsb.ops.dequant_q4_k(raw.to(cuda_dev)).cpu()
    assert torch.equal(got.view(torch.int16), ref_w.view(torch.int16))
    lin = torch.nn.Linear(1024, 72, bias=False).to(cuda_dev).bfloat16()
    p = _Q8Param(raw.to(cuda_dev))
    p.quant_dtype = type("QT", (), {"name": "Q4_K"})()
    lin.weight = p
    enable_b200_linear(lin, "bf16")
    x = torch.randn(40, 1024, generator=torch.Generator().manual_seed(3)).bfloat16()
    with b200_inference():
        y = lin(x.to(cuda_dev)).float().cpu()
    assert O.rel_l2(y, x.float() @ ref_w.float().t()) < 3e-3


@pytest.mark.parametrize("qtype", ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K"])
def test_gguf_every_block_format_is_bit_exact(dsb, cuda_dev, qtype):
    """``dsb_dequant_gguf`` against the reference-generated fixture (3 x 512 weights per format) and, on a larger
    seeded matrix, against the oracle restatement that the fixture pins: identical bf16 bits."""
    import os
    from safetensors.torch import load_file
    from oracle import gguf as OG
    GG = load_file(os.path.join(os.path.dirname(__file__), "golden", "gguf_blocks.safetensors"))
    got = dsb.ops.dequant_gguf(GG[f"{qtype}.raw"].to(cuda_dev), qtype).float().cpu()
    assert torch.equal(got, GG[f"{qtype}.bf16"])
    raw = OG.random_blocks(qtype, 40, 1024, 900)
    wide = torch.zeros(40, 1024 + 64, dtype=torch.bfloat16, device=cuda_dev)          # strided output rows
    dsb.ops.dequant_gguf(raw.to(cuda_dev), qtype, out=wide[:, :1024])
    assert torch.equal(wide[:, :1024].float().cpu(), OG.dequantize(raw, qtype, torch.bfloat16).float())
    assert float(wide[:, 1024:].abs().max()) == 0.0
    with pytest.raises(dsb.DsbError):
        dsb.ops.dequant_gguf(raw.to(cuda_dev), "Q9_9")


def test_gguf_q6_k_parameter_goes_through_enable_b200_linear(dsb, cuda_dev):
    """A Linear whose weight is a GGUF Q6_K parameter (a real Q4_K_S checkpoint mixes Q4_K with Q5_K / Q6_K tensors):
    dequantised once on the device, then the bf16 drop-in equals the reference's dequantise-then-linear."""
    from oracle import gguf as OG
    from diffsynth_engine_b200.quant import QuantLinearWeight, b200_inference, enable_b200_linear
    N, K = 64, 512
    raw = OG.random_blocks("Q6_K", N, K, 901)
    lin = nn.Linear(K, N, bias=False).to(cuda_dev)
    lin.weight = _Q8Param(raw.to(cuda_dev), "Q6_K")
    enable_b200_linear(lin, "bf16")
    assert isinstance(lin.weight, QuantLinearWeight)
    x = synth.randn((7, K), 902).bfloat16()
    with torch.no_grad(), b200_inference():
        y = lin(x.to(cuda_dev)).float().cpu()
    ref = x.float() @ OG.dequantize(raw, "Q6_K", torch.bfloat16).float().t()
    assert O.rel_l2(y, ref) < 4e-3
