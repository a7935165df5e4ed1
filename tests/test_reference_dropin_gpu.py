"""The reference's OWN modules on the GPU with this library installed behind their seams:

    enable_b200_linear(block, fmt)                          # instead of enable_fp8_linear
    set_attn_implementation("b200", flux_dit, wan_dit)      # flux_dit._attn_func / wan_dit.attention
    with b200_inference():                                  # instead of fp8_inference
        block(...)

``FluxJointTransformerBlock`` (models/flux/flux_dit.py:197-236), ``FluxSingleTransformerBlock`` (:273-321) and
``DiTBlock`` (models/wan/wan_dit.py:155-193) run unchanged; only ``F.linear`` and the attention callables are
replaced.  Compared with the exact fp32 oracle next to the reference's stock GPU path (cuBLAS + SDPA in bf16):
the drop-in may not be further from exact math than the stock path is (bf16), and stays within the FP8 bound the
reference's own FP8 path is measured against.  Needs ``baseline/_ref`` (``python baseline/install_reference.py``);
skipped otherwise."""
import importlib
import os
import sys

import pytest
import torch
import torch.nn.functional as F

from oracle import flux as OF
from oracle import ops as O
from oracle import wan as OW
from oracle.linear import LinearEval

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
synth = importlib.import_module("diffsynth_engine_b200.synth")


@pytest.fixture(scope="module")
def ref():
    import install_reference
    r = install_reference.import_reference()
    if r is None:
        pytest.skip("baseline/_ref is not installed")
    return r


def _load(module, sd, dev):
    res = torch.nn.Module.load_state_dict(module, sd, strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    return module.to(dev, torch.bfloat16).eval()     # two Linears of these classes ignore the device/dtype arguments


def _flux_ids(S_txt, side):
    ids = torch.zeros(S_txt + side * side, 3)
    r = torch.arange(side, dtype=torch.float32)
    ids[S_txt:, 1] = r[:, None].expand(side, side).reshape(-1)
    ids[S_txt:, 2] = r[None, :].expand(side, side).reshape(-1)
    return ids


def _run_three_ways(dsb, ref, make_block, call, fmts):
    """stock bf16 path, then the drop-in with each weight format; returns {name: output on the CPU in fp32}."""
    from diffsynth_engine_b200.attention import set_attn_implementation
    from diffsynth_engine_b200.quant import QuantLinearWeight, b200_inference, enable_b200_linear
    outs = {}
    with torch.no_grad():
        outs["stock"] = call(make_block())
        for fmt in fmts:
            blk = make_block()
            enable_b200_linear(blk, fmt)
            assert any(isinstance(p, QuantLinearWeight) for p in blk.parameters())
            set_attn_implementation("b200", ref.flux_dit, ref.wan_dit)
            n0 = dsb._lib.launches
            try:
                with b200_inference():
                    outs[fmt] = call(blk)
            finally:
                set_attn_implementation("sdpa", ref.flux_dit, ref.wan_dit)
            assert dsb._lib.launches > n0            # the library's kernels ran, not a fallback
            assert F.linear is torch.nn.functional.linear
    dsb.ops.check_status(0)
    return outs


def _report_and_check(what, outs, exact):
    err = {k: O.rel_l2(v, exact) for k, v in outs.items()}
    print(f"{what}: rel-L2 vs exact fp32 -> " + ", ".join(f"{k} {e:.3e}" for k, e in err.items()))
    # bf16: the drop-in is no further from exact math than the reference's own GPU path (small allowance for noise)
    assert err["bf16"] < 1.25 * err["stock"] + 5e-4
    # FP8 / INT8: per-row and per-tensor (or per-channel) scales keep the block well inside what the reference's
    # unit-scale FP8 path achieves on such weights (7e-2 on this block shape)
    for k in outs:
        if k not in ("stock", "bf16"):
            assert err[k] < 5e-2, (k, err[k])


def test_reference_flux_double_block_through_the_seams(dsb, cuda_dev, ref):
    d, H, side, S_txt = 1024, 8, 24, 80
    sd = {k: v.bfloat16().float() for k, v in synth.make_state_dict(synth.flux_block_shapes("", d, H, "double"), seed=90).items()}
    xa, xb, temb = (synth.randn(s, 91 + i).bfloat16() for i, s in enumerate(((1, side * side, d), (1, S_txt, d), (1, d))))
    ids = _flux_ids(S_txt, side)
    rope = ref.transformer_helper.RoPEEmbedding(d, 10000, [16, 56, 56])(ids[None]).to(cuda_dev)
    ya, yb = OF.double_block(xa[0].float(), xb[0].float(), temb[0].float(), O.flux_rope_table(ids), sd, "", H,
                             LinearEval("fp32"))
    exact = torch.cat([yb, ya])

    def make():
        return _load(ref.flux_dit.FluxJointTransformerBlock(d, H, device="cpu", dtype=torch.float32), sd, cuda_dev)

    def call(blk):
        a, b = blk(xa.to(cuda_dev), xb.to(cuda_dev), temb.to(cuda_dev), rope)
        return torch.cat([b[0], a[0]]).float().cpu()

    outs = _run_three_ways(dsb, ref, make, call, ("bf16", "fp8_tensor", "int8_channel"))
    _report_and_check("reference FluxJointTransformerBlock d=1024", outs, exact)


def test_reference_flux_single_block_through_the_seams(dsb, cuda_dev, ref):
    d, H, side, S_txt = 1024, 8, 24, 80
    sd = {k: v.bfloat16().float() for k, v in synth.make_state_dict(synth.flux_block_shapes("", d, H, "single"), seed=94).items()}
    x, temb = synth.randn((1, S_txt + side * side, d), 95).bfloat16(), synth.randn((1, d), 96).bfloat16()
    ids = _flux_ids(S_txt, side)
    rope = ref.transformer_helper.RoPEEmbedding(d, 10000, [16, 56, 56])(ids[None]).to(cuda_dev)
    exact = OF.single_block(x[0].float(), temb[0].float(), O.flux_rope_table(ids), sd, "", H, LinearEval("fp32"))

    def make():
        return _load(ref.flux_dit.FluxSingleTransformerBlock(d, H, device="cpu", dtype=torch.float32), sd, cuda_dev)

    def call(blk):
        return blk(x.to(cuda_dev), None, temb.to(cuda_dev), rope)[0][0].float().cpu()

    outs = _run_three_ways(dsb, ref, make, call, ("bf16", "fp8_tensor"))
    _report_and_check("reference FluxSingleTransformerBlock d=1024", outs, exact)


def test_reference_wan_block_through_the_seams(dsb, cuda_dev, ref):
    d, H, ffn = 1024, 8, 2816
    fr, hh, ww = 3, 12, 20
    S = fr * hh * ww
    sd = {k: v.bfloat16().float() for k, v in synth.make_state_dict(synth.wan_block_shapes("", d, ffn), seed=97).items()}
    x, ctx, tmod = synth.randn((1, S, d), 98).bfloat16(), synth.randn((1, 77, d), 99).bfloat16(), (synth.randn((1, 6, d), 100) * 0.1).bfloat16()
    table = O.wan_rope_table(fr, hh, ww)
    exact = OW.wan_block(x[0].float(), ctx[0].float(), tmod[0].float(), table, sd, "", H, LinearEval("fp32"))
    f_, h_, w_ = ref.wan_dit.precompute_freqs_cis_3d(d // H)
    freqs = torch.cat([f_[:fr].view(fr, 1, 1, -1).expand(fr, hh, ww, -1), h_[:hh].view(1, hh, 1, -1).expand(fr, hh, ww, -1),
                       w_[:ww].view(1, 1, ww, -1).expand(fr, hh, ww, -1)], dim=-1).reshape(S, 1, -1).to(cuda_dev)

    def make():
        return _load(ref.wan_dit.DiTBlock(False, d, H, ffn, 1e-6, device="cpu", dtype=torch.float32), sd, cuda_dev)

    def call(blk):
        return blk(x.to(cuda_dev), ctx.to(cuda_dev), tmod.to(cuda_dev), freqs)[0].float().cpu()

    outs = _run_three_ways(dsb, ref, make, call, ("bf16", "fp8_channel"))
    _report_and_check("reference DiTBlock d=1024", outs, exact)
