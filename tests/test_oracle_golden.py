"""Pins the CPU oracle: every restated function against outputs of the reference itself
(``tests/golden/reference_outputs.safetensors``, made by ``tests/golden/make_golden.py``), including the two
fixtures of the reference's own test-suite for the sampler and the scheduler."""
import os

import pytest
import torch
from safetensors.torch import load_file

from oracle import flux as OF
from oracle import ops as O
from oracle import wan as OW
from oracle.linear import LinearEval

synth = __import__("importlib").import_module("diffsynth_engine_b200.synth")
G = load_file(os.path.join(os.path.dirname(__file__), "golden", "reference_outputs.safetensors"))
TOL = 2e-5  # fp32 restatement vs fp32 reference: accumulation order only


def flux_ids(S_txt, side):
    ids = torch.zeros(S_txt + side * side, 3)
    r = torch.arange(side, dtype=torch.float32)
    ids[S_txt:, 1] = r[:, None].expand(side, side).reshape(-1)
    ids[S_txt:, 2] = r[None, :].expand(side, side).reshape(-1)
    return ids


def test_rope_table():
    t = O.flux_rope_table(G["rope.ids"])
    ref = G["rope.table"]  # [[cos, -sin], [sin, cos]]
    assert torch.equal(t[..., 0], ref[..., 0, 0]) and torch.equal(t[..., 1], ref[..., 1, 0])
    assert torch.equal(-t[..., 1], ref[..., 0, 1]) and torch.equal(t[..., 0], ref[..., 1, 1])


def test_timestep_embeddings():
    assert torch.allclose(O.timestep_embedding_flux(G["timestep.t"]), G["timestep.emb"], rtol=0, atol=1e-6)
    assert torch.allclose(O.sinusoidal_embedding_wan(256, G["timestep.t"]).float(), G["wan_sinusoid"], rtol=0,
                          atol=1e-7)


def test_wan_rope():
    table = O.wan_rope_table(3, 4, 5)
    assert torch.allclose(table, G["wan_rope.cos_sin"], rtol=0, atol=1e-7)
    x = synth.randn((1, 60, 256), 11)
    got = OW._rope(x[0], table, 2)
    assert O.rel_l2(got, G["wan_rope.applied"][0]) < 1e-6


def test_rmsnorm():
    w = 1 + 0.1 * synth.randn((128,), 12)
    assert O.rel_l2(O.rmsnorm(synth.randn((2, 3, 5, 128), 13), w), G["rmsnorm.out"]) < 1e-6


def test_flux_double_block_small():
    d, H, side, S_txt = 256, 2, 8, 32
    w = synth.make_state_dict(synth.flux_block_shapes("", d, H, "double"), seed=0)
    xa, xb, temb = synth.randn((1, side * side, d), 1)[0], synth.randn((1, S_txt, d), 2)[0], synth.randn((1, d), 3)[0]
    ya, yb = OF.double_block(xa, xb, temb, O.flux_rope_table(flux_ids(S_txt, side)), w, "", H, LinearEval("fp32"))
    assert O.rel_l2(ya, G["flux_double_small.out_a"]) < TOL
    assert O.rel_l2(yb, G["flux_double_small.out_b"]) < TOL


def test_flux_double_block_c1_config():
    """The CPU-runnable benchmark configuration: one double-stream block, hidden 3072, 24 heads, 1024 image + 512 text
    tokens, fp32."""
    d, H, side, S_txt = 3072, 24, 32, 512
    w = synth.make_state_dict(synth.flux_block_shapes("", d, H, "double"), seed=0)
    xa, xb, temb = synth.randn((1, side * side, d), 1)[0], synth.randn((1, S_txt, d), 2)[0], synth.randn((1, d), 3)[0]
    ya, yb = OF.double_block(xa, xb, temb, O.flux_rope_table(flux_ids(S_txt, side)), w, "", H, LinearEval("fp32"))
    assert O.rel_l2(ya[G["flux_double_c1.rows_a"]], G["flux_double_c1.out_a"]) < TOL
    assert O.rel_l2(yb[G["flux_double_c1.rows_b"]], G["flux_double_c1.out_b"]) < TOL


def test_flux_single_block_small():
    d, H, side, S_txt = 256, 2, 8, 32
    w = synth.make_state_dict(synth.flux_block_shapes("", d, H, "single"), seed=4)
    x, temb = synth.randn((1, S_txt + side * side, d), 5)[0], synth.randn((1, d), 6)[0]
    y = OF.single_block(x, temb, O.flux_rope_table(flux_ids(S_txt, side)), w, "", H, LinearEval("fp32"))
    assert O.rel_l2(y, G["flux_single_small.out"]) < TOL


def test_flux_dit_forward_glue():
    """FluxDiT.forward (embedders, patchify, block order, text/image concat, final AdaLN, unpatchify) with one
    double and one single block at the real width."""
    w = synth.make_state_dict(synth.flux_dit_shapes(n_double=1, n_single=1), seed=7)
    lat, pe, pooled = synth.randn((1, 16, 16, 16), 8), synth.randn((1, 32, 4096), 9), synth.randn((1, 768), 10)
    y = OF.flux_dit_forward(w, lat, torch.tensor([500.0]), pe, pooled, torch.tensor([3.5]), n_double=1, n_single=1)
    assert O.rel_l2(y, G["flux_dit_1p1.out"]) < TOL


def test_wan_block_small():
    d, H, ffn = 256, 2, 512
    w = synth.make_state_dict(synth.wan_block_shapes("", d, ffn), seed=20)
    x, ctx, tmod = synth.randn((1, 60, d), 21)[0], synth.randn((1, 16, d), 22)[0], synth.randn((1, 6, d), 23)[0] * 0.1
    y = OW.wan_block(x, ctx, tmod, O.wan_rope_table(3, 4, 5), w, "", H, LinearEval("fp32"))
    assert O.rel_l2(y, G["wan_block_small.out"]) < TOL


def test_wan_dit_tiny():
    w = synth.make_state_dict(synth.wan_dit_shapes(d=256, ffn=512, num_layers=2, text_dim=64), seed=24)
    y = OW.wan_dit_forward(w, synth.randn((1, 16, 3, 8, 10), 25), synth.randn((1, 16, 64), 26),
                           torch.tensor([417.0]), num_layers=2, H=2)
    assert O.rel_l2(y, G["wan_dit_tiny.out"]) < TOL


def test_wan_dit_tiny_image_to_video():
    w = synth.make_state_dict(synth.wan_dit_shapes(d=256, ffn=512, num_layers=2, text_dim=64, in_dim=36,
                                                   has_image_input=True), seed=27)
    y = OW.wan_dit_forward(w, synth.randn((1, 16, 3, 8, 10), 25), synth.randn((1, 16, 64), 26),
                           torch.tensor([417.0]), num_layers=2, H=2, clip_feature=synth.randn((1, 257, 1280), 28),
                           y=synth.randn((1, 20, 3, 8, 10), 29))
    assert O.rel_l2(y, G["wan_dit_tiny_i2v.out"]) < TOL


def test_reference_suite_sampler_fixture():
    """tests/test_algorithm/test_sampler.py:22-42 of the reference, on a row subsample of its fixture."""
    mu = (1024 // 16 * 1024 // 16) * ((1.15 - 0.5) / (4096 - 256)) + (0.5 - ((1.15 - 0.5) / (4096 - 256)) * 256)
    sigmas, _ = O.rectified_flow_schedule(20, sigma_min=1.0 / 20, sigma_max=1.0, mu=mu)
    got = O.euler_step(G["ref_tests.euler.origin_sample"], G["ref_tests.euler.model_output"], sigmas, 10)
    assert torch.allclose(got, G["ref_tests.euler.prev_sample"], atol=1e-3, rtol=1e-3)  # the reference's tolerance
    assert O.rel_l2(got, G["ref_tests.euler.prev_sample"]) < 1e-6


def test_reference_suite_scheduler_fixture():
    """tests/test_algorithm/test_scheduler.py:44-58 of the reference."""
    mu = (1024 // 16 * 1024 // 16) * ((1.15 - 0.5) / (4096 - 256)) + (0.5 - ((1.15 - 0.5) / (4096 - 256)) * 256)
    sigmas, timesteps = O.rectified_flow_schedule(20, sigma_min=1.0 / 20, sigma_max=1.0, mu=mu)
    assert torch.allclose(sigmas, G["ref_tests.sigmas"], atol=1e-6, rtol=1e-6)
    assert torch.allclose(timesteps, G["ref_tests.timesteps"], atol=1e-3, rtol=1e-6)


def test_fp8_unit_scale_linear_matches_reference_path():
    """The reference's shipped FP8 Linear (unit scales, utils/fp8_linear.py:27-60): cast both operands to e4m3,
    fp32 accumulate, add bias, round to bf16."""
    W, b, x = synth.randn((128, 256), 30) * 0.5, synth.randn((128,), 31) * 0.1, synth.randn((2, 24, 256), 32)
    xq = x.bfloat16().reshape(-1, 256).to(torch.float8_e4m3fn).float()
    y = (xq @ W.to(torch.float8_e4m3fn).float().t() + b.bfloat16().float()).bfloat16().float().reshape(2, 24, 128)
    # cuBLAS-free CPU fallback of _scaled_mm rounds once to bf16, like this restatement; allow one bf16 ulp
    assert O.rel_l2(y, G["fp8_linear_unit_scale.out"]) < 4e-3


def lora_case():
    """Inputs of the ``lora_linear.out`` fixture: (x, W, b, [(coef, up, down)])."""
    W, b = synth.randn((192, 256), 60) * 0.05, synth.randn((192,), 61) * 0.1
    loras = [(0.8 * 16 / 8, synth.randn((192, 8), 62) * 0.02, synth.randn((8, 256), 63) * 0.06),
             (1.0 * 4 / 4, synth.randn((192, 4), 64) * 0.02, synth.randn((4, 256), 65) * 0.06)]
    return synth.randn((40, 256), 66), W, b, loras


def test_lora_linear_restatement_and_quantised_extension():
    from oracle.linear import lora_linear_quant, lora_reference
    x, W, b, loras = lora_case()
    ref = lora_reference(x, W, b, loras)
    assert O.rel_l2(ref, G["lora_linear.out"]) < TOL
    # the K-extension form reproduces the LoRA sum to quantisation accuracy, and the LoRA part itself (not just the
    # main product) is resolved: its error is small against the size of the LoRA contribution
    delta = ref - (x @ W.t() + b)
    for mode in ("fp8_tensor", "fp8_channel", "int8_channel"):
        y = lora_linear_quant(x, W, b, loras, mode)
        base = LinearEval(mode)(x, W, b)
        assert O.rel_l2(y, ref) < 5e-2
        assert O.rel_l2(y - base, delta) < 5e-2, mode


def test_q8_0_dequantisation_matches_reference():
    raw = G["q8_0.raw"]
    assert torch.equal(raw, O.q8_0_quantize(synth.randn((24, 128), 67) * 0.05))
    assert torch.equal(O.q8_0_dequantize(raw, torch.bfloat16).float(), G["q8_0.dequant_bf16"])
    assert torch.equal(O.q8_0_dequantize(raw, torch.float32), G["q8_0.dequant_f32"])
    w = synth.randn((24, 128), 67) * 0.05
    assert O.rel_l2(G["q8_0.dequant_f32"], w) < 1e-2     # Q8_0 itself: 8-bit blocks of 32


def test_q4_k_dequantisation_matches_reference():
    raw = G["q4_k.raw"]
    assert torch.equal(raw, O.q4_k_random_blocks(6, 512, 68))
    assert torch.equal(O.q4_k_dequantize(raw, torch.bfloat16).float(), G["q4_k.dequant_bf16"])
    assert torch.equal(O.q4_k_dequantize(raw, torch.float32), G["q4_k.dequant_f32"])


@pytest.mark.parametrize("qtype", ["Q4_0", "Q4_1", "Q5_0", "Q5_1", "Q8_0", "Q2_K", "Q3_K", "Q4_K", "Q5_K", "Q6_K"])
def test_gguf_block_formats_match_reference(qtype):
    """Every GGUF block format the reference dequantises (utils/gguf.py:171-368): the element-by-element restatement
    in oracle/gguf.py against what the reference's ``dequantize`` made of the same seeded bytes, bit for bit, with bf16
    and with fp32 as compute dtype."""
    from oracle import gguf as OG
    GG = load_file(os.path.join(os.path.dirname(__file__), "golden", "gguf_blocks.safetensors"))
    raw = GG[f"{qtype}.raw"]
    i = sorted(OG.SIZES).index(qtype)
    assert torch.equal(raw, OG.random_blocks(qtype, 3, 512, 700 + i))
    assert torch.equal(OG.dequantize(raw, qtype, torch.bfloat16).float(), GG[f"{qtype}.bf16"])
    assert torch.equal(OG.dequantize(raw, qtype, torch.float32), GG[f"{qtype}.f32"])
