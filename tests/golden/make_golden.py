"""Generates the fixtures in this directory by EXECUTING THE REFERENCE (modelscope/DiffSynth-Engine
v0.1.1, imported from its source tree) on seeded inputs.  Run where the reference is mounted:

    python tests/golden/make_golden.py <path to the DiffSynth-Engine source tree>             # reference_outputs.safetensors
    python tests/golden/make_golden.py <path to the DiffSynth-Engine source tree> --gguf      # gguf_blocks.safetensors

Only outputs (and small inputs) are stored; weights and large inputs are regenerated from their seeds by
``diffsynth-engine_b200/synth.py``, which the reference run, the oracle and the CUDA path all share.
The package's ``__init__`` pulls in download/video helpers whose dependencies are absent, so the
hot-path modules are imported through a bare namespace package instead.
"""
import os
import sys
import types

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from tests.conftest import load_package  # noqa: E402

synth = __import__("importlib").import_module("diffsynth_engine_b200.synth") if load_package() else None


def import_reference(ref_root):
    m = types.ModuleType("diffsynth_engine")
    m.__path__ = [os.path.join(ref_root, "diffsynth_engine")]
    sys.modules["diffsynth_engine"] = m
    from diffsynth_engine.models.flux import flux_dit
    from diffsynth_engine.models.wan import wan_dit
    from diffsynth_engine.models.basic import transformer_helper, timestep
    from diffsynth_engine.utils import fp8_linear
    return flux_dit, wan_dit, transformer_helper, timestep, fp8_linear


def load_into(module, sd):
    # nn.Module's own loader: PreTrainedModel.load_state_dict routes through a key converter and returns None
    res = torch.nn.Module.load_state_dict(module, sd, strict=True)
    assert not res.missing_keys and not res.unexpected_keys, res
    return module


def sample_rows(n):
    """Row subset stored for large outputs: the first three rows and every 97th."""
    idx = sorted(set([0, 1, 2] + list(range(0, n, 97)) + [n - 1]))
    return torch.tensor(idx)


def flux_ids(S_txt, side):
    ids = torch.zeros(S_txt + side * side, 3)
    r = torch.arange(side, dtype=torch.float32)
    ids[S_txt:, 1] = r[:, None].expand(side, side).reshape(-1)
    ids[S_txt:, 2] = r[None, :].expand(side, side).reshape(-1)
    return ids


@torch.no_grad()
def gguf_fixtures(ref_root):
    """``gguf_blocks.safetensors``: for every GGUF block format the reference dequantises (utils/gguf.py:137-147),
    seeded well-formed random blocks and what the reference's ``dequantize`` makes of them with bf16 and fp32 as
    compute dtype."""
    import_reference(ref_root)
    import gguf as gguf_pkg
    from diffsynth_engine.utils import gguf as ref_gguf
    from oracle import gguf as OG
    out = {}
    for i, qt in enumerate(sorted(OG.SIZES)):
        raw = OG.random_blocks(qt, 3, 512, 700 + i)
        qd = getattr(gguf_pkg.GGMLQuantizationType, qt)
        out[f"{qt}.raw"] = raw
        out[f"{qt}.bf16"] = ref_gguf.dequantize(raw, quant_dtype=qd, compute_dtype=torch.bfloat16).float()
        out[f"{qt}.f32"] = ref_gguf.dequantize(raw, quant_dtype=qd, compute_dtype=torch.float32)
    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(HERE, "gguf_blocks.safetensors"))
    print("wrote gguf_blocks.safetensors:", sorted(out))


@torch.no_grad()
def main(ref_root):
    flux_dit, wan_dit, th, ts, fp8 = import_reference(ref_root)
    out = {}
    torch.manual_seed(0)

    # ---- elementary pieces
    ids = flux_ids(8, 4)
    out["rope.ids"] = ids
    out["rope.table"] = th.RoPEEmbedding(3072, 10000, [16, 56, 56])(ids[None])[0, 0].contiguous()  # [S,64,2,2]
    t = torch.tensor([0.0, 1.0, 500.0, 999.0, 37.25])
    out["timestep.t"] = t
    out["timestep.emb"] = ts.get_timestep_embedding(t, 256, flip_sin_to_cos=True, downscale_freq_shift=0)
    out["wan_sinusoid"] = wan_dit.sinusoidal_embedding_1d(256, t.double()).float()
    f_, h_, w_ = wan_dit.precompute_freqs_cis_3d(128)
    fr = torch.cat([f_[:3].view(3, 1, 1, -1).expand(3, 4, 5, -1), h_[:4].view(1, 4, 1, -1).expand(3, 4, 5, -1),
                    w_[:5].view(1, 1, 5, -1).expand(3, 4, 5, -1)], dim=-1).reshape(60, -1)
    out["wan_rope.cos_sin"] = torch.stack([fr.real, fr.imag], dim=-1).float()
    x = synth.randn((1, 60, 2 * 128), 11)
    out["wan_rope.applied"] = wan_dit.rope_apply(x, fr.reshape(60, 1, -1), 2)
    rn = th.RMSNorm(128, eps=1e-6, device="cpu", dtype=torch.float32)
    rn.weight.copy_(1 + 0.1 * synth.randn((128,), 12))
    out["rmsnorm.out"] = rn(synth.randn((2, 3, 5, 128), 13))

    # ---- Flux double block, small (d=256, 2 heads) and the benchmark's CPU config (d=3072, 24 heads)
    for tag, d, H, side, S_txt in (("flux_double_small", 256, 2, 8, 32), ("flux_double_c1", 3072, 24, 32, 512)):
        sd = synth.make_state_dict(synth.flux_block_shapes("", d, H, "double"), seed=0)
        blk = load_into(flux_dit.FluxJointTransformerBlock(d, H, device="cpu", dtype=torch.float32), sd)
        xa, xb, temb = synth.randn((1, side * side, d), 1), synth.randn((1, S_txt, d), 2), synth.randn((1, d), 3)
        rope = th.RoPEEmbedding(d, 10000, [16, 56, 56])(flux_ids(S_txt, side)[None])
        ya, yb = blk(xa, xb, temb, rope)
        if d == 256:
            out[f"{tag}.out_a"], out[f"{tag}.out_b"] = ya[0], yb[0]
        else:
            ia, ib = sample_rows(ya.shape[1]), sample_rows(yb.shape[1])
            out[f"{tag}.rows_a"], out[f"{tag}.rows_b"] = ia, ib
            out[f"{tag}.out_a"], out[f"{tag}.out_b"] = ya[0, ia].contiguous(), yb[0, ib].contiguous()

    # ---- Flux single block, small
    d, H, side, S_txt = 256, 2, 8, 32
    sd = synth.make_state_dict(synth.flux_block_shapes("", d, H, "single"), seed=4)
    blk = load_into(flux_dit.FluxSingleTransformerBlock(d, H, device="cpu", dtype=torch.float32), sd)
    x, temb = synth.randn((1, S_txt + side * side, d), 5), synth.randn((1, d), 6)
    rope = th.RoPEEmbedding(d, 10000, [16, 56, 56])(flux_ids(S_txt, side)[None])
    out["flux_single_small.out"] = blk(x, None, temb, rope)[0][0]

    # ---- FluxDiT.forward glue: the reference's forward on a model with 1 double + 1 single block
    class OneOfEach(flux_dit.FluxDiT):
        def __init__(self):  # same attributes as FluxDiT.__init__ (flux_dit.py:341-364), fewer blocks
            torch.nn.Module.__init__(self)
            kw = dict(device="cpu", dtype=torch.float32)
            self.pos_embedder = th.RoPEEmbedding(3072, 10000, [16, 56, 56])
            self.time_embedder = ts.TimestepEmbeddings(256, 3072, **kw)
            self.guidance_embedder = ts.TimestepEmbeddings(256, 3072, **kw)
            self.pooled_text_embedder = torch.nn.Sequential(torch.nn.Linear(768, 3072), torch.nn.SiLU(),
                                                            torch.nn.Linear(3072, 3072))
            self.context_embedder = torch.nn.Linear(4096, 3072)
            self.x_embedder = torch.nn.Linear(64, 3072)
            self.blocks = torch.nn.ModuleList([flux_dit.FluxJointTransformerBlock(3072, 24, **kw)])
            self.single_blocks = torch.nn.ModuleList([flux_dit.FluxSingleTransformerBlock(3072, 24, **kw)])
            self.final_norm_out = flux_dit.AdaLayerNormContinuous(3072, **kw)
            self.final_proj_out = torch.nn.Linear(3072, 64)

    sd = synth.make_state_dict(synth.flux_dit_shapes(n_double=1, n_single=1), seed=7)
    model = load_into(OneOfEach(), sd).eval()
    lat, pe, pooled = synth.randn((1, 16, 16, 16), 8), synth.randn((1, 32, 4096), 9), synth.randn((1, 768), 10)
    out["flux_dit_1p1.out"] = model(lat, torch.tensor([500.0]), pe, pooled, torch.tensor([3.5]),
                                    torch.zeros(1, 32, 3))
    del model, sd

    # ---- Wan block (small) and a tiny complete WanDiT
    d, H, ffn = 256, 2, 512
    sd = synth.make_state_dict(synth.wan_block_shapes("", d, ffn), seed=20)
    blk = load_into(wan_dit.DiTBlock(False, d, H, ffn, 1e-6, device="cpu", dtype=torch.float32), sd)
    x, ctx, tmod = synth.randn((1, 60, d), 21), synth.randn((1, 16, d), 22), synth.randn((1, 6, d), 23) * 0.1
    out["wan_block_small.out"] = blk(x, ctx, tmod, fr.reshape(60, 1, -1))[0]

    cfg = dict(dim=256, in_dim=16, ffn_dim=512, out_dim=16, text_dim=64, freq_dim=256, eps=1e-6, patch_size=(1, 2, 2),
               num_heads=2, num_layers=2, has_image_input=False)
    sd = synth.make_state_dict(synth.wan_dit_shapes(d=256, ffn=512, num_layers=2, text_dim=64), seed=24)
    model = load_into(wan_dit.WanDiT(**cfg, device="cpu", dtype=torch.float32), sd).eval()
    out["wan_dit_tiny.out"] = model(synth.randn((1, 16, 3, 8, 10), 25), synth.randn((1, 16, 64), 26),
                                    torch.tensor([417.0]))

    # ---- the image-to-video variant of the same tiny model (CLIP-token branch of the cross-attention, img_emb MLP)
    cfg_i2v = dict(cfg, in_dim=36, has_image_input=True)
    sd = synth.make_state_dict(synth.wan_dit_shapes(d=256, ffn=512, num_layers=2, text_dim=64, in_dim=36,
                                                    has_image_input=True), seed=27)
    model = load_into(wan_dit.WanDiT(**cfg_i2v, device="cpu", dtype=torch.float32), sd).eval()
    out["wan_dit_tiny_i2v.out"] = model(synth.randn((1, 16, 3, 8, 10), 25), synth.randn((1, 16, 64), 26),
                                        torch.tensor([417.0]), clip_feature=synth.randn((1, 257, 1280), 28),
                                        y=synth.randn((1, 20, 3, 8, 10), 29))

    # ---- LoRALinear with two unfused adapters (models/basic/lora.py:137-141), fp32
    from diffsynth_engine.models.basic.lora import LoRALinear
    ll = LoRALinear(256, 192)
    ll.weight.copy_(synth.randn((192, 256), 60) * 0.05)
    ll.bias.copy_(synth.randn((192,), 61) * 0.1)
    ll.add_lora("a", 0.8, 8, 16, synth.randn((192, 8), 62) * 0.02, synth.randn((8, 256), 63) * 0.06, "cpu", torch.float32)
    ll.add_lora("b", 1.0, 4, 4, synth.randn((192, 4), 64) * 0.02, synth.randn((4, 256), 65) * 0.06, "cpu", torch.float32)
    out["lora_linear.out"] = ll(synth.randn((40, 256), 66))

    # ---- GGUF Q8_0 block dequantisation (utils/gguf.py:113-135,171-175) on seeded raw bytes
    import gguf as gguf_pkg
    from diffsynth_engine.utils import gguf as ref_gguf
    from oracle.ops import q8_0_quantize
    raw = q8_0_quantize(synth.randn((24, 128), 67) * 0.05)
    out["q8_0.raw"] = raw
    out["q8_0.dequant_bf16"] = ref_gguf.dequantize(raw, quant_dtype=gguf_pkg.GGMLQuantizationType.Q8_0,
                                                   compute_dtype=torch.bfloat16).float()
    out["q8_0.dequant_f32"] = ref_gguf.dequantize(raw, quant_dtype=gguf_pkg.GGMLQuantizationType.Q8_0,
                                                  compute_dtype=torch.float32)

    from oracle.ops import q4_k_random_blocks
    raw4 = q4_k_random_blocks(6, 512, 68)
    out["q4_k.raw"] = raw4
    out["q4_k.dequant_bf16"] = ref_gguf.dequantize(raw4, quant_dtype=gguf_pkg.GGMLQuantizationType.Q4_K,
                                                   compute_dtype=torch.bfloat16).float()
    out["q4_k.dequant_f32"] = ref_gguf.dequantize(raw4, quant_dtype=gguf_pkg.GGMLQuantizationType.Q4_K,
                                                  compute_dtype=torch.float32)

    # ---- the reference's FP8 Linear as shipped (unit scales) on a small case, for the drop-in patch
    lin = torch.nn.Linear(256, 128)
    lin.weight.copy_(synth.randn((128, 256), 30) * 0.5)
    lin.bias.copy_(synth.randn((128,), 31) * 0.1)
    x = synth.randn((2, 24, 256), 32)
    fp8.enable_fp8_linear(lin)
    with fp8.fp8_inference(True):
        out["fp8_linear_unit_scale.out"] = lin(x.bfloat16()).float()

    # ---- the fixtures the reference's own test-suite ships for the op either side of the DiT step
    # (tests/test_algorithm/test_sampler.py:22-42, test_scheduler.py:44-58): kept as a row subsample
    from safetensors.torch import load_file
    exp = os.path.join(ref_root, "tests", "data", "expect", "algorithm")
    fm = load_file(os.path.join(exp, "flow_match_euler_i10.safetensors"))
    rows = sample_rows(fm["origin_sample"].shape[1])
    out["ref_tests.euler_rows"] = rows
    for k in ("origin_sample", "model_output", "prev_sample"):
        out[f"ref_tests.euler.{k}"] = fm[k][:, rows].contiguous()
    sch = load_file(os.path.join(exp, "recifited_flow_20steps_flux.safetensors"))
    out["ref_tests.sigmas"], out["ref_tests.timesteps"] = sch["sigmas"], sch["timesteps"]

    save_file({k: v.contiguous() for k, v in out.items()}, os.path.join(HERE, "reference_outputs.safetensors"))
    for k, v in out.items():
        print(f"{k:40s} {tuple(v.shape)} {v.dtype}")


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.expanduser("~"), "reference")
    if "--gguf" in sys.argv:
        gguf_fixtures(root)
    else:
        main(root)
