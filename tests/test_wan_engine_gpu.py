"""The Wan step engine against the CPU oracle (reduced width/depth), and its sequence-parallel form on two GPUs
against the single-GPU result."""
import os

import pytest
import torch

from oracle import ops as O
from oracle import wan as OW
from oracle.flux import round_bf16
from oracle.linear import LinearEval

pytestmark = pytest.mark.gpu
synth = __import__("importlib").import_module("diffsynth_engine_b200.synth")

CFG = dict(d=256, ffn=512, num_layers=2, text_dim=64)
H = 2


def _case(seed=24, grid=(3, 8, 10), ctx=16):
    w = synth.make_state_dict(synth.wan_dit_shapes(**CFG), seed=seed)
    w = {k: v.bfloat16().float() for k, v in w.items()}
    x = synth.randn((1, 16, *grid), seed + 1).bfloat16().float()
    context = synth.randn((1, ctx, CFG["text_dim"]), seed + 2).bfloat16().float()
    return w, x, context, torch.tensor([417.0])


@pytest.mark.parametrize("fmt", ["fp8_channel", "fp8_tensor", "int8_channel", "bf16"])
def test_wan_engine_matches_oracle(dsb, cuda_dev, fmt):
    from diffsynth_engine_b200.wan import WanDiTEngine
    w, x, context, t = _case()
    ref = OW.wan_dit_forward(w, x, context, t, num_layers=2, H=H, lin=LinearEval(fmt), rt=round_bf16)
    eng = WanDiTEngine(dict(w), fmt=fmt, device=cuda_dev, num_layers=2, num_heads=H)
    out = eng(x.to(cuda_dev), context.to(cuda_dev), t.to(cuda_dev)).float().cpu()
    dsb.ops.check_status(0)
    err = O.rel_l2(out, ref)
    exact = O.rel_l2(out, OW.wan_dit_forward(w, x, context, t, num_layers=2, H=H))
    print(f"wan tiny model {fmt}: rel-L2 vs same-quantisation oracle {err:.3e}, vs exact fp32 {exact:.3e}")
    assert out.shape == ref.shape
    assert err < (4e-3 if fmt == "bf16" else 2e-2)


def _i2v_case(seed=40, grid=(3, 8, 10), ctx=16):
    w = synth.make_state_dict(synth.wan_dit_shapes(**CFG, in_dim=36, has_image_input=True), seed=seed)
    w = {k: v.bfloat16().float() for k, v in w.items()}
    x = synth.randn((1, 16, *grid), seed + 1).bfloat16().float()
    y = synth.randn((1, 20, *grid), seed + 2).bfloat16().float()
    clip = synth.randn((1, 257, 1280), seed + 3).bfloat16().float()
    context = synth.randn((1, ctx, CFG["text_dim"]), seed + 4).bfloat16().float()
    return w, x, context, torch.tensor([417.0]), clip, y


@pytest.mark.parametrize("fmt", ["fp8_channel", "bf16"])
def test_wan_image_to_video_engine_matches_oracle(dsb, cuda_dev, fmt):
    """Image-to-video weights: 36 input channels (x | y), the CLIP-feature MLP (exact GELU, LayerNorm eps 1e-5) and
    the second key/value projection of every cross-attention over the 257 CLIP tokens."""
    from diffsynth_engine_b200.wan import WanDiTEngine
    w, x, context, t, clip, y = _i2v_case()
    ref = OW.wan_dit_forward(w, x, context, t, num_layers=2, H=H, lin=LinearEval(fmt), rt=round_bf16,
                             clip_feature=clip, y=y)
    eng = WanDiTEngine(dict(w), fmt=fmt, device=cuda_dev, num_layers=2, num_heads=H)
    dev = cuda_dev
    out = eng(x.to(dev), context.to(dev), t.to(dev), clip_feature=clip.to(dev), y=y.to(dev)).float().cpu()
    dsb.ops.check_status(0)
    err = O.rel_l2(out, ref)
    exact = O.rel_l2(out, OW.wan_dit_forward(w, x, context, t, num_layers=2, H=H, clip_feature=clip, y=y))
    print(f"wan tiny image-to-video model {fmt}: rel-L2 vs same-quantisation oracle {err:.3e}, vs exact fp32 {exact:.3e}")
    assert out.shape == ref.shape
    # whole model at width 256: every e4m3 rounding that falls on the other side of a tie between the two
    # implementations is a 6 % change of that element, and this model has more quantised Linears in series than the
    # text-to-video one (measured 2.6e-2; the bf16 run of the same dataflow sits at 2.9e-3)
    assert err < (4e-3 if fmt == "bf16" else 3e-2)
    with pytest.raises(ValueError):
        eng(x.to(dev), context.to(dev), t.to(dev))       # image-to-video weights without the image inputs


def test_wan_rope_table_matches_oracle(dsb, cuda_dev):
    from diffsynth_engine_b200.wan import wan_rope_table
    assert torch.equal(wan_rope_table(3, 4, 5, device=cuda_dev).cpu(), O.wan_rope_table(3, 4, 5))


def test_chunked_layout_kernels(dsb, cuda_dev):
    """rmsnorm_full writing the [P][rows][D/P] send layout and quant_rows reading it back."""
    g = torch.Generator().manual_seed(5)
    M, Hh, P = 50, 4, 2
    D = Hh * 128
    x = torch.randn(M, D, generator=g).bfloat16()
    wgt = 1 + 0.1 * torch.randn(D, generator=g)
    table = O.wan_rope_table(2, 5, 5)
    ref = O.apply_rope_pairs(O.rmsnorm(x, wgt).reshape(M, Hh, 128).transpose(0, 1), table[:M]).transpose(0, 1)
    ref = ref.reshape(M, D)
    out = torch.zeros(P, M, D // P, dtype=torch.bfloat16, device=cuda_dev)
    dsb.ops.rmsnorm_full(x.to(cuda_dev), wgt.to(cuda_dev), table.to(cuda_dev), 0, 1e-6, out=out, chunks=P)
    got = out.permute(1, 0, 2).reshape(M, D).float().cpu()
    assert O.rel_l2(got, ref) < 3e-3
    q, s = dsb.ops.quant_rows_chunked(out)
    q_ref, s_ref = O.quant_rows_e4m3(out.permute(1, 0, 2).reshape(M, D).float().cpu())
    assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu().view(torch.uint8), q_ref.view(torch.uint8))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("fmt,exchange", [("fp8_channel", "nccl"), ("bf16", "nccl"), ("fp8_channel", "peer"),
                                          ("bf16", "peer")])
def test_sequence_parallel_two_gpus_matches_one(dsb, cuda_dev, fmt, exchange):
    """UlyssesParallelModel (2 ranks) against the single-GPU engine on the same weights and inputs, with q and the
    attention output crossing ranks by all-to-all ("nccl") or inside the attention kernel over mapped peer memory
    ("peer": 240 tokens, 128-row slices, 16 padded rows on the second rank)."""
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from diffsynth_engine_b200.parallel import UlyssesParallelModel
    from diffsynth_engine_b200.wan import WanDiTEngine
    w, x, context, t = _case(seed=30, grid=(3, 16, 20) if exchange == "peer" else (3, 8, 10))
    one = WanDiTEngine(dict(w), fmt=fmt, device=cuda_dev, num_layers=2, num_heads=H)
    ref = one(x.to(cuda_dev), context.to(cuda_dev), t.to(cuda_dev)).float().cpu()
    model = UlyssesParallelModel(dict(w), sp_degree=2, master_port=29641, device="cuda", timeout_s=120, fmt=fmt,
                                 num_layers=2, num_heads=H, exchange=exchange)
    try:
        out = model(x=x, context=context, timestep=t).float().cpu()
        out2 = model(x=x, context=context, timestep=t).float().cpu()
    finally:
        model.close()
    # same kernels on the same numbers, only the attention tiling (heads per rank) differs
    assert O.rel_l2(out, ref) < 3e-3
    assert torch.equal(out, out2)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_parallel_image_to_video_two_gpus_matches_one(dsb, cuda_dev):
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from diffsynth_engine_b200.parallel import UlyssesParallelModel
    from diffsynth_engine_b200.wan import WanDiTEngine
    w, x, context, t, clip, y = _i2v_case(seed=50)
    dev = cuda_dev
    one = WanDiTEngine(dict(w), fmt="fp8_channel", device=dev, num_layers=2, num_heads=H)
    ref = one(x.to(dev), context.to(dev), t.to(dev), clip_feature=clip.to(dev), y=y.to(dev)).float().cpu()
    model = UlyssesParallelModel(dict(w), sp_degree=2, master_port=29643, device="cuda", timeout_s=120,
                                 fmt="fp8_channel", num_layers=2, num_heads=H)
    try:
        out = model(x=x, context=context, timestep=t, clip_feature=clip, y=y).float().cpu()
    finally:
        model.close()
    assert O.rel_l2(out, ref) < 3e-3


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_parallel_pads_a_token_count_that_does_not_split(dsb, cuda_dev):
    """3 x 7 x 5 = 105 tokens over two ranks: one padded row on the second rank, which must not act as a key and
    whose output is dropped."""
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from diffsynth_engine_b200.parallel import UlyssesParallelModel
    from diffsynth_engine_b200.wan import WanDiTEngine
    w, x, context, t = _case(seed=60, grid=(3, 14, 10))
    dev = cuda_dev
    one = WanDiTEngine(dict(w), fmt="fp8_channel", device=dev, num_layers=2, num_heads=H)
    ref = one(x.to(dev), context.to(dev), t.to(dev)).float().cpu()
    model = UlyssesParallelModel(dict(w), sp_degree=2, master_port=29645, device="cuda", timeout_s=120,
                                 fmt="fp8_channel", num_layers=2, num_heads=H)
    try:
        out = model(x=x, context=context, timestep=t).float().cpu()
    finally:
        model.close()
    assert out.shape == ref.shape
    assert O.rel_l2(out, ref) < 3e-3


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sequence_parallel_falls_back_to_all_to_all_without_peer_memory(dsb, cuda_dev):
    """``exchange="auto"`` on a system whose ranks cannot map each other's memory (the mapping raises on every rank):
    the engine says so on stderr, uses the all-to-all for all four tensors and still matches one GPU."""
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from diffsynth_engine_b200.parallel import UlyssesParallelModel
    from diffsynth_engine_b200.wan import WanDiTEngine
    from tests.parallel_helpers import wan_engine_factory_without_peer_memory
    w, x, context, t = _case(seed=70, grid=(3, 8, 10))
    one = WanDiTEngine(dict(w), fmt="fp8_channel", device=cuda_dev, num_layers=2, num_heads=H)
    ref = one(x.to(cuda_dev), context.to(cuda_dev), t.to(cuda_dev)).float().cpu()
    model = UlyssesParallelModel(dict(w), sp_degree=2, master_port=29647, device="cuda", timeout_s=120,
                                 factory=wan_engine_factory_without_peer_memory, fmt="fp8_channel", num_layers=2,
                                 num_heads=H, exchange="auto")
    try:
        out = model(x=x, context=context, timestep=t).float().cpu()
    finally:
        model.close()
    assert O.rel_l2(out, ref) < 3e-3
