"""Seeded synthetic weights and inputs with the shapes of the benchmark configurations
(random-init N(0, 0.02) Linear weights and biases, N(0,1) activations); no checkpoint is read.

Parameter names follow the reference's modules (``FluxDiT`` / ``WanDiT`` state-dict keys) so the same
dictionaries drive the reference, the CPU oracle and this library."""
from typing import Dict, Tuple

import torch


def _normal(shape, std, gen, device, dtype=torch.float32):
    return (torch.randn(shape, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)


def init_param(name: str, shape, gen, device="cpu", dtype=torch.float32):
    """N(0,0.02) for Linear/Conv weights and biases; 1 + N(0,0.02) for norm weights; N(0,1)/sqrt(dim) for the
    Wan ``modulation`` tables (as models/wan/wan_dit.py:183,232 initialises them)."""
    if name.endswith("modulation"):
        return _normal(shape, 1.0 / shape[-1] ** 0.5, gen, device, dtype)
    is_norm = (".norm_q" in name or ".norm_k" in name or "norm3" in name or name.startswith("img_emb.proj.0")
               or name.startswith("img_emb.proj.4")) and name.endswith("weight")
    t = _normal(shape, 0.02, gen, device, dtype)
    return t + 1.0 if is_norm else t


def flux_block_shapes(pre: str, d: int, H: int, kind: str) -> Dict[str, Tuple[int, ...]]:
    hd = d // H
    s = {}
    def lin(n, o, i):
        s[pre + n + ".weight"] = (o, i)
        s[pre + n + ".bias"] = (o,)
    if kind == "double":
        lin("norm1_a.linear", 6 * d, d)
        lin("norm1_b.linear", 6 * d, d)
        lin("attn.a_to_qkv", 3 * d, d)
        lin("attn.b_to_qkv", 3 * d, d)
        for n in ("norm_q_a", "norm_k_a", "norm_q_b", "norm_k_b"):
            s[pre + f"attn.{n}.weight"] = (hd,)
        lin("attn.a_to_out", d, d)
        lin("attn.b_to_out", d, d)
        lin("ff_a.0", 4 * d, d)
        lin("ff_a.2", d, 4 * d)
        lin("ff_b.0", 4 * d, d)
        lin("ff_b.2", d, 4 * d)
    else:
        lin("norm.linear", 3 * d, d)
        lin("to_qkv_mlp", 7 * d, d)
        s[pre + "norm_q_a.weight"] = (hd,)
        s[pre + "norm_k_a.weight"] = (hd,)
        lin("proj_out", d, 5 * d)
    return s


def flux_dit_shapes(d=3072, H=24, n_double=19, n_single=38, in_ch=64, txt_dim=4096, pooled_dim=768,
                    guidance=True) -> Dict[str, Tuple[int, ...]]:
    s = {}
    def lin(n, o, i):
        s[n + ".weight"] = (o, i)
        s[n + ".bias"] = (o,)
    lin("time_embedder.timestep_embedder.0", d, 256)
    lin("time_embedder.timestep_embedder.2", d, d)
    if guidance:
        lin("guidance_embedder.timestep_embedder.0", d, 256)
        lin("guidance_embedder.timestep_embedder.2", d, d)
    lin("pooled_text_embedder.0", d, pooled_dim)
    lin("pooled_text_embedder.2", d, d)
    lin("context_embedder", d, txt_dim)
    lin("x_embedder", d, in_ch)
    for i in range(n_double):
        s.update(flux_block_shapes(f"blocks.{i}.", d, H, "double"))
    for i in range(n_single):
        s.update(flux_block_shapes(f"single_blocks.{i}.", d, H, "single"))
    lin("final_norm_out.linear", 2 * d, d)
    lin("final_proj_out", in_ch, d)
    return s


def wan_block_shapes(pre: str, d: int, ffn: int, has_image_input: bool = False) -> Dict[str, Tuple[int, ...]]:
    s = {}
    def lin(n, o, i):
        s[pre + n + ".weight"] = (o, i)
        s[pre + n + ".bias"] = (o,)
    for a in ("self_attn", "cross_attn"):
        for n in ("q", "k", "v", "o"):
            lin(f"{a}.{n}", d, d)
        s[pre + f"{a}.norm_q.weight"] = (d,)
        s[pre + f"{a}.norm_k.weight"] = (d,)
    s[pre + "norm3.weight"] = (d,)
    s[pre + "norm3.bias"] = (d,)
    lin("ffn.0", ffn, d)
    lin("ffn.2", d, ffn)
    s[pre + "modulation"] = (1, 6, d)
    if has_image_input:   # image-to-video: second key/value projection for the CLIP tokens (wan_dit.py:131-134)
        lin("cross_attn.k_img", d, d)
        lin("cross_attn.v_img", d, d)
        s[pre + "cross_attn.norm_k_img.weight"] = (d,)
    return s


def wan_dit_shapes(d=5120, ffn=13824, num_layers=40, in_dim=16, out_dim=16, text_dim=4096,
                   freq_dim=256, has_image_input: bool = False, clip_dim: int = 1280) -> Dict[str, Tuple[int, ...]]:
    """``has_image_input``: the image-to-video variant (``in_dim`` is then 36 in the released models: 16 latent +
    20 conditioning channels) with the CLIP-feature MLP ``img_emb`` (wan_dit.py:196-216,297-298)."""
    s = {"patch_embedding.weight": (d, in_dim, 1, 2, 2), "patch_embedding.bias": (d,)}
    def lin(n, o, i):
        s[n + ".weight"] = (o, i)
        s[n + ".bias"] = (o,)
    lin("text_embedding.0", d, text_dim)
    lin("text_embedding.2", d, d)
    lin("time_embedding.0", d, freq_dim)
    lin("time_embedding.2", d, d)
    lin("time_projection.1", 6 * d, d)
    for i in range(num_layers):
        s.update(wan_block_shapes(f"blocks.{i}.", d, ffn, has_image_input))
    lin("head.head", out_dim * 4, d)
    s["head.modulation"] = (1, 2, d)
    if has_image_input:
        s["img_emb.proj.0.weight"], s["img_emb.proj.0.bias"] = (clip_dim,), (clip_dim,)
        lin("img_emb.proj.1", clip_dim, clip_dim)
        lin("img_emb.proj.3", d, clip_dim)
        s["img_emb.proj.4.weight"], s["img_emb.proj.4.bias"] = (d,), (d,)
    return s


def make_state_dict(shapes: Dict[str, Tuple[int, ...]], seed=0, device="cpu", dtype=torch.float32):
    """One generator, parameters drawn in the dictionary's order."""
    gen = torch.Generator(device=device).manual_seed(seed)
    return {k: init_param(k, shp, gen, device, dtype) for k, shp in shapes.items()}


def randn(shape, seed, device="cpu", dtype=torch.float32):
    gen = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=gen, device=device, dtype=torch.float32).to(dtype)
