"""Wan2.1 DiT forward restated functionally over a reference-named state dict (fp32 on the CPU).
Citations: ``diffsynth_engine/models/wan/wan_dit.py`` of modelscope/DiffSynth-Engine v0.1.1."""
import torch
import torch.nn.functional as F

from . import ops as O
from .linear import LinearEval


IMG_TOKENS = 257   # CLIP tokens at the head of the context of image-to-video models (wan_dit.py:138-139)


def _ident(x):
    return x


def _mh(x, H):
    return x.reshape(x.shape[0], H, -1).transpose(0, 1)  # [H, S, D]


def _attend(q, k, v, H, rt=_ident):
    """wan_dit.py:18-22.  With a rounding ``rt`` (the same-rounding oracle) the probabilities are rounded to bf16 as a
    GPU flash kernel does."""
    attn = O.attention if rt is _ident else O.attention_bf16_probs
    o = attn(_mh(q, H)[None], _mh(k, H)[None], _mh(v, H)[None])[0]
    return o.transpose(0, 1).reshape(q.shape[0], -1)


def _rope(x, table, H):
    """wan_dit.py:54-58 (complex multiply of adjacent pairs == the 2x2 rotation)."""
    return O.apply_rope_pairs(_mh(x, H), table).transpose(0, 1).reshape(x.shape[0], -1)


def wan_block(x, context, t_mod, table, w, pre, H, lin: LinearEval, rt=_ident, eps=1e-6, other_kv=None):
    """DiTBlock.forward, wan_dit.py:185-193.  x [S,d], context [L,d], t_mod [6,d].
    ``other_kv = (k, v)``: keys and values (normalised and rotated, [S', d]) of tokens OUTSIDE ``x`` that the
    self-attention also attends to - the block as one rank of a sequence-parallel group evaluates it (its own token
    slice as queries, everybody's tokens as keys); used by the benchmark's CPU arm to time a 1/P share of a block."""
    mod = w[pre + "modulation"].float().reshape(6, -1) + t_mod.float()
    sh_msa, sc_msa, g_msa, sh_mlp, sc_mlp, g_mlp = mod
    def L(inp, name, **kw):
        return lin(inp, w[pre + name + ".weight"], w[pre + name + ".bias"], **kw)
    # self-attention, wan_dit.py:101-107
    n = O.ln_modulate(x, sh_msa, sc_msa, eps)
    # the projection is rounded (it is stored), norm and rotation then run in one pass with one rounding at its end
    q = O.rmsnorm(rt(L(n, "self_attn.q", from_fp32=True)), w[pre + "self_attn.norm_q.weight"], eps)
    k = O.rmsnorm(rt(L(n, "self_attn.k", from_fp32=True)), w[pre + "self_attn.norm_k.weight"], eps)
    v = rt(L(n, "self_attn.v", from_fp32=True))
    q, k = rt(_rope(q, table, H)), rt(_rope(k, table, H))
    if other_kv is not None:
        k, v = torch.cat([k, other_kv[0]], dim=0), torch.cat([v, other_kv[1]], dim=0)
    x = rt(x.float() + g_msa * L(rt(_attend(q, k, v, H, rt)), "self_attn.o"))
    # cross-attention, wan_dit.py:136-152; norm3 is an affine LayerNorm (:178,190).  Image-to-video models carry
    # k_img/v_img: the first 257 context rows are CLIP tokens with their own key/value projection, attended
    # separately, and the two attention outputs are summed before the output projection (:137-152).
    has_img = (pre + "cross_attn.k_img.weight") in w
    img, ctx = (context[:IMG_TOKENS], context[IMG_TOKENS:]) if has_img else (None, context)
    n3 = O.layer_norm(x, eps) * w[pre + "norm3.weight"].float() + w[pre + "norm3.bias"].float()
    q = rt(O.rmsnorm(rt(L(n3, "cross_attn.q", from_fp32=True)), w[pre + "cross_attn.norm_q.weight"], eps))
    k = rt(O.rmsnorm(rt(L(ctx, "cross_attn.k")), w[pre + "cross_attn.norm_k.weight"], eps))
    v = rt(L(ctx, "cross_attn.v"))
    att = rt(_attend(q, k, v, H, rt))
    if has_img:
        k_i = rt(O.rmsnorm(rt(L(img, "cross_attn.k_img")), w[pre + "cross_attn.norm_k_img.weight"], eps))
        v_i = rt(L(img, "cross_attn.v_img"))
        att = rt(att + rt(_attend(q, k_i, v_i, H, rt)))
    x = rt(x + L(att, "cross_attn.o"))
    # FFN, wan_dit.py:179-182,191-192
    n2 = O.ln_modulate(x, sh_mlp, sc_mlp, eps)
    hid = O.gelu_tanh(L(n2, "ffn.0", from_fp32=True))
    if getattr(lin, "unit_scale_acts", False):   # FP8 weights: the first FFN GEMM emits e4m3 (unit scale) directly
        return rt(x + g_mlp * L(hid, "ffn.2", act_quant="unit"))
    return rt(x + g_mlp * L(rt(hid), "ffn.2"))


def patchify(x, w, lin):
    """Conv3d with kernel = stride = (1,2,2) == a Linear over (c, 1, y, z) patches, then
    b c f h w -> b (f h w) c (wan_dit.py:271-273,301-305).  x: [1, C, F, Hh, Ww]."""
    _, C, Fr, Hh, Ww = x.shape
    p = x[0].reshape(C, Fr, Hh // 2, 2, Ww // 2, 2).permute(1, 2, 4, 0, 3, 5).reshape(Fr * (Hh // 2) * (Ww // 2), C * 4)
    Wc = w["patch_embedding.weight"]
    return lin(p, Wc.reshape(Wc.shape[0], -1), w["patch_embedding.bias"]), (Fr, Hh // 2, Ww // 2)


def unpatchify(x, grid, out_dim):
    """b (f h w) (x y z c) -> b c (f x) (h y) (w z) with (x,y,z) = (1,2,2) (wan_dit.py:307-317)."""
    f, h, ww = grid
    return x.reshape(f, h, ww, 1, 2, 2, out_dim).permute(6, 0, 3, 1, 4, 2, 5).reshape(1, out_dim, f, h * 2, ww * 2)


def img_emb(clip_feature, w, lin, rt=_ident):
    """MLP of wan_dit.py:196-216 on the CLIP feature [257, 1280]: LayerNorm (eps 1e-5, affine) -> Linear -> exact
    GELU -> Linear -> LayerNorm."""
    def ln(t, i):
        return O.layer_norm(t, 1e-5) * w[f"img_emb.proj.{i}.weight"].float() + w[f"img_emb.proj.{i}.bias"].float()
    h = rt(F.gelu(lin(ln(clip_feature, 0), w["img_emb.proj.1.weight"], w["img_emb.proj.1.bias"], from_fp32=True)))
    return rt(ln(rt(lin(h, w["img_emb.proj.3.weight"], w["img_emb.proj.3.bias"])), 4))


def wan_dit_forward(w, x, context, timestep, num_layers, H, freq_dim=256, eps=1e-6, lin: LinearEval = None,
                    rt=_ident, clip_feature=None, y=None, return_hidden=False):
    """WanDiT.forward, wan_dit.py:319-351, batch 1.  With ``clip_feature`` [1,257,1280] and ``y`` (conditioning
    latents, concatenated to x on the channel axis) the image-to-video branch (:330-333)."""
    lin = lin or LinearEval("fp32")
    d = w["time_embedding.0.weight"].shape[0]
    def L(inp, name, **kw):
        return lin(inp, w[name + ".weight"], w[name + ".bias"], **kw)
    sin = rt(O.sinusoidal_embedding_wan(freq_dim, timestep).float())
    t = L(F.silu(L(sin, "time_embedding.0", act_quant=False)), "time_embedding.2", act_quant=False)   # [1,d]
    t_mod = L(F.silu(t), "time_projection.1", act_quant=False).reshape(6, d)
    ctx = rt(L(rt(O.gelu_tanh(L(context[0], "text_embedding.0"))), "text_embedding.2"))
    if clip_feature is not None:
        x = torch.cat([x, y], dim=1)
        ctx = torch.cat([img_emb(clip_feature[0].float(), w, lin, rt), ctx], dim=0)
    h, grid = patchify(x, w, lin)
    h = rt(h)
    table = O.wan_rope_table(*grid, head_dim=d // H)
    h_in = h
    for i in range(num_layers):
        h = wan_block(h, ctx, t_mod, table, w, f"blocks.{i}.", H, lin, rt, eps)
    mod = w["head.modulation"].float().reshape(2, d) + t[0]
    shift, scale = mod
    out = rt(L(O.ln_modulate(h, shift, scale, eps), "head.head", from_fp32=True))
    out = unpatchify(out, grid, out.shape[1] // 4)
    return (out, h_in, h) if return_hidden else out      # hidden state before the first and after the last block
