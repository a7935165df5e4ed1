"""Flux MMDiT forward restated functionally over a reference-named state dict (fp32 on the CPU).
Citations: ``diffsynth_engine/models/flux/flux_dit.py`` and ``models/basic/{transformer_helper,timestep}.py``
of modelscope/DiffSynth-Engine v0.1.1.

``rt`` is the rounding applied wherever the CUDA path materialises a bf16 tensor (identity for the
exact oracle); ``lin`` is a ``LinearEval``.  With a rounding ``rt`` the attention also rounds its probabilities to
bf16 (``ops.attention_bf16_probs``) and the RoPE factors are the fp16 values the projection's epilogue reads."""
import torch
import torch.nn.functional as F

from . import ops as O
from .linear import LinearEval


UNIT_SCALE = True   # see LinearEval.unit_scale_acts (False restores per-row scales everywhere, for comparison)


def _ident(x):
    return x


def round_bf16(x):
    return x.bfloat16().float()


def _heads(x, H):
    S = x.shape[0]
    return x.reshape(S, H, -1).transpose(0, 1)  # [H, S, D]


def joint_attention(qkv_b, qkv_a, w, pre, H, table, rt=_ident):
    """flux_dit.py:161-188: per-stream q/k RMSNorm, text rows first then image rows, RoPE, attention.
    qkv_*: [S_*, 3*H*D] with feature layout [q | k | v], head-major inside each (flux_dit.py:166-167)."""
    d = qkv_a.shape[1] // 3
    def split(qkv, nq, nk):
        # qkv is the UNROUNDED projection: the projection's epilogue normalises and rotates q and k from its fp32
        # accumulator and rounds once, after the rotation (the reference rounds the projection first,
        # flux_dit.py:164-171: one rounding more); v is rounded as it is stored
        q, k, v = qkv[:, :d], qkv[:, d:2 * d], rt(qkv[:, 2 * d:])
        return O.rmsnorm(_heads(q, H), w[pre + nq]), O.rmsnorm(_heads(k, H), w[pre + nk]), _heads(v, H)
    q_a, k_a, v_a = split(qkv_a, "norm_q_a.weight", "norm_k_a.weight")
    if qkv_b is not None:
        q_b, k_b, v_b = split(qkv_b, "norm_q_b.weight", "norm_k_b.weight")
        q, k, v = torch.cat([q_b, q_a], 1), torch.cat([k_b, k_a], 1), torch.cat([v_b, v_a], 1)
    else:
        q, k, v = q_a, k_a, v_a
    q, k = rt(O.apply_rope_pairs(q, table)), rt(O.apply_rope_pairs(k, table))
    attn = O.attention if rt is _ident else O.attention_bf16_probs
    o = attn(q[None], k[None], v[None])[0]              # [H, S, D]
    return rt(o.transpose(0, 1).reshape(o.shape[1], -1))  # flux_dit.py:183


def double_block(xa, xb, temb, table, w, pre, H, lin: LinearEval, rt=_ident):
    """FluxJointTransformerBlock.forward, flux_dit.py:219-236 (a = image stream, b = text stream).
    xa: [S_img, d], xb: [S_txt, d], temb: [d]."""
    def ada(x, name):  # transformer_helper.py:13-22
        emb = lin(F.silu(temb.float())[None], w[pre + name + ".linear.weight"], w[pre + name + ".linear.bias"],
                  act_quant=False)[0]
        sh_msa, sc_msa, g_msa, sh_mlp, sc_mlp, g_mlp = emb.chunk(6)
        return O.ln_modulate(x, sh_msa, sc_msa), g_msa, sh_mlp, sc_mlp, g_mlp
    na, g_msa_a, sh_mlp_a, sc_mlp_a, g_mlp_a = ada(xa, "norm1_a")
    nb, g_msa_b, sh_mlp_b, sc_mlp_b, g_mlp_b = ada(xb, "norm1_b")
    qkv_a = lin(na, w[pre + "attn.a_to_qkv.weight"], w[pre + "attn.a_to_qkv.bias"], from_fp32=True)
    qkv_b = lin(nb, w[pre + "attn.b_to_qkv.weight"], w[pre + "attn.b_to_qkv.bias"], from_fp32=True)
    att = joint_attention(qkv_b, qkv_a, w, pre + "attn.", H, table, rt)
    Sb = xb.shape[0]
    att_b, att_a = att[:Sb], att[Sb:]
    def tail(x, att_x, g_msa, sh_mlp, sc_mlp, g_mlp, s):
        x = rt(x.float() + g_msa * lin(att_x, w[pre + f"attn.{s}_to_out.weight"], w[pre + f"attn.{s}_to_out.bias"]))
        n = O.ln_modulate(x, sh_mlp, sc_mlp)
        hid = O.gelu_tanh(lin(n, w[pre + f"ff_{s}.0.weight"], w[pre + f"ff_{s}.0.bias"], from_fp32=True))
        if not getattr(lin, "unit_scale_acts", False) or not UNIT_SCALE:
            hid = rt(hid)    # otherwise the projection's epilogue emits e4m3 straight from its fp32 values
        return rt(x + g_mlp * lin(hid, w[pre + f"ff_{s}.2.weight"], w[pre + f"ff_{s}.2.bias"],
                                  act_quant="unit" if UNIT_SCALE else True))
    xa = tail(xa, att_a, g_msa_a, sh_mlp_a, sc_mlp_a, g_mlp_a, "a")
    xb = tail(xb, att_b, g_msa_b, sh_mlp_b, sc_mlp_b, g_mlp_b, "b")
    return xa, xb


def single_block(x, temb, table, w, pre, H, lin: LinearEval, rt=_ident):
    """FluxSingleTransformerBlock.forward, flux_dit.py:308-321.  x: [S_txt + S_img, d]."""
    d = x.shape[1]
    emb = lin(F.silu(temb.float())[None], w[pre + "norm.linear.weight"], w[pre + "norm.linear.bias"],
              act_quant=False)[0]
    shift, scale, gate = emb.chunk(3)  # transformer_helper.py:32-36
    n = O.ln_modulate(x, shift, scale)
    h = lin(n, w[pre + "to_qkv_mlp.weight"], w[pre + "to_qkv_mlp.bias"], from_fp32=True)
    qkv, mlp = h[:, :3 * d], O.gelu_tanh(h[:, 3 * d:])
    if not getattr(lin, "unit_scale_acts", False) or not UNIT_SCALE:
        mlp = rt(mlp)
    att = joint_attention(None, qkv, w, pre, H, table, rt)
    out = lin(torch.cat([att, mlp], dim=1), w[pre + "proj_out.weight"], w[pre + "proj_out.bias"],
              act_quant="unit" if UNIT_SCALE else True)
    return rt(x.float() + gate * out)


def timestep_mlp(t_emb, w, pre, lin):
    """TimestepEmbeddings.timestep_embedder (timestep.py:73-81) / pooled_text_embedder (flux_dit.py:348-352)."""
    h = F.silu(lin(t_emb, w[pre + "0.weight"], w[pre + "0.bias"], act_quant=False))
    return lin(h, w[pre + "2.weight"], w[pre + "2.bias"], act_quant=False)


def patchify(x):
    """B C (H P) (W Q) -> B (H W) (C P Q), P=Q=2 (flux_dit.py:366-368)."""
    B, C, Hh, Ww = x.shape
    return x.reshape(B, C, Hh // 2, 2, Ww // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(B, (Hh // 2) * (Ww // 2), C * 4)


def unpatchify(x, height, width):
    """B (H W) (C P Q) -> B C (H P) (W Q) (flux_dit.py:370-374)."""
    B, _, CPQ = x.shape
    C = CPQ // 4
    return x.reshape(B, height // 2, width // 2, C, 2, 2).permute(0, 3, 1, 4, 2, 5).reshape(B, C, height, width)


def image_ids(height, width):
    """flux_dit.py:376-390: (0, row, col) per 2x2 patch."""
    ids = torch.zeros(height // 2, width // 2, 3)
    ids[..., 1] += torch.arange(height // 2)[:, None]
    ids[..., 2] += torch.arange(width // 2)[None, :]
    return ids.reshape(-1, 3)


def flux_dit_forward(w, latents, timestep, prompt_emb, pooled, guidance, text_ids=None, n_double=19, n_single=38,
                     H=24, lin: LinearEval = None, rt=_ident, use_guidance=True, return_hidden=False):
    """FluxDiT.forward, flux_dit.py:392-461, batch 1.  latents [1,C,h,w], timestep [1] (0..1000 units),
    prompt_emb [1,S_txt,4096], pooled [1,768], guidance [1]."""
    lin = lin or LinearEval("fp32")
    S_txt = prompt_emb.shape[1]
    height, width = latents.shape[-2:]
    ids = torch.cat([torch.zeros(S_txt, 3) if text_ids is None else text_ids.reshape(-1, 3).float(),
                     image_ids(height, width)], dim=0)
    # conditioning: time + guidance + pooled, in this order (flux_dit.py:409-415); the sinusoid is rounded to the
    # model dtype before the MLP (timestep.py:79) - rt models that
    cond = timestep_mlp(rt(O.timestep_embedding_flux(timestep)), w, "time_embedder.timestep_embedder.", lin)
    if use_guidance:
        cond = cond + timestep_mlp(rt(O.timestep_embedding_flux(guidance * 1000)), w,
                                   "guidance_embedder.timestep_embedder.", lin)
    cond = (cond + timestep_mlp(pooled[0:1].float(), w, "pooled_text_embedder.", lin))[0]
    xb = rt(lin(prompt_emb[0], w["context_embedder.weight"], w["context_embedder.bias"]))
    table = O.flux_rope_table(ids)
    if rt is not _ident:
        table = table.half().float()   # the rotation factors reach the projection's epilogue as fp16 (exact to 2^-12)
    xa = rt(lin(patchify(latents)[0], w["x_embedder.weight"], w["x_embedder.bias"]))
    for i in range(n_double):
        xa, xb = double_block(xa, xb, cond, table, w, f"blocks.{i}.", H, lin, rt)
    x = torch.cat([xb, xa], dim=0)
    for i in range(n_single):
        x = single_block(x, cond, table, w, f"single_blocks.{i}.", H, lin, rt)
    hidden = x
    x = x[S_txt:]
    emb = lin(F.silu(cond)[None], w["final_norm_out.linear.weight"], w["final_norm_out.linear.bias"],
              act_quant=False)[0]
    scale, shift = emb.chunk(2)  # flux_dit.py:333: scale first
    x = O.ln_modulate(x, shift, scale)
    x = rt(lin(x, w["final_proj_out.weight"], w["final_proj_out.bias"], from_fp32=True))
    out = unpatchify(x[None], height, width)
    return (out, hidden) if return_hidden else out
