"""Elementary operations of the DiT step, restated in fp32 on the CPU.  Paths cite
modelscope/DiffSynth-Engine v0.1.1 (``diffsynth_engine/...``)."""
import math

import torch
import torch.nn.functional as F

E4M3_MAX = 448.0
INT8_MAX = 127.0


# ------------------------------------------------------------------ normalisation / modulation
def layer_norm(x, eps=1e-6):
    """nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6): models/basic/transformer_helper.py:11,30;
    models/flux/flux_dit.py:207,212,329; models/wan/wan_dit.py:176-177,231."""
    return F.layer_norm(x.float(), (x.shape[-1],), eps=eps)


def ln_modulate(x, shift, scale, eps=1e-6):
    """norm(x) * (1 + scale) + shift: models/basic/transformer_helper.py:17,21,35;
    models/flux/flux_dit.py:228,233,334; models/wan/wan_dit.py:25-26."""
    return layer_norm(x, eps) * (1.0 + scale.float()) + shift.float()


def gate_residual(x, y, gate=None):
    """x + gate * y: models/flux/flux_dit.py:227,229,318-319; models/wan/wan_dit.py:189-192."""
    return x.float() + (y.float() if gate is None else gate.float() * y.float())


def rmsnorm(x, weight, eps=1e-6):
    """x * rsqrt(mean(x^2) + eps) * weight over the last dimension:
    models/basic/transformer_helper.py:73-78 (per head) and models/wan/wan_dit.py:74-78 (full width).
    The reference rounds to the input dtype before the weight multiply; in fp32 that is a no-op."""
    x = x.float()
    var = x.square().mean(-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight.float()


def gelu_tanh(x):
    """nn.GELU(approximate="tanh"): models/flux/flux_dit.py:209,215,315; models/wan/wan_dit.py:180."""
    return F.gelu(x.float(), approximate="tanh")


# ------------------------------------------------------------------------------------ RoPE
def flux_rope_table(ids, axes_dim=(16, 56, 56), theta=10000):
    """(cos, sin) per pair, [S, 64, 2] fp32, from position ids [S, 3].
    models/basic/transformer_helper.py:46-64: omega in fp64, angle = pos * omega, table rounded to fp32.
    The reference stores [[cos, -sin], [sin, cos]]; (cos, sin) carries the same information."""
    cols = []
    for i, d in enumerate(axes_dim):
        scale = torch.arange(0, d, 2, dtype=torch.float64) / d
        omega = 1.0 / (theta ** scale)
        ang = ids[..., i].to(torch.float64)[:, None] * omega[None, :]
        cols.append(torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1))
    return torch.cat(cols, dim=1).float()


def apply_rope_pairs(x, table):
    """Rotate adjacent pairs (2j, 2j+1) of the last dimension: out0 = cos*x0 - sin*x1, out1 = sin*x0 + cos*x1.
    models/flux/flux_dit.py:154-159.  x: [..., S, 128]; table: [S, 64, 2]."""
    x = x.float()
    xp = x.reshape(*x.shape[:-1], -1, 2)
    cos, sin = table[..., 0], table[..., 1]
    o0 = cos * xp[..., 0] - sin * xp[..., 1]
    o1 = sin * xp[..., 0] + cos * xp[..., 1]
    return torch.stack([o0, o1], dim=-1).reshape(x.shape)


def wan_rope_table(f, h, w, head_dim=128, theta=10000.0):
    """(cos, sin) per pair for the (f, h, w) grid in raster order, [f*h*w, 64, 2] fp32.
    models/wan/wan_dit.py:38-51 (frequencies in fp64, split 44/42/42 of the 128 dims) and :335-346."""
    def freqs(dim, end):
        fr = 1.0 / (theta ** (torch.arange(0, dim, 2)[: dim // 2].double() / dim))
        return torch.outer(torch.arange(end, dtype=torch.float64), fr)

    d_h = head_dim // 3
    d_f = head_dim - 2 * d_h
    af, ah, aw = freqs(d_f, f), freqs(d_h, h), freqs(d_h, w)
    ang = torch.cat([
        af.view(f, 1, 1, -1).expand(f, h, w, -1),
        ah.view(1, h, 1, -1).expand(f, h, w, -1),
        aw.view(1, 1, w, -1).expand(f, h, w, -1),
    ], dim=-1).reshape(f * h * w, -1)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float()


# ------------------------------------------------------------------------------- attention
def attention(q, k, v, sm_scale=None):
    """softmax(q k^T / sqrt(d)) v without mask; q,k,v: [B, H, S, D].
    models/flux/flux_dit.py:21 (default _attn_func = SDPA); models/wan/wan_dit.py:18-22."""
    return F.scaled_dot_product_attention(q.float(), k.float(), v.float(), scale=sm_scale)


def attention_bf16_probs(q, k, v, sm_scale=None):
    """The same attention as GPU flash kernels evaluate it (the SDPA kernel the reference reaches on CUDA, and this
    library's): fp32 scores from bf16 operands, probabilities ROUNDED TO BF16 for the P.V product, fp32 row sum of the
    unrounded probabilities.  The probabilities are taken relative to an integer power of two,
    ``p = exp2(s*c - M)`` with ``M = ceil(rowmax * c)`` and ``c = scale * log2(e)``: scaling by 2^integer is exact, so
    the rounded values - and with them the result - do not depend on which integer ``M`` an implementation uses or on
    how it tiles the keys.  q, k, v: [B, H, S, D]; the same-rounding counterpart of :func:`attention`."""
    B, H, Sq, D = q.shape
    scale = (1.0 / math.sqrt(D)) if sm_scale is None else sm_scale
    c = torch.tensor(scale, dtype=torch.float32) * torch.tensor(1.4426950408889634, dtype=torch.float32)
    out = torch.empty(B, H, Sq, v.shape[-1])
    for b in range(B):
        for h in range(H):
            s = q[b, h].float() @ k[b, h].float().t()
            m = torch.ceil(s.amax(dim=1) * c)
            p = torch.exp2(s * c - m[:, None])
            out[b, h] = (p.bfloat16().float() @ v[b, h].float()) / p.sum(dim=1, keepdim=True)
    return out


# ---------------------------------------------------------------------------- quantisation
def quant_rows_e4m3(x):
    """Dynamic per-row FP8 quantisation: s = amax/448 (1 for an all-zero row), q = e4m3(clamp(x * (1/s))).
    The reference casts with unit scale (utils/fp8_linear.py:35); the scale is this library's extension."""
    x = x.float()
    amax = x.abs().amax(dim=1)
    s = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (x * (1.0 / s)[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q, s


def quant_rows_int8(x):
    x = x.float()
    amax = x.abs().amax(dim=1)
    s = torch.where(amax > 0, amax / INT8_MAX, torch.ones_like(amax))
    q = torch.round(x * (1.0 / s)[:, None]).clamp(-INT8_MAX, INT8_MAX).to(torch.int8)
    return q, s


def quant_weight(W, fmt="fp8_tensor"):
    """Weight prepack rule: fp8_tensor: s = amax|W|/448; fp8_channel: s_n = amax|W[n,:]|/448;
    int8_channel: s_n = amax/127 with round-half-even.  q = clamp(W / s).  (An all-zero row gets s = 1.)
    The reference only casts (utils/fp8_linear.py:12-17)."""
    W = W.float()
    if fmt == "fp8_tensor":
        amax = W.abs().amax().reshape(1)
    else:
        amax = W.abs().amax(dim=1)
    qmax = INT8_MAX if fmt == "int8_channel" else E4M3_MAX
    s = torch.where(amax > 0, amax / qmax, torch.ones_like(amax))
    sd = s if fmt == "fp8_tensor" else s[:, None]
    q = (W / sd).clamp(-qmax, qmax)
    q = torch.round(q).to(torch.int8) if fmt == "int8_channel" else q.to(torch.float8_e4m3fn)
    return q, s


def q8_0_quantize(W):
    """GGUF Q8_0 as published (ggml): blocks of 32 along the last axis, each ``fp16 d = amax / 127`` followed by 32
    ``int8 q = round(x / d)``; returns the raw bytes ``[N, K / 32 * 34]`` (uint8).  Only used to make test inputs."""
    N, K = W.shape
    blk = W.float().reshape(N, K // 32, 32)
    d = (blk.abs().amax(dim=-1, keepdim=True) / 127.0)
    q = torch.where(d > 0, blk / d, torch.zeros_like(blk)).round().clamp(-127, 127).to(torch.int8)
    raw = torch.cat([d.to(torch.float16).view(torch.uint8), q.view(torch.uint8)], dim=-1)     # [N, K/32, 2 + 32]
    return raw.reshape(N, K // 32 * 34).contiguous()


def q8_0_dequantize(raw, dtype=torch.bfloat16):
    """``dequantize_blocks_Q8_0`` (utils/gguf.py:171-175): ``d.view(fp16).to(dtype) * q.view(int8)``, the product
    taken in ``dtype``.  raw: uint8 ``[N, K / 32 * 34]`` -> ``[N, K]``."""
    N = raw.shape[0]
    blocks = raw.reshape(-1, 34)
    d = blocks[:, :2].contiguous().view(torch.float16).to(dtype)
    q = blocks[:, 2:].contiguous().view(torch.int8)
    return (d * q).reshape(N, -1)


def q4_k_random_blocks(N, K, seed):
    """Well-formed random GGUF Q4_K bytes ``[N, K / 256 * 144]`` (test input only): per 256 weights an fp16 d, an fp16
    dmin, 12 bytes holding eight 6-bit scales and eight 6-bit mins, and 128 bytes of 4-bit quants (ggml's layout)."""
    g = torch.Generator().manual_seed(seed)
    nb = N * (K // 256)
    d = (torch.rand(nb, 1, generator=g) * 0.01 + 0.001).to(torch.float16).view(torch.uint8)
    dmin = (torch.rand(nb, 1, generator=g) * 0.02).to(torch.float16).view(torch.uint8)
    rest = torch.randint(0, 256, (nb, 12 + 128), generator=g, dtype=torch.uint8)
    return torch.cat([d, dmin, rest], dim=1).reshape(N, (K // 256) * 144).contiguous()


def q4_k_dequantize(raw, dtype=torch.bfloat16):
    """``dequantize_blocks_Q4_K`` with ``get_scale_min`` (utils/gguf.py:158-168,298-315): sub-block j of 32 weights is
    ``(d * sc_j) * q - (dmin * m_j)``, every product and the difference taken in ``dtype``.  Scales and mins are
    6-bit: j < 4: sc = s[j] & 63, m = s[j+4] & 63; j >= 4: sc = (s[j+4] & 15) | ((s[j-4] >> 6) << 4),
    m = (s[j+4] >> 4) | ((s[j] >> 6) << 4).  Quants: bytes [32g, 32g+32) carry sub-block 2g in their low and sub-block
    2g+1 in their high nibbles."""
    N = raw.shape[0]
    blk = raw.reshape(-1, 144)
    nb = blk.shape[0]
    d = blk[:, 0:2].contiguous().view(torch.float16).to(dtype)
    dmin = blk[:, 2:4].contiguous().view(torch.float16).to(dtype)
    s = blk[:, 4:16].to(torch.int32)
    sc = torch.empty(nb, 8, dtype=torch.int32)
    mn = torch.empty(nb, 8, dtype=torch.int32)
    for j in range(4):
        sc[:, j] = s[:, j] & 63
        mn[:, j] = s[:, j + 4] & 63
        sc[:, j + 4] = (s[:, j + 8] & 15) | ((s[:, j] >> 6) << 4)
        mn[:, j + 4] = (s[:, j + 8] >> 4) | ((s[:, j + 4] >> 6) << 4)
    dsc = (d * sc.to(torch.uint8)).reshape(nb, 8, 1)
    dm = (dmin * mn.to(torch.uint8)).reshape(nb, 8, 1)
    qs = blk[:, 16:].reshape(nb, 4, 32)
    q = torch.stack([qs & 0x0F, qs >> 4], dim=2).reshape(nb, 8, 32)
    return (dsc * q - dm).reshape(N, -1)


def linear_quant(x_q, x_s, W_q, W_s, bias=None):
    """Quantised Linear with fp32 accumulation: ((x_q W_q^T) * x_s[m] * W_s[n]) + bias.
    Dataflow of utils/fp8_linear.py:33-50 with scales added; products of e4m3 (or int8) values are exact in fp32
    only up to accumulation order, so comparisons use a tolerance, not bit equality."""
    acc = x_q.float() @ W_q.float().t()
    ws = W_s if W_s.numel() > 1 else W_s.reshape(1)
    y = acc * x_s[:, None] * ws[None, :]
    return y if bias is None else y + bias.float()


# ------------------------------------------------------------------------------- embeddings
def timestep_embedding_flux(t, dim=256, max_period=10000):
    """[cos | sin] sinusoid in fp32 (flip_sin_to_cos=True, downscale_freq_shift=0):
    models/basic/timestep.py:6-44 as configured at :68-70."""
    half = dim // 2
    exponent = -math.log(max_period) * torch.arange(0, half, dtype=torch.float32) / half
    emb = t[:, None].float() * torch.exp(exponent)[None, :]
    return torch.cat([torch.cos(emb), torch.sin(emb)], dim=-1)


def sinusoidal_embedding_wan(dim, position):
    """[cos | sin] from an fp64 outer product: models/wan/wan_dit.py:29-35."""
    sinusoid = torch.outer(position.double(),
                           torch.pow(10000, -torch.arange(dim // 2, dtype=torch.float64).div(dim // 2)))
    return torch.cat([torch.cos(sinusoid), torch.sin(sinusoid)], dim=1)


# ------------------------------------------------------------------------ sampler / scheduler
def euler_step(latents, model_out, sigmas, i, init=None, mask=None):
    """algorithm/sampler/flow_match/flow_match_euler.py:11-19."""
    if mask is not None:
        model_out = model_out * mask + init * (1 - mask)
    dt = sigmas[i + 1] - sigmas[i]
    out = latents.to(torch.float32) + model_out * dt
    return out.to(model_out.dtype)


def cfg_combine(pos, neg, cfg_scale):
    """noise_pred = negative + cfg_scale * (positive - negative): pipelines/wan_video.py:230,248;
    pipelines/flux_image.py:387,398 (evaluated in the tensors' own dtype, as PyTorch does)."""
    return neg + cfg_scale * (pos - neg)


def rectified_flow_schedule(num_steps, shift=1.0, sigma_min=0.001, sigma_max=1.0, num_train_timesteps=1000,
                            mu=None):
    """algorithm/noise_scheduler/flow_match/recifited_flow.py:34-50 (mu given = dynamic shifting, as Flux uses)."""
    sigmas = torch.linspace(sigma_max, sigma_min, num_steps)
    if mu is not None:
        sigmas = math.exp(mu) / (math.exp(mu) + (1 / sigmas - 1) ** 1.0)
    else:
        sigmas = shift * sigmas / (1 + (shift - 1) * sigmas)
    timesteps = sigmas * num_train_timesteps
    sigmas = torch.cat([sigmas, sigmas.new_zeros([1])])
    return sigmas, timesteps


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
