"""GGUF block dequantisation restated element by element (CPU, torch).  Each function follows one
``dequantize_blocks_*`` of ``diffsynth_engine/utils/gguf.py`` (v0.1.1, lines cited per function) - the torch port of
ggml's block formats the reference dequantises with - including its rounding: with a 16-bit compute dtype every
product and every sum is rounded to that dtype, in the order the reference evaluates them.

Written as explicit index arithmetic ("value v of the block comes from byte b, bits s..") instead of the reference's
reshape-and-shift chains, so that the two agree only if both read the format the same way.
``tests/test_oracle_golden.py`` pins every function bit for bit against outputs of the reference itself
(``tests/golden/gguf_blocks.safetensors``)."""
import torch

# bytes per block, values per block
SIZES = {"Q4_0": (18, 32), "Q4_1": (20, 32), "Q5_0": (22, 32), "Q5_1": (24, 32), "Q8_0": (34, 32),
         "Q2_K": (84, 256), "Q3_K": (110, 256), "Q4_K": (144, 256), "Q5_K": (176, 256), "Q6_K": (210, 256)}
# byte offsets of the fp16 fields of a block (the rest may be arbitrary bytes)
F16_FIELDS = {"Q4_0": (0,), "Q4_1": (0, 2), "Q5_0": (0,), "Q5_1": (0, 2), "Q8_0": (0,), "Q2_K": (80, 82),
              "Q3_K": (108,), "Q4_K": (0, 2), "Q5_K": (0, 2), "Q6_K": (208,)}


def random_blocks(qtype: str, N: int, K: int, seed: int) -> torch.Tensor:
    """Well-formed random bytes ``[N, K / block * bytes]`` (test input only): every bit pattern in the integer fields,
    small finite values in the fp16 fields."""
    tsz, bsz = SIZES[qtype]
    g = torch.Generator().manual_seed(seed)
    nb = N * (K // bsz)
    raw = torch.randint(0, 256, (nb, tsz), generator=g, dtype=torch.uint8)
    for off in F16_FIELDS[qtype]:
        v = ((torch.rand(nb, generator=g) - 0.3) * 0.02).to(torch.float16)
        raw[:, off:off + 2] = v.view(torch.uint8).reshape(nb, 2)
    return raw.reshape(N, (K // bsz) * tsz).contiguous()


def _f16(blk, off, dtype):
    return blk[:, off:off + 2].contiguous().view(torch.float16).to(dtype)          # [nb, 1]


def _k_scales(s12):
    """The eight 6-bit (scale, min) pairs of a K-quant super-block (``get_scale_min``, gguf.py:158-168):
    j < 4: sc = s[j] & 63, m = s[j+4] & 63; j >= 4: sc = (s[j+4] & 15) | ((s[j-4] >> 6) << 4),
    m = (s[j+4] >> 4) | ((s[j] >> 6) << 4)."""
    s = s12.to(torch.int32)
    nb = s.shape[0]
    sc = torch.empty(nb, 8, dtype=torch.int32)
    mn = torch.empty(nb, 8, dtype=torch.int32)
    for j in range(4):
        sc[:, j] = s[:, j] & 63
        mn[:, j] = s[:, j + 4] & 63
        sc[:, j + 4] = (s[:, j + 8] & 15) | ((s[:, j] >> 6) << 4)
        mn[:, j + 4] = (s[:, j + 8] >> 4) | ((s[:, j + 4] >> 6) << 4)
    return sc.to(torch.uint8), mn.to(torch.uint8)


def _nibbles32(qs16):
    """32 4-bit values of 16 bytes: values 0..15 are the low nibbles, 16..31 the high nibbles."""
    return torch.cat([qs16 & 15, qs16 >> 4], dim=1)


def _bit_of_u32(b4, n=32):
    """bits 0..n-1 of the little-endian 32-bit word in 4 bytes -> [nb, n] of 0/1"""
    w = b4.to(torch.int64)
    word = w[:, 0] | (w[:, 1] << 8) | (w[:, 2] << 16) | (w[:, 3] << 24)
    return ((word[:, None] >> torch.arange(n)[None, :]) & 1).to(torch.uint8)


def _deq_q4_0(blk, dtype):   # gguf.py:237-247
    d = _f16(blk, 0, dtype)
    q = _nibbles32(blk[:, 2:18]).to(torch.int8) - 8
    return d * q


def _deq_q4_1(blk, dtype):   # gguf.py:222-234
    d, m = _f16(blk, 0, dtype), _f16(blk, 2, dtype)
    return d * _nibbles32(blk[:, 4:20]) + m


def _deq_q5_0(blk, dtype):   # gguf.py:201-219
    d = _f16(blk, 0, dtype)
    q = (_nibbles32(blk[:, 6:22]) | (_bit_of_u32(blk[:, 2:6]) << 4)).to(torch.int8) - 16
    return d * q


def _deq_q5_1(blk, dtype):   # gguf.py:178-198
    d, m = _f16(blk, 0, dtype), _f16(blk, 2, dtype)
    q = _nibbles32(blk[:, 8:24]) | (_bit_of_u32(blk[:, 4:8]) << 4)
    return d * q + m


def _deq_q8_0(blk, dtype):   # gguf.py:171-175
    return _f16(blk, 0, dtype) * blk[:, 2:].contiguous().view(torch.int8)


def _two_bit_planes(qs64):
    """256 2-bit values of 64 bytes: value v = 128 h + 32 s + t is bits (2s, 2s+1) of byte 32 h + t."""
    h = qs64.reshape(-1, 2, 1, 32)
    sh = torch.tensor([0, 2, 4, 6], dtype=torch.uint8).reshape(1, 1, 4, 1)
    return ((h >> sh) & 3).reshape(-1, 256)


def _deq_q2_k(blk, dtype):   # gguf.py:349-368: 16 sub-blocks of 16: (d * (s & 15)) * q - dmin * (s >> 4)
    sc, qs = blk[:, 0:16], blk[:, 16:80]
    d, dmin = _f16(blk, 80, dtype), _f16(blk, 82, dtype)
    dl = (d * (sc & 15)).reshape(-1, 16, 1)
    ml = (dmin * (sc >> 4)).reshape(-1, 16, 1)
    q = _two_bit_planes(qs).reshape(-1, 16, 16)
    return (dl * q - ml).reshape(-1, 256)


def _deq_q3_k(blk, dtype):   # gguf.py:317-346
    hmask, qs, s = blk[:, 0:32], blk[:, 32:96], blk[:, 96:108]
    d = _f16(blk, 108, dtype)
    nb = blk.shape[0]
    k = torch.arange(16)
    low = torch.where(k[None, :] < 8, s[:, k % 8] & 15, s[:, k % 8] >> 4)                 # 4 low bits of scale k
    high = (s[:, 8 + (k % 4)] >> (2 * (k // 4)).to(torch.uint8)[None, :]) & 3             # 2 high bits
    scale = (low | (high << 4)).to(torch.int8) - 32
    dl = (d * scale).reshape(nb, 16, 1)
    ql = _two_bit_planes(qs)                                                               # value v as in Q2_K
    v = torch.arange(256)
    hbit = ((hmask[:, v % 32] >> (v // 32).to(torch.uint8)[None, :]) & 1) ^ 1              # inverted high bit
    q = ql.to(torch.int8) - (hbit << 2).to(torch.int8)
    return (dl * q.reshape(nb, 16, 16)).reshape(nb, 256)


def _deq_q4_k(blk, dtype):   # gguf.py:298-315
    d, dmin = _f16(blk, 0, dtype), _f16(blk, 2, dtype)
    sc, mn = _k_scales(blk[:, 4:16])
    qs = blk[:, 16:144].reshape(-1, 4, 32)
    q = torch.stack([qs & 15, qs >> 4], dim=2).reshape(-1, 8, 32)         # sub-block 2g low, 2g+1 high nibbles
    return ((d * sc).reshape(-1, 8, 1) * q - (dmin * mn).reshape(-1, 8, 1)).reshape(-1, 256)


def _deq_q5_k(blk, dtype):   # gguf.py:270-295: as Q4_K with bit j of qh[t] as fifth bit of value t of sub-block j
    d, dmin = _f16(blk, 0, dtype), _f16(blk, 2, dtype)
    sc, mn = _k_scales(blk[:, 4:16])
    qh, qs = blk[:, 16:48], blk[:, 48:176].reshape(-1, 4, 32)
    ql = torch.stack([qs & 15, qs >> 4], dim=2).reshape(-1, 8, 32)
    hb = (qh[:, None, :] >> torch.arange(8, dtype=torch.uint8).reshape(1, 8, 1)) & 1
    q = ql | (hb << 4)
    return ((d * sc).reshape(-1, 8, 1) * q - (dmin * mn).reshape(-1, 8, 1)).reshape(-1, 256)


def _deq_q6_k(blk, dtype):   # gguf.py:250-267
    ql, qh, sc = blk[:, 0:128], blk[:, 128:192], blk[:, 192:208]
    d = _f16(blk, 208, dtype)
    nb = blk.shape[0]
    dl = (d * sc.contiguous().view(torch.int8).to(dtype)).reshape(nb, 16, 1)
    v = torch.arange(256)
    h, r = v // 128, v % 128                                   # which 128-value half, position inside it
    lo = (ql[:, h * 64 + (r % 64)] >> (4 * (r // 64)).to(torch.uint8)[None, :]) & 15
    hi = (qh[:, h * 32 + (r % 32)] >> (2 * (r // 32)).to(torch.uint8)[None, :]) & 3
    q = (lo | (hi << 4)).to(torch.int8) - 32
    return (dl * q.reshape(nb, 16, 16)).reshape(nb, 256)


_FUNCS = {"Q4_0": _deq_q4_0, "Q4_1": _deq_q4_1, "Q5_0": _deq_q5_0, "Q5_1": _deq_q5_1, "Q8_0": _deq_q8_0,
          "Q2_K": _deq_q2_k, "Q3_K": _deq_q3_k, "Q4_K": _deq_q4_k, "Q5_K": _deq_q5_k, "Q6_K": _deq_q6_k}


def dequantize(raw: torch.Tensor, qtype: str, dtype=torch.bfloat16) -> torch.Tensor:
    """``dequantize`` (gguf.py:113-135) for raw rows ``[N, bytes]`` (uint8) -> ``[N, K]`` in ``dtype``."""
    tsz, bsz = SIZES[qtype]
    N = raw.shape[0]
    blk = raw.reshape(-1, tsz)
    return _FUNCS[qtype](blk, dtype).reshape(N, -1)
