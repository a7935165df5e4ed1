"""Thin torch-tensor front end of the C ABI (``include/dsb.h``).  Tensors only carry device memory
and the current stream; all arithmetic happens in ``libdsb.so``."""
import ctypes
import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import ACT_GELU, ACT_GELU_TANH, ACT_NONE, ACT_SILU, FMT_BF16, FMT_E4M3, FMT_INT8, check  # noqa: F401

_status = {}


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*ts):
    """Every tensor of a call must live on the CURRENT CUDA device: kernels launch on its current stream, and the
    status word and the static scratch of ``dsb_linear_static`` belong to it."""
    cur = None
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise _lib.DsbError("dsb ops take CUDA tensors only (no CPU fallback exists)")
        if cur is None:
            cur = torch.cuda.current_device()
        if t.device.index != cur:
            raise _lib.DsbError(f"tensor on cuda:{t.device.index} but the current device is cuda:{cur}: wrap the call "
                                "in torch.cuda.device(tensor.device)")


def _require_bf16(t, what):
    if t.dtype != torch.bfloat16:
        raise _lib.DsbError(f"{what} takes bf16 rows, got {t.dtype}")


def status_word(device) -> torch.Tensor:
    """Per-device int32 the kernels set to DSB_ERR_TIMEOUT when a bounded wait runs out."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status[key]


def check_status(device=None):
    """Synchronising read of the status word; raises if a kernel reported a timeout."""
    dev = torch.cuda.current_device() if device is None else device
    code = int(status_word(dev).item())
    if code != 0:
        status_word(dev).zero_()
        _lib.check(code, "device kernel")


def selftest_wait_timeout(limit_cycles: int = 2_000_000, device=None):
    """Runs ``dsb_selftest_wait_timeout`` on its own status word; returns ``(status, neighbour_left)`` as Python
    ints (synchronises).  A healthy library returns ``(ERR_TIMEOUT, 1)`` after about ``limit_cycles`` SM cycles."""
    dev = torch.device("cuda", torch.cuda.current_device() if device is None else device)
    with torch.cuda.device(dev):
        words = torch.zeros(2, dtype=torch.int32, device=dev)
        rc = _lib.lib().dsb_selftest_wait_timeout(int(limit_cycles), ctypes.c_void_p(words.data_ptr()),
                                                  ctypes.c_void_p(words.data_ptr() + 4), _stream())
        check(rc, "dsb_selftest_wait_timeout")
        status, left = words.tolist()
    return status, left


def _fmt_of(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return FMT_BF16
    if t.dtype == torch.float8_e4m3fn:
        return FMT_E4M3
    if t.dtype == torch.int8:
        return FMT_INT8
    raise _lib.DsbError(f"unsupported operand dtype {t.dtype}")


_OUT_DTYPE = {FMT_BF16: torch.bfloat16, FMT_E4M3: torch.float8_e4m3fn, FMT_INT8: torch.int8}


def _rows(t: torch.Tensor) -> Tuple[int, int, int]:
    """(M, D, ld) of a 2-D row view with unit inner stride."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise _lib.DsbError("expected a 2-D tensor with contiguous rows")
    return t.shape[0], t.shape[1], t.stride(0)


def _check_gemm_io(M, N, out, out1, split_col, resid=None, row_scale=None, col_scale=None, bias=None, gate=None,
                   e4m3_ok=False):
    """The C entry points take raw pointers: every shape and dtype they rely on is checked here, so that a wrong
    buffer raises instead of being written out of bounds."""
    n0 = N if (out1 is None or split_col is None) else split_col
    ok_out = (torch.bfloat16, torch.float8_e4m3fn) if e4m3_ok else (torch.bfloat16,)
    for name, t, cols in (("out", out, n0), ("out1", out1, N - n0)):
        if t is None:
            continue
        if t.dtype not in ok_out:
            raise _lib.DsbError(f"gemm {name} must be bfloat16" + (" or float8_e4m3fn" if e4m3_ok else
                                " (use gemm_group for an e4m3 output)"))
        if t.dim() != 2 or t.stride(1) != 1 or t.shape[0] != M or t.shape[1] < cols:
            raise _lib.DsbError(f"gemm {name} must be a [{M}, >={cols}] row view, got {tuple(t.shape)}")
    if out1 is not None and not 0 < n0 < N:
        raise _lib.DsbError("split_col must lie inside (0, N) when out1 is given")
    if resid is not None and (resid.dtype != torch.bfloat16 or resid.dim() != 2 or resid.stride(1) != 1
                              or resid.shape[0] != M or resid.shape[1] < N):
        raise _lib.DsbError(f"gemm resid must be a bfloat16 [{M}, >={N}] row view")
    for name, t, n in (("row_scale", row_scale, M), ("bias", bias, N), ("gate", gate, N),
                       ("col_scale", col_scale, 1 if (col_scale is not None and col_scale.numel() == 1) else N)):
        if t is not None and (t.dtype != torch.float32 or t.numel() < n or not t.is_contiguous()):
            raise _lib.DsbError(f"gemm {name} must be contiguous float32 with at least {n} elements")


def ln_modulate(x, shift, scale, eps=1e-6, out_fmt=FMT_BF16, out=None, row_scale=None, split_row=None,
                shift_b=None, scale_b=None):
    """LayerNorm (no affine) then ``* (1 + scale) + shift``; optionally quantised per row.  With ``split_row``
    rows from that index on use ``(shift_b, scale_b)`` instead.  Returns ``(y, row_scale)`` (row_scale is None
    for bf16 output)."""
    _require_cuda(x, shift, scale, shift_b, scale_b)
    M, D, ld_x = _rows(x)
    if out is None:
        out = torch.empty((M, D), dtype=_OUT_DTYPE[out_fmt], device=x.device)
    if out_fmt != FMT_BF16 and row_scale is None:
        row_scale = torch.empty(M, dtype=torch.float32, device=x.device)
    if split_row is None:
        rc = _lib.lib().dsb_ln_modulate(_ptr(x), ld_x, _ptr(shift), _ptr(scale), _ptr(out), out.stride(0),
                                        _ptr(row_scale), M, D, eps, out_fmt, _stream())
    else:
        rc = _lib.lib().dsb_ln_modulate2(_ptr(x), ld_x, _ptr(shift), _ptr(scale), split_row, _ptr(shift_b),
                                         _ptr(scale_b), _ptr(out), out.stride(0), _ptr(row_scale), M, D, eps, out_fmt,
                                         _stream())
    check(rc, "dsb_ln_modulate")
    return out, row_scale


def gate_residual(x, y, gate=None, out=None):
    _require_cuda(x, y, gate)
    M, D, ld_x = _rows(x)
    if out is None:
        out = torch.empty((M, D), dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().dsb_gate_residual(_ptr(x), ld_x, _ptr(y), y.stride(0), _ptr(gate), _ptr(out), out.stride(0), M, D,
                                      _stream())
    check(rc, "dsb_gate_residual")
    return out


def rmsnorm_rope_heads(buf, H, w_q, w_k=None, rope=None, rope_row0=0, eps=1e-6):
    """In place on ``buf[S, ld]``: the first H (w_k None) or 2H heads of each row."""
    _require_cuda(buf, w_q, w_k, rope)
    S, _, ld = _rows(buf)
    rc = _lib.lib().dsb_rmsnorm_rope_heads(_ptr(buf), ld, S, H, 128, 1 if w_k is None else 2, _ptr(w_q), _ptr(w_k),
                                           _ptr(rope), rope_row0, eps, _stream())
    check(rc, "dsb_rmsnorm_rope_heads")
    return buf


def rmsnorm_full(buf, w, rope=None, rope_row0=0, eps=1e-6, out=None, chunks=1):
    """RMSNorm over whole rows (+RoPE); in place unless ``out`` is given.  ``chunks`` = P > 1 writes ``out`` as
    ``[P, M, D/P]`` (contiguous), the send layout of the head exchange."""
    _require_cuda(buf, w, rope, out)
    M, D, ld = _rows(buf)
    if out is None:
        out, ld_out, cc, cs = buf, ld, 0, 0
    elif chunks > 1:
        if tuple(out.shape) != (chunks, M, D // chunks) or not out.is_contiguous():
            raise _lib.DsbError("chunked rmsnorm_full output must be a contiguous [P, M, D/P] tensor")
        ld_out, cc, cs = D // chunks, D // chunks, M * (D // chunks)
    else:
        ld_out, cc, cs = out.stride(0), 0, 0
    rc = _lib.lib().dsb_rmsnorm_full(_ptr(buf), ld, _ptr(out), ld_out, cc, cs, M, D, _ptr(w), _ptr(rope), rope_row0,
                                     eps, _stream())
    check(rc, "dsb_rmsnorm_full")
    return out


def quant_rows(x, out_fmt=FMT_E4M3, out=None, row_scale=None):
    _require_cuda(x, out, row_scale)
    _require_bf16(x, "quant_rows")
    M, K, ld_x = _rows(x)
    if out is None:
        out = torch.empty((M, K), dtype=_OUT_DTYPE[out_fmt], device=x.device)
    if row_scale is None:
        row_scale = torch.empty(M, dtype=torch.float32, device=x.device)
    rc = _lib.lib().dsb_quant_rows(_ptr(x), ld_x, _ptr(out), out.stride(0), _ptr(row_scale), M, K, out_fmt, _stream())
    check(rc, "dsb_quant_rows")
    return out, row_scale


def quant_rows_chunked(x3, out_fmt=FMT_E4M3, out=None, row_scale=None):
    """Quantise rows delivered as ``[P, M, K/P]`` (contiguous) into plain ``[M, K]`` rows."""
    _require_cuda(x3)
    if x3.dim() != 3 or not x3.is_contiguous():
        raise _lib.DsbError("quant_rows_chunked takes a contiguous [P, M, K/P] tensor")
    P, M, C = x3.shape
    K = P * C
    if out is None:
        out = torch.empty((M, K), dtype=_OUT_DTYPE[out_fmt], device=x3.device)
    if row_scale is None:
        row_scale = torch.empty(M, dtype=torch.float32, device=x3.device)
    rc = _lib.lib().dsb_quant_rows_chunked(_ptr(x3), C, C, M * C, _ptr(out), out.stride(0), _ptr(row_scale), M, K,
                                           out_fmt, _stream())
    check(rc, "dsb_quant_rows_chunked")
    return out, row_scale


def dequant_q8_0(raw, out=None):
    """GGUF Q8_0 bytes ``[N, K/32*34]`` (uint8) -> bf16 ``[N, K]``."""
    _require_cuda(raw, out)
    if raw.dtype != torch.uint8 or raw.dim() != 2 or raw.stride(1) != 1 or raw.shape[1] % 34:
        raise _lib.DsbError("dequant_q8_0 takes uint8 rows of 34-byte blocks")
    N, K = raw.shape[0], raw.shape[1] // 34 * 32
    if out is None:
        out = torch.empty((N, K), dtype=torch.bfloat16, device=raw.device)
    rc = _lib.lib().dsb_dequant_q8_0(_ptr(raw), raw.stride(0), N, K, _ptr(out), out.stride(0), _stream())
    check(rc, "dsb_dequant_q8_0")
    return out


def dequant_q4_k(raw, out=None):
    """GGUF Q4_K bytes ``[N, K/256*144]`` (uint8) -> bf16 ``[N, K]``."""
    _require_cuda(raw, out)
    if raw.dtype != torch.uint8 or raw.dim() != 2 or raw.stride(1) != 1 or raw.shape[1] % 144:
        raise _lib.DsbError("dequant_q4_k takes uint8 rows of 144-byte super-blocks")
    N, K = raw.shape[0], raw.shape[1] // 144 * 256
    if out is None:
        out = torch.empty((N, K), dtype=torch.bfloat16, device=raw.device)
    rc = _lib.lib().dsb_dequant_q4_k(_ptr(raw), raw.stride(0), N, K, _ptr(out), out.stride(0), _stream())
    check(rc, "dsb_dequant_q4_k")
    return out


# ggml type number, bytes per block, weights per block
GGUF_TYPES = {"Q4_0": (2, 18, 32), "Q4_1": (3, 20, 32), "Q5_0": (6, 22, 32), "Q5_1": (7, 24, 32), "Q8_0": (8, 34, 32),
              "Q2_K": (10, 84, 256), "Q3_K": (11, 110, 256), "Q4_K": (12, 144, 256), "Q5_K": (13, 176, 256),
              "Q6_K": (14, 210, 256)}


def dequant_gguf(raw, qtype: str, out=None):
    """GGUF bytes ``[N, K / block * bytes]`` (uint8) of block format ``qtype`` -> bf16 ``[N, K]``."""
    _require_cuda(raw, out)
    if qtype not in GGUF_TYPES:
        raise _lib.DsbError(f"unsupported GGUF block format {qtype}")
    code, tsz, bsz = GGUF_TYPES[qtype]
    if raw.dtype != torch.uint8 or raw.dim() != 2 or raw.stride(1) != 1 or raw.shape[1] % tsz:
        raise _lib.DsbError(f"dequant_gguf({qtype}) takes uint8 rows of {tsz}-byte blocks")
    N, K = raw.shape[0], raw.shape[1] // tsz * bsz
    if out is None:
        out = torch.empty((N, K), dtype=torch.bfloat16, device=raw.device)
    rc = _lib.lib().dsb_dequant_gguf(code, _ptr(raw), raw.stride(0), N, K, _ptr(out), out.stride(0), _stream())
    check(rc, "dsb_dequant_gguf")
    return out


def cast_quant(x, out, out_fmt=FMT_E4M3, split=False):
    """Saturating cast of bf16 ``x [M, D]`` into the 8-bit window ``out`` (may be a column slice): ``[M, D]``, or
    with ``split`` (e4m3) ``[M, 3D]`` = [head | remainder | head]."""
    _require_cuda(x, out)
    M, D, ld_x = _rows(x)
    if out.shape[0] != M or out.shape[1] != (3 * D if split else D):
        raise _lib.DsbError("cast_quant: output window has the wrong shape")
    rc = _lib.lib().dsb_cast_quant(_ptr(x), ld_x, _ptr(out), out.stride(0), M, D, out_fmt, int(split), _stream())
    check(rc, "dsb_cast_quant")
    return out


def gemv(W, x, w_scale=None, bias=None, act_in=ACT_NONE, act_out=ACT_NONE, out=None, accumulate=False):
    """y = act_out((W @ act_in(x)) * w_scale + bias) for one fp32 activation row."""
    _require_cuda(W, x, w_scale, bias)
    N, K, ld_w = _rows(W)
    if out is None:
        out = torch.empty(N, dtype=torch.float32, device=x.device)
    stride = 0 if (w_scale is None or w_scale.numel() == 1) else 1
    rc = _lib.lib().dsb_gemv(_ptr(W), ld_w, _fmt_of(W), _ptr(x), _ptr(w_scale), stride, _ptr(bias), _ptr(out), N, K,
                             act_in, act_out, 1 if accumulate else 0, _stream())
    check(rc, "dsb_gemv")
    return out


def timestep_embedding(t, dim=256, t_scale=1.0, mode=0, round_bf16=False, out=None):
    """[n, dim] fp32 sinusoid of a device fp32 vector t (mode 0 Flux fp32 angles, 1 Wan fp64 angles)."""
    _require_cuda(t)
    n = t.numel()
    if out is None:
        out = torch.empty((n, dim), dtype=torch.float32, device=t.device)
    rc = _lib.lib().dsb_timestep_embedding(_ptr(t), n, dim, float(t_scale), mode, 1 if round_bf16 else 0, _ptr(out),
                                           _stream())
    check(rc, "dsb_timestep_embedding")
    return out


def euler_step(latents, model_out, dt: float, init=None, mask=None, out=None):
    _require_cuda(latents, model_out, init, mask)
    if out is None:
        out = torch.empty_like(model_out)
    is_f32 = 1 if model_out.dtype == torch.float32 else 0
    rc = _lib.lib().dsb_euler_step(_ptr(latents), _ptr(model_out), _ptr(init), _ptr(mask), float(dt), _ptr(out),
                                   latents.numel(), is_f32, _stream())
    check(rc, "dsb_euler_step")
    return out


def cfg_euler_step(latents, pos, neg, cfg_scale: float, dt: float, out=None):
    """``latents + (neg + cfg_scale * (pos - neg)) * dt`` in one pass (CFG combine + flow-match Euler update)."""
    _require_cuda(latents, pos, neg)
    if out is None:
        out = torch.empty_like(pos)
    rc = _lib.lib().dsb_cfg_euler_step(_ptr(latents), _ptr(pos), _ptr(neg), float(cfg_scale), float(dt), _ptr(out),
                                       latents.numel(), 1 if pos.dtype == torch.float32 else 0, _stream())
    check(rc, "dsb_cfg_euler_step")
    return out


def gemm(a, w, row_scale=None, col_scale=None, bias=None, act=ACT_NONE, act_col0=0, gate=None, resid=None, out=None,
         out1=None, split_col=None):
    """out = epilogue(a @ w.T): see ``dsb_gemm`` in include/dsb.h.  a: [M,K], w: [N,K] of one format."""
    _require_cuda(a, w, row_scale, col_scale, bias, gate, resid, out, out1)
    M, K, lda = _rows(a)
    N, Kw, ldw = _rows(w)
    if K != Kw or _fmt_of(a) != _fmt_of(w):
        raise _lib.DsbError("gemm operands disagree in K or format")
    if out is None:
        n0 = N if out1 is None else split_col
        out = torch.empty((M, n0), dtype=torch.bfloat16, device=a.device)
    if torch.float8_e4m3fn in (out.dtype, None if out1 is None else out1.dtype):
        # an e4m3 output selects the unit-scale 8-bit epilogue, which only the grouped entry point describes
        gemm_group([dict(a=a, w=w, row_scale=row_scale, col_scale=col_scale, bias=bias, act=act, act_col0=act_col0,
                         gate=gate, resid=resid, out=out, out1=out1, split_col=split_col)])
        return out
    _check_gemm_io(M, N, out, out1, split_col, resid, row_scale, col_scale, bias, gate)
    cs_stride = 0 if (col_scale is None or col_scale.numel() == 1) else 1
    rc = _lib.lib().dsb_gemm(
        _ptr(a), lda, _ptr(w), ldw, _fmt_of(a), M, N, K, _ptr(row_scale), _ptr(col_scale), cs_stride, _ptr(bias), act,
        act_col0, _ptr(gate), _ptr(resid), 0 if resid is None else resid.stride(0), _ptr(out), out.stride(0),
        _ptr(out1), 0 if out1 is None else out1.stride(0), N if split_col is None else split_col,
        _ptr(status_word(a.device)), _stream())
    check(rc, "dsb_gemm")
    return out


def _check_rope_table(rope, rows_needed):
    """The GEMM epilogue reads the RoPE table through a TMA map: fp16 [rows, 64, 2] (cos, sin), contiguous."""
    if rope is None:
        return
    if rope.dtype != torch.float16 or not rope.is_contiguous() or rope.numel() % 128 or rope.numel() // 128 < rows_needed:
        raise _lib.DsbError("the fused-RoPE GEMM takes a contiguous float16 [rows, 64, 2] table covering rope_row0 + M rows")


def gemm_qkv(a, w, nq_w, nk_w, d_model, rope=None, rope_row0=0, eps=1e-6, row_scale=None, col_scale=None, bias=None,
             act=ACT_NONE, act_col0=0, out=None, out1=None, split_col=None):
    """``dsb_gemm_qkv``: the fused q|k|v(|mlp) projection with per-head RMSNorm + RoPE on the q and k columns.
    ``rope``: float16 [rows, 64, 2] (cos, sin)."""
    _require_cuda(a, w, nq_w, nk_w, rope, row_scale, col_scale, bias, out, out1)
    _check_rope_table(rope, rope_row0 + a.shape[0])
    M, K, lda = _rows(a)
    N, Kw, ldw = _rows(w)
    if K != Kw or _fmt_of(a) != _fmt_of(w):
        raise _lib.DsbError("gemm operands disagree in K or format")
    if out is None:
        out = torch.empty((M, N if out1 is None else split_col), dtype=torch.bfloat16, device=a.device)
    if torch.float8_e4m3fn in (out.dtype, None if out1 is None else out1.dtype):
        gemm_group([dict(a=a, w=w, row_scale=row_scale, col_scale=col_scale, bias=bias, act=act, act_col0=act_col0,
                         out=out, out1=out1, split_col=split_col, nq_w=nq_w, nk_w=nk_w, d_model=d_model, rope=rope,
                         rope_row0=rope_row0, eps=eps)])
        return out
    _check_gemm_io(M, N, out, out1, split_col, None, row_scale, col_scale, bias, None)
    cs_stride = 0 if (col_scale is None or col_scale.numel() == 1) else 1
    rc = _lib.lib().dsb_gemm_qkv(
        _ptr(a), lda, _ptr(w), ldw, _fmt_of(a), M, N, K, _ptr(row_scale), _ptr(col_scale), cs_stride, _ptr(bias), act,
        act_col0, _ptr(out), out.stride(0), _ptr(out1), 0 if out1 is None else out1.stride(0),
        N if split_col is None else split_col, _ptr(nq_w), _ptr(nk_w), d_model, _ptr(rope), rope_row0, float(eps),
        _ptr(status_word(a.device)), _stream())
    check(rc, "dsb_gemm_qkv")
    return out


def gemm_group(problems):
    """``dsb_gemm_group``: one persistent launch for up to two GEMMs of one format.  Each problem is a dict with
    the keyword arguments of :func:`gemm` / :func:`gemm_qkv` (``a``, ``w``, ``out`` required; ``nq_w`` present
    selects the fused QK-RMSNorm/RoPE epilogue).  Outputs must be preallocated; an output of dtype float8_e4m3fn is
    written as the saturating e4m3 cast of the epilogue value (unit scale)."""
    if not 1 <= len(problems) <= 2:
        raise _lib.DsbError("gemm_group takes one or two problems")
    arr = (_lib.GemmArgs * len(problems))()
    fmt = _fmt_of(problems[0]["a"])
    keep = []
    for i, pr in enumerate(problems):
        a, w, out = pr["a"], pr["w"], pr["out"]
        out1, resid = pr.get("out1"), pr.get("resid")
        _require_cuda(a, w, out, out1, resid)
        M, K, lda = _rows(a)
        N, Kw, ldw = _rows(w)
        if K != Kw or _fmt_of(a) != fmt or _fmt_of(w) != fmt:
            raise _lib.DsbError("gemm_group operands disagree in K or format")
        if pr.get("nq_w") is not None:
            _check_rope_table(pr.get("rope"), pr.get("rope_row0", 0) + M)
        cs = pr.get("col_scale")
        _check_gemm_io(M, N, out, out1, pr.get("split_col"), resid, pr.get("row_scale"), cs, pr.get("bias"),
                       pr.get("gate"), e4m3_ok=True)
        g = arr[i]
        g.A, g.lda, g.W, g.ldw, g.M, g.N, g.K = a.data_ptr(), lda, w.data_ptr(), ldw, M, N, K
        for name, key in (("row_scale", "row_scale"), ("col_scale", "col_scale"), ("bias", "bias"), ("gate", "gate"),
                          ("resid", "resid"), ("out1", "out1"), ("nq_w", "nq_w"), ("nk_w", "nk_w"), ("rope", "rope")):
            t = pr.get(key)
            setattr(g, name, None if t is None else t.data_ptr())
            keep.append(t)
        g.col_scale_stride = 0 if (cs is None or cs.numel() == 1) else 1
        g.act, g.act_col0 = pr.get("act", ACT_NONE), pr.get("act_col0", 0)
        g.ld_resid = 0 if resid is None else resid.stride(0)
        g.out0, g.ld_out0 = out.data_ptr(), out.stride(0)
        g.ld_out1 = 0 if out1 is None else out1.stride(0)
        # an e4m3 output tensor selects the unit-scale 8-bit epilogue for that column range
        g.out0_fmt = FMT_E4M3 if out.dtype == torch.float8_e4m3fn else FMT_BF16
        g.out1_fmt = FMT_E4M3 if (out1 is not None and out1.dtype == torch.float8_e4m3fn) else FMT_BF16
        g.split_col = N if pr.get("split_col") is None else pr["split_col"]
        g.d_model, g.rope_row0, g.norm_eps = pr.get("d_model", 0), pr.get("rope_row0", 0), float(pr.get("eps", 1e-6))
    rc = _lib.lib().dsb_gemm_group(arr, len(problems), fmt, _ptr(status_word(problems[0]["a"].device)), _stream())
    check(rc, "dsb_gemm_group")


def flash_attn(q, k, v, out=None, sm_scale=None):
    """q: [B, Sq, H, 128], k/v: [B, Sk, H, 128] views (any strides that are multiples of 8, unit inner
    stride); returns o as [B, Sq, H, 128] contiguous unless ``out`` is given.  An ``out`` of dtype float8_e4m3fn
    receives the saturating e4m3 cast of the bf16 result (``dsb_flash_attn_out8``)."""
    _require_cuda(q, k, v, out)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    for t in (q, k, v):
        if t.stride(3) != 1 or t.dtype != torch.bfloat16:
            raise _lib.DsbError("flash_attn needs bf16 tensors with a contiguous head dimension")
    if k.shape != (B, Sk, H, D) or v.shape != k.shape:
        raise _lib.DsbError("flash_attn: k and v must be [B, Sk, H, 128] with the batch and heads of q")
    if out is None:
        out = torch.empty((B, Sq, H, D), dtype=torch.bfloat16, device=q.device)
    if out.dtype not in (torch.bfloat16, torch.float8_e4m3fn) or tuple(out.shape) != (B, Sq, H, D) or out.stride(3) != 1:
        raise _lib.DsbError("flash_attn out must be a bf16 or e4m3 [B, Sq, H, 128] view with a contiguous head dimension")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    fn = _lib.lib().dsb_flash_attn_out8 if out.dtype == torch.float8_e4m3fn else _lib.lib().dsb_flash_attn
    rc = fn(
        _ptr(q), _ptr(k), _ptr(v), _ptr(out), B, H, Sq, Sk, D,
        q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1), k.stride(2),
        v.stride(0), v.stride(1), v.stride(2), out.stride(0), out.stride(1), out.stride(2),
        float(sm_scale), _ptr(status_word(q.device)), _stream())
    check(rc, "dsb_flash_attn")
    return out


def _addr_array(items):
    """Host array of device addresses for the C side; items are tensors or integer addresses (memory of another GPU
    that this process has mapped has no tensor here)."""
    arr = (ctypes.c_void_p * len(items))()
    for i, it in enumerate(items):
        arr[i] = it.data_ptr() if isinstance(it, torch.Tensor) else int(it)
    return arr


def flash_attn_workspace(device) -> torch.Tensor:
    """A workspace large enough for any ``flash_attn_parts`` call on ``device`` (``dsb_flash_attn_workspace_bytes``;
    80 MB on a 148-SM part): lets the kernel cut the items of a partly filled last wave along the keys."""
    with torch.cuda.device(device):
        n = int(_lib.lib().dsb_flash_attn_workspace_bytes())
    return torch.empty(n, dtype=torch.uint8, device=device)


def flash_attn_parts(q_parts, q_rows_per_part, q_strides, k, v, o_parts, o_rows_per_part, o_strides, H, Sq,
                     sm_scale=None, workspace=None):
    """``dsb_flash_attn_parts``: one sample whose query rows come from ``q_parts[i]`` (``q_rows_per_part`` rows each,
    a multiple of 128) and whose output row s goes to ``o_parts[s // o_rows_per_part]``.  Parts are tensors or raw
    device addresses (peer memory); ``q_strides`` / ``o_strides`` are the (token, head) strides in elements inside a
    part.  k, v: [1, Sk, H, 128] views on the current device.  ``workspace`` (``flash_attn_workspace``): optional,
    lets a partly filled last wave be cut along the keys."""
    _require_cuda(k, v, *[t for t in list(q_parts) + list(o_parts) if isinstance(t, torch.Tensor)])
    if k.dim() != 4 or k.shape[0] != 1 or k.shape[2] != H or k.shape[3] != 128 or v.shape != k.shape:
        raise _lib.DsbError("flash_attn_parts takes k and v as [1, Sk, H, 128]")
    for t in (k, v):
        if t.stride(3) != 1 or t.dtype != torch.bfloat16:
            raise _lib.DsbError("flash_attn needs bf16 tensors with a contiguous head dimension")
    for parts, rows, (ss, sh) in ((q_parts, q_rows_per_part, q_strides), (o_parts, o_rows_per_part, o_strides)):
        if not 1 <= len(parts) <= 8 or rows <= 0 or len(parts) * rows < Sq:
            raise _lib.DsbError("flash_attn_parts: 1..8 parts that together cover Sq rows")
        for i, t in enumerate(parts):
            if isinstance(t, torch.Tensor):
                # query parts are read in whole tiles: each holds all its rows; output rows past Sq are not written
                n_rows = rows if parts is q_parts else max(0, min(rows, Sq - i * rows))
                need = 0 if n_rows == 0 else (n_rows - 1) * ss + (H - 1) * sh + 128
                if t.dtype != torch.bfloat16 or t.untyped_storage().nbytes() // 2 - t.storage_offset() < need:
                    raise _lib.DsbError("flash_attn_parts: a part is not bf16 or too small for its rows")
    if q_rows_per_part % 128:
        raise _lib.DsbError("flash_attn_parts: q_rows_per_part must be a multiple of 128")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(128)
    qa, oa = _addr_array(q_parts), _addr_array(o_parts)
    if workspace is not None:
        _require_cuda(workspace)
        if workspace.dtype != torch.uint8 or not workspace.is_contiguous():
            raise _lib.DsbError("flash_attn_parts workspace must be a contiguous uint8 tensor")
    rc = _lib.lib().dsb_flash_attn_parts(
        qa, len(q_parts), q_rows_per_part, _ptr(k), _ptr(v), oa, len(o_parts), o_rows_per_part, H, Sq, k.shape[1], 128,
        q_strides[0], q_strides[1], k.stride(1), k.stride(2), v.stride(1), v.stride(2), o_strides[0], o_strides[1],
        float(sm_scale), _ptr(workspace), 0 if workspace is None else workspace.numel(),
        _ptr(status_word(k.device)), _stream())
    check(rc, "dsb_flash_attn_parts")


def rank_barrier(flag_arrays, rank, epoch, limit_cycles=20_000_000_000, status=None):
    """``dsb_rank_barrier`` on the current stream: ``flag_arrays[r]`` is rank r's int32 flag array (tensor or raw
    device address mapped in this process).  ``limit_cycles`` SM cycles (default: about ten seconds) bound the wait;
    a timeout lands in the device status word (``check_status``)."""
    n = len(flag_arrays)
    st = status if status is not None else status_word(torch.device("cuda", torch.cuda.current_device()))
    rc = _lib.lib().dsb_rank_barrier(_addr_array(flag_arrays), n, rank, int(epoch), int(limit_cycles), _ptr(st), _stream())
    check(rc, "dsb_rank_barrier")


def patchify(latents, row0=0, n_rows=None, out_fmt=FMT_BF16, out=None, row_scale=None):
    """``dsb_patchify``: latents ``[C, F, 2gh, 2gw]`` (bf16, contiguous; a leading batch of 1 is accepted) -> token
    rows ``[n_rows, C*4]`` from token ``row0`` on; 8-bit formats also return the per-row scale."""
    _require_cuda(latents, out, row_scale)
    _require_bf16(latents, "patchify")
    lat = latents[0] if latents.dim() == 5 else latents
    if lat.dim() != 4 or not lat.is_contiguous() or lat.shape[2] % 2 or lat.shape[3] % 2:
        raise _lib.DsbError("patchify takes contiguous [C, F, H, W] latents with even H and W")
    C, F, gh, gw = lat.shape[0], lat.shape[1], lat.shape[2] // 2, lat.shape[3] // 2
    if n_rows is None:
        n_rows = F * gh * gw - row0
    if out is None:
        out = torch.empty((n_rows, C * 4), dtype=_OUT_DTYPE[out_fmt], device=lat.device)
    if out.dtype != _OUT_DTYPE[out_fmt] or out.dim() != 2 or out.stride(1) != 1 or out.shape[0] < n_rows or out.shape[1] < C * 4:
        raise _lib.DsbError("patchify output must be [>= n_rows, >= C*4] rows of the requested format")
    if out_fmt != FMT_BF16:
        if row_scale is None:
            row_scale = torch.empty(n_rows, dtype=torch.float32, device=lat.device)
        if row_scale.dtype != torch.float32 or row_scale.numel() < n_rows or not row_scale.is_contiguous():
            raise _lib.DsbError("patchify row_scale must be contiguous float32 [n_rows]")
    rc = _lib.lib().dsb_patchify(_ptr(lat), C, F, gh, gw, row0, n_rows, out_fmt, _ptr(out), out.stride(0),
                                 _ptr(row_scale) if out_fmt != FMT_BF16 else None, _stream())
    check(rc, "dsb_patchify")
    return out, (row_scale if out_fmt != FMT_BF16 else None)


def unpatchify(tokens, C, F, gh, gw, c_fastest, out=None):
    """``dsb_unpatchify``: token rows ``[F*gh*gw, >= C*4]`` (bf16) -> latents ``[1, C, F, 2gh, 2gw]``."""
    _require_cuda(tokens, out)
    _require_bf16(tokens, "unpatchify")
    if tokens.dim() != 2 or tokens.stride(1) != 1 or tokens.shape[0] < F * gh * gw or tokens.shape[1] < C * 4:
        raise _lib.DsbError("unpatchify takes [>= F*gh*gw, >= C*4] token rows")
    if out is None:
        out = torch.empty((1, C, F, 2 * gh, 2 * gw), dtype=torch.bfloat16, device=tokens.device)
    if out.dtype != torch.bfloat16 or not out.is_contiguous() or out.numel() != C * F * 4 * gh * gw:
        raise _lib.DsbError("unpatchify output must be a contiguous bf16 [C, F, 2gh, 2gw] tensor")
    rc = _lib.lib().dsb_unpatchify(_ptr(tokens), tokens.stride(0), C, F, gh, gw, 1 if c_fastest else 0, _ptr(out), _stream())
    check(rc, "dsb_unpatchify")
    return out


def pack_quant_weight(W, fmt=FMT_E4M3, per_channel=False):
    """Quantise a [N,K] fp32/bf16 weight on the device; returns (payload, scales)."""
    _require_cuda(W)
    N, K, ld = _rows(W)
    if W.dtype not in (torch.float32, torch.bfloat16):
        raise _lib.DsbError("pack_quant_weight takes fp32 or bf16 weights")
    payload = torch.empty((N, K), dtype=_OUT_DTYPE[fmt], device=W.device)
    scales = torch.empty(N if per_channel else 1, dtype=torch.float32, device=W.device)
    work = torch.zeros(1, dtype=torch.float32, device=W.device)
    rc = _lib.lib().dsb_pack_quant_weight(_ptr(W), ld, 1 if W.dtype == torch.bfloat16 else 0, _ptr(payload), K,
                                          _ptr(scales), N, K, fmt, 1 if per_channel else 0, _ptr(work), _stream())
    check(rc, "dsb_pack_quant_weight")
    return payload, scales


def linear_static(x, w_payload, w_scale, bias=None, act=ACT_NONE, out=None):
    """``dsb_linear_static``: quantise the bf16 rows of ``x`` and multiply by the prepacked ``w_payload`` without
    any caller-provided scratch - the intermediates live in a fixed array inside the library (see
    include/dsb.h for who needs that, the size limit and the sharing rules).  Only the output is allocated here,
    and not at all when ``out`` is given."""
    _require_cuda(x, w_payload, w_scale, bias, out)
    _require_bf16(x, "linear_static")
    M, K, ld_x = _rows(x)
    N, Kw, ld_w = _rows(w_payload)
    if K != Kw:
        raise _lib.DsbError("linear_static operands disagree in K")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    stride = 0 if w_scale.numel() == 1 else 1
    rc = _lib.lib().dsb_linear_static(_ptr(x), ld_x, _ptr(w_payload), ld_w, _fmt_of(w_payload), M, N, K,
                                      _ptr(w_scale), stride, _ptr(bias), act, _ptr(out), out.stride(0),
                                      _ptr(status_word(x.device)), _stream())
    check(rc, "dsb_linear_static")
    return out
