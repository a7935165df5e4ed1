"""ctypes binding of ``libdsb.so``.  There is no fallback: if the library is missing or does not
load, every op raises - the CUDA path is the only path."""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdsb.so")
HEADER = os.path.join(os.path.dirname(HERE), "include", "dsb.h")

OK, ERR_ARG, ERR_CUDA, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_TOO_LARGE = 0, -1, -2, -3, -4, -5
FMT_BF16, FMT_E4M3, FMT_INT8 = 0, 1, 2
ACT_NONE, ACT_GELU_TANH, ACT_SILU, ACT_GELU = 0, 1, 2, 3

_ERR_NAMES = {
    ERR_ARG: "DSB_ERR_ARG (bad pointer, size, alignment or flag combination)",
    ERR_CUDA: "DSB_ERR_CUDA (a CUDA call failed)",
    ERR_TIMEOUT: "DSB_ERR_TIMEOUT (a bounded device wait ran out)",
    ERR_UNSUPPORTED: "DSB_ERR_UNSUPPORTED (shape outside what the kernel supports)",
    ERR_TOO_LARGE: "DSB_ERR_TOO_LARGE (the problem does not fit the fixed scratch of a *_static entry point: "
                   "M*K <= 64 Mi elements and M <= 65536)",
}

c_i, c_i64, c_f, c_p = ctypes.c_int, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p

# argument lists, in the order of include/dsb.h
_SIGS = {
    "dsb_version": [],
    "dsb_selftest_wait_timeout": [ctypes.c_longlong, c_p, c_p, c_p],
    "dsb_patchify": [c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_p, c_i64, c_p, c_p],
    "dsb_unpatchify": [c_p, c_i64, c_i, c_i, c_i, c_i, c_i, c_p, c_p],
    "dsb_rank_barrier": [c_p, c_i, c_i, c_i, ctypes.c_longlong, c_p, c_p],
    "dsb_flash_attn_parts": [c_p, c_i, c_i, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i] + [c_i64] * 8 + [c_f, c_p, c_i64, c_p, c_p],
    "dsb_flash_attn_workspace_bytes": [],
    "dsb_ln_modulate": [c_p, c_i64, c_p, c_p, c_p, c_i64, c_p, c_i, c_i, c_f, c_i, c_p],
    "dsb_ln_modulate2": [c_p, c_i64, c_p, c_p, c_i, c_p, c_p, c_p, c_i64, c_p, c_i, c_i, c_f, c_i, c_p],
    "dsb_gate_residual": [c_p, c_i64, c_p, c_i64, c_p, c_p, c_i64, c_i, c_i, c_p],
    "dsb_rmsnorm_rope_heads": [c_p, c_i64, c_i, c_i, c_i, c_i, c_p, c_p, c_p, c_i, c_f, c_p],
    "dsb_rmsnorm_full": [c_p, c_i64, c_p, c_i64, c_i, c_i64, c_i, c_i, c_p, c_p, c_i, c_f, c_p],
    "dsb_quant_rows_chunked": [c_p, c_i64, c_i, c_i64, c_p, c_i64, c_p, c_i, c_i, c_i, c_p],
    "dsb_quant_rows": [c_p, c_i64, c_p, c_i64, c_p, c_i, c_i, c_i, c_p],
    "dsb_dequant_q8_0": [c_p, c_i64, c_i, c_i, c_p, c_i64, c_p],
    "dsb_dequant_q4_k": [c_p, c_i64, c_i, c_i, c_p, c_i64, c_p],
    "dsb_dequant_gguf": [c_i, c_p, c_i64, c_i, c_i, c_p, c_i64, c_p],
    "dsb_cast_quant": [c_p, c_i64, c_p, c_i64, c_i, c_i, c_i, c_i, c_p],
    "dsb_gemv": [c_p, c_i64, c_i, c_p, c_p, c_i, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_p],
    "dsb_timestep_embedding": [c_p, c_i, c_i, c_f, c_i, c_i, c_p, c_p],
    "dsb_cfg_euler_step": [c_p, c_p, c_p, c_f, c_f, c_p, c_i64, c_i, c_p],
    "dsb_euler_step": [c_p, c_p, c_p, c_p, c_f, c_p, c_i64, c_i, c_p],
    "dsb_gemm": [c_p, c_i64, c_p, c_i64, c_i, c_i, c_i, c_i, c_p, c_p, c_i, c_p, c_i, c_i, c_p, c_p, c_i64, c_p,
                 c_i64, c_p, c_i64, c_i, c_p, c_p],
    "dsb_gemm_qkv": [c_p, c_i64, c_p, c_i64, c_i, c_i, c_i, c_i, c_p, c_p, c_i, c_p, c_i, c_i, c_p, c_i64, c_p, c_i64, c_i,
                     c_p, c_p, c_i, c_p, c_i, c_f, c_p, c_p],
    "dsb_flash_attn": [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i] + [c_i64] * 12 + [c_f, c_p, c_p],
    "dsb_flash_attn_out8": [c_p, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i] + [c_i64] * 12 + [c_f, c_p, c_p],
    "dsb_pack_quant_weight": [c_p, c_i64, c_i, c_p, c_i64, c_p, c_i, c_i, c_i, c_i, c_p, c_p],
    "dsb_linear_static": [c_p, c_i64, c_p, c_i64, c_i, c_i, c_i, c_i, c_p, c_i, c_p, c_i, c_p, c_i64, c_p, c_p],
}



class GemmArgs(ctypes.Structure):
    """``dsb_gemm_args`` of include/dsb.h."""
    _fields_ = [("A", c_p), ("lda", c_i64), ("W", c_p), ("ldw", c_i64), ("M", c_i), ("N", c_i), ("K", c_i),
                ("row_scale", c_p), ("col_scale", c_p), ("col_scale_stride", c_i), ("bias", c_p), ("act", c_i),
                ("act_col0", c_i), ("gate", c_p), ("resid", c_p), ("ld_resid", c_i64), ("out0", c_p),
                ("ld_out0", c_i64), ("out1", c_p), ("ld_out1", c_i64), ("split_col", c_i), ("nq_w", c_p),
                ("nk_w", c_p), ("d_model", c_i), ("rope", c_p), ("rope_row0", c_i), ("norm_eps", c_f),
                ("out0_fmt", c_i), ("out1_fmt", c_i)]


_SIGS["dsb_gemm_group"] = [ctypes.POINTER(GemmArgs), c_i, c_i, c_p, c_p]

_lib = None


class DsbError(RuntimeError):
    pass


def declared_symbols():
    """Names of every function declared in include/dsb.h."""
    with open(HEADER) as f:
        text = f.read()
    return sorted(set(re.findall(r"^int\s+(dsb_\w+)\s*\(", text, flags=re.M)))


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise DsbError(
                f"{LIB_PATH} is missing: build it with `python diffsynth-engine_b200/build.py` "
                "(there is no CPU or PyTorch fallback)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, args in _SIGS.items():
            fn = getattr(handle, name)
            fn.argtypes = args
            fn.restype = c_i64 if name == "dsb_flash_attn_workspace_bytes" else c_i
        _lib = handle
    return _lib


launches = 0  # successful op calls so far (one kernel launch each on the step's path)


def check(rc: int, what: str):
    global launches
    launches += 1
    if rc != OK:
        raise DsbError(f"{what} failed: {_ERR_NAMES.get(rc, rc)}")
