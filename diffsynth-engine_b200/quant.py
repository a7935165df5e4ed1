"""Quantised-Linear drop-in behind the reference's own seam.

DiffSynth-Engine switches its FP8 Linear on by (a) ``enable_fp8_linear(module)``, which rewrites every
``nn.Linear`` weight in place, and (b) the context manager ``fp8_inference()`` that swaps
``torch.nn.functional.linear`` for the duration of ``FluxDiT.forward`` (utils/fp8_linear.py:7-64).  Quantised
weights that need metadata travel as a ``Parameter`` subclass (``GGUFParameter``, utils/gguf.py:9-59) because
``F.linear`` never sees the module.  The same two pieces, same names and argument meaning, backed by
``dsb_quant_rows`` + ``dsb_gemm`` / ``dsb_gemv``:

    enable_b200_linear(dit, fmt="fp8_tensor")        # once, weights already on the GPU
    with b200_inference():
        dit(...)                                      # every Linear whose weight is a QuantLinearWeight runs here

Anything that is not a ``QuantLinearWeight`` (VAE, text encoders, LoRA side matrices) falls through to the
original ``F.linear`` untouched; ``lora.fuse_lora(dit)`` folds loaded-but-unfused LoRAs into the quantised GEMM.  Unlike the reference's context manager this one restores ``F.linear`` in a
``finally`` block.
"""
from contextlib import contextmanager

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .packed import FORMATS, act_format


class QuantLinearWeight(nn.Parameter):
    """``[N, K]`` quantised payload (float8_e4m3fn / int8, or bf16 for fmt="bf16") carrying ``scale``
    (fp32 ``[1]`` or ``[N]``) and ``fmt``."""

    def __new__(cls, payload: torch.Tensor, scale, fmt: str):
        self = torch.Tensor._make_subclass(cls, payload, False)
        self.scale = scale
        self.fmt = fmt
        self._bias_f32 = None
        self.lora_ext = None      # unfused LoRAs riding in the GEMM as extra K columns (lora.fuse_lora)
        self._lora_sig = None
        return self

    __torch_function__ = torch._C._disabled_torch_function_impl

    def bias_f32(self, bias):
        """fp32 copy of the module's bias (the GEMM epilogue adds an fp32 bias); cached per bias tensor."""
        if bias is None:
            return None
        key = (bias.data_ptr(), bias._version)
        if self._bias_f32 is None or self._bias_f32[0] != key:
            self._bias_f32 = (key, bias.detach().float().contiguous())
        return self._bias_f32[1]


def _gguf_type(weight):
    """The block format name ("Q8_0", "Q4_K", "Q6_K", ...) of a ``GGUFParameter`` (utils/gguf.py:9-59: raw uint8 rows
    plus a ``quant_dtype`` tag) if it is one this library dequantises itself - every format the reference does -
    else None."""
    qd = getattr(weight, "quant_dtype", None)
    name = None if qd is None else getattr(qd, "name", str(qd))
    return name if name in ops.GGUF_TYPES else None


def _is_gguf_q8_0(weight) -> bool:
    return _gguf_type(weight) == "Q8_0"


def _raw_bytes(weight) -> torch.Tensor:
    """The stored bytes of a GGUFParameter (its ``shape``/``dtype`` properties describe the dequantised weight)."""
    t = torch.Tensor._make_subclass(torch.Tensor, weight.detach(), False)
    return t.view(torch.uint8) if t.dtype != torch.uint8 else t


def _enable_b200_linear(module: nn.Module, fmt: str):
    if isinstance(module, nn.Linear) and _gguf_type(module.weight) is not None:
        # GGUF Q8_0 / Q4_K: dequantise ONCE, exactly as the reference does per call, then prepack like any other weight
        raw = _raw_bytes(module.weight)
        if not raw.is_cuda:
            raise ops._lib.DsbError("enable_b200_linear: move the module to the GPU first (no CPU path exists)")
        raw = raw.reshape(raw.shape[0], -1).contiguous()
        qt = _gguf_type(module.weight)
        w = (ops.dequant_q8_0(raw) if qt == "Q8_0" else ops.dequant_q4_k(raw) if qt == "Q4_K"
             else ops.dequant_gguf(raw, qt))
        if fmt == "bf16":
            payload, scale = w, None
        else:
            code = ops.FMT_INT8 if fmt == "int8_channel" else ops.FMT_E4M3
            payload, scale = ops.pack_quant_weight(w, code, per_channel=(fmt != "fp8_tensor"))
        module.weight = QuantLinearWeight(payload, scale, fmt)
    elif isinstance(module, nn.Linear) and torch.is_floating_point(module.weight.data) \
            and not isinstance(module.weight, QuantLinearWeight):
        w = module.weight.data
        if not w.is_cuda:
            raise ops._lib.DsbError("enable_b200_linear: move the module to the GPU first (no CPU path exists)")
        if w.dtype not in (torch.float32, torch.bfloat16):
            w = w.float()
        if fmt == "bf16":
            payload, scale = w.to(torch.bfloat16).contiguous(), None
        else:
            code = ops.FMT_INT8 if fmt == "int8_channel" else ops.FMT_E4M3
            payload, scale = ops.pack_quant_weight(w.contiguous(), code, per_channel=(fmt != "fp8_tensor"))
        module.weight = QuantLinearWeight(payload, scale, fmt)
    for sub in module.children():
        _enable_b200_linear(sub, fmt)


def enable_b200_linear(module: nn.Module, fmt: str = "fp8_tensor"):
    """Counterpart of ``enable_fp8_linear`` (utils/fp8_linear.py:7-17): prepack every floating ``nn.Linear``
    weight below ``module`` and mark the module.  GGUF Q8_0 and Q4_K weights (``GGUFParameter``) are dequantised once on the
    device (``fmt="bf16"`` keeps exactly the values the reference's ``gguf_linear`` multiplies with) and then take
    the same path, so they no longer depend on ``gguf_inference`` re-materialising them in every call."""
    if fmt not in FORMATS:
        raise ValueError(f"fmt must be one of {FORMATS}, but got '{fmt}'")
    _enable_b200_linear(module, fmt)
    setattr(module, "b200_linear_enabled", True)


def b200_linear(input: torch.Tensor, weight: torch.Tensor, bias=None, _origin=F.linear) -> torch.Tensor:
    """``F.linear`` for a ``QuantLinearWeight``: flatten leading dims, quantise rows, tensor-core GEMM with the
    scales and bias in its epilogue, output in the input dtype (the dataflow of utils/fp8_linear.py:27-60)."""
    if not isinstance(weight, QuantLinearWeight):
        return _origin(input, weight, bias)
    if not input.is_cuda:
        raise ops._lib.DsbError("b200_linear got a CPU tensor: there is no CPU fallback")
    N, K = weight.shape
    lead = input.shape[:-1]
    x = input.reshape(-1, K)
    M = x.shape[0]
    b32 = weight.bias_f32(bias)
    payload = weight.data
    ext = getattr(weight, "lora_ext", None)
    if ext is not None:
        from .lora import linear_lora
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        if xb.stride(-1) != 1 or (xb.stride(0) % 8) or (xb.data_ptr() % 16):
            xb = xb.contiguous()
        return linear_lora(xb, payload, weight.scale, b32, ext).to(input.dtype).reshape(*lead, N)
    if M <= 4:  # conditioning vectors: bandwidth-bound GEMV on fp32 activations, weights dequantised on the fly
        xf = x.float().contiguous()
        rows = [ops.gemv(payload, xf[i], weight.scale, b32) for i in range(M)]
        y = torch.stack(rows) if M > 1 else rows[0][None]
        return y.to(input.dtype).reshape(*lead, N)
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    if xb.stride(-1) != 1 or (xb.stride(0) % 8) or (xb.data_ptr() % 16):
        xb = xb.contiguous()
    afmt = act_format(weight.fmt)
    if afmt == ops.FMT_BF16:
        y = ops.gemm(xb, payload, bias=b32)
    else:
        xq, rs = ops.quant_rows(xb, afmt)
        y = ops.gemm(xq, payload, row_scale=rs, col_scale=weight.scale, bias=b32)
    return y.to(input.dtype).reshape(*lead, N)


@contextmanager
def b200_inference(enabled: bool = True):
    """Counterpart of ``fp8_inference`` (utils/fp8_linear.py:20-64): patches ``torch.nn.functional.linear``;
    nests with the reference's ``gguf_inference`` the same way (the patched function keeps the previous one as
    its fall-through)."""
    if not enabled:
        yield
        return
    origin = F.linear

    def patched(input, weight, bias=None):
        return b200_linear(input, weight, bias, _origin=origin)

    F.linear = patched
    try:
        yield
    finally:
        F.linear = origin
