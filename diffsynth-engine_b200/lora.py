"""Unfused LoRA inside the quantised Linear.

The reference keeps loaded-but-unfused LoRAs as two extra bf16 Linears per adapter and adds
``scale * alpha / rank * up(down(x))`` to the main Linear's output (models/basic/lora.py:29-32,137-141): two more
GEMM launches, a scaling pass and an in-place add over ``[M, N]`` per adapter.  Here the adapters ride in the main
tensor-core GEMM as extra K columns:

    stacked  D = cat(down_i) [R, K],  U = cat(coef_i * up_i) [N, R]          (R padded to a multiple of 64)
    offline  D_q, s_D  = per-row quantisation of D;   U_q = cast(U * tau / s_n)
             W_ext = [W_q | U_ext]                                            [N, K + E]
    per call x_q, s_m  = quant_rows(x)             -> columns [0, K) of the activation buffer
             t         = gemm(x_q, D_q) * (s_D / tau)   (no row scale: s_m cancels)        [M, R] bf16
             cast_quant(t)                          -> columns [K, K + E) of the same buffer
             y         = gemm([x_q | t_ext], W_ext) * s_m * s_n + bias        (any fused epilogue of the main GEMM)

because ``s_m s_n * t_q U_q = s_m s_n * (x.D_j / (s_m tau_j)) * (U_nj tau_j / s_n) = (x.D_j) U_nj``.  ``tau_j``
splits the 8-bit range between the two factors of rank column j (``_balance``: as much headroom as the range has
goes to t, whose bound is only statistical).  FP8: both factors are split into an e4m3 head and
an e4m3 remainder (E = 3R: t_ext = [t_hi | t_lo | t_hi] against U_ext = [U_hi | U_hi | U_lo]), so the LoRA term is
as accurate as the main product; INT8: E = R, errors in units of the main GEMM's quantisation step, like R more
weight columns.  A LoRA whose columns exceed the 8-bit range after balancing is rejected (keep it unfused).  With
bf16 weights the side matrices stay two bf16 GEMMs, the second one adding into the main output through the
residual epilogue.
"""
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from . import ops
from .packed import act_format

PAD = 64


@dataclass
class LoraExtension:
    fmt: str
    rank: int                       # padded stacked rank R
    ext_cols: int                   # E: K columns added to the main GEMM (3R for FP8, R for INT8, 0 for bf16)
    w_ext: Optional[torch.Tensor]   # [N, K + E] 8-bit payload (None for bf16 weights)
    down: torch.Tensor              # [R, K] in the operand format (bf16 for bf16 weights)
    down_scale: Optional[torch.Tensor]   # fp32 [R] = s_D / tau (None for bf16)
    up: Optional[torch.Tensor]      # bf16 [N, R] = coef * up (bf16 weights only)


def _balance(a: torch.Tensor, bmax: torch.Tensor, qmax: float) -> torch.Tensor:
    """tau_j for rank column j: the activation-side factor t_j = x_q.D_j / tau_j is expected to stay below
    ``a_j / tau_j``, the weight-side factor is bounded by ``bmax_j * tau_j``; both must fit ``qmax``.  The weight-side
    bound is exact, the activation-side one is a statistical estimate that an activation row aligned with D_j exceeds
    (by up to sqrt(K)), and a value past ``qmax`` would saturate in ``dsb_cast_quant``.  So the expected t is aimed at
    ``qmax / 8`` or the balanced point sqrt(a*bmax), whichever is smaller - but never below a*bmax/qmax, where the
    weight-side factor reaches ``qmax``: every bit of slack the 8-bit range has goes to the side whose bound is not
    exact."""
    prod = a * bmax
    target = torch.maximum(prod / qmax, torch.minimum(torch.sqrt(prod), torch.full_like(prod, qmax / 8.0)))
    tau = a / target.clamp_min(1e-30)
    return torch.where((a > 0) & (bmax > 0), tau, torch.ones_like(tau))


def build_lora_extension(payload: torch.Tensor, scale: Optional[torch.Tensor], fmt: str,
                         loras: Sequence[Tuple[float, torch.Tensor, torch.Tensor]]) -> LoraExtension:
    """``loras``: (coef, up [N, r], down [r, K]) with coef = scale * alpha / rank.  ``payload``/``scale``: the
    prepacked main weight (``pack_linear`` / ``QuantLinearWeight``)."""
    if not loras:
        raise ValueError("no LoRA to attach")
    dev = payload.device
    N, K = payload.shape
    D = torch.cat([d.to(dev, torch.float32) for _, _, d in loras], dim=0)
    U = torch.cat([float(c) * u.to(dev, torch.float32) for c, u, _ in loras], dim=1)
    if D.shape[1] != K or U.shape[0] != N or U.shape[1] != D.shape[0]:
        raise ValueError("LoRA matrices do not match the Linear: need up [N, r] and down [r, K]")
    R = D.shape[0]
    Rp = (R + PAD - 1) // PAD * PAD
    D = torch.cat([D, torch.zeros(Rp - R, K, device=dev)], dim=0).contiguous()
    U = torch.cat([U, torch.zeros(N, Rp - R, device=dev)], dim=1)
    afmt = act_format(fmt)
    if afmt == ops.FMT_BF16:
        return LoraExtension(fmt, Rp, 0, None, D.to(torch.bfloat16), None, U.to(torch.bfloat16).contiguous())
    qmax = 127.0 if afmt == ops.FMT_INT8 else 448.0
    D_q, s_D = ops.pack_quant_weight(D, afmt, per_channel=True)
    s_n = scale.float().reshape(-1, 1) if scale.numel() > 1 else scale.float().reshape(1, 1)
    a = qmax * D.norm(dim=1)                 # 4-sigma estimate of |x_q . D_j| for activations uncorrelated with D_j
    bmax = (U / s_n).abs().amax(dim=0)       # exact bound of the other factor
    tau = _balance(a, bmax, qmax)
    Up = U * tau[None, :] / s_n
    if float(Up.abs().amax()) > qmax * (1.0 + 1e-4):
        raise ValueError("a LoRA column is larger than the quantised weight's range allows; keep it unfused")
    Up = Up.clamp(-qmax, qmax)
    if afmt == ops.FMT_INT8:
        U_q = torch.clamp(torch.round(Up), -127, 127).to(torch.int8)
    else:
        U_hi = Up.to(torch.float8_e4m3fn)
        U_lo = (Up - U_hi.float()).to(torch.float8_e4m3fn)
        U_q = torch.cat([U_hi, U_hi, U_lo], dim=1)
    w_ext = torch.cat([payload.view(torch.uint8), U_q.view(torch.uint8)], dim=1).contiguous().view(payload.dtype)
    return LoraExtension(fmt, Rp, U_q.shape[1], w_ext, D_q, (s_D.float() / tau).contiguous(), None)


def linear_lora(x: torch.Tensor, payload: torch.Tensor, scale, bias, ext: LoraExtension, out=None, **epilogue):
    """``x [M, K]`` bf16 -> ``[M, N]`` bf16: the main Linear plus its attached LoRAs.  ``epilogue``: the keyword
    arguments of :func:`ops.gemm` (``act``, ``gate``, ``resid`` ...)."""
    M, K = x.shape
    afmt = act_format(ext.fmt)
    if afmt == ops.FMT_BF16:
        t = ops.gemm(x, ext.down)
        y = ops.gemm(x, payload, bias=bias, out=out, **epilogue)
        return ops.gemm(t, ext.up, resid=y, out=y)
    qdt = torch.float8_e4m3fn if afmt == ops.FMT_E4M3 else torch.int8
    xq = torch.empty((M, K + ext.ext_cols), dtype=qdt, device=x.device)
    rs = torch.empty(M, dtype=torch.float32, device=x.device)
    ops.quant_rows(x, afmt, out=xq[:, :K], row_scale=rs)
    t = ops.gemm(xq[:, :K], ext.down, col_scale=ext.down_scale)
    ops.cast_quant(t, xq[:, K:], afmt, split=(afmt == ops.FMT_E4M3))
    return ops.gemm(xq, ext.w_ext, row_scale=rs, col_scale=scale, bias=bias, out=out, **epilogue)


# ---------------------------------------------------------------------- the reference's module seam
def _adapters(module) -> List[Tuple[float, torch.Tensor, torch.Tensor]]:
    out = []
    for lora in module._lora_dict.values():
        up = lora.up.weight if hasattr(lora.up, "weight") else lora.up
        down = lora.down.weight if hasattr(lora.down, "weight") else lora.down
        out.append((float(lora.scale) * float(lora.alpha) / float(lora.rank), up.detach(), down.detach()))
    return out


def _signature(module):
    return tuple((name, float(l.scale), float(l.alpha), float(l.rank),
                  (l.up.weight if hasattr(l.up, "weight") else l.up).data_ptr(),
                  (l.down.weight if hasattr(l.down, "weight") else l.down).data_ptr())
                 for name, l in module._lora_dict.items())


def _fused_forward(self, x):
    """Replacement of ``LoRALinear.forward`` (lora.py:137-141) once the adapters ride in the quantised weight:
    one patched ``F.linear`` call, no side-matrix loop.  Rebuilds the extension when adapters or scales changed."""
    import torch.nn.functional as F
    w = self.weight
    sig = _signature(self)
    if getattr(w, "_lora_sig", None) != sig:
        w.lora_ext = build_lora_extension(w.data, w.scale, w.fmt, _adapters(self)) if sig else None
        w._lora_sig = sig
    return F.linear(x, w, self.bias)


def fuse_lora(module: torch.nn.Module) -> int:
    """For every ``LoRALinear``-like module below ``module`` (an ``nn.Linear`` with a ``_lora_dict`` of adapters
    carrying ``scale``/``alpha``/``rank``/``up``/``down``) whose weight was prepacked by ``enable_b200_linear``:
    route its forward through the fused path.  ``modify_scale``, ``add_lora`` and ``clear`` of the reference keep
    working (the extension is rebuilt on the next call).  Returns the number of modules switched."""
    from .quant import QuantLinearWeight
    n = 0
    for sub in module.modules():
        if isinstance(sub, torch.nn.Linear) and hasattr(sub, "_lora_dict") and isinstance(sub.weight, QuantLinearWeight) \
                and not getattr(type(sub), "_b200_fused_lora", False):
            cls = type(sub)
            sub.__class__ = type("B200Fused" + cls.__name__, (cls,), {"forward": _fused_forward,
                                                                      "_b200_fused_lora": True, "_b200_base": cls})
            n += 1
    return n


def unfuse_lora(module: torch.nn.Module) -> int:
    n = 0
    for sub in module.modules():
        if getattr(type(sub), "_b200_fused_lora", False):
            sub.__class__ = type(sub)._b200_base
            sub.weight.lora_ext, sub.weight._lora_sig = None, None
            n += 1
    return n
