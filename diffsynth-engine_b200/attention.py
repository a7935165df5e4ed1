"""Attention drop-in behind the reference's dispatch points.

* Flux: the module global ``flux_dit._attn_func`` is called as ``_attn_func(q, k, v)`` with ``[B, H, S, D]``
  tensors (q, k fresh from RoPE; v possibly a strided view of the fused projection) and must return
  ``[B, H, S, D]`` (models/flux/flux_dit.py:21,182,267,303); ``FluxDiT.set_attn_implementation(name)`` rebinds it
  (:480-504).
* Wan: the module function ``wan_dit.attention(q, k, v, num_heads)`` takes and returns ``[B, S, H*D]``
  (models/wan/wan_dit.py:18-22) and is looked up at call time.
"""
import torch

from . import ops

SUPPORTED = ("sdpa", "b200")


def _check(t):
    if not t.is_cuda:
        raise ops._lib.DsbError("b200 attention got a CPU tensor: there is no CPU fallback")
    if t.dtype != torch.bfloat16:
        raise ops._lib.DsbError(f"b200 attention takes bf16 tensors, got {t.dtype}")
    return t if t.stride(-1) == 1 and all(s % 8 == 0 for s in t.stride()[:-1]) else t.contiguous()


def b200_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, **kwargs) -> torch.Tensor:
    """``_attn_func`` replacement: ``[B, H, S, D]`` in and out.  The result's memory is ``[B, S, H, D]``, so the
    caller's ``transpose(1, 2).reshape(B, S, H*D)`` (flux_dit.py:183) is a view, not a copy."""
    if kwargs:
        raise TypeError(f"b200_attn supports the unmasked default call only, got {sorted(kwargs)}")
    q, k, v = _check(q), _check(k), _check(v)
    out = ops.flash_attn(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return out.transpose(1, 2)


def b200_wan_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_heads: int) -> torch.Tensor:
    """``wan_dit.attention`` replacement: ``[B, S, H*D]`` in and out; the kernel reads that layout directly."""
    q, k, v = _check(q), _check(k), _check(v)
    B, Sq, HD = q.shape
    D = HD // num_heads
    out = ops.flash_attn(q.unflatten(2, (num_heads, D)), k.unflatten(2, (num_heads, D)),
                         v.unflatten(2, (num_heads, D)))
    return out.flatten(2)


def set_attn_implementation(attn_implementation: str, flux_dit_module=None, wan_dit_module=None):
    """Mirror of ``FluxDiT.set_attn_implementation`` (flux_dit.py:480-504) with the extra name "b200":
    rebinds ``flux_dit._attn_func`` and/or ``wan_dit.attention`` in the given reference modules."""
    if attn_implementation not in SUPPORTED:
        raise ValueError(f"attn_implementation must be one of {SUPPORTED}, but got '{attn_implementation}'")
    if flux_dit_module is not None:
        flux_dit_module._attn_func = (b200_attn if attn_implementation == "b200"
                                      else torch.nn.functional.scaled_dot_product_attention)
    if wan_dit_module is not None:
        if attn_implementation == "b200":
            if not hasattr(wan_dit_module, "_sdpa_attention"):
                wan_dit_module._sdpa_attention = wan_dit_module.attention
            wan_dit_module.attention = b200_wan_attention
        elif hasattr(wan_dit_module, "_sdpa_attention"):
            wan_dit_module.attention = wan_dit_module._sdpa_attention
