"""Prepacked Linear weights: the quantised payload ``[N, K]`` (K contiguous, exactly what the GEMM's TMA
reads), its dequantisation scale(s) and an fp32 bias."""
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from . import ops

FORMATS = ("bf16", "fp8_tensor", "fp8_channel", "int8_channel")
_ACT_FMT = {"bf16": ops.FMT_BF16, "fp8_tensor": ops.FMT_E4M3, "fp8_channel": ops.FMT_E4M3,
            "int8_channel": ops.FMT_INT8}


def act_format(fmt: str) -> int:
    """Element format the GEMM's activation operand must have for weights packed as ``fmt``."""
    return _ACT_FMT[fmt]


@dataclass
class PackedLinear:
    w: torch.Tensor                 # [N, K] bf16 / float8_e4m3fn / int8
    scale: Optional[torch.Tensor]   # fp32 [1] (per tensor), [N] (per channel) or None (bf16)
    bias: Optional[torch.Tensor]    # fp32 [N]
    fmt: str

    @property
    def out_features(self):
        return self.w.shape[0]

    @property
    def in_features(self):
        return self.w.shape[1]


def pack_linear(weight: torch.Tensor, bias: Optional[torch.Tensor], fmt: str, device) -> PackedLinear:
    """Quantise one ``[N, K]`` weight on the device with the library's prepack kernel."""
    if fmt not in FORMATS:
        raise ValueError(f"fmt must be one of {FORMATS}, but got '{fmt}'")
    w = weight.reshape(weight.shape[0], -1)
    w = w.to(device=device)
    if w.dtype not in (torch.float32, torch.bfloat16):
        w = w.float()
    w = w.contiguous()
    b = None if bias is None else bias.to(device=device, dtype=torch.float32).contiguous()
    if fmt == "bf16":
        return PackedLinear(w.to(torch.bfloat16), None, b, fmt)
    code = ops.FMT_INT8 if fmt == "int8_channel" else ops.FMT_E4M3
    q, s = ops.pack_quant_weight(w, code, per_channel=(fmt != "fp8_tensor"))
    return PackedLinear(q, s, b, fmt)


def stack_for_gemv(parts: List[PackedLinear]) -> PackedLinear:
    """Concatenate Linears that share their input (the AdaLN modulation layers of every block all read
    SiLU(conditioning)) into one row-stacked matrix with a per-row scale, so one GEMV launch serves them all."""
    fmt = parts[0].fmt
    w = torch.cat([p.w for p in parts], dim=0)
    scale = None
    if fmt != "bf16":
        scale = torch.cat([p.scale if p.scale.numel() > 1 else p.scale.expand(p.w.shape[0]) for p in parts]).contiguous()
    bias = torch.cat([p.bias for p in parts]).contiguous()
    return PackedLinear(w, scale, bias, fmt)
