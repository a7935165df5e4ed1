"""How the oracle evaluates a Linear: exact fp32, or with the library's quantisation rules applied
(weights prepacked per tensor / per channel, activations quantised per row), always accumulating in fp32."""
import torch

from . import ops as O

MODES = ("fp32", "bf16", "fp8_tensor", "fp8_channel", "int8_channel")


class LinearEval:
    """``lin(x, W, b)`` for 2-D ``x``.  ``mode``:
      fp32          exact
      bf16          operands rounded to bf16 (what a bf16 tensor-core GEMM sees), fp32 accumulate
      fp8_* / int8  W quantised by ``ops.quant_weight``; activations quantised per row by
                    ``ops.quant_rows_*`` when ``act_quant`` (the M=S GEMMs) and left in fp32 otherwise
                    (the M=1 modulation / embedding GEMVs).
    Quantised weights are cached by tensor identity."""

    def __init__(self, mode="fp32"):
        assert mode in MODES
        self.mode = mode
        self._cache = {}

    def _wq(self, W):
        key = id(W)
        if key not in self._cache:
            self._cache[key] = O.quant_weight(W, self.mode)
        return self._cache[key]

    def __call__(self, x, W, b=None, act_quant=True):
        x = x.float()
        if self.mode == "fp32":
            y = x @ W.float().t()
        elif self.mode == "bf16":
            y = x.bfloat16().float() @ W.bfloat16().float().t()
        else:
            q, s = self._wq(W)
            sd = s if s.numel() == 1 else s[:, None]
            if act_quant:
                xq, xs = (O.quant_rows_int8 if self.mode == "int8_channel" else O.quant_rows_e4m3)(x.bfloat16())
                y = O.linear_quant(xq, xs, q, s)
            else:
                y = x @ (q.float() * sd).t()
        return y if b is None else y + b.float()
