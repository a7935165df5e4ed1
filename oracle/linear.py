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

    def __init__(self, mode="fp32", shuffle_k=None):
        """``shuffle_k`` (a seed): evaluate every product with the K axis of both operands permuted.  The result is
        mathematically the same and differs only in fp32 summation order (about 1e-7 relative) - the disagreement of
        two such evaluations after a few low-precision roundings is the floor below which no two implementations of
        this arithmetic can be expected to agree."""
        assert mode in MODES
        self.mode = mode
        self.shuffle_k = shuffle_k
        self._cache = {}
        self._perms = {}

    def _perm(self, K):
        if K not in self._perms:
            self._perms[K] = torch.randperm(K, generator=torch.Generator().manual_seed(self.shuffle_k + K))
        return self._perms[K]

    def _mm(self, a, b_t):
        """a [M,K] @ b_t[N,K]^T in fp32, optionally with the K axis shuffled."""
        if self.shuffle_k is not None:
            p = self._perm(a.shape[1])
            a, b_t = a[:, p], b_t[:, p]
        return a @ b_t.t()

    def _wq(self, W):
        key = id(W)
        if key not in self._cache:
            self._cache[key] = O.quant_weight(W, self.mode)
        return self._cache[key]

    @property
    def unit_scale_acts(self):
        """FP8 weights: the post-GELU hidden and (single blocks) the attention output reach their Linear as e4m3 with
        unit scale - the reference's own activation rule (utils/fp8_linear.py:35) - because the producing kernels
        emit e4m3 directly; a per-row scale would need the finished row."""
        return self.mode in ("fp8_tensor", "fp8_channel")

    def __call__(self, x, W, b=None, act_quant=True, from_fp32=False):
        """``act_quant``: True = per-row dynamic scale, False = fp32 activations, "unit" = e4m3 cast with scale 1.
        ``from_fp32``: the activation is quantised straight from its fp32 values - the case of a Linear fed by a
        LayerNorm, whose kernel emits the 8-bit rows itself - instead of from a bf16 tensor (one rounding less)."""
        x = x.float()
        if self.mode == "fp32":
            y = self._mm(x, W.float())
        elif self.mode == "bf16":
            # the M = 1 Linears (modulation, embedders) run as GEMVs on fp32 activations
            y = self._mm(x if act_quant is False else x.bfloat16().float(), W.bfloat16().float())
        else:
            q, s = self._wq(W)
            sd = s if s.numel() == 1 else s[:, None]
            ws = s.reshape(1) if s.numel() == 1 else s
            if act_quant == "unit" and self.unit_scale_acts:
                xq = x.clamp(-448, 448).to(torch.float8_e4m3fn)
                y = self._mm(xq.float(), q.float()) * ws[None, :]          # ops.linear_quant with unit row scales
            elif act_quant:
                xq, xs = (O.quant_rows_int8 if self.mode == "int8_channel" else O.quant_rows_e4m3)(
                    x if from_fp32 else x.bfloat16())
                y = self._mm(xq.float(), q.float()) * xs[:, None] * ws[None, :]   # ops.linear_quant
            else:
                y = self._mm(x, q.float() * sd)
        return y if b is None else y + b.float()


# ------------------------------------------------------------------ LoRA side matrices
def lora_reference(x, W, b, loras):
    """``LoRALinear.forward`` (models/basic/lora.py:137-141 with ``LoRA.forward`` :29-32) in exact fp32:
    ``x W^T + b + sum_i scale_i * alpha_i / rank_i * (x down_i^T) up_i^T``.  ``loras``: (coef, up [N,r], down [r,K])
    with coef = scale * alpha / rank."""
    y = x.float() @ W.float().t()
    if b is not None:
        y = y + b.float()
    for coef, up, down in loras:
        y = y + coef * ((x.float() @ down.float().t()) @ up.float().t())
    return y


def _e4m3(t):
    return torch.clamp(t, -448, 448).to(torch.float8_e4m3fn).float()


def lora_extension(W_q, W_s, mode, loras, pad=64):
    """The library's K-extension of a quantised weight by unfused LoRAs (no reference counterpart: the reference
    runs the side matrices as two more bf16 Linears).  Stacks ``D = cat(down_i)`` [R, K] and
    ``U = cat(coef_i * up_i)`` [N, R] (R padded with zeros to a multiple of ``pad``), quantises D per row, and
    returns (W_ext_q [N, K+E], D_q, D_colscale [R]) such that
    ``(x_q W_q^T + t_ext U_ext^T) * s_m * s_n`` with ``t = bf16(x_q D_q^T * D_colscale)`` reproduces the LoRA sum;
    tau splits the 8-bit range between the two factors per rank column (headroom goes to t, whose bound is statistical).  FP8: both factors are split into an e4m3
    head and an e4m3 remainder, t_ext = [t_hi | t_lo | t_hi] against U_ext = [U_hi | U_hi | U_lo] (E = 3R), which
    leaves only the remainder-times-remainder term out.  INT8: single columns (E = R)."""
    qmax = 127.0 if mode == "int8_channel" else 448.0
    N, K = W_q.shape
    D = torch.cat([d.float() for _, _, d in loras], dim=0)
    U = torch.cat([c * u.float() for c, u, _ in loras], dim=1)
    R = D.shape[0]
    Rp = (R + pad - 1) // pad * pad
    D = torch.cat([D, torch.zeros(Rp - R, K)], dim=0)
    U = torch.cat([U, torch.zeros(N, Rp - R)], dim=1)
    D_q, D_s = O.quant_weight(D, "int8_channel" if mode == "int8_channel" else "fp8_channel")
    s_n = W_s.float().reshape(-1, 1) if W_s.numel() > 1 else W_s.float().reshape(1, 1)
    a = qmax * D.norm(dim=1)                                  # 4-sigma estimate of |x_q . D_j| for rows with amax qmax
    bmax = (U / s_n).abs().amax(dim=0)
    # expected t aimed at min(balanced point, qmax/8), but not below the point where the weight-side factor reaches qmax
    prod = a * bmax
    target = torch.maximum(prod / qmax, torch.minimum(torch.sqrt(prod), torch.full_like(prod, qmax / 8.0)))
    tau = a / target.clamp_min(1e-30)
    tau = torch.where((a > 0) & (bmax > 0), tau, torch.ones_like(tau))
    Up = U * tau[None, :] / s_n
    assert float(Up.abs().amax()) <= qmax * (1.0 + 1e-4), "LoRA column beyond the quantised weight's range: the library keeps it unfused"
    Up = Up.clamp(-qmax, qmax)
    if mode == "int8_channel":
        U_ext = torch.clamp(torch.round(Up), -127, 127).to(torch.int8)
    else:
        U_hi = _e4m3(Up)
        U_lo = _e4m3(Up - U_hi)
        U_ext = torch.cat([U_hi, U_hi, U_lo], dim=1).to(torch.float8_e4m3fn)
    return torch.cat([W_q, U_ext], dim=1), D_q, (D_s.float() / tau).contiguous()


def lora_linear_quant(x, W, b, loras, mode):
    """Same-quantisation restatement of the library's fused LoRA Linear for ``mode`` in fp8_tensor / fp8_channel /
    int8_channel (bf16 activations in, fp32 out before the final bf16 rounding)."""
    W_q, W_s = O.quant_weight(W, mode)
    W_ext, D_q, D_cs = lora_extension(W_q, W_s, mode, loras)
    int8 = mode == "int8_channel"
    x_q, x_s = (O.quant_rows_int8 if int8 else O.quant_rows_e4m3)(x.bfloat16())
    t = (x_q.float() @ D_q.float().t()) * D_cs[None, :]
    t = t.bfloat16().float()
    if int8:
        t_ext = torch.clamp(torch.round(t), -127, 127)
    else:
        t_hi = _e4m3(t)
        t_ext = torch.cat([t_hi, _e4m3(t - t_hi), t_hi], dim=1)
    acc = torch.cat([x_q.float(), t_ext], dim=1) @ W_ext.float().t()
    s_n = W_s.float().reshape(1, -1) if W_s.numel() > 1 else W_s.float().reshape(1, 1)
    y = acc * x_s.float().reshape(-1, 1) * s_n
    return y if b is None else y + b.float()
