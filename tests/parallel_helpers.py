"""Picklable worker models for the CPU (gloo) tests of the multi-GPU wrapper."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def oracle_wan_attention(q, k, v, num_heads):
    """``wan_dit.attention`` semantics ([B, S, H*D] in and out) on the CPU oracle."""
    from oracle import ops as O
    mh = lambda t: t.unflatten(2, (num_heads, t.shape[2] // num_heads)).transpose(1, 2)
    return O.attention(mh(q), mh(k), mh(v)).transpose(1, 2).flatten(2)


class SliceAttentionModel:
    """Each rank attends with its slice of the tokens through the head exchange, then the slices are gathered."""

    def __init__(self, payload, rank, group, device):
        import torch.distributed as dist
        from diffsynth_engine_b200.parallel import HeadExchangeAttention
        self.dist, self.group = dist, group
        self.P, self.r = dist.get_world_size(group), dist.get_rank(group)
        self.num_heads = payload["num_heads"]
        self.fail_rank = payload.get("fail_rank")
        self.die_rank = payload.get("die_rank")
        self.rank = rank
        self.attn = HeadExchangeAttention(group, inner=oracle_wan_attention)

    def __call__(self, q, k, v):
        if self.fail_rank == self.rank:
            raise RuntimeError("injected failure")
        if self.die_rank == self.rank:
            os._exit(17)
        S = q.shape[1]
        Sl = S // self.P
        sl = slice(self.r * Sl, (self.r + 1) * Sl)
        o = self.attn(q[:, sl].contiguous(), k[:, sl].contiguous(), v[:, sl].contiguous(), self.num_heads)
        out = [torch.empty_like(o) for _ in range(self.P)]
        self.dist.all_gather(out, o.contiguous(), group=self.group)
        return torch.cat(out, dim=1)


def slice_attention_factory(payload, rank, group, device):
    return SliceAttentionModel(payload, rank, group, device)


class EchoModel:
    """Returns a checksum of everything it was given: checks that nested keyword arguments (lists of tensors,
    dtypes, plain Python values) reach every rank intact."""

    def __init__(self, payload, rank, group, device):
        import torch.distributed as dist
        self.dist, self.group = dist, group

    def __call__(self, x, extras, flag=None, scale=1.0):
        acc = x.double().sum() * scale + sum(t.double().sum() for t in extras["list"]) + extras["k"]
        acc = acc + (1000.0 if flag == "on" else 0.0) + (1.0 if extras["list"][1].dtype == torch.int64 else 0.0)
        t = torch.tensor([[float(acc)]], dtype=torch.float64)
        self.dist.all_reduce(t, group=self.group)      # every rank must have computed the same number
        return t / self.dist.get_world_size(self.group)


def echo_factory(payload, rank, group, device):
    return EchoModel(payload, rank, group, device)


def wan_engine_factory_without_peer_memory(state_dict, rank, sp_group, device, **engine_kwargs):
    """The Wan engine on a system where the ranks cannot map each other's memory: the mapping raises on every rank,
    and an engine created with ``exchange="auto"`` has to fall back to the all-to-all for every tensor."""
    from diffsynth_engine_b200 import wan

    def unavailable(*a, **k):
        raise RuntimeError("peer memory is switched off in this test")

    wan.PeerMemory = unavailable
    eng = wan.WanDiTEngine(state_dict, device=device, group=sp_group, **engine_kwargs)
    return _ExchangeReporting(eng)


class _ExchangeReporting:
    """Forwards the call and appends nothing; after the first call the engine must have settled on the all-to-all."""

    def __init__(self, eng):
        self.eng = eng

    def __call__(self, **kw):
        out = self.eng(**kw)
        if self.eng.exchange != "nccl":
            raise RuntimeError(f"expected the all-to-all fallback, engine uses {self.eng.exchange}")
        return out
