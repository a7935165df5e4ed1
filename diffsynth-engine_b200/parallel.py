"""Multi-GPU wrapper with the contract of the reference's ``ParallelModel`` (utils/parallel.py:149-188 of
DiffSynth-Engine): the constructor spawns one worker process per GPU, ``forward(**kwargs)`` ships the step's
inputs to the workers and returns one tensor, ``__del__`` sends the terminate message.  Where the reference
shards the model with a DTensor tensor-parallel plan, this wrapper shards the *sequence* (Ulysses): every worker
holds the whole (FP8) model and ``S / sp_degree`` tokens, and self-attention exchanges heads for tokens.

Differences that a caller can observe:
  * ``sp_degree`` replaces ``tensor_parallelism``/``tp_plan`` (there is no plan to pass);
  * every wait has a deadline: ``forward`` raises ``ParallelWorkerError`` if a worker dies, reports an exception,
    or does not answer within ``timeout_s`` (the reference blocks forever in ``conn.recv()``, parallel.py:181);
  * a worker that fails sends its traceback to the parent before leaving.
The optional 2-way "CFG/batch parallel" of the reference (parallel.py:105-109,123,127-132) is kept: with
``batch_parallelism = 2`` the batch dimension of every tensor input is split over two groups of ``sp_degree`` ranks
and the two results are gathered in order.
"""
import datetime
import os
import time
import traceback
from typing import Callable, Optional

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

TERMINATE = "TERMINATE"


class ParallelWorkerError(RuntimeError):
    pass


def map_tensors(tree, fn):
    """A copy of a nest of dicts / lists / tuples with ``fn`` applied to every tensor leaf (sequences come back as
    lists, other leaves unchanged)."""
    if torch.is_tensor(tree):
        return fn(tree)
    if isinstance(tree, dict):
        return {key: map_tensors(value, fn) for key, value in tree.items()}
    if isinstance(tree, (list, tuple)):
        return [map_tensors(value, fn) for value in tree]
    return tree


def batch_slice(tree, parts: int, index: int):
    """Part ``index`` of ``parts`` equal slices along dimension 0 of every tensor leaf: the batch split of the
    reference's CFG / batch parallelism (utils/parallel.py:50-59 raises the same ValueError for a batch that is too
    small)."""
    def take(t):
        if t.shape[0] < parts:
            raise ValueError("data.shape[0] < num, batch split failed")
        step = t.shape[0] // parts
        return t.narrow(0, index * step, step)
    return map_tensors(tree, take) if parts > 1 else tree


def wan_engine_factory(state_dict, rank, sp_group, device, **engine_kwargs):
    """Default worker model: a sequence-parallel ``WanDiTEngine`` over ``sp_group``."""
    from .wan import WanDiTEngine
    return WanDiTEngine(state_dict, device=device, group=sp_group, **engine_kwargs)


def flux_engine_factory(state_dict, rank, sp_group, device, **engine_kwargs):
    """Worker model for the Flux / MMDiT step: a sequence-parallel ``FluxDiTEngine`` over ``sp_group``; called with
    the keyword arguments of ``FluxDiT.forward``."""
    from .flux import FluxDiTEngine
    return FluxDiTEngine(state_dict, device=device, group=sp_group, **engine_kwargs)


def _share_step_inputs(kwargs, rank: int, dev):
    """Rank 0 hands one step's keyword arguments to every rank.  The reference pickles the whole dict, tensors
    included, through ``broadcast_object_list`` every step (utils/parallel.py:112-116); here only the structure is
    pickled (names, shapes, dtypes, non-tensor values) and each tensor leaf travels as one collective broadcast on the
    workers' device (NCCL on GPUs, gloo on CPU ranks).  Returns the dict with tensors on ``dev`` (or TERMINATE)."""
    leaves = []

    def strip(v):
        if isinstance(v, dict):
            return {k: strip(x) for k, x in v.items()}
        if isinstance(v, (tuple, list)):
            return [strip(x) for x in v]
        if isinstance(v, torch.Tensor):
            leaves.append(v)
            return ("__tensor__", len(leaves) - 1, tuple(v.shape), v.dtype)
        return v

    def fill(v):
        if isinstance(v, dict):
            return {k: fill(x) for k, x in v.items()}
        if isinstance(v, tuple) and len(v) == 4 and v[0] == "__tensor__":
            return leaves[v[1]]
        if isinstance(v, list):
            return [fill(x) for x in v]
        return v

    meta = [strip(kwargs) if rank == 0 else None, None]
    if rank == 0:
        meta[1] = [(tuple(t.shape), t.dtype) for t in leaves]
    dist.broadcast_object_list(meta, src=0)
    skeleton, specs = meta
    if isinstance(skeleton, str) and skeleton == TERMINATE:
        return TERMINATE
    if rank == 0:
        leaves = [t.to(dev).contiguous() for t in leaves]
    else:
        leaves = [torch.empty(shape, dtype=dtype, device=dev) for shape, dtype in specs]
    for t in leaves:
        dist.broadcast(t, src=0)
    return fill(skeleton)


def _worker_loop(rank: int, world_size: int, conn, payload, factory: Callable, sp_degree: int, batch_parallelism: int,
                 master_port: int, device: str, backend: str, timeout_s: float, engine_kwargs: dict):
    model = None
    try:
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(world_size)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(master_port)
        if device.startswith("cuda"):
            # A worker that fails leaves between steps, but the parent may also end survivors (close()).  A rank that
            # dies while its buffers are bound to an NVLink multicast object can fault the GPUs of the other ranks, so
            # this wrapper's NCCL never uses NVLS; the head exchange is an all-to-all, which NVLS does not serve anyway.
            os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            torch.cuda.set_device(rank)
            dev = f"cuda:{rank}"
        else:
            dev = device
        dist.init_process_group(backend=backend, init_method="env://", world_size=world_size, rank=rank,
                                timeout=datetime.timedelta(seconds=timeout_s))
        # rank = bp_row * sp_degree + sp_rank
        sp_groups = [dist.new_group([r * sp_degree + i for i in range(sp_degree)]) for r in range(batch_parallelism)]
        bp_group = dist.new_group([r * sp_degree for r in range(batch_parallelism)])
        bp_row, sp_rank = divmod(rank, sp_degree)
        model = factory(payload, rank, sp_groups[bp_row], dev, **engine_kwargs)
        if rank == 0:
            conn.send(("READY", None))
        while True:
            kwargs = _share_step_inputs(conn.recv() if rank == 0 else None, rank, dev)
            if isinstance(kwargs, str) and kwargs == TERMINATE:
                break
            kwargs = batch_slice(kwargs, batch_parallelism, bp_row)
            with torch.no_grad():
                result = model(**kwargs)
            if sp_rank == 0 and batch_parallelism > 1:
                gathered = torch.zeros((batch_parallelism, *result.shape[1:]), dtype=result.dtype, device=result.device)
                dist.all_gather_into_tensor(gathered, result.contiguous(), group=bp_group)
                result = gathered
            if rank == 0:
                conn.send(("OK", result.detach().to("cpu")))
            dist.barrier()
    except Exception as e:  # report, then leave: the parent must not wait for a worker that is gone
        tb = traceback.format_exc()
        try:
            conn.send(("ERROR", f"rank {rank}: {e}\n{tb}"))
        except Exception:
            pass
    finally:
        del model
        try:
            conn.close()
        except Exception:
            pass
        if device.startswith("cuda") and torch.cuda.is_available():
            torch.cuda.synchronize()
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


class UlyssesParallelModel(nn.Module):
    """``ParallelModel`` with sequence parallelism.  ``model`` is the reference's ``WanDiT`` module (its
    ``state_dict()`` is shipped to the workers), a state dict, or any picklable payload for a custom ``factory``."""

    def __init__(self, model, sp_degree: int = 4, batch_parallelism: int = 1, master_port: int = 29500,
                 device: str = "cuda", backend: Optional[str] = None, timeout_s: float = 600.0,
                 factory: Callable = wan_engine_factory, **engine_kwargs):
        super().__init__()
        self.world_size = sp_degree * batch_parallelism
        self.device = device
        self.timeout_s = timeout_s
        backend = backend or ("nccl" if device.startswith("cuda") else "gloo")
        payload = model.state_dict() if isinstance(model, nn.Module) else model
        ctx = mp.get_context("spawn")
        self.conn_main, conn_worker = ctx.Pipe(duplex=True)
        # every worker gets the pipe end; only rank 0 answers on it, the others use it for error reports
        self._ctx = mp.spawn(
            _worker_loop,
            args=(self.world_size, conn_worker, payload, factory, sp_degree, batch_parallelism, master_port, device,
                  backend, timeout_s, engine_kwargs),
            nprocs=self.world_size, join=False)
        self._closed = False
        self._recv("READY")

    def _recv(self, expect):
        deadline = time.time() + self.timeout_s
        while True:
            if self.conn_main.poll(0.05):
                try:
                    tag, value = self.conn_main.recv()
                except (EOFError, OSError) as e:
                    raise ParallelWorkerError(f"worker pipe closed: {e}")
                if tag == "ERROR":
                    self._closed = True
                    raise ParallelWorkerError(f"a worker failed:\n{value}")
                if tag == expect or (expect == "READY" and tag == "OK"):
                    return value
                continue
            dead = [i for i, p in enumerate(self._ctx.processes) if not p.is_alive()]
            if dead:
                self._closed = True
                codes = [self._ctx.processes[i].exitcode for i in dead]
                raise ParallelWorkerError(f"worker(s) {dead} exited (exit codes {codes}) before answering")
            if time.time() > deadline:
                self._closed = True
                raise ParallelWorkerError(f"no answer from the workers within {self.timeout_s} s")

    def forward(self, **kwargs):
        if self._closed:
            raise ParallelWorkerError("the worker group is no longer running")
        self.conn_main.send(kwargs)
        result = self._recv("OK")
        return result.to(self.device) if isinstance(result, torch.Tensor) and self.device.startswith("cuda") else result

    def close(self, grace_s: float = 10.0):
        if hasattr(self, "conn_main") and not self._closed:
            self._closed = True
            try:
                self.conn_main.send(TERMINATE)
            except Exception:
                pass
        if hasattr(self, "_ctx"):
            end = time.time() + grace_s
            for p in self._ctx.processes:
                p.join(max(0.0, end - time.time()))
            for p in self._ctx.processes:
                if p.is_alive():
                    p.terminate()  # exact process objects this wrapper started
        if hasattr(self, "conn_main"):
            try:
                self.conn_main.close()
            except Exception:
                pass

    def __del__(self):
        try:
            self.close(grace_s=2.0)
        except Exception:
            pass


__all__ = ["UlyssesParallelModel", "ParallelWorkerError", "HeadExchangeAttention", "wan_engine_factory",
           "flux_engine_factory"]


class HeadExchangeAttention:
    """Sequence-parallel attention as a drop-in for ``wan_dit.attention(q, k, v, num_heads)``
    (models/wan/wan_dit.py:18-22) when q, k, v hold this rank's ``S/P`` tokens: heads are exchanged for tokens,
    ``inner(q, k, v, num_heads / P)`` runs on the full sequence, and the result is exchanged back.  ``inner``
    defaults to the library's flash attention; tests on CPU ranks pass the oracle's attention."""

    def __init__(self, group=None, inner: Optional[Callable] = None):
        from .wan import HeadExchange
        self.xchg = HeadExchange(group)
        self.inner = inner

    def __call__(self, q, k, v, num_heads: int):
        P = self.xchg.world
        inner = self.inner
        if inner is None:
            from .attention import b200_wan_attention as inner
        if P == 1:
            return inner(q, k, v, num_heads)
        B, Sl, HD = q.shape
        if B != 1 or num_heads % P:
            raise ValueError("head exchange needs batch 1 and a head count divisible by the group size")
        C = HD // P

        def fwd(t):  # [1, S/P, H*D] -> [1, S, H/P*D]
            send = t[0].reshape(t.shape[1], P, C).permute(1, 0, 2).contiguous()
            return self.xchg(send).reshape(1, P * t.shape[1], C)

        o = inner(fwd(q), fwd(k), fwd(v), num_heads // P)          # [1, S, C]
        back = self.xchg(o[0].reshape(P, Sl, C).contiguous())      # chunk p = head group p of the own tokens
        return back.permute(1, 0, 2).reshape(1, Sl, HD)
