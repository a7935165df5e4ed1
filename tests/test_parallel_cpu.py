"""The multi-GPU wrapper on CPU ranks (gloo, world size 2 and 4): the head exchange reproduces full attention,
the control plane (pipe, per-step broadcast, batch split + ordered gather, terminate) works, and failures made
on the host (an exception in one worker, a worker that exits) surface as errors within the deadline instead of
blocking the parent the way the reference's ``conn.recv()`` does (utils/parallel.py:181)."""
import time

import pytest
import torch

from tests.parallel_helpers import oracle_wan_attention, slice_attention_factory

import diffsynth_engine_b200  # noqa: F401  (registers the package alias used by the worker processes)
from diffsynth_engine_b200.parallel import ParallelWorkerError, UlyssesParallelModel, batch_slice, map_tensors

_PORT = [29720]


def _port():
    _PORT[0] += 1
    return _PORT[0]


def _qkv(B, S, H, seed):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(B, S, H * 16, generator=g) for _ in range(3))


@pytest.mark.parametrize("sp", [2, 4])
def test_head_exchange_matches_full_attention(sp):
    H, S = 4, 24
    q, k, v = _qkv(1, S, H, 1)
    model = UlyssesParallelModel({"num_heads": H}, sp_degree=sp, batch_parallelism=1, master_port=_port(),
                                 device="cpu", timeout_s=60, factory=slice_attention_factory)
    try:
        out = model(q=q, k=k, v=v)
        ref = oracle_wan_attention(q, k, v, H)
        assert out.shape == ref.shape
        assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5)
        out2 = model(q=q * 2, k=k, v=v)          # a second step through the same workers
        assert torch.allclose(out2, oracle_wan_attention(q * 2, k, v, H), atol=1e-5, rtol=1e-5)
    finally:
        model.close()


def test_batch_parallel_split_and_ordered_gather():
    """batch_parallelism=2 x sp_degree=2: positive/negative halves of a batch-2 input go to the two groups and come
    back in order (the reference's CFG parallel, utils/parallel.py:123,127-132)."""
    H, S = 2, 16
    q, k, v = _qkv(2, S, H, 2)
    model = UlyssesParallelModel({"num_heads": H}, sp_degree=2, batch_parallelism=2, master_port=_port(),
                                 device="cpu", timeout_s=60, factory=slice_attention_factory)
    try:
        out = model(q=q, k=k, v=v)
        ref = torch.cat([oracle_wan_attention(q[i:i + 1], k[i:i + 1], v[i:i + 1], H) for i in range(2)])
        assert torch.allclose(out, ref, atol=1e-5, rtol=1e-5)
    finally:
        model.close()


def test_step_inputs_reach_every_rank_with_structure_and_dtypes():
    """Per step only the structure of the keyword arguments is pickled; every tensor leaf is broadcast as a tensor.
    Nested containers, integer tensors and non-tensor values must arrive unchanged on all ranks."""
    from tests.parallel_helpers import echo_factory
    model = UlyssesParallelModel({}, sp_degree=3, batch_parallelism=1, master_port=_port(), device="cpu", timeout_s=60,
                                 factory=echo_factory)
    try:
        x = torch.arange(12, dtype=torch.float32).reshape(1, 3, 4)
        extras = {"list": [torch.ones(2, 2, dtype=torch.bfloat16), torch.tensor([[5, 6]], dtype=torch.int64)], "k": 7}
        out = model(x=x, extras=extras, flag="on", scale=2.0)
        assert float(out) == 66.0 * 2 + 4 + 11 + 7 + 1000 + 1
    finally:
        model.close()


def test_worker_exception_reaches_the_parent():
    q, k, v = _qkv(1, 8, 2, 3)
    model = UlyssesParallelModel({"num_heads": 2, "fail_rank": 1}, sp_degree=2, master_port=_port(), device="cpu",
                                 timeout_s=30, factory=slice_attention_factory)
    t0 = time.time()
    try:
        with pytest.raises(ParallelWorkerError, match="injected failure"):
            model(q=q, k=k, v=v)
        assert time.time() - t0 < 25
        with pytest.raises(ParallelWorkerError):   # the group is marked dead, no second hang
            model(q=q, k=k, v=v)
    finally:
        model.close(grace_s=1.0)


def test_worker_exit_is_detected():
    q, k, v = _qkv(1, 8, 2, 4)
    model = UlyssesParallelModel({"num_heads": 2, "die_rank": 1}, sp_degree=2, master_port=_port(), device="cpu",
                                 timeout_s=30, factory=slice_attention_factory)
    t0 = time.time()
    try:
        # either the parent sees the dead process first, or a surviving rank reports its broken collective
        with pytest.raises(ParallelWorkerError, match="exited|closed by peer|failed"):
            model(q=q, k=k, v=v)
        assert time.time() - t0 < 25
    finally:
        model.close(grace_s=1.0)


def test_batch_slice_matches_reference_contract():
    """The batch split of utils/parallel.py:50-59 of the reference: every tensor leaf, other leaves untouched, the
    same ValueError for a batch smaller than the number of parts."""
    d = {"a": torch.arange(8).reshape(4, 2), "b": [torch.zeros(2, 1), "keep"], "c": 3}
    s = batch_slice(d, 2, 1)
    assert s["a"].tolist() == [[4, 5], [6, 7]] and s["b"][0].shape == (1, 1) and s["b"][1] == "keep" and s["c"] == 3
    assert batch_slice(d, 1, 0) is d
    with pytest.raises(ValueError, match="batch split failed"):
        batch_slice(torch.zeros(1, 3), 2, 0)
    doubled = map_tensors(d, lambda t: t * 2)
    assert doubled["a"].tolist()[0] == [0, 2] and doubled["c"] == 3 and doubled["b"][1] == "keep"


def test_joint_sequence_slices_cover_every_token_once():
    """The text+image split of the sequence-parallel MMDiT step: for every group size the ranks' text and image rows
    tile the unpadded sequence exactly, padding only at the end of the last ranks."""
    flux = __import__("importlib").import_module("diffsynth_engine_b200.flux")
    for S_txt, S_img in ((256, 6889), (512, 4096), (41, 84), (72, 54), (8, 64), (1, 1), (5, 0)):
        for world in (1, 2, 3, 4, 8):
            text_rows, image_rows, pad = [], [], 0
            for rank in range(world):
                sl = flux.sequence_slice(S_txt, S_img, world, rank)
                assert sl["S_pad"] % world == 0 and 0 <= sl["S_pad"] - sl["S"] < world
                assert 0 <= sl["t_loc"] <= sl["n_loc"] <= sl["Sl"]
                g0 = sl["g0"]
                text_rows += list(range(g0, g0 + sl["t_loc"]))
                image_rows += list(range(g0 + sl["t_loc"], g0 + sl["n_loc"]))
                pad += sl["Sl"] - sl["n_loc"]
            assert text_rows == list(range(S_txt))
            assert image_rows == list(range(S_txt, S_txt + S_img))
            assert pad == sl["S_pad"] - sl["S"]


def test_peer_exchange_addressing_equals_full_attention():
    """The addressing of the sequence-parallel attention over mapped peer memory (``wan.py`` with
    ``exchange="peer"``), restated on the CPU for P = 4 emulated ranks: rank r keeps its normalised queries as
    ``qn_r [Sl, d]`` and owns a return buffer ``ao_back_r [P][Sl][C]``.  Rank g (head group g) reads query part p from
    ``qn_p`` at column offset g*C with strides (d, 128), attends over all real tokens, and writes output row s to
    chunk g of ``ao_back_{s // Sl}`` at row s % Sl with strides (C, 128).  Afterwards
    ``ao_back_r.permute(1, 0, 2).reshape(Sl, d)`` is rank r's slice of the full attention output; padded rows never act
    as keys."""
    from oracle import ops as O
    P, H, S = 4, 8, 437                       # S does not split evenly: slices are padded to a multiple of 128
    d, C, Hl = H * 128, H * 128 // P, H // P
    Sl = ((S + P - 1) // P + 127) // 128 * 128
    S_pad = Sl * P
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(S_pad, d, generator=g) for _ in range(3))
    q[S:], k[S:], v[S:] = 7.0, 9.0, -3.0      # padded rows hold junk that must not leak into real rows
    full = O.attention(*(t[:S].reshape(1, S, H, 128).transpose(1, 2) for t in (q, k, v)))[0].transpose(0, 1).reshape(S, d)
    qn = [q[r * Sl:(r + 1) * Sl].clone() for r in range(P)]
    ao_back = [torch.zeros(P, Sl, C) for _ in range(P)]
    for grp in range(P):                      # what rank grp's attention kernel does
        cols = slice(grp * C, (grp + 1) * C)
        q_all = torch.cat([qn[p][:, cols] for p in range(P)])                    # query part p comes from rank p
        k_g, v_g = k[:S, cols], v[:S, cols]                                      # arrived by all-to-all; real tokens only
        o = O.attention(*(t.reshape(1, -1, Hl, 128).transpose(1, 2) for t in (q_all, k_g, v_g)))[0]
        o = o.transpose(0, 1).reshape(S_pad, C)
        for s in range(S_pad):
            ao_back[s // Sl][grp, s % Sl] = o[s]
    got = torch.cat([ao_back[r].permute(1, 0, 2).reshape(Sl, d) for r in range(P)])
    assert O.rel_l2(got[:S], full) < 1e-6
