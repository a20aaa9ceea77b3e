"""The multi-GPU partition on CPU ranks (gloo, world size 2): plans are disjoint and complete, a
rank's head shard computed alone equals the same heads of the whole call, and the optional
all-gather rebuilds the whole output.  The arithmetic on each rank is the CPU oracle here - what is
under test is the partition and the collective, which never touch a kernel."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dashmag_b200 import sharding
from oracle import attention_oracle as oracle


def test_head_shards_cover_every_head_once():
    for hkv, group, world in [(8, 4, 1), (8, 4, 2), (8, 4, 8), (3, 2, 2), (2, 4, 4), (1, 8, 2)]:
        shards = sharding.head_shards(hkv, group, world)
        kv = [h for s, _ in shards for h in range(s.start, s.stop)]
        qh = [h for _, s in shards for h in range(s.start, s.stop)]
        assert kv == list(range(hkv)) and qh == list(range(hkv * group))
        for s_kv, s_q in shards:
            assert (s_q.start, s_q.stop) == (s_kv.start * group, s_kv.stop * group)


def test_training_plan_splits_sequences_when_heads_run_out():
    lengths = [8192, 1024, 4000, 3000, 6000, 2500, 7000, 1200, 5000, 900, 4400, 3100, 2000, 8000, 1500, 6800]
    plan = sharding.training_plan(lengths, hkv=4, group=4, world=8, window_left=4096)
    seen = {}
    for seqs, kv, qh in plan:
        assert kv.stop - kv.start == 1 and qh.stop - qh.start == 4
        for s in seqs:
            seen.setdefault(kv.start, []).append(s)
    for head in range(4):
        assert sorted(seen[head]) == list(range(len(lengths)))  # every sequence once per head
    loads = {}
    for seqs, kv, _ in plan:
        loads.setdefault(kv.start, []).append(sum(sharding.causal_pairs(lengths[s], 4096) for s in seqs))
    for pair in loads.values():
        assert max(pair) / min(pair) < 1.1  # the two ranks of a head carry nearly the same work
    # with enough heads nobody splits sequences
    plan = sharding.training_plan(lengths, hkv=8, group=4, world=8)
    assert all(seqs == list(range(len(lengths))) for seqs, _, _ in plan)


def test_training_share_cuts_heads_in_place_and_gathers_sequence_bins():
    lengths = [5, 3, 7, 2]
    q = torch.arange(17 * 8 * 2, dtype=torch.float32).reshape(1, 17, 8, 2)
    k = torch.arange(17 * 2 * 2, dtype=torch.float32).reshape(1, 17, 2, 2)
    whole = sharding.training_plan(lengths, hkv=2, group=4, world=2)
    for r, entry in enumerate(whole):
        ls, qs, ks, vs, gs = sharding.training_share(entry, lengths, q, k, k, q)
        assert ls == lengths and qs.data_ptr() == q[:, :, 4 * r:].data_ptr() and qs.stride() == q.stride()  # a view
        assert torch.equal(qs, q[:, :, 4 * r:4 * r + 4]) and torch.equal(ks, k[:, :, r:r + 1]) and torch.equal(gs, qs)
    bins = sharding.training_plan(lengths, hkv=2, group=4, world=4)   # two ranks per head split the sequences
    covered = {0: [], 1: []}
    for entry in bins:
        seqs, kv, qh = entry
        ls, qs, ks, vs, gs = sharding.training_share(entry, lengths, q, k, k, q)
        assert ls == [lengths[i] for i in seqs] and qs.shape == (1, sum(ls), 4, 2) and ks.shape == (1, sum(ls), 1, 2)
        starts = np.concatenate([[0], np.cumsum(lengths)])
        want = torch.cat([q[:, starts[i]:starts[i + 1], qh] for i in seqs], dim=1)
        assert torch.equal(qs, want)
        covered[kv.start] += list(seqs)
    assert sorted(covered[0]) == sorted(covered[1]) == [0, 1, 2, 3]


def test_decode_plan_balances_cache_lengths():
    rng = np.random.default_rng(3)
    lengths = rng.integers(1024, 32769, size=64)
    plan = sharding.decode_plan(lengths, 8)
    assert sorted(i for part in plan for i in part) == list(range(64))
    loads = [int(lengths[part].sum()) for part in plan]
    assert max(loads) / min(loads) < 1.05


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, result):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, t, hq, hkv, d = 1, 96, 6, 3, 32
        q, k, v = (oracle.seeded(s, seed) for s, seed in (((b, t, hq, d), 11), ((b, t, hkv, d), 12), ((b, t, hkv, d), 13)))
        cu = np.array([0, 40, 41, 96], np.int64)
        kw = dict(cu_q=cu, cu_k=cu, causal=True)
        whole, whole_lse = oracle.forward(q, k, v, **kw)
        tq, tk, tv = (torch.from_numpy(x) for x in (q, k, v))
        lq, lk, lv = sharding.shard_heads(tq, tk, tv, rank, world)
        assert not lq.is_contiguous() or lq.shape[2] == hq  # a view of the caller's tensor
        local, local_lse = oracle.forward(lq.numpy(), lk.numpy(), lv.numpy(), **kw)
        # a shard computed alone is the same heads of the whole call, to the bit
        _, qh = sharding.head_shards(hkv, hq // hkv, world)[rank]
        assert np.array_equal(local, whole[:, :, qh]) and np.array_equal(local_lse, whole_lse[:, :, qh])
        full = sharding.all_gather_heads(torch.from_numpy(local), hq, group=hq // hkv)
        assert np.array_equal(full.numpy(), whole)
        # max over ranks of a per-rank time, as the benchmark takes it
        tmax = torch.tensor([float(rank + 1)], dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        assert tmax.item() == float(world)
        result[rank] = "ok"
    except Exception as e:  # surfaced by the parent
        result[rank] = f"{type(e).__name__}: {e}"
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_heads_and_gather_the_output():
    world = 2
    with mp.Manager() as manager:
        result = manager.dict()
        mp.spawn(_rank_main, args=(world, _free_port(), result), nprocs=world, join=True)
        assert dict(result) == {0: "ok", 1: "ok"}
