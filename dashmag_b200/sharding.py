"""How the attention path is cut across the GPUs of one box.

Every unit of the path is independent: a (batch element or packed sequence, key-value head) pair
in the training passes - the key and value gradients sum only over the query heads of their own
group and the queries of their own sequence - and a (batch element, key-value head) pair in the
decoding step.  So ranks take disjoint units, read their slices of the caller's tensors in place
through strides, and exchange nothing while computing.  The reference has no multi-GPU path at all
(``crates/dash-mag/src/lib.rs:1-3``: device pooling "planned and not started"); this module is the
partition the benchmark's configurations name, plus the one optional collective: an all-gather of
the output's head shards when a caller wants the whole output on every rank.

Nothing here touches a kernel; it is index arithmetic and one ``torch.distributed`` call, so it is
tested on CPU ranks (gloo).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def head_shards(hkv: int, group: int, world: int) -> List[Tuple[slice, slice]]:
    """Per rank, the slice of key-value heads and the slice of query heads it owns.

    Key-value heads are dealt out in contiguous runs as evenly as they go (ranks beyond ``hkv``
    get empty slices); a rank's query heads are the groups of its key-value heads, which are
    contiguous because query head ``h`` reads key-value head ``h // group``.
    """
    out = []
    base, extra = divmod(hkv, world)
    start = 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append((slice(start, start + n), slice(start * group, (start + n) * group)))
        start += n
    return out


def causal_pairs(length: int, window_left=None) -> int:
    """Visible (query, key) pairs of one causal self-attention sequence."""
    if window_left is None or length <= window_left + 1:
        return length * (length + 1) // 2
    w = window_left
    return (w + 1) * (w + 2) // 2 + (length - w - 1) * (w + 1)


def balanced_bins(work: Sequence[int], bins: int) -> List[List[int]]:
    """Indices of ``work`` dealt into ``bins`` by falling work, each to the lightest bin so far
    (longest-processing-time first); ties go to the lower bin, so the plan is deterministic."""
    order = sorted(range(len(work)), key=lambda i: (-work[i], i))
    loads = [0] * bins
    out: List[List[int]] = [[] for _ in range(bins)]
    for i in order:
        b = min(range(bins), key=lambda j: (loads[j], j))
        out[b].append(i)
        loads[b] += work[i]
    return [sorted(x) for x in out]


def training_plan(lengths: Sequence[int], hkv: int, group: int, world: int, window_left=None):
    """Which (sequences, key-value heads) each rank takes for packed causal training.

    Heads first: with ``hkv >= world`` every rank takes whole key-value heads of every sequence.
    With fewer key-value heads than ranks, ``world // hkv`` ranks share each head and split the
    sequences between them, balanced by visible pairs.  Returns, per rank,
    ``(sequence indices, kv-head slice, query-head slice)``.
    """
    if world <= hkv:
        everything = list(range(len(lengths)))
        return [(everything, kv, qh) for kv, qh in head_shards(hkv, group, world)]
    per_head = world // hkv
    bins = balanced_bins([causal_pairs(int(n), window_left) for n in lengths], per_head)
    plan = []
    for r in range(world):
        head, part = divmod(r, per_head)
        if head >= hkv:
            plan.append(([], slice(0, 0), slice(0, 0)))
        else:
            plan.append((bins[part], slice(head, head + 1), slice(head * group, (head + 1) * group)))
    return plan


def decode_plan(lengths: Sequence[int], world: int) -> List[List[int]]:
    """Batch elements per rank for the decoding step, balanced by cache length: the cache lives
    with its sequence, so the batch is what is cut."""
    return balanced_bins([int(n) for n in lengths], world)


def training_share(entry, lengths: Sequence[int], q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *more: torch.Tensor):
    """One rank's part of a packed batch ``[1, T, H, D]`` under a plan entry of :func:`training_plan`:
    ``(lengths of its sequences, q, k, v, *more)`` with ``more`` cut like ``q`` (the output's
    gradient, the output).  With every sequence on the rank the parts are head slices of the
    caller's tensors, read in place through their strides; with a bin of the sequences the bin's
    tokens are gathered into packed tensors of their own (a rank that owns some of the sequences
    holds those sequences, not the whole batch)."""
    seqs, kv, qh = entry
    lengths = [int(n) for n in lengths]
    cut_q = [t[:, :, qh] for t in (q,) + tuple(more)]
    cut_kv = [t[:, :, kv] for t in (k, v)]
    if list(seqs) != list(range(len(lengths))):
        starts = [0]
        for n in lengths:
            starts.append(starts[-1] + n)
        tokens = lambda t: (torch.cat([t[:, starts[i]:starts[i + 1]] for i in seqs], dim=1) if len(seqs)
                            else t[:, :0].contiguous())
        cut_q, cut_kv = [tokens(t) for t in cut_q], [tokens(t) for t in cut_kv]
    return ([lengths[i] for i in seqs], cut_q[0], cut_kv[0], cut_kv[1], *cut_q[1:])


def shard_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rank: int, world: int):
    """This rank's head slices of ``[B,T,H,D]`` tensors: views, read in place through strides."""
    hkv, group = k.shape[2], q.shape[2] // k.shape[2]
    kv, qh = head_shards(hkv, group, world)[rank]
    return q[:, :, qh], k[:, :, kv], v[:, :, kv]


def all_gather_heads(local: torch.Tensor, hq: int, group: int = None) -> torch.Tensor:
    """The whole ``[B,T,Hq,D]`` tensor on every rank from each rank's head shard.

    The one collective of the path, and only for callers that want the full output (or query
    gradient) everywhere.  Shards may differ in size, so each rank's is padded to the largest,
    gathered with one ``all_gather_into_tensor`` (NCCL over NVLink on GPUs, gloo on CPU ranks) and
    cut back.  ``group`` is the query heads per key-value head, needed when ``local`` holds query
    heads and the shards follow the key-value heads.
    """
    world, rank = dist.get_world_size(), dist.get_rank()
    group = group or 1
    sizes = [s.stop - s.start for _, s in head_shards(hq // group, group, world)]
    assert local.shape[2] == sizes[rank], f"rank {rank} holds {local.shape[2]} heads, its shard has {sizes[rank]}"
    b, t, _, d = local.shape
    widest = max(sizes)
    padded = local.new_zeros((b, t, widest, d))
    padded[:, :, : sizes[rank]] = local
    flat = local.new_empty((world * b, t, widest, d))
    dist.all_gather_into_tensor(flat, padded.contiguous())
    gathered = flat.view(world, b, t, widest, d)
    return torch.cat([gathered[r, :, :, : sizes[r]] for r in range(world)], dim=2)
