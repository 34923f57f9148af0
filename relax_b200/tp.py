"""Tensor-parallel sharding of the quantised projections (column-/row-parallel matmul).

The reference has no sharding or collective; this follows the usual split of a decoder layer:

* column-parallel (shard the rows of W = the outputs, no exchange): q, k, v (by heads), gate, up;
* row-parallel (shard K = the inputs, ONE sum over ranks afterwards): o, down.

Shards are contiguous copies in the benchmark layout (uint32 [N, K/8], fp16 [N, K/32]), so every
rank calls the same kernels on smaller tensors.  K slices are multiples of 256 so that the
TMA-fed skinny kernel takes them; 11008 = 43 * 256 therefore splits unevenly (e.g. 6,6,6,5,5,5,5,5
blocks over 8 ranks), which is stated in the slice table instead of padding the weights.

Everything here is index arithmetic on array-likes (numpy arrays or torch tensors).
"""
from __future__ import annotations

K_BLOCK = 256   # granularity of a K slice (one 256-k chunk of the skinny kernel's tensor map)


def split_blocks(total: int, parts: int, block: int = K_BLOCK):
    """[(start, stop)] * parts: `total` (a multiple of `block`) cut into `parts` contiguous ranges
    of whole blocks, the first `nblocks % parts` ranges one block longer."""
    if total % block:
        raise ValueError(f"{total} is not a multiple of {block}")
    nb = total // block
    if nb < parts:
        raise ValueError(f"cannot cut {nb} blocks of {block} into {parts} non-empty parts")
    base, extra = divmod(nb, parts)
    out, start = [], 0
    for r in range(parts):
        n = (base + (1 if r < extra else 0)) * block
        out.append((start, start + n))
        start += n
    return out


def shard_rows(wq, scales, rows: slice):
    """Column-parallel: keep the output rows `rows`."""
    return wq[rows], scales[rows]


def shard_k(wq, scales, k0: int, k1: int):
    """Row-parallel: keep input columns [k0, k1) (multiples of 32)."""
    if k0 % 32 or k1 % 32:
        raise ValueError("K slices must be multiples of the group size 32")
    return wq[:, k0 // 8:k1 // 8], scales[:, k0 // 32:k1 // 32]


def _cat(parts):
    first = parts[0]
    if hasattr(first, "numpy") or type(first).__module__.startswith("torch"):
        import torch

        return torch.cat(list(parts), dim=0).contiguous()
    import numpy as np

    return np.ascontiguousarray(np.concatenate(list(parts), axis=0))


def _contig(a):
    if hasattr(a, "contiguous"):
        return a.contiguous()
    import numpy as np

    return np.ascontiguousarray(a)


def shard_layer(full: dict, rank: int, world: int, hidden: int, inter: int):
    """Shard of one decoder layer for `rank`.

    `full` holds (wq, scales) under 'qkv' ([3H, H] rows = q | k | v), 'o' ([H, H]), 'gu'
    ([2I, H] rows = gate | up), 'down' ([H, I]) and fp16 vectors 'norm1', 'norm2'.
    Returns the same keys with this rank's slices plus 'hidden_local' and 'inter_local'."""
    if hidden % (world * K_BLOCK) and world > 1:
        raise ValueError(f"hidden {hidden} does not split into {world} slices of whole {K_BLOCK}-blocks")
    hl = hidden // world
    h0, h1 = rank * hl, (rank + 1) * hl
    i0, i1 = split_blocks(inter, world)[rank]
    out = {"norm1": full["norm1"], "norm2": full["norm2"], "hidden_local": hl, "inter_local": i1 - i0}
    wq, s = full["qkv"]
    out["qkv"] = (_cat([wq[h0:h1], wq[hidden + h0:hidden + h1], wq[2 * hidden + h0:2 * hidden + h1]]),
                  _cat([s[h0:h1], s[hidden + h0:hidden + h1], s[2 * hidden + h0:2 * hidden + h1]]))
    wq, s = full["o"]
    a, b = shard_k(wq, s, h0, h1)
    out["o"] = (_contig(a), _contig(b))
    wq, s = full["gu"]
    out["gu"] = (_cat([wq[i0:i1], wq[inter + i0:inter + i1]]), _cat([s[i0:i1], s[inter + i0:inter + i1]]))
    wq, s = full["down"]
    a, b = shard_k(wq, s, i0, i1)
    out["down"] = (_contig(a), _contig(b))
    return out


# ---------------------------------------------------------------------------------- host-side checks
class ShardingMismatch(ValueError):
    """The ranks of a tensor-parallel group hold shards that do not fit together."""


class RankLeft(RuntimeError):
    """A rank of the tensor-parallel group announced that it is leaving (or stopped answering)."""


def shard_signature(shard: dict, hidden: int, inter_range=None):
    """What the other ranks need to know about one rank's layer shard: its sizes as integers."""
    def shape(a):
        return [int(d) for d in a.shape]

    sig = [int(shard["hidden_local"]), int(shard["inter_local"]), int(hidden)]
    for key in ("qkv", "o", "gu", "down"):
        sig += shape(shard[key][0]) + shape(shard[key][1])
    return sig


def verify_sharding(shards, rank: int, world: int, hidden: int, inter: int, group=None):
    """Checks on the host, before anything is launched, that every rank's layer shards fit together:
    equal head slices, local shapes consistent with hidden_local / inter_local, and K slices of the
    row-parallel matmuls that add up to `inter`.  Every rank gathers every rank's sizes
    (torch.distributed.all_gather_object on `group`, any backend) and raises ShardingMismatch on ALL
    ranks when something disagrees, so no rank goes on to a collective the others never join."""
    import torch.distributed as dist

    mine = [shard_signature(s, hidden) for s in shards]
    if world > 1:
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
    else:
        everyone = [mine]
    problems = []
    nl = len(mine)
    for r, sigs in enumerate(everyone):
        if len(sigs) != nl:
            problems.append(f"rank {r} holds {len(sigs)} layers, rank {rank} holds {nl}")
            continue
        for li, sig in enumerate(sigs):
            hl, il, h = sig[0], sig[1], sig[2]
            want = [hl, il, h,
                    3 * hl, h // 8, 3 * hl, h // 32,        # qkv
                    h, hl // 8, h, hl // 32,                # o
                    2 * il, h // 8, 2 * il, h // 32,        # gate | up
                    h, il // 8, h, il // 32]                # down
            if h != hidden or hl * world != hidden:
                problems.append(f"rank {r} layer {li}: hidden {h} / hidden_local {hl} do not give {hidden} over {world} ranks")
            elif sig != want:
                problems.append(f"rank {r} layer {li}: shard shapes {sig[3:]} do not match hidden_local {hl}, inter_local {il}")
    for li in range(nl):
        if all(len(s) == nl for s in everyone):
            tot = sum(s[li][1] for s in everyone)
            if tot != inter:
                problems.append(f"layer {li}: the ranks' K slices of the down projection add up to {tot}, not {inter}")
    if problems:
        raise ShardingMismatch("; ".join(problems[:4]))


class StepGuard:
    """Host-side liveness check between decode steps.  Every rank calls check() before it launches a
    step: one tiny all-reduce (MIN of "I am staying") on a CPU-capable process group.  A rank that
    wants to leave calls leave() INSTEAD of check(), between steps, with none of its kernels or
    collectives in flight; the others then get RankLeft from the same collective and launch nothing.
    A rank that disappears without announcing it makes the collective fail or time out (the group's
    timeout), which is reported as RankLeft too.  Nothing here touches a GPU."""

    def __init__(self, group=None):
        self.group = group

    def _exchange(self, staying: int) -> int:
        import torch
        import torch.distributed as dist

        t = torch.tensor([staying], dtype=torch.int32)
        try:
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        except Exception as e:  # a peer that is gone: connection closed, or the group's timeout ran out
            raise RankLeft(f"a rank of the group stopped answering: {e}") from e
        return int(t.item())

    def check(self):
        if self._exchange(1) != 1:
            raise RankLeft("a rank of the tensor-parallel group has left; no further step is launched")

    def leave(self):
        self._exchange(0)
