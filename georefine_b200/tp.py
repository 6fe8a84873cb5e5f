"""Tensor-parallel shards of a compressed linear: one process per GPU over torch.distributed.

The reference has no multi-GPU execution of a linear (its only multi-device code places whole layers,
``glc_loader/tbe_device_map.py:46-56``); the split below follows the row-local structure of its formats
(``glc_serve/tbe_desc.py:1-13``: fused groups are row concatenations).

* Column parallel (QKV, gate|up): rank r owns the weight rows [n0, n1) of every fused member and produces
  y[:, n0:n1].  No communication.
* Row parallel (O, down): rank r owns the weight columns [k0, k1), k0 and k1 multiples of 128 (one chunk of the
  resident layout), multiplies x[:, k0:k1] and the partial outputs are summed across ranks: NCCL all-reduce of
  the BF16 partials, or, with ``reduce="ordered"``, an all-gather followed by a sum in rank order, which
  gives the same bits whatever the message size, or, with ``reduce="peer"``, the library's own kernel over peer
  memory (``peer.PeerReducer``: rank-ordered FP32 sum, the same bits on every rank, capturable in a CUDA graph).

``local_factory(words) -> callable(x2d) -> y2d`` builds the per-rank linear; the default builds a
``ResidentWeight`` on the current CUDA device.  Tests inject a CPU stand-in to exercise the sharding and the
collectives under gloo.
"""
from __future__ import annotations

import numpy as np

CHUNK = 128


def row_range(n: int, rank: int, world: int, multiple: int = 1):
    """Contiguous, balanced split of n units of size `multiple` (the last rank takes the ragged tail)."""
    units = (n + multiple - 1) // multiple
    lo = units * rank // world * multiple
    hi = min(n, units * (rank + 1) // world * multiple)
    return lo, hi


def column_parallel_rows(member_rows, rank: int, world: int):
    """Row ranges of this rank inside each member of a fused group (q|k|v, gate|up), so that the concatenated
    local output is the rank's slice of every member."""
    out, base = [], 0
    for n in member_rows:
        lo, hi = row_range(n, rank, world)
        out.append((base + lo, base + hi))
        base += n
    return out


def _default_factory(device=None, max_m=128):
    def make(words):
        import torch

        from .resident import ResidentWeight

        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        w = ResidentWeight.from_words(words, dev, max_m=max_m)

        def run(x):
            return w.linear(x)

        run.weight = w
        return run

    return make


class ColumnParallelLinear:
    """y_local = x @ W[rows of this rank].T; members lists the row counts of the fused group."""

    def __init__(self, words, rank: int, world: int, *, members=None, local_factory=None, gather_output=False, group=None):
        words = np.asarray(words)
        members = [words.shape[0]] if members is None else list(members)
        if sum(members) != words.shape[0]:
            raise ValueError("member rows do not add up to the weight rows")
        self.ranges = column_parallel_rows(members, rank, world)
        local = np.concatenate([words[lo:hi] for lo, hi in self.ranges], axis=0)
        self.local_rows = local.shape[0]
        self.rank, self.world, self.group, self.gather_output = rank, world, group, gather_output
        self.linear = (local_factory or _default_factory())(np.ascontiguousarray(local))

    def __call__(self, x):
        y = self.linear(x)
        if not self.gather_output or self.world == 1:
            return y
        import torch
        import torch.distributed as dist

        parts = [torch.empty_like(y) for _ in range(self.world)]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)


class RowParallelLinear:
    """y = sum over ranks of x[:, k0:k1] @ W[:, k0:k1].T."""

    def __init__(self, words, rank: int, world: int, *, local_factory=None, reduce="nccl", group=None, peer=None, slot=None):
        words = np.asarray(words)
        if reduce not in ("nccl", "ordered", "peer"):
            raise ValueError("reduce must be 'nccl', 'ordered' or 'peer'")
        if reduce == "peer" and (peer is None or slot is None):
            raise ValueError("reduce='peer' needs a PeerReducer and the name of one of its slots")
        self.peer, self.slot = peer, slot
        self.k0, self.k1 = row_range(words.shape[1], rank, world, CHUNK)
        if self.k1 <= self.k0:
            raise ValueError("more ranks than 128-column chunks")
        self.rank, self.world, self.group, self.reduce = rank, world, group, reduce
        self.linear = (local_factory or _default_factory())(np.ascontiguousarray(words[:, self.k0:self.k1]))

    def __call__(self, x):
        part = self.linear(x[..., self.k0:self.k1])
        if self.world == 1:
            return part
        import torch
        import torch.distributed as dist

        if self.reduce == "nccl":
            dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
            return part
        if self.reduce == "peer":
            flat = part.reshape(-1, part.shape[-1])
            self.peer.slot(self.slot, flat.shape[0], flat.shape[1]).copy_(flat)
            return self.peer.reduce(self.slot, torch.empty_like(flat)).view(part.shape)
        parts = [torch.empty_like(part) for _ in range(self.world)]
        dist.all_gather(parts, part.contiguous(), group=self.group)
        total = parts[0].float()
        for p in parts[1:]:
            total = total + p.float()
        return total.to(part.dtype)
