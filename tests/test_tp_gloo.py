"""Tensor-parallel sharding and collectives on CPU (gloo, world size 2) with a stand-in local linear."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from georefine_b200 import tp

MEMBERS = [96, 32, 32]


def _cpu_factory(words):
    w = torch.from_numpy(np.ascontiguousarray(words).view(np.int16)).view(torch.bfloat16).float()

    def run(x):
        return (x.float() @ w.T).to(torch.bfloat16)

    return run


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, words, x, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        col = tp.ColumnParallelLinear(words, rank, world, members=MEMBERS, local_factory=_cpu_factory)
        y_local = col(x)
        parts = [torch.empty_like(y_local) for _ in range(world)]
        dist.all_gather(parts, y_local)
        row_nccl = tp.RowParallelLinear(words, rank, world, local_factory=_cpu_factory, reduce="nccl")(x)
        row_ord = tp.RowParallelLinear(words, rank, world, local_factory=_cpu_factory, reduce="ordered")(x)
        if rank == 0:
            out.put({"col_parts": [p.float().numpy() for p in parts], "row_nccl": row_nccl.float().numpy(),
                     "row_ord": row_ord.float().numpy()})
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_row_ranges_cover_and_align():
    for n, world in ((5120, 8), (17408, 4), (300, 2), (128, 1)):
        spans = [tp.row_range(n, r, world, 128) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:])) and all(lo % 128 == 0 for lo, _ in spans)
    got = tp.column_parallel_rows([5120, 1024, 1024], 1, 2)
    assert got == [(2560, 5120), (5120 + 512, 5120 + 1024), (6144 + 512, 6144 + 1024)]
    with pytest.raises(ValueError):
        tp.RowParallelLinear(np.zeros((8, 128), dtype=np.uint16), 0, 2, local_factory=_cpu_factory)


@pytest.mark.timeout(120)
def test_two_rank_column_and_row_parallel_match_the_unsharded_product():
    from oracle import bcx_oracle as orc

    words = orc.synthetic_weight_words(160, 512, 77)
    x = torch.randn(5, 512, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16)
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, words, x, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = out.get(timeout=100)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    full = _cpu_factory(words)(x).float().numpy()
    # column parallel: rank r holds its slice of every member of the fused group
    rebuilt = np.empty_like(full)
    for r, part in enumerate(res["col_parts"]):
        at = 0
        for lo, hi in tp.column_parallel_rows(MEMBERS, r, 2):
            rebuilt[:, lo:hi] = part[:, at:at + hi - lo]
            at += hi - lo
    assert np.array_equal(rebuilt, full)
    scale = np.abs(full).max()
    assert np.abs(res["row_nccl"] - full).max() <= 2e-2 * scale
    assert np.abs(res["row_ord"] - full).max() <= 2e-2 * scale
