"""Ranks of the peer all-reduce test: launched by tests/test_gpu_peer_reduce.py (or by hand) with

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P tests/peer_ranks.py

Every rank writes a rank-dependent BF16 pattern into its slot, all ranks reduce, every rank checks the result against
the sum computed locally in rank order (bit-exact), eagerly and replayed from a CUDA graph, and a row-parallel linear
summed this way is compared with the product of the whole weight."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from georefine_b200.peer import PeerReducer  # noqa: E402


def pattern(rank, rows, cols, step, device):
    g = torch.Generator(device="cpu").manual_seed(1000 * step + rank)
    return (torch.randn(rows, cols, generator=g) * (1 + rank)).to(torch.bfloat16).to(device)


def expected(world, rows, cols, step, device):
    total = pattern(0, rows, cols, step, device).float()
    for r in range(1, world):
        total = total + pattern(r, rows, cols, step, device).float()   # FP32, rank order: what the kernel does
    return total.to(torch.bfloat16)


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    shapes = {"small": (1, 5120), "ragged": (3, 1000), "large": (128, 5120)}
    red = PeerReducer({k: r * c for k, (r, c) in shapes.items()}, device=device)
    failures = 0
    for step in range(3):
        for name, (rows, cols) in shapes.items():
            red.slot(name, rows, cols).copy_(pattern(rank, rows, cols, step, device))
            out = torch.empty(rows, cols, dtype=torch.bfloat16, device=device)
            red.reduce(name, out)
            if not torch.equal(out, expected(world, rows, cols, step, device)):
                failures += 1
    # the same call replayed from a CUDA graph (the call counter lives on the device)
    rows, cols = shapes["large"]
    src = pattern(rank, rows, cols, 7, device)
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=device)
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            red.slot("large", rows, cols).copy_(src)
            red.reduce("large", out, stream=side)
    torch.cuda.current_stream().wait_stream(side)
    want = expected(world, rows, cols, 7, device)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        if not torch.equal(out, want):
            failures += 1
    # a row-parallel linear whose partial outputs are summed this way, against the dense product
    import numpy as np

    from georefine_b200 import tp
    from oracle import bcx_oracle as orc

    words = orc.synthetic_weight_words(256, 512, 5)
    red2 = PeerReducer({"lin": 8 * 256}, device=device)
    lin = tp.RowParallelLinear(words, rank, world, reduce="peer", peer=red2, slot="lin")
    x = (torch.randn(8, 512, generator=torch.Generator().manual_seed(3)) * 0.5).to(torch.bfloat16).to(device)
    got = lin(x).float()
    dense = torch.from_numpy(words.view(np.int16)).view(torch.bfloat16).to(device).float()
    want_lin = x.float() @ dense.T
    if not torch.allclose(got, want_lin, rtol=2e-2, atol=2e-2 * float(want_lin.abs().max())):
        failures += 1
    if red2.check_status():
        failures += 1
    red2.close()
    status = red.check_status()
    bad = torch.tensor([failures + (1 if status else 0)], device=device)
    dist.all_reduce(bad)
    if rank == 0:
        print(f"peer all-reduce: world {world}, failures {int(bad.item())}, status {status}", flush=True)
    red.close()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(1 if int(bad.item()) else 0)


if __name__ == "__main__":
    main()
