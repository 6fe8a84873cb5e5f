"""Benchmark of the fused decode-GEMM path on the hybrid-decoder linear shapes (hidden 5120).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layout window4|window|rans]

One step = the four linears of a decoder layer (QKV 5120->7168, O 5120->5120, gate|up 5120->2x17408,
down 17408->5120), each at batch M = 1, 64 and 128: twelve fused decode-GEMM launches over synthetic
weights N(0, 0.02) x LogNormal(0, 0.25) per row (seed 1) held in HBM as compressed resident images.
The coded working set (~440 MB) is larger than the L2, so no flush is needed between iterations.

metric    fused decode-GEMM effective BF16 weight bandwidth: dense BF16 bytes of the weights the step
          multiplies by (2*N*K per launch) divided by the step time, GB/s, whole job.
value     inputs resident in HBM, CUDA events around exactly K steps, max over ranks; the K-step region is
          repeated until at least half a second has been timed and the median region is reported.
roofline  algorithmic bytes of the step (coded images + activations in + outputs out) over the same
          ms_per_step, against the measured copy bandwidth.
e2e       the same step through the descriptor call with activations in pinned host memory copied in and
          the down-projection outputs copied back every step.
parity    outside the timed region: the decode twin reproduces every weight's digest, every output is
          within 1e-2 (relative) of the FP32 product, rows are bitwise equal across M.
With --gpus N (torchrun) the layer is tensor-parallel: QKV and gate|up split by weight rows (no traffic), O
and down by weight columns followed by the sum of the BF16 partials across GPUs; total work is fixed
(strong scaling).  --impl reference times the reference's own CPU decode + matmul on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fused_decode_gemm_effective_bf16_weight_bandwidth"
UNIT = "GB/s"
HIDDEN, FFN = 5120, 17408
# name, N (weight rows), K, parallel kind, members of the fused group
LINEARS = [("qkv", 7168, HIDDEN, "col", [5120, 1024, 1024]), ("o", HIDDEN, HIDDEN, "row", None),
           ("gate_up", 2 * FFN, HIDDEN, "col", [FFN, FFN]), ("down", HIDDEN, FFN, "row", None)]
BATCHES = (1, 64, 128)
SEED = 1
REL_TOL = 1e-2
MIN_TIMED_SECONDS = 0.5
# dram__bytes_read + dram__bytes_write over the algorithmic bytes of one launch, from one ncu capture per layout of the
# step's largest launch (gate|up at M = 128; the entropy-coded layout: the down projection at M = 1).  The window4
# figure is of a launch in a chain of launches, captured cold: 299.3 MB read + 4.1 MB written for 278.9 MB; 29 MB of the
# reads are the first eight blobs per CTA of the NEXT image, asked into L2 for the launch after (which then does not
# read them from DRAM), so in a warm stream the launch's own traffic is its algorithmic bytes or a little less (part of y
# is still in L2 when it ends; the FP32 partial tiles never reach DRAM).
DRAM_TRAFFIC_RATIO = {"window4": 1.088, "window": 1.055, "rans": 1.04}
KERNEL_OF = {"window4": "bxq_kernel", "window": "bxw_kernel", "rans": "bxr_kernel"}
FALLBACK_HBM_GBS = 6650.0


def synthetic_words(generator, rows, cols):
    """BF16 bit patterns of N(0, 0.02) weights with a LogNormal(0, 0.25) scale per row."""
    import torch

    w = torch.randn(rows, cols, generator=generator) * 0.02
    w = w * torch.exp(0.25 * torch.randn(rows, 1, generator=generator))
    return w.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def all_weights():
    import torch

    g = torch.Generator().manual_seed(SEED)
    return {name: synthetic_words(g, n, k) for name, n, k, _, _ in LINEARS}


def measured_hbm_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except (KeyError, ValueError):
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples, each stamped with its arrival time.  Started before the weights
    are built (the tool takes a while to produce its first line on a machine with many GPUs), read over the window of
    the timed region only."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.thread = index, None, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line))

    def wait_first_sample(self, seconds=8.0):
        t0 = time.monotonic()
        while self.proc is not None and not self.lines and time.monotonic() - t0 < seconds:
            time.sleep(0.02)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            if self.thread is not None:
                self.thread.join(timeout=2)

    def summary(self, t0, t1):
        """Over [t0, t1] (monotonic seconds), widened by one sampling period on either side."""
        sm, mx, reasons = [], [], set()
        for at, line in list(self.lines):
            if at < t0 - 0.03 or at > t1 + 0.05:
                continue
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ CPU arm
def cpu_reference_run(sample_rows, steps, warmup, threads):
    """The reference's CPU path on slabs of the benchmark weights: decode every frame, then F.linear at every
    batch size.  Returns (GB/s, seconds per step, description); the description splits the CPU seconds into decode
    and matmul.  Uses oracle/_ref (the reference's coder compiled from its sources) when it was built, else the
    plain-C oracle port."""
    import torch
    import torch.nn.functional as F

    from oracle import bcx_oracle as orc

    kind = "reference" if orc.ref_available() else "port"
    coder = orc.Coder("ref" if kind == "reference" else "oracle")
    g = torch.Generator().manual_seed(SEED)
    slab = 128
    frames = []
    for name, n, k, _, _ in LINEARS:
        rows = min(n, sample_rows)
        words = synthetic_words(g, rows, k)
        for lo in range(0, rows, slab):
            frames.append((k, coder.encode(np.ascontiguousarray(words[lo:lo + slab]))))
    xs = {(m, k): torch.randn(m, k, generator=g).to(torch.bfloat16) for m in BATCHES for k in (HIDDEN, FFN)}
    dense_bytes = sum(2 * min(n, sample_rows) * k for _, n, k, _, _ in LINEARS) * len(BATCHES)
    torch.set_num_threads(1)

    def one(job):
        k, frame = job
        decode_s = matmul_s = 0.0
        for m in BATCHES:          # the reference decodes the whole weight on every forward call
            t0 = time.perf_counter()
            w = torch.from_numpy(coder.decode(frame).view(np.int16)).view(torch.bfloat16)
            t1 = time.perf_counter()
            F.linear(xs[(m, k)], w)
            decode_s += t1 - t0
            matmul_s += time.perf_counter() - t1
        return decode_s, matmul_s

    def step():
        with ThreadPoolExecutor(threads) as pool:
            parts = list(pool.map(one, frames))
        return sum(p[0] for p in parts), sum(p[1] for p in parts)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    decode_s = matmul_s = 0.0
    for _ in range(steps):
        d, mm = step()
        decode_s += d
        matmul_s += mm
    dt = (time.perf_counter() - t0) / max(steps, 1)
    sample = f"first {sample_rows} rows of each of the four weights as {slab}-row BCTX frames, decode + F.linear at M=1,64,128"
    return dense_bytes / dt / 1e9, dt, {"kind": kind, "cores": threads, "sample": sample,
                                        "decode_cpu_seconds_per_step": round(decode_s / max(steps, 1), 3),
                                        "matmul_cpu_seconds_per_step": round(matmul_s / max(steps, 1), 3)}


# ------------------------------------------------------------------------------------------------ GPU arm
class Layer:
    """The four linears of one decoder layer on this rank, as resident images (tensor-parallel when world > 1)."""

    def __init__(self, rank, world, device, layout="window4", weights=None, with_peer=True):
        import torch

        from georefine_b200 import tp
        from georefine_b200.resident import ResidentWeight

        self.rank, self.world, self.device = rank, world, device
        weights = dict(all_weights() if weights is None else weights)
        self.entries = []
        for name, n, k, kind, members in LINEARS:
            w = weights.pop(name)
            if kind == "col":
                spans = tp.column_parallel_rows(members, rank, world)
                local = np.concatenate([w[lo:hi] for lo, hi in spans], axis=0)
                k0, k1 = 0, k
            else:
                spans = [(0, n)]
                k0, k1 = tp.row_range(k, rank, world, tp.CHUNK)
                local = w[:, k0:k1]
            local = np.ascontiguousarray(local)
            res = ResidentWeight.from_words(local, device, max_m=max(BATCHES), verify=False, layout=layout)
            self.entries.append({"name": name, "kind": kind, "n": n, "k": k, "k0": k0, "k1": k1, "res": res, "spans": spans,
                                 "words": local, "y": {m: torch.empty(m, res.N, device=device, dtype=torch.bfloat16) for m in BATCHES}})
            del w
        # the order of the launches is fixed: every weight knows which one the stream reads next (an L2 prefetch hint)
        for e, nxt in zip(self.entries, self.entries[1:] + self.entries[:1]):
            e["res"].then(nxt["res"])
        g = torch.Generator().manual_seed(SEED + 1)
        self.x_host = {(m, k): torch.randn(m, k, generator=g).to(torch.bfloat16).pin_memory() for m in BATCHES for k in (HIDDEN, FFN)}
        self.x = {key: v.to(device) for key, v in self.x_host.items()}
        self.y_host = {m: torch.empty(m, HIDDEN, dtype=torch.bfloat16).pin_memory() for m in BATCHES}
        self.xv = {(m, e["name"]): self.x[(m, e["k"])][:, e["k0"]:e["k1"]] for m in BATCHES for e in self.entries}
        # More than one rank: the down projection multiplies this rank's FFN columns only, so the host hands the rank only
        # that slice of the FFN-width activations (a contiguous pinned buffer, a contiguous device buffer): the end-to-end
        # loop then copies 2 M (hidden + FFN / world) bytes per batch instead of 2 M (hidden + FFN).  The hidden-width
        # input is needed whole (QKV and gate|up read all of it).
        self.ffn_host, self.ffn_local = {}, {}
        if world > 1:
            down = next(e for e in self.entries if e["name"] == "down")
            for m in BATCHES:
                self.ffn_host[m] = self.x_host[(m, FFN)][:, down["k0"]:down["k1"]].contiguous().pin_memory()
                self.ffn_local[m] = self.ffn_host[m].to(device)
                self.xv[(m, "down")] = self.ffn_local[m]
        self.launches_per_step = len(LINEARS) * len(BATCHES)
        # More than one rank: the partial outputs of the column-split linears (O, down) are summed over peer memory by
        # the library's own kernel, which can be captured in a CUDA graph with the fused launches.  The linear writes its
        # partial into the reducer's slot (e["y"]), the sum lands in e["sum"].  NCCL is the fallback if the buffers cannot
        # be mapped on every rank.
        self.peer, self.reduce_kind = None, "none"
        if world > 1 and with_peer:
            self.peer, self.reduce_kind = self._peer_reducer(), "nccl"
            if self.peer is not None:
                self.reduce_kind = "peer"
                for e in self.entries:
                    if e["kind"] == "row":
                        e["sum"] = {m: torch.empty(m, e["res"].N, device=device, dtype=torch.bfloat16) for m in BATCHES}
                        e["y"] = {m: self.peer.slot(f'{e["name"]}:{m}', m, e["res"].N) for m in BATCHES}
                self.launches_per_step += sum(len(BATCHES) for e in self.entries if e["kind"] == "row")

    def _peer_reducer(self):
        import torch
        import torch.distributed as dist

        from georefine_b200.peer import PeerReducer

        slots = {f'{e["name"]}:{m}': (m * e["res"].N + 7) // 8 * 8 for e in self.entries if e["kind"] == "row" for m in BATCHES}
        peer, ok = None, 1
        try:
            peer = PeerReducer(slots, device=self.device)
        except Exception as exc:  # noqa: BLE001
            print(f"[bench] rank {self.rank}: peer-memory all-reduce unavailable ({type(exc).__name__}: {exc}); using NCCL", file=sys.stderr)
            ok = 0
        flag = torch.tensor([ok], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return peer if int(flag.item()) else None

    def peer_is_healthy(self):
        """After the first eager steps: did every rank's peer reductions complete?  A wait that ran out (a peer that is
        not there, a mapping that does not work) must not be paid two seconds at a time for the rest of the run: all
        ranks fall back to NCCL together.  The slots stay where they are (the linears keep writing into them)."""
        import torch
        import torch.distributed as dist

        if self.peer is None:
            return True
        bad = torch.tensor([1 if self.peer.check_status() else 0], device=self.device)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            self._retired_peer, self.peer, self.reduce_kind = self.peer, None, "nccl (the peer reduction reported a timeout)"
            self.launches_per_step = len(LINEARS) * len(BATCHES)
            return False
        return True

    def result(self, e, m):
        """Where the finished output of a linear is."""
        return e["sum"][m] if (self.peer is not None and e["kind"] == "row") else e["y"][m]

    def all_reduce(self, e, m):
        import torch.distributed as dist

        if self.peer is not None:
            self.peer.reduce(f'{e["name"]}:{m}', e["sum"][m])
        else:
            dist.all_reduce(e["y"][m])

    def dense_bytes_per_step(self):
        return sum(2 * n * k for _, n, k, _, _ in LINEARS) * len(BATCHES)

    def algorithmic_bytes(self, e, m):
        """What one launch must move: the coded image once, the activations in, the outputs out."""
        return e["res"].coded_bytes + 2 * m * (e["k1"] - e["k0"]) + 2 * m * e["res"].N

    def step(self):
        """The twelve launches.  More than one rank: the sums of the column-split linears' partial outputs run on a side
        stream, in launch order, each behind the linear that feeds it; the step's launches do not read one another's
        outputs, so a sum (mostly a wait for the peers' flags) overlaps the next linear instead of standing between two.
        The side stream joins before the step ends; captured, this is one graph with two branches."""
        import torch

        side = self._side_stream() if (self.peer is not None and self.world > 1) else None
        main = torch.cuda.current_stream(self.device) if side is not None else None
        for m in BATCHES:
            for e in self.entries:
                e["res"].gemm(self.xv[(m, e["name"])], e["y"][m])
                if e["kind"] == "row" and self.world > 1:
                    if side is None:
                        self.all_reduce(e, m)
                    else:
                        ready = torch.cuda.Event()
                        ready.record(main)
                        side.wait_event(ready)
                        self.peer.reduce(f'{e["name"]}:{m}', e["sum"][m], stream=side)
        if side is not None:
            done = torch.cuda.Event()
            done.record(side)
            main.wait_event(done)

    def _side_stream(self):
        import torch

        if getattr(self, "_side", None) is None:
            self._side = torch.cuda.Stream(self.device)
        return self._side

    def segmented_step(self):
        """Multi-rank step as CUDA graphs of the fused launches with the NCCL all-reduces launched between them
        (no collective is ever captured).  Returns a callable, or None if a capture failed on any rank."""
        import torch
        import torch.distributed as dist

        plan, ok = [], 1
        try:
            for m in BATCHES:
                run = []
                for e in self.entries:
                    run.append(e)
                    if e["kind"] == "row":
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g, capture_error_mode="thread_local"):
                            for f in run:
                                f["res"].gemm(self.xv[(m, f["name"])], f["y"][m])
                        plan.append((g, e["y"][m]))
                        run = []
        except Exception:  # noqa: BLE001
            ok = 0
        flag = torch.tensor([ok], device=self.device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if not int(flag.item()):
            return None

        def step():
            for g, y in plan:
                g.replay()
                dist.all_reduce(y)

        return step

    def copy_inputs(self, m):
        """Pinned host -> device: the activations batch m needs on this rank (asynchronous, current stream)."""
        self.x[(m, HIDDEN)].copy_(self.x_host[(m, HIDDEN)], non_blocking=True)
        if self.world > 1:
            self.ffn_local[m].copy_(self.ffn_host[m], non_blocking=True)
        else:
            self.x[(m, FFN)].copy_(self.x_host[(m, FFN)], non_blocking=True)

    def h2d_bytes_per_step(self):
        ffn = self.ffn_host[BATCHES[0]].shape[1] if self.world > 1 else FFN
        return sum(2 * m * (HIDDEN + ffn) for m in BATCHES)

    def step_e2e(self):
        """Host buffers in, host buffers out, through the descriptor call `weight(x, y)` a serving engine makes:
        every activation is copied from pinned host memory first, the down projection's output is copied back."""
        import torch

        for m in BATCHES:
            self.copy_inputs(m)
            for e in self.entries:
                e["res"](self.xv[(m, e["name"])], e["y"][m])
                if e["kind"] == "row" and self.world > 1:
                    self.all_reduce(e, m)
            self.y_host[m].copy_(self.result(self.entries[-1], m), non_blocking=True)   # the down projection's output
        torch.cuda.current_stream().synchronize()

    def e2e_graph(self):
        """The end-to-end step as one CUDA graph, the way the reference's serving engines replay a whole decode step
        (glc_serve/fastdec.py capture/replay): the pinned-host -> device copies of every batch run on a side stream and
        overlap the launches of the batches before them, the descriptor calls follow on the main stream, and each
        batch's result goes back to the host on the side stream while the next batch runs.  With more than one rank only
        when the sums go over peer memory (no NCCL collective is ever captured).  Returns a callable that
        replays the graph and waits until the results are in host memory."""
        import torch

        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream(self.device)
        with torch.cuda.graph(graph):
            main = torch.cuda.current_stream()
            side.wait_stream(main)
            ready = {}
            with torch.cuda.stream(side):
                for m in BATCHES:
                    self.copy_inputs(m)
                    ready[m] = torch.cuda.Event()
                    ready[m].record(side)
            sums = self._side_stream() if self.peer is not None else None   # the cross-rank sums, as in step()
            for m in BATCHES:
                main.wait_event(ready[m])
                for e in self.entries:
                    e["res"](self.xv[(m, e["name"])], e["y"][m])
                    if e["kind"] == "row" and sums is not None:
                        partial = torch.cuda.Event()
                        partial.record(main)
                        sums.wait_event(partial)
                        self.peer.reduce(f'{e["name"]}:{m}', e["sum"][m], stream=sums)
                done = torch.cuda.Event()
                done.record(main if sums is None else sums)
                with torch.cuda.stream(side):   # the down projection's output goes back while the next batch runs
                    side.wait_event(done)
                    self.y_host[m].copy_(self.result(self.entries[-1], m), non_blocking=True)
            main.wait_stream(side)
            if sums is not None:
                main.wait_stream(sums)

        def step():
            graph.replay()
            torch.cuda.current_stream().synchronize()

        return step

    def status(self):
        return sum(e["res"].check_status() for e in self.entries) + (self.peer.check_status() if self.peer is not None else 0)

    # ---- checks outside the timed region --------------------------------------------------------------------
    def parity(self):
        """This rank's images and outputs against FP32 arithmetic on the source words: the decode twin must reproduce
        the digest of the words the image was built from; every fused product must be within REL_TOL of the FP32
        product (relative to the call's largest magnitude); rows must be bitwise the same at every batch size."""
        import hashlib

        import torch

        worst, rows_equal, digests = 0.0, True, True
        for e in self.entries:
            res = e["res"]
            got = res.decode(check=False).view(torch.int16).cpu().numpy().view(np.uint16)
            digests = digests and hashlib.sha256(got.tobytes()).digest() == hashlib.sha256(e["words"].tobytes()).digest()
            w = torch.from_numpy(e["words"].view(np.int16)).view(torch.bfloat16).to(self.device)
            top = None
            for m in sorted(BATCHES, reverse=True):
                x = self.xv[(m, e["name"])]
                y = torch.empty(m, res.N, device=self.device, dtype=torch.bfloat16)
                res.gemm(x, y)
                ref = x.float() @ w.float().T
                worst = max(worst, float((y.float() - ref).abs().max() / ref.abs().max()))
                # the same leading rows of the activations at every batch size? they are separate draws: compare the
                # rows of a batch cut from the largest one instead
                if top is None:
                    top = (x, y.clone())
                else:
                    ycut = torch.empty(m, res.N, device=self.device, dtype=torch.bfloat16)
                    res.gemm(top[0][:m], ycut)
                    rows_equal = rows_equal and bool(torch.equal(ycut.view(torch.int16), top[1][:m].view(torch.int16)))
            del w
        return {"max_rel": float(f"{worst:.3e}"), "tolerance": REL_TOL, "rows_equal": bool(rows_equal), "decode_digests_ok": bool(digests),
                "status_word": self.status()}

    def tp_parity(self, full_weights):
        """More than one rank: the summed outputs of the column-split linears (O, down) on this rank against the FP32
        product with the WHOLE weight, computed on this GPU alone."""
        import torch

        worst = 0.0
        for e in self.entries:
            if e["kind"] != "row":
                continue
            w = torch.from_numpy(full_weights[e["name"]].view(np.int16)).view(torch.bfloat16).to(self.device)
            for m in BATCHES:
                ref = self.x[(m, e["k"])].float() @ w.float().T
                got = self.result(e, m).float()
                worst = max(worst, float((got - ref).abs().max() / ref.abs().max()))
            del w
        return {"max_rel": float(f"{worst:.3e}"), "tolerance": REL_TOL, "checked": "summed O and down outputs vs the one-GPU FP32 product"}


def timed_regions(fn, steps, warmup, world, min_seconds=MIN_TIMED_SECONDS, max_regions=400):
    """W warm-up steps, then regions of exactly K steps, each bracketed by a barrier and a device synchronise on both
    sides and timed with CUDA events (max over ranks), repeated until min_seconds have been timed.  Returns the list of
    per-region milliseconds per step and the (monotonic) host times around the whole measurement."""
    import torch
    import torch.distributed as dist

    def region():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device="cuda")
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(warmup):
        fn()
    t0 = time.monotonic()
    out = [region()]
    want = int(min(max_regions, max(1, -(-min_seconds * 1e3 // max(out[0] * steps, 1e-6)))))   # same on every rank
    while len(out) < want:
        out.append(region())
    return out, t0, time.monotonic()


def launch_times(layer):
    """Microseconds of every (linear, batch size) launch in a stream of such launches, rotating over enough copies of
    the image that the weights never come from the L2 (the practice of the reference's tuner,
    glc_serve/tbe_desc.py:160-175)."""
    import torch

    from georefine_b200 import tune

    out = {}
    for e in layer.entries:
        res = e["res"]
        first = res.clone()
        copies = [first] + [res.clone() for _ in range(tune.copies_for(res.coded_bytes) - 1)]
        for a, b in zip(copies, copies[1:] + copies[:1]):
            a.then(b)
        for m in BATCHES:
            x, y = layer.xv[(m, e["name"])], e["y"][m]
            reps = max(20, int(1e9 // res.coded_bytes))
            out[(e["name"], m)] = tune.rotation_us(lambda i: copies[i].gemm(x, y), len(copies), reps)
        for c in copies:
            c.then(None)
        del copies, first
        torch.cuda.empty_cache()
    return out


def dense_times(layer):
    """The dense BF16 yardsticks on the same GPU and the same (local) weights: the library's own GEMV at M = 1 and
    torch.matmul at every batch size, rotating over copies like launch_times."""
    import torch

    from georefine_b200 import tune
    from georefine_b200.dense import dense_gemv

    own, lib = {}, {}
    for e in layer.entries:
        w = torch.from_numpy(e["words"].view(np.int16)).view(torch.bfloat16).to(layer.device)
        copies = [w] + [w.clone() for _ in range(tune.copies_for(w.numel() * 2) - 1)]
        reps = max(20, int(1e9 // (w.numel() * 2)))
        for m in BATCHES:
            x, y = layer.xv[(m, e["name"])].contiguous(), torch.empty(m, w.shape[0], device=layer.device, dtype=torch.bfloat16)
            lib[(e["name"], m)] = tune.rotation_us(lambda i: torch.matmul(x, copies[i].T, out=y), len(copies), reps)
            if m == 1:
                own[e["name"]] = tune.rotation_us(lambda i: dense_gemv(copies[i], x, y), len(copies), reps)
        del copies, w
        torch.cuda.empty_cache()
    return own, lib


def indexed_decode_times(device):
    """Decode of UNCHANGED BCTX streams on the GPU (what an embedding gather and ``CudaContextTensor.decode`` run): the
    configuration-0 matrix (4096 x 4096, seed 0) through this library's kernel and - when the reference's own modules
    have been staged under baseline/_ref/ - through the reference's Triton kernels followed by F.linear at M = 1, the
    reference's simple path on the same GPU."""
    import torch
    import torch.nn.functional as F

    from georefine_b200 import codec
    from georefine_b200.gpu import CudaContextTensor

    words = synthetic_words(torch.Generator().manual_seed(0), 4096, 4096)
    frame = codec.encode(words)
    x = torch.randn(1, 4096, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(device)

    def timed_us(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps * 1e3

    out = {"matrix": "4096x4096 seed 0", "frame_bytes": len(frame)}
    # walk_stride = words per lane of the device walk.  1024 is the reference's geometry (one lane per restart block of
    # the caller's stride); CudaContextTensor(frame, stride=1024) builds its index at 128 by default.
    for walk in (1024, 128):
        t = CudaContextTensor(frame, stride=1024, walk_stride=walk, device=device, fused=False)
        ok = bool(np.array_equal(t.decode().view(torch.int16).cpu().numpy().view(np.uint16), words))
        us = timed_us(lambda: t.decode(check=False))
        out[f"bctx_decode_kernel_stride{walk}"] = {"us": round(us, 1), "dense_GBps": round(2 * words.size / us / 1e3, 1), "bit_exact": ok,
                                                   "index_bytes": int(sum(v.numel() * v.element_size() for k, v in t.buffers.items()
                                                                          if k.endswith(("_states", "_offsets"))))}
        if walk == 1024:
            us = timed_us(lambda: F.linear(x, t.decode(check=False)))
            out["decode_plus_linear_m1_us"] = round(us, 1)
        del t
    t = CudaContextTensor(frame, stride=1024, device=device, fused=False)
    out["default"] = {"stride": 1024, "walk_stride": t.walk_stride, "decode_us": round(timed_us(lambda: t.decode(check=False)), 1),
                      "decode_plus_linear_m1_us": round(timed_us(lambda: F.linear(x, t.decode(check=False))), 1)}
    del t
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "georefine_context_runtime" / "bitexact_context_gpu.py").is_file():
        out["reference_triton"] = {"unavailable": "the reference's modules are not staged under baseline/_ref"}
        return out
    try:
        import importlib
        import tempfile

        os.environ.setdefault("BITEXACT_CONTEXT_CACHE_DIR", tempfile.mkdtemp(prefix="bctx-ref-"))
        sys.path.insert(0, str(ref_root))
        ref_gpu = importlib.import_module("georefine_context_runtime.bitexact_context_gpu")
        t = ref_gpu.CudaContextTensor(frame, stride=1024, device=str(device))
        ok = bool(np.array_equal(t.decode().view(torch.int16).cpu().numpy().view(np.uint16), words))
        us_decode = timed_us(lambda: t.decode(check=False), reps=3)
        us_both = timed_us(lambda: F.linear(x, t.decode()), reps=3)          # the reference's BctxLinear.forward, check included
        out["reference_triton"] = {"decode_us": round(us_decode, 1), "decode_plus_linear_m1_us": round(us_both, 1),
                                   "dense_GBps": round(2 * words.size / us_decode / 1e3, 1), "bit_exact": ok,
                                   "what": "the reference's CudaContextTensor.decode() (Triton decode_words) + F.linear, unmodified, stride 1024"}
    except Exception as exc:  # noqa: BLE001
        out["reference_triton"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    finally:
        if str(ref_root) in sys.path:
            sys.path.remove(str(ref_root))
    return out


def capture(step, eager_steps=2):
    """The step as one CUDA graph (the entry points neither allocate nor synchronise)."""
    import torch

    for _ in range(eager_steps):
        step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    return graph.replay


def _deadline(seconds):
    """Ends the process if the whole run takes longer than `seconds`: a stuck collective must not hold GPUs."""
    def fire():
        sys.stderr.write(f"bench.py: no result after {seconds} s, giving up\n")
        sys.stderr.flush()
        os._exit(3)

    t = threading.Timer(seconds, fire)
    t.daemon = True
    t.start()
    return t


def run_ours(args):
    import torch
    import torch.distributed as dist

    _deadline(540)

    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused path has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    clocks = ClockSampler(local).start()
    if world > 1:
        import datetime

        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=180))
    weights = all_weights()
    layer = Layer(rank, world, device, layout=args.layout, weights=weights)

    # The timed step is replayed from a CUDA graph, so the host's launch cost is not part of `value`; the e2e figure
    # below goes through the public descriptor call.  NCCL collectives are never captured: with the NCCL fallback
    # multi-rank runs replay graphs of the fused launches only and issue the collectives eagerly between them.
    step_fn, launch = layer.step, "eager"
    if world > 1 and layer.peer is not None:
        for _ in range(2):
            layer.step()
        torch.cuda.synchronize()
        layer.peer_is_healthy()
    whole_graph = world == 1 or layer.peer is not None   # nothing of NCCL inside the step
    if not args.no_graph and whole_graph:
        try:
            step_fn, launch = capture(layer.step), "cuda_graph" + (" (peer-memory all-reduce inside)" if world > 1 else "")
        except Exception as exc:  # noqa: BLE001
            launch = f"eager (graph capture failed: {type(exc).__name__})"
        if world > 1:   # every rank must replay the same thing: one failed capture sends all of them to eager launches
            agreed = torch.tensor([1 if step_fn is not layer.step else 0], device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if not int(agreed.item()):
                step_fn, launch = layer.step, "eager (graph capture failed on some rank)"
    if not args.no_graph and world > 1 and not whole_graph:
        for _ in range(2):
            layer.step()
        torch.cuda.synchronize()
        seg = layer.segmented_step()
        if seg is not None:
            step_fn, launch = seg, "cuda_graph segments + eager all-reduce"
    clocks.wait_first_sample()
    regions, t_begin, t_end = timed_regions(step_fn, args.steps, args.warmup, world)
    clock_summary = clocks.summary(t_begin, t_end)
    ms = float(np.median(regions))

    e2e_fn, e2e_launch = layer.step_e2e, "eager"
    if not args.no_graph and whole_graph:
        try:
            layer.step_e2e()
            e2e_fn, e2e_launch = layer.e2e_graph(), "cuda_graph, copies on a side stream"
        except Exception as exc:  # noqa: BLE001
            e2e_launch = f"eager (graph capture failed: {type(exc).__name__})"
        if world > 1:
            agreed = torch.tensor([1 if e2e_fn is not layer.step_e2e else 0], device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if not int(agreed.item()):
                e2e_fn, e2e_launch = layer.step_e2e, "eager (graph capture failed on some rank)"
    e2e_regions, _, _ = timed_regions(e2e_fn, args.steps, args.warmup, world)
    ms_e2e = float(np.median(e2e_regions))
    y_check = [layer.y_host[m].clone() for m in BATCHES]
    layer.step_e2e()                                     # the eager public-API path must land the same outputs
    e2e_same = all(bool((a.view(torch.int16) == layer.y_host[m].view(torch.int16)).all()) for a, m in zip(y_check, BATCHES))
    tp_check = layer.tp_parity(weights) if world > 1 else None
    status = layer.status()
    clocks.stop()

    dense = layer.dense_bytes_per_step()
    peak, peak_kind = measured_hbm_peak()
    algo = sum(layer.algorithmic_bytes(e, m) for m in BATCHES for e in layer.entries)     # this rank's bytes per step
    achieved = algo / (ms * 1e-3) / 1e9
    top_e = max(layer.entries, key=lambda e: e["res"].coded_bytes)
    top_bytes = layer.algorithmic_bytes(top_e, max(BATCHES))
    mhz = clock_summary["sm_mhz"]
    line = {
        "metric": METRIC, "value": round(dense / (ms * 1e-3) / 1e9, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "hybrid-decoder linears hidden=5120 (QKV 7168x5120, O 5120x5120, gate|up 34816x5120, down 5120x17408), "
                               "seed 1, fused decode-GEMM at M=1,64,128", "parallelism": f"tp{world}",
                   "l2": "coded working set ~440 MB exceeds the 126 MB L2; no flush between iterations",
                   "resident_format": "BXR1/" + args.layout, "launch": launch, "all_reduce": layer.reduce_kind, "status_word": status},
        "timing": {"regions": len(regions), "steps_per_region": args.steps, "timed_seconds": round(sum(regions) * args.steps / 1e3, 3),
                   "ms_per_step_median": round(ms, 4), "ms_per_step_min": round(min(regions), 4), "ms_per_step_max": round(max(regions), 4),
                   "ms_times_sm_mhz": None if not mhz else round(ms * mhz, 1)},
        "e2e": {"value": round(dense / (ms_e2e * 1e-3) / 1e9, 2), "unit": UNIT, "ms_per_step": round(ms_e2e, 4),
                "h2d_bytes_per_step": layer.h2d_bytes_per_step(), "d2h_bytes_per_step": sum(2 * m * HIDDEN for m in BATCHES),
                "launch": e2e_launch, "outputs_match_eager_path": e2e_same, "regions": len(e2e_regions)},
        "gpu_launches": layer.launches_per_step * args.steps * len(regions),
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": round(top_bytes * DRAM_TRAFFIC_RATIO[args.layout]), "peak_source": peak_kind,
                     "algorithmic_bytes_per_step": algo,
                     "how": "achieved = algorithmic_bytes_per_step (this rank's coded images + x + y of the 12 launches) / ms_per_step; "
                            "traffic = DRAM bytes of the step's largest launch (gate|up at M=128): its algorithmic bytes x the "
                            "dram read+write ratio of one ncu capture of that launch",
                     "kernel": KERNEL_OF[args.layout] + "<kUmma, NB>, the 12 launches of a step"},
        "clocks": clock_summary,
    }
    # ---- outside the timed region: parity, per-launch breakdown, dense yardsticks, the other layouts
    line["parity"] = layer.parity()
    if tp_check is not None:
        line["tp_parity"] = tp_check
    ktimes = launch_times(layer)
    per_m = {}
    for m in BATCHES:
        t = sum(ktimes[(e["name"], m)] for e in layer.entries) * 1e-3
        coded = sum(layer.algorithmic_bytes(e, m) for e in layer.entries)
        per_m[str(m)] = {"kernel_ms": round(t, 4), "effective_bf16_GBps": round(dense / len(BATCHES) / world / t / 1e6, 1),
                         "coded_GBps": round(coded / t / 1e6, 1), "frac_of_hbm_peak": round(coded / t / 1e6 / peak, 4),
                         "linears_only_tok_s_64_layers": round(m / (64 * t * 1e-3), 1)}
    line["per_m"] = per_m
    line["per_launch"] = {f"{name}:{m}": {"us": round(us, 2), "algorithmic_bytes": layer.algorithmic_bytes(next(e for e in layer.entries if e["name"] == name), m),
                                          "frac_of_hbm_peak": round(layer.algorithmic_bytes(next(e for e in layer.entries if e["name"] == name), m) / us / 1e3 / peak, 4)}
                          for (name, m), us in ktimes.items()}
    top = (top_e["name"], max(BATCHES))
    line["roofline"]["top_launch"] = {"linear": top[0], "m": top[1], "us": round(ktimes[top], 2), "algorithmic_bytes": top_bytes,
                                      "GBps": round(top_bytes / ktimes[top] / 1e3, 1), "frac": round(top_bytes / ktimes[top] / 1e3 / peak, 4),
                                      "how": "in a stream of such launches over rotating copies of the image"}
    own, lib = dense_times(layer)
    fused_m1 = {e["name"]: ktimes[(e["name"], 1)] for e in layer.entries}
    line["dense_gemv"] = {
        "own_kernel_us_m1": {k: round(v, 2) for k, v in own.items()}, "torch_matmul_us": {f"{k[0]}:{k[1]}": round(v, 2) for k, v in lib.items()},
        "fused_us_m1": {k: round(v, 2) for k, v in fused_m1.items()},
        "speedup_vs_own_gemv_m1": {k: round(own[k] / fused_m1[k], 3) for k in own},
        "speedup_vs_own_gemv_m1_step": round(sum(own.values()) / sum(fused_m1.values()), 3),
        "speedup_vs_torch_matmul": {str(m): round(sum(lib[(e["name"], m)] for e in layer.entries) / sum(ktimes[(e["name"], m)] for e in layer.entries), 3)
                                    for m in BATCHES},
        "target": "> 1.3x a dense BF16 GEMV on the same GPU",
        "own_gemv_GBps_m1": {e["name"]: round(2 * e["words"].size / own[e["name"]] / 1e3, 1) for e in layer.entries}}
    if world == 1 and not args.skip_layouts:
        line["per_layout"] = {args.layout: {"value": line["value"], "ms_per_step": line["ms_per_step"], "roofline_frac": line["roofline"]["frac"],
                                            "bytes_per_weight": round(sum(e["res"].coded_bytes for e in layer.entries) / sum(e["words"].size for e in layer.entries), 4)}}
        del layer
        torch.cuda.empty_cache()
        for other in ("window4", "window", "rans"):
            if other == args.layout:
                continue
            alt = Layer(rank, world, device, layout=other, weights=weights)
            fn = alt.step if args.no_graph else capture(alt.step)
            r, _, _ = timed_regions(fn, args.steps, args.warmup, world, min_seconds=0.2)
            t = float(np.median(r))
            a = sum(alt.algorithmic_bytes(e, m) for m in BATCHES for e in alt.entries)
            gate_up = next(e for e in alt.entries if e["name"] == "gate_up")
            us1 = launch_times_one(alt, gate_up, 1)
            line["per_layout"][other] = {"value": round(dense / (t * 1e-3) / 1e9, 2), "ms_per_step": round(t, 4),
                                         "roofline_frac": round(a / (t * 1e-3) / 1e9 / peak, 4),
                                         "bytes_per_weight": round(sum(e["res"].coded_bytes for e in alt.entries) / sum(e["words"].size for e in alt.entries), 4),
                                         "gate_up_m1_us": round(us1, 2),
                                         "gate_up_m1_frac": round(alt.algorithmic_bytes(gate_up, 1) / us1 / 1e3 / peak, 4),
                                         "status_word": alt.status()}
            del alt
            torch.cuda.empty_cache()
    if world == 1 and rank == 0:
        line["indexed_decode"] = indexed_decode_times(device)
        fused_c0 = None
        try:
            from georefine_b200 import tune as _tune

            fused_c0 = _tune.tune_shape(4096, 4096, device, ms=(1,), workers=[128], reps=200, log=lambda m: None,
                                        words=synthetic_words(torch.Generator().manual_seed(0), 4096, 4096))["us"]["window4,128,M1"]
        except Exception:  # noqa: BLE001
            pass
        line["indexed_decode"]["fused_linear_m1_us"] = fused_c0
    if world == 1 and not args.skip_decode:
        # the other half of the headline metric: whole-stack decode tokens per second at 1, 64 and 128 concurrent sequences
        torch.cuda.empty_cache()
        rec = decode_measurement(device, [1, 64, 128], generate=128)
        line["decode"] = {"tok_s": {n: r["tok_s"] for n, r in rec["results"].items()}, "ms_per_step": {n: r["ms_per_step"] for n, r in rec["results"].items()},
                          "weight_bytes_per_step": rec["weight_bytes_per_step"], "kv_bytes_per_step": {n: r["kv_bytes_per_step"] for n, r in rec["results"].items()},
                          "frac_of_hbm_peak": {n: r["frac_of_hbm_peak"] for n, r in rec["results"].items()}, "config": rec["config"],
                          "generated_tokens_timed": 128, "status_word": sum(r["status_word"] for r in rec["results"].values())}
    if rank == 0 and world == 1:
        value, dt, info = cpu_reference_run(sample_rows=2048, steps=1, warmup=0, threads=os.cpu_count() or 1)
        line["cpu_baseline"] = {"value": round(value, 4), "unit": UNIT, **info, "seconds": round(dt, 2)}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def launch_times_one(layer, e, m):
    from georefine_b200 import tune

    res = e["res"]
    copies = [res.clone() for _ in range(tune.copies_for(res.coded_bytes))]
    for a, b in zip(copies, copies[1:] + copies[:1]):
        a.then(b)
    x, y = layer.xv[(m, e["name"])], e["y"][m]
    return tune.rotation_us(lambda i: copies[i].gemm(x, y), len(copies), max(20, int(1e9 // res.coded_bytes)))


def run_decode(args):
    """Whole-stack decode throughput (BASELINE.json configs 2 and 3): the 64-layer random-init decoder (hidden 5120, 40
    query / 8 KV heads x 128, FFN 17408, vocabulary 152064) with compressed weights, continuous batching at the given
    numbers of concurrent sequences, a 2048-token context per sequence and 128 generated tokens, from random token IDs.
    The context's KV entries are synthetic (random pages written directly: processing 128 x 2048 prompt tokens would
    take longer than the measurement and is not what the configuration times); every timed step is the engine's real
    step - embedding, 64 x (norm, QKV, rotary + append, paged attention, O, norm, gate|up, SwiGLU, down), final norm,
    output head, arg-max, device-side advance - replayed from one CUDA graph.  Layers beyond --distinct-layers reuse
    device copies of the first ones (the same bytes stream from HBM; building 64 distinct layers on the host takes
    minutes).  One JSON line: tok/s per configuration, with the weight and KV bytes a step streams."""
    import torch

    _deadline(1500)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:    # BASELINE.json config 4: the same stack under tensor parallelism (see decode_measurement)
        import datetime

        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    line = decode_measurement(dev, [int(v) for v in args.seqs.split(",")], layers=args.layers, distinct_layers=args.distinct_layers,
                              spec=args.spec and world == 1, generate=128, rank=rank, world=world)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


def _same_on_every_rank(tensor, dev) -> bool:
    """Do all ranks hold the same values (the tokens of a step: they must, or the ranks' hosts would drift apart)?"""
    import torch
    import torch.distributed as dist

    lo, hi = tensor.clone().to(torch.int64), tensor.clone().to(torch.int64)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return bool(torch.equal(lo, hi))


def decode_measurement(dev, seqs, *, layers=64, distinct_layers=2, spec=False, generate=128, rank=0, world=1):
    """See run_decode.  Returns the JSON-ready record.  With world > 1 (one process per GPU under torchrun) the stack is
    tensor-parallel: QKV and gate|up split by weight rows - a rank keeps its query heads, its KV heads (and their
    cache) and its FFN columns -, O and down by weight columns with their partial outputs summed over peer memory
    inside the step's graph; embedding, norms and the output head are replicated.  Times are the maximum over the
    ranks; the byte counts are per rank."""
    import torch

    from georefine_b200 import serve

    cfg = serve.DecoderConfig(layers=layers, tp_world=world, tp_rank=rank)
    t0 = time.time()
    weights = serve.DecoderWeights.synthetic(cfg, dev, seed=SEED, distinct_layers=distinct_layers, max_m=128)
    build_s = time.time() - t0
    context, k = 2048, 5
    spec_rows = max(seqs) * (k + 1)
    d = serve.BatchDecoder(weights, max_rows=spec_rows if spec else max(seqs), max_slots=max(seqs), max_context=context + generate + 2 * k + 2, device=dev)
    for part in d.kv.view(-1, d.kv.shape[-3] * d.kv.shape[-2] * d.kv.shape[-1]).split(4096):
        part.uniform_(-0.5, 0.5)                                   # a synthetic context in every page
    peak, peak_kind = measured_hbm_peak()
    g = torch.Generator().manual_seed(SEED)
    line = {"metric": "decode_tokens_per_second", "unit": "tok/s", "n_gpus": world, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{cfg.layers}-layer decoder hidden={cfg.hidden} heads={cfg.heads}/{cfg.kv_heads}x{cfg.head_dim} ffn={cfg.ffn} "
                                   f"vocab={cfg.vocab}, {context}-token context, {generate} generated tokens, random token IDs",
                       "parallelism": f"tp{world}", "distinct_layers": weights.notes["distinct_layers"], "resident_format": "BXR1/window4",
                       "launch": "cuda_graph per row bucket" + (", sums of O and down over peer memory inside the graph" if world > 1 else ""),
                       "host_build_seconds": round(build_s, 1)},
            "weight_bytes_per_step": weights.streamed_bytes(), "results": {}}
    clocks = ClockSampler(dev.index or 0).start()
    for n in seqs:
        b = serve.Batcher(d)
        for _ in range(n):                                         # admit n sequences whose context is already "in the cache"
            slot = d.open_slot()
            d.ensure_pages(slot, context + generate + 2 * k + 1)
            b.active[slot] = {"pos": context, "tokens": [int(torch.randint(0, cfg.vocab, (1,), generator=g))]}
        b._dirty = True
        for _ in range(3):                                         # warm-up steps (captures the bucket's graph)
            b.step(fetch=False)
        b.sync_tokens()
        for s in b.active.values():
            s["pos"], s["tokens"] = context, s["tokens"][-1:]
        b._dirty = True
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_begin = time.monotonic()
        e0.record()
        for _ in range(generate):
            b.step(fetch=False)
        e1.record()
        torch.cuda.synchronize()
        t_end = time.monotonic()
        ms = e0.elapsed_time(e1) / generate
        if world > 1:
            import torch.distributed as dist

            slowest = torch.tensor([ms], device=dev)
            dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
            ms = float(slowest.item())
        mean_context = context + generate / 2
        kv = d.streamed_bytes([mean_context] * n)["kv"]
        res = {"ms_per_step": round(ms, 3), "tok_s": round(n / (ms * 1e-3), 1), "kv_bytes_per_step": int(kv),
               "streamed_GBps": round((kv + weights.streamed_bytes()) / (ms * 1e-3) / 1e9, 1),
               "frac_of_hbm_peak": round((kv + weights.streamed_bytes()) / (ms * 1e-3) / 1e9 / peak, 4),
               "status_word": sum(w.check_status() for w in weights.linears()) + (d.peer.check_status() if d.peer is not None else 0),
               "clocks": clocks.summary(t_begin, t_end)}
        if world > 1:
            res["per_gpu_streamed_GBps"] = res["streamed_GBps"]
            res["tokens_agree_across_ranks"] = _same_on_every_rank(d.next_token[:n], dev)
        if spec:                                              # config 3: exact speculation, k = 5, verify pass at n x 6 rows
            b.sync_tokens()
            for s in b.active.values():
                s["pos"], s["tokens"] = context, s["tokens"][-1:]
            cycles, emitted = 12, 0
            rnd = lambda: {slot: torch.randint(0, cfg.vocab, (k,), generator=g).tolist() for slot in b.active}
            b.verify(rnd())                                        # warm-up (captures the verify graph)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(cycles):
                emitted += sum(len(v) for v in b.verify(rnd()).values())
            e1.record()
            torch.cuda.synchronize()
            cyc = e0.elapsed_time(e1) / cycles
            res["speculation_k5"] = {"rows_per_verify_pass": n * (k + 1), "ms_per_cycle": round(cyc, 3), "drafts": "random token IDs",
                                     "tokens_per_cycle_per_sequence": round(emitted / cycles / n, 3),
                                     "tok_s_random_drafts": round(emitted / cycles / (cyc * 1e-3), 1),
                                     "tok_s_if_every_draft_were_accepted": round(n * (k + 1) / (cyc * 1e-3), 1),
                                     "cycle_over_plain_step": round(cyc / ms, 3)}
        line["results"][str(n)] = res
        for slot in list(b.active):
            b.retire(slot)
    clocks.stop()
    line["value"] = line["results"][str(max(seqs))]["tok_s"]
    line["peak_hbm_GBps"] = peak
    del b, d, weights
    torch.cuda.empty_cache()
    return line


def run_reference(args):
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    value, dt, info = cpu_reference_run(sample_rows=2048, steps=args.steps, warmup=min(args.warmup, 1), threads=threads)
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 2), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "hybrid-decoder linears hidden=5120, seed 1, CPU decode + F.linear at M=1,64,128 on a bounded sample"},
            "cpu_baseline": {"value": round(value, 4), "unit": UNIT, **info},
            "e2e": {"value": round(value, 4), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of CUDA graph replays")
    ap.add_argument("--layout", choices=("rans", "window", "window4"), default="window4",
                    help="resident layout of the weights: fixed 4-bit window codes (default), fixed 3-bit window codes, or "
                         "entropy-coded exponent streams")
    ap.add_argument("--skip-layouts", action="store_true", help="do not time the other two layouts after the main run")
    ap.add_argument("--skip-decode", action="store_true", help="do not time the whole-stack decode step after the main run")
    ap.add_argument("--workload", choices=("linears", "decode"), default="linears",
                    help="linears: the fused decode-GEMM step (the headline metric); decode: whole-stack tokens per second")
    ap.add_argument("--seqs", default="64,128", help="decode workload: concurrent sequences, comma separated")
    ap.add_argument("--layers", type=int, default=64, help="decode workload: decoder layers")
    ap.add_argument("--distinct-layers", type=int, default=2, help="decode workload: layers built on the host (the rest are device copies)")
    ap.add_argument("--spec", action="store_true", help="decode workload: also time exact speculation (k = 5, verify at 6 rows per sequence)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "decode":
        run_decode(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
