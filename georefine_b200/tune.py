"""Per-shape tune records for the fused linears: which resident layout and how many persistent CTAs a weight of a given
shape is built for, chosen by measured time on the GPU at hand.

Counterpart of the reference's per-shape tune JSON (``glc_serve/tbe_desc.py:160-215`` ``tune_tbe_per_m``,
``glc_serve/fastdec.py:283-285`` ``load_tune``, ``glc_serve/tunes/fastdec_sm120.json``; ``untuned_config`` for a shape
the record does not know).  One difference follows from the arithmetic: the reference's candidates are bitwise
equivalent, so it may pick a different one per batch size; here the worker count fixes the split of K and with it the
order of additions, so a choice is made per SHAPE only - every batch size of a weight then runs the same image and rows
stay bitwise independent of M.  The figure of merit is the sum of the times over the batch sizes asked for.

Timing follows the reference's practice (``glc_serve/tbe_desc.py:160-175``): CUDA events around back-to-back launches in
one stream, rotating over enough copies of the weight that the working set exceeds the L2.

    python -m georefine_b200.tune --shape 34816x5120 --m 1,64,128 --out tune.json      # one shape, default candidates
    python -m georefine_b200.tune --shape 5120x5120 --m 128 --layout window4 --workers 120 --reps 3   # one launch kind, a few launches
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np

from . import resident

L2_BYTES = 126 << 20
ROTATION_BYTES = 400_000_000      # working set of one rotation: more than three times the L2
SCHEMA = "georefine_b200.tune.v1"


def synthetic_words(rows: int, cols: int, seed: int = 1):
    """BF16 bit patterns of N(0, 0.02) weights with a LogNormal(0, 0.25) scale per row: the distribution tune records
    and benchmarks are taken on when no checkpoint is at hand."""
    import torch

    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * 0.02
    w = w * torch.exp(0.25 * torch.randn(rows, 1, generator=g))
    return w.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def untuned_config(rows: int, cols: int, sms: int):
    """(layout, workers) for a shape no record covers."""
    return resident.DEFAULT_LAYOUT, resident.default_workers(rows, cols, sms)


def worker_candidates(rows: int, cols: int, sms: int):
    """One CTA per SM, and - for weights with fewer 128-row blocks than SMs - the multiples of the row-block count below
    it (every row block is then cut into the same number of whole CTAs)."""
    row_blocks = -(-rows // 128)
    out = {sms}
    if 0 < row_blocks < sms:
        for mult in range(1, sms // row_blocks + 1):
            if row_blocks * mult >= sms // 2:
                out.add(row_blocks * mult)
    return sorted(out)


def rotation_us(launch, copies: int, reps: int) -> float:
    """Mean microseconds of launch(i % copies), issued back to back in the current stream after a warm-up round."""
    import torch

    for i in range(max(3, copies)):
        launch(i % copies)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(reps):
        launch(i % copies)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps * 1e3


def copies_for(nbytes: int) -> int:
    return max(2, -(-ROTATION_BYTES // max(int(nbytes), 1)))


def chained_copies(weight: "resident.ResidentWeight"):
    """Enough copies of the image to exceed the L2 in one rotation, each told that the next one follows it (the hint a
    serving engine gives with ``then``)."""
    copies = [weight.clone() for _ in range(copies_for(weight.coded_bytes))]
    for a, b in zip(copies, copies[1:] + copies[:1]):
        a.then(b)
    return copies


def time_weight(weight: "resident.ResidentWeight", m: int, *, reps: int | None = None, entry: str = "gemm", copies=None) -> float:
    """Microseconds per fused launch at batch m, in a stream of such launches over rotating copies of the image."""
    import torch

    images = copies if copies is not None else chained_copies(weight)
    x = torch.randn(m, weight.K, device=weight.device).to(torch.bfloat16)
    y = torch.empty(m, weight.N, device=weight.device, dtype=torch.bfloat16)
    reps = reps or max(20, int(2e9 // weight.coded_bytes))
    return rotation_us(lambda i: getattr(images[i], entry)(x, y), len(images), reps)


def tune_shape(rows: int, cols: int, device, *, ms=(1, 64, 128), layouts=(resident.DEFAULT_LAYOUT,), workers=None, words=None,
               reps: int | None = None, log=print):
    """Times every (layout, workers) candidate of one shape at every batch size of ``ms``.  Returns
    {"layout", "workers", "us": {"layout,workers,M": microseconds}, "coded_bytes", "coded_GBps": {M: ...}}."""
    import torch

    sms = resident.sm_count(device)
    words = synthetic_words(rows, cols) if words is None else words
    table, best = {}, None
    for layout in layouts:
        for w in (worker_candidates(rows, cols, sms) if workers is None else workers):
            res = resident.ResidentWeight.from_words(words, device, max_m=max(ms), workers=w, layout=layout, verify=False)
            built = {v: k for k, v in resident.LAYOUTS.items()}[res.mode]
            copies = chained_copies(res)
            total = 0.0
            for m in ms:
                us = time_weight(res, m, reps=reps, copies=copies)
                table[f"{layout},{w},M{m}"] = round(us, 2)
                total += us
            if res.check_status() or any(c.check_status() for c in copies):
                raise RuntimeError(f"status word set while timing {rows}x{cols} {layout} workers={w}")
            if best is None or total < best[0]:
                best = (total, layout, w, built, res.coded_bytes)
            log(f"[tune] {rows}x{cols} {layout} (built {built}) workers {w}: " + " ".join(f"M{m}:{table[f'{layout},{w},M{m}']}us" for m in ms))
            del res, copies
            torch.cuda.empty_cache()
    _, layout, w, built, coded = best
    return {"layout": layout, "built": built, "workers": w, "us": table, "coded_bytes": coded,
            "coded_GBps": {str(m): round(coded / table[f"{layout},{w},M{m}"] / 1e3, 1) for m in ms}}


def tune_shapes(shapes, device, **kw):
    """A tune record for several shapes: {"schema", "device", "sms", "layout_version", "config": {"NxK": [layout, workers]},
    "detail": {...}}; ``save_tune`` writes it, ``load_tune`` reads the ``config`` part back."""
    import torch

    from . import _native

    detail = {f"{n}x{k}": tune_shape(n, k, device, **kw) for n, k in shapes}
    return {"schema": SCHEMA, "device": torch.cuda.get_device_name(device), "sms": resident.sm_count(device),
            "layout_version": int(_native.lib().bxr_layout_version()),
            "config": {key: [d["layout"], d["workers"]] for key, d in detail.items()}, "detail": detail}


def save_tune(record, path) -> None:
    Path(path).write_text(json.dumps(record, indent=1, sort_keys=True))


def load_tune(path):
    """{(N, K): (layout, workers)} from a record written by ``save_tune``.  Refuses a record of another schema."""
    record = json.loads(Path(path).read_text())
    if record.get("schema") != SCHEMA:
        raise ValueError(f"{path}: not a {SCHEMA} record")
    out = {}
    for key, (layout, workers) in record["config"].items():
        n, k = (int(v) for v in key.lower().split("x"))
        if layout not in resident.LAYOUTS or int(workers) < 1:
            raise ValueError(f"{path}: bad entry for {key}")
        out[(n, k)] = (layout, int(workers))
    return out


def config_for(rows: int, cols: int, sms: int, tune=None):
    """(layout, workers) for a shape: the record's entry if it has one, else ``untuned_config``."""
    if tune and (rows, cols) in tune:
        return tune[(rows, cols)]
    return untuned_config(rows, cols, sms)


def main(argv=None):
    ap = argparse.ArgumentParser(description="time the fused linear of one shape; choose its layout and worker count")
    ap.add_argument("--shape", required=True, action="append", help="NxK (weight rows x columns); may be given several times")
    ap.add_argument("--m", default="1,64,128", help="batch sizes, comma separated")
    ap.add_argument("--layout", default=resident.DEFAULT_LAYOUT, help="layouts to try, comma separated (window4, window, rans)")
    ap.add_argument("--workers", default=None, help="worker counts to try, comma separated (default: the shape's candidates)")
    ap.add_argument("--reps", type=int, default=None, help="timed launches per candidate and batch size (default: ~2 GB of traffic)")
    ap.add_argument("--out", default=None, help="write the record here as JSON")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("tuning needs a CUDA device")
    shapes = [tuple(int(v) for v in s.lower().split("x")) for s in args.shape]
    record = tune_shapes(shapes, torch.device(args.device), ms=tuple(int(v) for v in args.m.split(",")),
                         layouts=tuple(args.layout.split(",")), reps=args.reps,
                         workers=None if args.workers is None else [int(v) for v in args.workers.split(",")])
    if args.out:
        save_tune(record, args.out)
    print(json.dumps(record))


if __name__ == "__main__":
    main()
