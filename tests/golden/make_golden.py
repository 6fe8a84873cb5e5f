"""Regenerates tests/golden/bctx_golden.npz from the REFERENCE implementation.

Run where the reference checkout is available (path as argument, or $REFERENCE_ROOT):

    python tests/golden/make_golden.py [reference_root]

Frames come from the reference's own Python codec (``bitexact_context_codec.encode``), which compiles its
C++ coder into a scratch directory given by BITEXACT_CONTEXT_CACHE_DIR.  Restart points come from the
reference's ``bcx_checkpoint`` compiled by ``oracle/Makefile`` into ``oracle/_ref`` (its Python wrapper
builds beside its sources, which are read-only here).  The inputs mirror the reference's own tests:

  * tests/test_bitexact_context_gpu.py:9-29          special BF16 words 64x67, uniform 13x17 (raw mode)
  * tests/test_bitexact_context_gpu_index.py:75-137  9x17 random words, nr=4, nc=3, both stream kinds
  * context-runtime/tests/test_compact_rans_lookup.py:7-50  all words / constant / sparse
  * synthetic benchmark weights (N(0,0.02) x LogNormal(0,0.25) rows) and a frame whose residual is
    cheaper as a conditional stream (mode 128)

The file is a few hundred KB; large frames are stored as SHA-256 only.
"""
from __future__ import annotations

import hashlib
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def main():
    named = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("REFERENCE_ROOT")
    if not named:
        raise SystemExit("usage: make_golden.py <checkout of the reference project>   (or set REFERENCE_ROOT)")
    ref_root = Path(named)
    os.environ["BITEXACT_CONTEXT_CACHE_DIR"] = tempfile.mkdtemp(prefix="bctx-golden-")
    sys.path.insert(0, str(ref_root / "context-runtime"))
    from georefine_context_runtime import bitexact_context_codec as ref  # noqa: E402
    from oracle import bcx_oracle as orc  # noqa: E402

    orc.build()
    rlib = orc.Coder("ref")
    out = {}

    def put_frame(tag, words, nr, nc, strides=()):
        frame = ref.encode(words, row_classes=nr, col_classes=nc)
        assert np.array_equal(ref.decode(frame), words)
        out[tag + ".words"] = words
        out[tag + ".frame"] = np.frombuffer(frame, dtype=np.uint8)
        out[tag + ".classes"] = np.array([nr, nc], dtype=np.int64)
        f = orc.parse_frame(frame)
        for stride in strides:
            if f["mode"] == 1:
                continue
            st, of, main = rlib.checkpoint(f["main_stream"], f["main_freq"], f["rows"], f["columns"], *f["shape"],
                                           f["nr"], f["nc"], 0, stride)
            out[f"{tag}.s{stride}.main_states"] = st
            out[f"{tag}.s{stride}.main_offsets"] = of
            if f["mode"] == 128:
                st, of, _ = rlib.checkpoint(f["residual_stream"], f["residual_freq"], f["rows"], f["columns"],
                                            *f["shape"], f["nr"], f["nc"], 1, stride, main)
                out[f"{tag}.s{stride}.residual_states"] = st
                out[f"{tag}.s{stride}.residual_offsets"] = of
        return frame

    special = np.resize(np.array([0, 0x8000, 0x7F80, 0xFF80, 0x7FC1, 0xFFE5, 1, 0x8001], dtype=np.uint16), (64, 67))
    put_frame("special", special, 16, 4, strides=(1, 7, 128, 1024))
    put_frame("uniform13x17", np.random.default_rng(9).integers(0, 65536, (13, 17), dtype=np.uint16), 16, 4)

    # raw C-ABI cases of the index test (nc = 3 is legal at the ABI although no frame uses it)
    for kind in (0, 1):
        rng = np.random.default_rng(701 + kind)
        rows_n, cols_n, nr, nc = 9, 17, 4, 3
        vals = rng.integers(0, 65536, size=rows_n * cols_n, dtype=np.uint16).reshape(rows_n, cols_n)
        rc = (np.arange(rows_n, dtype=np.uint8) % nr).copy()
        cc = (np.arange(cols_n, dtype=np.uint8) % nc).copy()
        freq, stream = rlib.encode_stream(vals, rc, cc, nr, nc, kind)
        tag = f"abi9x17.k{kind}"
        out[tag + ".vals"] = vals
        out[tag + ".freq"] = freq
        out[tag + ".stream"] = np.frombuffer(stream, dtype=np.uint8)
        resctx = orc.split_words(vals)[0].ravel() if kind else None
        for stride in (1, 7, 19, 128):
            st, of, sym = rlib.checkpoint(stream, freq, rc, cc, rows_n, cols_n, nr, nc, kind, stride, resctx)
            out[f"{tag}.s{stride}.states"] = st
            out[f"{tag}.s{stride}.offsets"] = of
            out[f"{tag}.symbols"] = sym

    # distributions of the compact-lookup test: frame digests for every class configuration
    all_words = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    sparse = all_words.copy()
    sparse[:240] = 0x3F80
    dists = {"all_words": all_words, "constant": np.full((64, 128), 0x3F80, dtype=np.uint16), "sparse": sparse}
    for name, words in dists.items():
        for nr, nc in ((1, 1), (4, 4), (16, 4), (64, 16)):
            frame = ref.encode(words, row_classes=nr, col_classes=nc)
            assert np.array_equal(ref.decode(frame), words)
            out[f"dist.{name}.{nr}x{nc}.frame_sha256"] = np.frombuffer(hashlib.sha256(frame).digest(), dtype=np.uint8)
            out[f"dist.{name}.{nr}x{nc}.mode_len"] = np.array([frame[5], len(frame)], dtype=np.int64)
    put_frame("constant", dists["constant"], 16, 4, strides=(128, 1024))

    # the benchmark's weight distribution, small
    w = orc.synthetic_weight_words(64, 512, 0)
    put_frame("synthetic64x512", w, 16, 4, strides=(128, 1024))
    put_frame("synthetic48x320.r4c1", orc.synthetic_weight_words(48, 320, 3), 4, 1, strides=(1024,))

    # a frame where the conditional residual stream beats raw6: the low mantissa bits follow the exponent
    rng = np.random.default_rng(2024)
    expo = rng.integers(100, 132, size=(96, 160)).astype(np.uint16)
    low = ((expo * 7) % 32).astype(np.uint16)
    flip = rng.random((96, 160)) < 0.05
    low = np.where(flip, rng.integers(0, 32, size=low.shape).astype(np.uint16), low)
    cond_words = ((expo << 7) | (rng.integers(0, 4, size=expo.shape).astype(np.uint16) << 5) | low).astype(np.uint16)
    frame = put_frame("conditional96x160", cond_words, 4, 4, strides=(1, 100, 1024))
    assert frame[5] == 128, "expected the conditional residual mode"

    path = Path(__file__).with_name("bctx_golden.npz")
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
