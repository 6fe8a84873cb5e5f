"""Writes tests/golden/tbe_golden.npz: TBE containers made by the REFERENCE's own encoder
(context-runtime/glc_loader/tbe_container.py encode_tbe), with the words they were made from.

Run where a checkout of the reference is reachable: REFERENCE_ROOT=<checkout> python tests/golden/make_tbe_golden.py
The fixtures are committed; nothing at test time needs the reference."""
import os
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import bcx_oracle  # noqa: E402  (synthetic weights with the benchmark's distribution)

ref = os.environ.get("REFERENCE_ROOT") or str(ROOT.parent / "reference")
sys.path.insert(0, str(Path(ref) / "context-runtime"))
from glc_loader import tbe_container as tbe  # noqa: E402


def words_cases():
    rng = np.random.default_rng(7)
    every = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    sparse = bcx_oracle.synthetic_weight_words(40, 72, 3).copy()
    sparse[rng.random(sparse.shape) < 0.6] = 0                       # many zeros: the six-exponent mode with a zero code
    return {
        "weights_mma16": (bcx_oracle.synthetic_weight_words(96, 160, 1), "mma16"),
        "weights_flat64_ragged": (bcx_oracle.synthetic_weight_words(37, 53, 2), "flat64"),   # 1961 weights: a partial last tile
        "weights_mma16_ragged": (bcx_oracle.synthetic_weight_words(21, 45, 4), "mma16"),
        "weights_tile8x8": (bcx_oracle.synthetic_weight_words(64, 72, 5), "tile8x8"),
        "every_pattern_mma16": (every, "mma16"),
        "every_pattern_flat64": (every, "flat64"),
        "sparse_mma16": (sparse, "mma16"),
        "constant_flat64": (np.full((8, 24), 0x3F80, dtype=np.uint16), "flat64"),
    }


def main():
    out = {}
    for name, (words, layout) in words_cases().items():
        w = torch.from_numpy(words.view(np.int16).copy()).view(torch.bfloat16)
        c = tbe.encode_tbe(w, layout=layout)
        assert tbe.tbe_certify(c, w)["bitwise_ok"]
        out[name + ".words"] = words
        out[name + ".planes"] = c.planes.numpy().astype(np.uint32)
        out[name + ".smb"] = c.smb.numpy()
        out[name + ".esc"] = c.esc.numpy()
        out[name + ".sbbase"] = c.sbbase.numpy().astype(np.uint32)
        out[name + ".meta"] = np.array([c.shape[0], c.shape[1], LAYOUT_ID[layout], c.mode, c.base, c.tiles, c.escapes, c.superblock], dtype=np.int64)
        print(name, layout, "mode", c.mode, "base", c.base, "tiles", c.tiles, "escapes", c.escapes)
    np.savez_compressed(ROOT / "tests" / "golden" / "tbe_golden.npz", **out)


LAYOUT_ID = {"flat64": 0, "tile8x8": 1, "mma16": 2}

if __name__ == "__main__":
    main()
