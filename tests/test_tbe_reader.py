"""The reader of the reference's TBE containers (georefine_b200/tbe.py) against containers made by the reference's own
encoder (fixtures: tests/golden/tbe_golden.npz, written by tests/golden/make_tbe_golden.py): every layout, both modes,
partial last tiles, every BF16 bit pattern; and the checks that refuse containers whose arrays contradict each other."""
from types import SimpleNamespace

import numpy as np
import pytest

from georefine_b200 import tbe

LAYOUT = {0: "flat64", 1: "tile8x8", 2: "mma16"}
CASES = ["weights_mma16", "weights_flat64_ragged", "weights_mma16_ragged", "weights_tile8x8", "every_pattern_mma16",
         "every_pattern_flat64", "sparse_mma16", "constant_flat64"]


@pytest.fixture(scope="module")
def fixtures():
    from pathlib import Path

    with np.load(Path(__file__).resolve().parent / "golden" / "tbe_golden.npz") as z:
        return {k: z[k] for k in z.files}


def container(fixtures, name, **changes):
    rows, cols, layout, mode, base, tiles, escapes, superblock = (int(v) for v in fixtures[name + ".meta"])
    c = SimpleNamespace(shape=(rows, cols), layout=LAYOUT[layout], mode=mode, base=base, tiles=tiles, escapes=escapes,
                        planes=fixtures[name + ".planes"].copy(), smb=fixtures[name + ".smb"].copy(), esc=fixtures[name + ".esc"].copy(),
                        sbbase=fixtures[name + ".sbbase"].copy(), superblock=superblock)
    for k, v in changes.items():
        setattr(c, k, v)
    return c


@pytest.mark.parametrize("name", CASES)
def test_reader_reproduces_the_words_bit_for_bit(fixtures, name):
    words = tbe.decode_words(container(fixtures, name))
    assert words.dtype == np.uint16 and np.array_equal(words, fixtures[name + ".words"])


def test_torch_tensors_and_64_bit_planes_are_accepted(fixtures):
    import torch

    c = container(fixtures, "weights_mma16")
    c.planes = torch.from_numpy(c.planes.astype(np.int64))
    c.smb, c.esc = torch.from_numpy(c.smb), torch.from_numpy(c.esc)
    c.sbbase = None                                            # the per-group counts are optional
    assert np.array_equal(tbe.decode_words(c), fixtures["weights_mma16.words"])


def test_modes_are_both_covered(fixtures):
    assert int(fixtures["sparse_mma16.meta"][3]) == 1 and int(fixtures["weights_mma16.meta"][3]) == 0
    assert int(fixtures["every_pattern_mma16.meta"][6]) > 60000          # nearly every weight escapes there


def test_contradicting_containers_are_refused(fixtures):
    name = "weights_flat64_ragged"
    for changes in ({"layout": "rows"}, {"mode": 2}, {"tiles": 30}, {"escapes": 52}, {"shape": (37, 54)},
                    {"esc": fixtures[name + ".esc"][:-1]}, {"smb": fixtures[name + ".smb"][:-64]}, {"base": 300},
                    {"sbbase": fixtures[name + ".sbbase"] + 1}):
        with pytest.raises(tbe.TbeFormatError):
            tbe.decode_words(container(fixtures, name, **changes))
    flipped = container(fixtures, name)
    flipped.planes[3, 0, 0] ^= 1 << 5                          # one code bit: an escape appears or disappears, or a
    try:                                                       # window exponent changes - never silently the same words
        assert not np.array_equal(tbe.decode_words(flipped), fixtures[name + ".words"])
    except tbe.TbeFormatError:
        pass
    with pytest.raises(tbe.TbeFormatError):
        tbe.decode_words(container(fixtures, "weights_tile8x8", shape=(60, 76), tiles=72))   # 8 x 8 tiles need multiples of 8
    high = container(fixtures, "constant_flat64", base=250)    # code 7 would address exponent 256
    high.planes[:] = 0xFFFFFFFF
    with pytest.raises(tbe.TbeFormatError):
        tbe.decode_words(high)


@pytest.mark.gpu
def test_resident_image_from_a_tbe_container(fixtures):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    dev = torch.device("cuda:0")
    w = tbe.resident_from_tbe(container(fixtures, "weights_mma16"), dev, verify=True)
    words = fixtures["weights_mma16.words"]
    assert np.array_equal(w.decode().view(torch.int16).cpu().numpy().view(np.uint16), words)
    x = torch.randn(3, w.K).to(torch.bfloat16).to(dev)
    y = w.linear(x)
    ref = x.float() @ torch.from_numpy(words.view(np.int16)).to(dev).view(torch.bfloat16).float().T
    assert w.check_status() == 0 and ((y.float() - ref).abs().max() / ref.abs().max()).item() <= 1e-2


def test_bundle_directory_is_read_tensor_by_tensor(fixtures, tmp_path):
    """A bundle as the reference writes it: manifest.json + tbe_tensors.safetensors (written here by hand, 64-bit planes
    as its encoder returns them); raw entries are passed over, rank-3 entries use their coded 2-D shape."""
    import json
    import struct

    names = ["weights_mma16", "sparse_mma16", "weights_tile8x8"]
    header, payload, tensors = {}, b"", []
    for name in names:
        c = container(fixtures, name)
        parts = {"planes": c.planes.astype("<i8"), "smb": c.smb, "esc": c.esc, "sbbase": c.sbbase.astype("<i8")}
        for part, a in parts.items():
            raw = np.ascontiguousarray(a).tobytes()
            header[f"model.{name}.weight.{part}"] = {"dtype": "I64" if a.dtype.itemsize == 8 else "U8", "shape": list(a.shape),
                                                      "data_offsets": [len(payload), len(payload) + len(raw)]}
            payload += raw
        shape = [2, c.shape[0] // 2, c.shape[1]] if name == "weights_mma16" else list(c.shape)     # an expert stack
        tensors.append({"name": f"model.{name}.weight", "kind": "tbe", "shape": shape, "coded_shape": list(c.shape), "layout": c.layout,
                        "mode": c.mode, "base": c.base, "tiles": c.tiles, "escapes": c.escapes, "superblock": c.superblock})
    tensors.append({"name": "model.norm.weight", "kind": "raw", "shape": [8]})
    text = json.dumps(header).encode()
    (tmp_path / "tbe_tensors.safetensors").write_bytes(struct.pack("<Q", len(text)) + text + payload)
    (tmp_path / "manifest.json").write_text(json.dumps({"schema": "georefine.tbe_transcode_manifest.v1", "tensors": tensors}))
    seen = []
    for c in tbe.iter_bundle(tmp_path):
        short = c.name.split(".")[1]
        assert np.array_equal(tbe.decode_words(c), fixtures[short + ".words"])
        seen.append((short, c.full_shape))
    assert [s for s, _ in seen] == names and seen[0][1] == (2, 48, 160)
    broken = json.loads((tmp_path / "manifest.json").read_text())
    broken["tensors"][1]["name"] = "model.absent.weight"
    (tmp_path / "manifest.json").write_text(json.dumps(broken))
    with pytest.raises(tbe.TbeFormatError):
        list(tbe.iter_bundle(tmp_path))
