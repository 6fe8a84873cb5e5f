"""Reading the reference's TBE containers.

The reference's fast linears stream weights from its TBE container (``context-runtime/glc_loader/tbe_container.py:11-40``
describes it; ``encode_tbe`` / ``decode_tbe`` at ``:259-404``): per 2-D BF16 tensor a 3-bit code per weight over one
exponent window of the whole tensor, in tiles of 64 weights (three 64-bit bit planes per tile), the sign and mantissa
byte of every weight verbatim in tile order, and the raw exponents of the weights outside the window ("escapes") in tile
order.  This library keeps weights in another resident layout (a window per ROW, 128 x 128 chunk blobs: ``csrc/
bxr_format.h``), built at load time from decoded words; this module is the bridge for a deployment that holds TBE
bundles rather than BCTX frames: it turns a container back into the tensor's BF16 words, exactly, on the host, with
numpy, and ``resident_from_tbe`` builds the resident image from them.

A container is any object with the fields of the reference's ``TBETensor``: ``shape``, ``layout`` ("flat64", "tile8x8" or
"mma16"), ``mode`` (0: codes 1..7 address seven exponents from ``base``; 1: codes 1..6 address six, code 7 is exponent
0), ``base``, ``tiles``, ``escapes``, ``planes`` [tiles, 3, 2] (32-bit words in 32- or 64-bit integers), ``smb``
[tiles * 64] bytes, ``esc`` [escapes] bytes and, optionally, ``sbbase`` / ``superblock`` (escapes in front of every
group of tiles: redundant for a front-to-back decode, checked when present).  Arrays may be numpy arrays or torch
tensors.
"""
from __future__ import annotations

import numpy as np

TILE = 64
LAYOUTS = ("flat64", "tile8x8", "mma16")


class TbeFormatError(ValueError):
    """The container's arrays contradict its own description."""


def _array(value, dtype):
    if hasattr(value, "detach"):            # a torch tensor
        value = value.detach().cpu().numpy()
    return np.ascontiguousarray(value).astype(dtype, copy=False)


def _place_in_tile(layout: str) -> np.ndarray:
    """place[j] = where, among a tile's 64 stored positions, the j-th weight of the tile (in reading order) sits."""
    stored = np.arange(TILE)
    if layout != "mma16":
        return stored
    # stored position p holds weight 16 * ((p >> 2) & 3) + 2 * (p >> 4) + (0, 1, 8, 9)[p & 3]: the 16 weights of one lane
    # of a 16 x 8 matrix fragment end up side by side
    weight_at = 16 * ((stored >> 2) & 3) + 2 * (stored >> 4) + np.array([0, 1, 8, 9])[stored & 3]
    place = np.empty(TILE, dtype=np.int64)
    place[weight_at] = stored
    return place


def decode_words(container) -> np.ndarray:
    """The tensor's BF16 words, uint16 [rows, cols], bit for bit (every NaN payload, both zeros, denormals: the
    container stores the three fields of a word, not a value)."""
    rows, cols = (int(v) for v in container.shape)
    layout, mode, base = str(container.layout), int(container.mode), int(container.base)
    if layout not in LAYOUTS or mode not in (0, 1) or rows <= 0 or cols <= 0 or not 0 <= base <= 255:
        raise TbeFormatError("unknown layout or mode, empty shape, or exponent base outside a byte")
    if layout == "tile8x8":
        if rows % 8 or cols % 8:
            raise TbeFormatError("the 8 x 8 layout needs both dimensions divisible by 8")
        tiles = (rows // 8) * (cols // 8)
    else:
        tiles = -(-rows * cols // TILE)
    planes = _array(container.planes, np.int64)
    sign_mantissa = _array(container.smb, np.uint8)
    raw = _array(container.esc, np.uint8)
    if int(container.tiles) != tiles or planes.shape != (tiles, 3, 2) or sign_mantissa.shape != (tiles * TILE,):
        raise TbeFormatError("tile count or array shapes do not fit the tensor's shape")
    if planes.min(initial=0) < 0 or planes.max(initial=0) > 0xFFFFFFFF:
        raise TbeFormatError("a plane word does not fit 32 bits")

    # codes: bit b of the code of stored position j of tile t is bit j % 32 of planes[t, b, j // 32]
    bit = np.arange(32, dtype=np.int64)
    code = np.zeros((tiles, 2, 32), dtype=np.int64)
    for b in range(3):
        code |= ((planes[:, b, :, None] >> bit) & 1) << b
    code = code.reshape(tiles, TILE)

    exponent = code - 1 + base
    if mode == 1:
        exponent[code == 7] = 0
    outside = code == 0                      # escapes: raw exponents, tile after tile, stored positions ascending
    if int(outside.sum()) != raw.size or int(container.escapes) != raw.size:
        raise TbeFormatError("the number of escape codes differs from the number of stored exponents")
    exponent[outside] = raw
    if exponent.max(initial=0) > 255:
        raise TbeFormatError("a code addresses an exponent beyond 255")
    counts = getattr(container, "sbbase", None)
    if counts is not None:
        group = int(getattr(container, "superblock", 32))
        counts = _array(counts, np.int64)
        per_tile = outside.sum(axis=1)
        want = np.concatenate([[0], np.cumsum(per_tile)])[0:tiles:group] if tiles else np.zeros(0, dtype=np.int64)
        if group <= 0 or counts.shape != want.shape or not np.array_equal(counts, want):
            raise TbeFormatError("the escape counts per group of tiles do not match the codes")

    sm = sign_mantissa.reshape(tiles, TILE).astype(np.int64)
    stored_words = ((sm & 0x80) << 8) | (exponent << 7) | (sm & 0x7F)
    words = stored_words[:, _place_in_tile(layout)]          # back to reading order inside every tile
    if layout == "tile8x8":
        blocks = words.reshape(rows // 8, cols // 8, 8, 8).transpose(0, 2, 1, 3)
        return np.ascontiguousarray(blocks).reshape(rows, cols).astype(np.uint16)
    flat = words.reshape(-1)
    tail = flat[rows * cols:]
    if tail.size and (np.any(code.reshape(-1)[_tail_positions(layout, tiles, rows * cols)] != 1)):
        raise TbeFormatError("the padding of the last tile is not coded as the reference codes it")
    return flat[:rows * cols].reshape(rows, cols).astype(np.uint16)


def _tail_positions(layout: str, tiles: int, used: int) -> np.ndarray:
    """Stored positions (flat index into [tiles, 64]) of the padding weights of the last tile."""
    first_pad = used - (tiles - 1) * TILE
    return (tiles - 1) * TILE + _place_in_tile(layout)[first_pad:]


def resident_from_tbe(container, device, **kwargs):
    """A ``ResidentWeight`` (this library's fused linear) from a TBE container: decode on the host, re-code into the
    resident layout.  ``kwargs`` go to ``ResidentWeight.from_words`` (``layout``, ``workers``, ``max_m``, ``tune``)."""
    from .resident import ResidentWeight

    return ResidentWeight.from_words(decode_words(container), device, **kwargs)


# ---------------------------------------------------------------------------------------------- bundles on disk
_STORED = {"I32": np.dtype("<i4"), "I64": np.dtype("<i8"), "U8": np.dtype("u1"), "U32": np.dtype("<u4"), "U64": np.dtype("<u8")}


class BundleContainer:
    """One coded tensor of a bundle: the manifest entry plus its four arrays, read on demand."""

    def __init__(self, entry, arrays):
        coded = entry.get("coded_shape") or entry["shape"]          # the 2-D view the encoder saw (expert stacks are rank 3)
        if len(coded) != 2:
            raise TbeFormatError(f"{entry['name']}: the coded shape is not two-dimensional")
        self.name = str(entry["name"])
        self.shape = (int(coded[0]), int(coded[1]))
        self.full_shape = tuple(int(d) for d in entry["shape"])
        self.layout, self.mode, self.base = str(entry["layout"]), int(entry["mode"]), int(entry["base"])
        self.tiles, self.escapes, self.superblock = int(entry["tiles"]), int(entry["escapes"]), int(entry["superblock"])
        self.planes, self.smb, self.esc, self.sbbase = arrays


def iter_bundle(directory):
    """The coded tensors of a TBE bundle directory (``manifest.json`` with one entry per tensor - ``kind`` "tbe" for the
    coded ones, with ``name``, ``shape``, ``coded_shape``, ``layout``, ``mode``, ``base``, ``tiles``, ``escapes``,
    ``superblock`` - and ``tbe_tensors.safetensors`` holding ``<name>.planes``, ``.smb``, ``.esc``, ``.sbbase``; the layout
    the reference's ``glc_loader/tbe_artifact.py:511-540`` reads).  Yields ``BundleContainer`` objects, one tensor in
    memory at a time; ``decode_words`` / ``resident_from_tbe`` take them as they are."""
    import json
    from pathlib import Path

    from .package import _read_range, read_shard_header

    directory = Path(directory)
    manifest = json.loads((directory / "manifest.json").read_text())
    blob = directory / "tbe_tensors.safetensors"
    _, header, data_at = read_shard_header(blob)
    for entry in manifest["tensors"]:
        if entry.get("kind") != "tbe":
            continue
        arrays = []
        for part in ("planes", "smb", "esc", "sbbase"):
            stored = header.get(f"{entry['name']}.{part}")
            if stored is None or stored["dtype"] not in _STORED:
                raise TbeFormatError(f"{entry['name']}.{part} is missing from the bundle or has an unexpected type")
            begin, end = stored["data_offsets"]
            a = np.frombuffer(_read_range(blob, data_at + begin, data_at + end), dtype=_STORED[stored["dtype"]])
            arrays.append(a.reshape([int(d) for d in stored["shape"]]))
        yield BundleContainer(entry, arrays)
