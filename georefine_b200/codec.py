"""BCTX v1 frame codec: the host half of the path, with the reference module's public names.

Mirrors ``context-runtime/georefine_context_runtime/bitexact_context_codec.py`` (``encode`` :354, ``decode``
:377, ``CodecError`` :26, ``HEADER`` :19, ``_inflate_exact`` :328, ``_labels`` :183): same frame bytes, same
errors.  The integer work runs in libgeorefine_b200.so through the ``bcx_*`` C ABI.  Per-call decoding on the
GPU lives in ``georefine_b200.gpu``; this module is what an offline encoder or a loader calls once.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import struct
import zlib

import numpy as np

from . import _native

MAGIC = b"BCTX"
VERSION = 1
HEADER = struct.Struct("<4sBBBBIIQQQQ32s")
MAX_WORDS = 0xFFFFFFFF
ROWS = {1, 4, 16, 64}
COLS = {1, 4, 16}


class CodecError(ValueError):
    """Invalid input or malformed frame."""


def _lib():
    return _native.lib()


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def _input(words):
    a = np.asarray(words)
    if a.ndim != 2 or a.dtype.kind not in "ui" or a.dtype.itemsize != 2:
        raise CodecError("expected a 2D uint16 word array")
    if not all(a.shape) or a.size > MAX_WORDS:
        raise CodecError("invalid or oversized geometry")
    if a.dtype.kind == "i" and (np.any(a < 0) or np.any(a > 65535)):
        raise CodecError("word outside uint16 range")
    return np.ascontiguousarray(a, dtype="<u2")


def _labels(a, nr, nc):
    """Quantile class of every row and column by the sum of magnitudes (word & 0x7FFF), computed in row
    slabs so that very large tensors never materialise a second full-size array."""
    rows, cols = a.shape
    rs = np.zeros(rows, dtype=np.uint64)
    cs = np.zeros(cols, dtype=np.uint64)
    slab = max(1, min(rows, (1 << 20) // cols))
    for lo in range(0, rows, slab):
        mag = a[lo:lo + slab] & np.uint16(0x7FFF)
        rs[lo:lo + len(mag)] = mag.sum(axis=1, dtype=np.uint64)
        cs += mag.sum(axis=0, dtype=np.uint64)

    def classes(v, k):
        order = np.argsort(v, kind="stable")
        out = np.empty(len(v), dtype=np.uint8)
        out[order] = (np.arange(len(v), dtype=np.uint64) * np.uint64(k) // np.uint64(len(v))).astype(np.uint8)
        return out

    return classes(rs, nr), classes(cs, nc)


def _dims(kind, nr, nc):
    return (64, 1024) if kind else (1024, nr * nc)


def _encode_kind(lib, a, rc, cc, nr, nc, kind):
    vocab, nctx = _dims(kind, nr, nc)
    freq = np.zeros(nctx * vocab, dtype="<u4")
    rc = np.ascontiguousarray(rc, dtype=np.uint8)
    cc = np.ascontiguousarray(cc, dtype=np.uint8)
    ptr, length = _native.U8P(), ctypes.c_size_t()
    status = lib.bcx_encode(_p(a, ctypes.c_uint16), a.size, a.shape[0], a.shape[1], _p(rc, ctypes.c_uint8),
                            _p(cc, ctypes.c_uint8), nr, nc, kind, _p(freq, ctypes.c_uint32), ctypes.byref(ptr),
                            ctypes.byref(length))
    if status:
        raise CodecError(f"rANS encode failed ({status})")
    try:
        stream = ctypes.string_at(ptr, length.value)
    finally:
        lib.bcx_free(ptr)
    return freq.tobytes(), stream


def _frequencies_kind(lib, a, rc, cc, nr, nc, kind):
    vocab, nctx = _dims(kind, nr, nc)
    freq = np.zeros(nctx * vocab, dtype="<u4")
    rc = np.ascontiguousarray(rc, dtype=np.uint8)
    cc = np.ascontiguousarray(cc, dtype=np.uint8)
    status = lib.bcx_frequencies(_p(a, ctypes.c_uint16), a.size, a.shape[0], a.shape[1], _p(rc, ctypes.c_uint8),
                                 _p(cc, ctypes.c_uint8), nr, nc, kind, _p(freq, ctypes.c_uint32))
    if status:
        raise CodecError(f"frequency-only encode failed ({status})")
    return freq.tobytes()


def _decode_kind(lib, stream, freq, rc, cc, rows, cols, nr, nc, kind, main=None):
    choice = os.environ.get("GEOREFINE_CONTEXT_COMPACT_RANS")
    if choice not in (None, "0", "1"):
        raise CodecError("GEOREFINE_CONTEXT_COMPACT_RANS must be 0 or 1")
    decoder = lib.bcx_decode_compact if choice == "1" else lib.bcx_decode
    vocab, nctx = _dims(kind, nr, nc)
    if len(freq) != nctx * vocab * 4:
        raise CodecError("frequency table length mismatch")
    table = np.frombuffer(freq, dtype="<u4").copy()
    n = rows * cols
    out = np.empty(n, dtype="<u2")
    rc = np.ascontiguousarray(rc, dtype=np.uint8)
    cc = np.ascontiguousarray(cc, dtype=np.uint8)
    data = np.frombuffer(bytes(stream), dtype=np.uint8).copy() if len(stream) else np.zeros(1, dtype=np.uint8)
    ctx = _native.U16P() if main is None else _p(np.ascontiguousarray(main, dtype="<u2").ravel(), ctypes.c_uint16)
    if kind and main is None:
        raise CodecError("residual stream needs the main symbols")
    status = decoder(_p(data, ctypes.c_uint8), len(stream), n, rows, cols, _p(rc, ctypes.c_uint8), _p(cc, ctypes.c_uint8),
                     nr, nc, kind, ctx, _p(table, ctypes.c_uint32), _p(out, ctypes.c_uint16))
    if status:
        raise CodecError(f"rANS decode failed ({status})")
    return out if not kind else out.astype(np.uint8)


def _pack6(lib, a):
    ptr, length = _native.U8P(), ctypes.c_size_t()
    if lib.bcx_pack6(_p(a, ctypes.c_uint16), a.size, ctypes.byref(ptr), ctypes.byref(length)):
        raise CodecError("raw residual packing failed")
    try:
        return ctypes.string_at(ptr, length.value)
    finally:
        lib.bcx_free(ptr)


def _unpack6(lib, raw, n):
    out = np.empty(n, dtype="<u2")
    data = np.frombuffer(bytes(raw), dtype=np.uint8).copy() if len(raw) else np.zeros(1, dtype=np.uint8)
    if lib.bcx_unpack6(_p(data, ctypes.c_uint8), len(raw), n, _p(out, ctypes.c_uint16)):
        raise CodecError("invalid raw residual stream")
    return out


def _inflate_exact(data, expected):
    try:
        dec = zlib.decompressobj()
        raw = dec.decompress(data, expected + 1)
        if len(raw) > expected or dec.unconsumed_tail:
            raise CodecError("compressed section exceeds declared size")
        raw += dec.flush()
    except zlib.error as e:
        raise CodecError("invalid compressed section") from e
    if len(raw) != expected or not dec.eof or dec.unused_data:
        raise CodecError("compressed section length/trailing data mismatch")
    return raw


def _frame(mode, nr, nc, r, c, meta, table, sy, rs, raw, dig):
    body = HEADER.pack(MAGIC, VERSION, mode, nr, nc, r, c, len(meta), len(table), len(sy), len(rs), dig)
    body += meta + table + sy + rs + raw
    return body + hashlib.sha256(body).digest()


def join_words(main, residual):
    m = np.asarray(main).astype(np.uint32)
    q = np.asarray(residual).astype(np.uint32)
    return (((m >> 2) << 7) | ((m & 3) << 5) | (q & 31) | ((q >> 5) << 15)).astype("<u2")


def encode(words, *, row_classes=16, col_classes=4):
    """Encode a 2-D array of BF16 bit patterns into a self-contained frame (smallest of the raw6-residual
    frame, the conditional-residual frame and the raw fallback)."""
    a = _input(words)
    if row_classes not in ROWS or col_classes not in COLS:
        raise CodecError("unsupported class count")
    r, c = a.shape
    raw = a.tobytes()
    dig = hashlib.sha256(raw).digest()
    fallback = _frame(1, row_classes, col_classes, r, c, b"", b"", b"", b"", raw, dig)
    lib = _lib()
    rc, cc = _labels(a, row_classes, col_classes)
    meta = zlib.compress(rc.tobytes() + cc.tobytes(), 6)
    sf, sy = _encode_kind(lib, a, rc, cc, row_classes, col_classes, 0)
    crf, cr = _encode_kind(lib, a, rc, cc, row_classes, col_classes, 1)
    packed = _pack6(lib, a)
    raw6 = _frame(0, row_classes, col_classes, r, c, meta, zlib.compress(sf, 6), sy, packed, b"", dig)
    cond = _frame(128, row_classes, col_classes, r, c, meta, zlib.compress(sf + crf, 6), sy, cr, b"", dig)
    coded = min((raw6, cond), key=len)
    return coded if len(coded) < len(fallback) else fallback


def parse(frame):
    """Validated sections of a frame: header fields, labels, tables, stream slices (no entropy decoding)."""
    if not isinstance(frame, (bytes, bytearray, memoryview)) or len(frame) < HEADER.size + 32:
        raise CodecError("short frame")
    frame = bytes(frame)
    if hashlib.sha256(frame[:-32]).digest() != frame[-32:]:
        raise CodecError("frame checksum mismatch")
    try:
        magic, ver, mode, nr, nc, r, c, ml, tl, sl, dl, dig = HEADER.unpack_from(frame)
    except struct.error as e:
        raise CodecError("bad frame header") from e
    if magic != MAGIC or ver != VERSION or nr not in ROWS or nc not in COLS:
        raise CodecError("unsupported frame header")
    n = r * c
    if not r or not c or n > MAX_WORDS:
        raise CodecError("invalid geometry")
    end = HEADER.size + ml + tl + sl + dl
    out = {"mode": mode, "nr": nr, "nc": nc, "shape": (r, c), "digest": dig}
    if mode == 1:
        if ml or tl or sl or dl or len(frame) != end + 2 * n + 32:
            raise CodecError("invalid raw frame length")
        raw = frame[end:-32]
        if hashlib.sha256(raw).digest() != dig:
            raise CodecError("raw checksum mismatch")
        out["raw"] = np.frombuffer(raw, dtype="<u2").copy()
        return out
    if mode not in (0, 128) or len(frame) != end + 32:
        raise CodecError("invalid frame mode/length")
    p = HEADER.size
    meta = _inflate_exact(frame[p:p + ml], r + c)
    p += ml
    main_bytes = nr * nc * 1024 * 4
    table = _inflate_exact(frame[p:p + tl], main_bytes + (1024 * 64 * 4 if mode == 128 else 0))
    p += tl
    rc = np.frombuffer(meta[:r], dtype=np.uint8).copy()
    cc = np.frombuffer(meta[r:], dtype=np.uint8).copy()
    if rc.max(initial=0) >= nr or cc.max(initial=0) >= nc:
        raise CodecError("class outside declared range")
    out.update(rows=rc, columns=cc, main_table=table[:main_bytes], residual_table=table[main_bytes:] if mode == 128 else None,
               main_stream=frame[p:p + sl], residual_stream=frame[p + sl:p + sl + dl])
    return out


def decode(frame):
    """Decode a complete frame on the host and verify the source checksum; trailing data rejects."""
    f = parse(frame)
    r, c = f["shape"]
    if f["mode"] == 1:
        return f["raw"].reshape(r, c)
    lib = _lib()
    main = _decode_kind(lib, f["main_stream"], f["main_table"], f["rows"], f["columns"], r, c, f["nr"], f["nc"], 0)
    if f["mode"] == 128:
        residual = _decode_kind(lib, f["residual_stream"], f["residual_table"], f["rows"], f["columns"], r, c, f["nr"],
                                f["nc"], 1, main)
    else:
        residual = _unpack6(lib, f["residual_stream"], r * c)
    out = np.ascontiguousarray(join_words(main, residual).reshape(r, c))
    if hashlib.sha256(out.tobytes()).digest() != f["digest"]:
        raise CodecError("decoded checksum mismatch")
    return out
