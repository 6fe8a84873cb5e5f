"""BCTX v1 frame codec: the host half of the path, under the reference module's public names.

Drop-in for ``context-runtime/georefine_context_runtime/bitexact_context_codec.py``: ``encode`` (:354), ``decode``
(:377), ``CodecError`` (:26) and the constants ``MAGIC, VERSION, HEADER, ROWS, COLS, MAX_WORDS`` (:17-22) keep their
meaning, frames are byte-identical to the reference's, every malformed frame raises ``CodecError``; the helpers
``_inflate_exact``, ``_unpack6`` and ``_lib`` exist because the index module of the reference imports them
(bitexact_context_gpu.py:71-102).  The integer work runs in libgeorefine_b200.so through the ``bcx_*`` C ABI.  This
module is what an offline encoder or a loader calls once per tensor; per-call decoding on the GPU lives in
``georefine_b200.gpu``.

Wire format (little endian)::

    header   "<4sBBBBIIQQQQ32s"  magic, version, mode, row classes, column classes, rows, cols,
                                 bytes of [labels, tables, main stream, residual section], SHA-256 of the source words
    labels   zlib(row classes u8[rows] + column classes u8[cols])
    tables   zlib(main frequencies u32[nr * nc][1024] (+ residual frequencies u32[1024][64] in mode 128))
    main     rANS stream of the 10-bit symbols
    residual mode 0: 6-bit residuals packed MSB first; mode 128: rANS stream conditioned on the main symbol
    raw      mode 1 only: the source words themselves (every other section empty)
    trailer  SHA-256 of everything before it
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import struct
import zlib
from dataclasses import dataclass

import numpy as np

from . import _native

MAGIC = b"BCTX"
VERSION = 1
HEADER = struct.Struct("<4sBBBBIIQQQQ32s")
MAX_WORDS = 0xFFFFFFFF
ROWS = {1, 4, 16, 64}
COLS = {1, 4, 16}

MODE_RAW6, MODE_WORDS, MODE_CONDITIONAL = 0, 1, 128
_TRAILER = hashlib.sha256().digest_size
_MAIN_VOCAB, _RESIDUAL_VOCAB = 1024, 64


class CodecError(ValueError):
    """Invalid input or malformed frame."""


def _lib():
    return _native.lib()


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def _u8(a):
    return np.ascontiguousarray(a, dtype=np.uint8)


def _stream_array(data):
    """A byte string as an array the C ABI can take the address of (one zero byte stands in for an empty stream)."""
    return np.frombuffer(bytes(data), dtype=np.uint8).copy() if len(data) else np.zeros(1, dtype=np.uint8)


# ---------------------------------------------------------------------------------------------- frame layout
@dataclass(frozen=True)
class _Head:
    """The fixed header of a frame and the section boundaries that follow from it."""

    mode: int
    nr: int
    nc: int
    rows: int
    cols: int
    lengths: tuple          # bytes of labels, tables, main stream, residual section
    digest: bytes

    @property
    def words(self) -> int:
        return self.rows * self.cols

    @property
    def coded_end(self) -> int:
        return HEADER.size + sum(self.lengths)

    def pack(self) -> bytes:
        return HEADER.pack(MAGIC, VERSION, self.mode, self.nr, self.nc, self.rows, self.cols, *self.lengths, self.digest)

    def sections(self, frame: bytes):
        at, out = HEADER.size, []
        for n in self.lengths:
            out.append(frame[at:at + n])
            at += n
        return out

    @classmethod
    def read(cls, frame: bytes) -> "_Head":
        try:
            magic, version, mode, nr, nc, rows, cols, ml, tl, sl, dl, digest = HEADER.unpack_from(frame)
        except struct.error as exc:
            raise CodecError("bad frame header") from exc
        problems = {"unsupported frame header": magic != MAGIC or version != VERSION or nr not in ROWS or nc not in COLS,
                    "invalid geometry": rows == 0 or cols == 0 or rows * cols > MAX_WORDS}
        for message, bad in problems.items():
            if bad:
                raise CodecError(message)
        return cls(mode, nr, nc, rows, cols, (ml, tl, sl, dl), digest)


def _sealed(body: bytes) -> bytes:
    return body + hashlib.sha256(body).digest()


def _seal_is_intact(frame: bytes) -> bool:
    return len(frame) >= HEADER.size + _TRAILER and hashlib.sha256(frame[:-_TRAILER]).digest() == frame[-_TRAILER:]


def _inflate_exact(data, expected):
    """zlib-inflates a section that must yield exactly ``expected`` bytes and end exactly where the input ends; never
    produces more than one byte beyond the declared size, whatever the input claims."""
    inflater = zlib.decompressobj()
    try:
        out = inflater.decompress(data, expected + 1)
        overflow = len(out) > expected or bool(inflater.unconsumed_tail)
        if not overflow:
            out += inflater.flush()
    except zlib.error as exc:
        raise CodecError("invalid compressed section") from exc
    if overflow:
        raise CodecError("compressed section exceeds declared size")
    if len(out) != expected or not inflater.eof or inflater.unused_data:
        raise CodecError("compressed section length/trailing data mismatch")
    return out


# ---------------------------------------------------------------------------------------------- inputs and labels
def _input(words):
    """The caller's array as contiguous little-endian uint16 [rows, cols]; anything else is refused."""
    a = np.asarray(words)
    two_byte_integers = a.dtype.kind in "ui" and a.dtype.itemsize == 2
    if a.ndim != 2 or not two_byte_integers:
        raise CodecError("expected a 2D uint16 word array")
    if 0 in a.shape or a.size > MAX_WORDS:
        raise CodecError("invalid or oversized geometry")
    if a.dtype.kind == "i" and (a < 0).any():
        raise CodecError("word outside uint16 range")
    return np.ascontiguousarray(a, dtype="<u2")


def _quantile_classes(weight, k):
    """Class of every entry = its rank (stable sort by weight) scaled to 0..k-1: equal-population bins."""
    n = len(weight)
    rank = np.empty(n, dtype=np.uint64)
    rank[np.argsort(weight, kind="stable")] = np.arange(n, dtype=np.uint64)
    return (rank * np.uint64(k) // np.uint64(n)).astype(np.uint8)


def _labels(a, nr, nc):
    """Row and column classes by total magnitude (sum of word & 0x7FFF), accumulated over row slabs so that a very
    large tensor never needs a second array of its own size."""
    rows, cols = a.shape
    row_sum = np.zeros(rows, dtype=np.uint64)
    col_sum = np.zeros(cols, dtype=np.uint64)
    step = max(1, min(rows, (1 << 20) // cols))
    for lo in range(0, rows, step):
        magnitude = a[lo:lo + step] & np.uint16(0x7FFF)
        row_sum[lo:lo + step] = magnitude.sum(axis=1, dtype=np.uint64)
        col_sum += magnitude.sum(axis=0, dtype=np.uint64)
    return _quantile_classes(row_sum, nr), _quantile_classes(col_sum, nc)


# ---------------------------------------------------------------------------------------------- C ABI calls
def _dims(kind, nr, nc):
    """(vocabulary, number of contexts) of a stream kind: 0 = main symbols, 1 = residuals conditioned on the main symbol."""
    return (_RESIDUAL_VOCAB, _MAIN_VOCAB) if kind else (_MAIN_VOCAB, nr * nc)


def _encode_kind(lib, a, rc, cc, nr, nc, kind):
    vocab, nctx = _dims(kind, nr, nc)
    freq = np.zeros(nctx * vocab, dtype="<u4")
    rc, cc = _u8(rc), _u8(cc)
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
    rc, cc = _u8(rc), _u8(cc)
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
    if kind and main is None:
        raise CodecError("residual stream needs the main symbols")
    table = np.frombuffer(freq, dtype="<u4").copy()
    out = np.empty(rows * cols, dtype="<u2")
    rc, cc, data = _u8(rc), _u8(cc), _stream_array(stream)
    context = _native.U16P() if main is None else _p(np.ascontiguousarray(main, dtype="<u2").ravel(), ctypes.c_uint16)
    status = decoder(_p(data, ctypes.c_uint8), len(stream), rows * cols, rows, cols, _p(rc, ctypes.c_uint8),
                     _p(cc, ctypes.c_uint8), nr, nc, kind, context, _p(table, ctypes.c_uint32), _p(out, ctypes.c_uint16))
    if status:
        raise CodecError(f"rANS decode failed ({status})")
    return out.astype(np.uint8) if kind else out


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
    data = _stream_array(raw)
    if lib.bcx_unpack6(_p(data, ctypes.c_uint8), len(raw), n, _p(out, ctypes.c_uint16)):
        raise CodecError("invalid raw residual stream")
    return out


def join_words(main, residual):
    """BF16 words from their two halves: main = exponent << 2 | mantissa[6:5], residual = sign << 5 | mantissa[4:0]."""
    m = np.asarray(main).astype(np.uint32)
    q = np.asarray(residual).astype(np.uint32)
    return (((m >> 2) << 7) | ((m & 3) << 5) | (q & 31) | ((q >> 5) << 15)).astype("<u2")


# ---------------------------------------------------------------------------------------------- public API
def encode(words, *, row_classes=16, col_classes=4):
    """Encode a 2-D array of BF16 bit patterns into a self-contained frame: the smaller of the two coded forms (6-bit
    residuals stored raw, or entropy-coded under the main symbol), unless the plain words are no larger."""
    a = _input(words)
    if row_classes not in ROWS or col_classes not in COLS:
        raise CodecError("unsupported class count")
    rows, cols = a.shape
    source = a.tobytes()
    digest = hashlib.sha256(source).digest()

    def frame(mode, labels=b"", tables=b"", main=b"", residual=b"", raw=b""):
        head = _Head(mode, row_classes, col_classes, rows, cols, (len(labels), len(tables), len(main), len(residual)), digest)
        return _sealed(head.pack() + labels + tables + main + residual + raw)

    lib = _lib()
    rc, cc = _labels(a, row_classes, col_classes)
    labels = zlib.compress(rc.tobytes() + cc.tobytes(), 6)
    main_table, main_stream = _encode_kind(lib, a, rc, cc, row_classes, col_classes, 0)
    cond_table, cond_stream = _encode_kind(lib, a, rc, cc, row_classes, col_classes, 1)
    candidates = [   # in order of preference at equal size
        frame(MODE_RAW6, labels, zlib.compress(main_table, 6), main_stream, _pack6(lib, a)),
        frame(MODE_CONDITIONAL, labels, zlib.compress(main_table + cond_table, 6), main_stream, cond_stream),
    ]
    best = min(candidates, key=len)
    plain = frame(MODE_WORDS, raw=source)
    return best if len(best) < len(plain) else plain


def parse(frame):
    """Validated sections of a frame: header fields, labels, tables, stream slices (no entropy decoding)."""
    if not isinstance(frame, (bytes, bytearray, memoryview)) or len(frame) < HEADER.size + _TRAILER:
        raise CodecError("short frame")
    frame = bytes(frame)
    if not _seal_is_intact(frame):
        raise CodecError("frame checksum mismatch")
    head = _Head.read(frame)
    out = {"mode": head.mode, "nr": head.nr, "nc": head.nc, "shape": (head.rows, head.cols), "digest": head.digest}
    if head.mode == MODE_WORDS:
        if any(head.lengths) or len(frame) != HEADER.size + 2 * head.words + _TRAILER:
            raise CodecError("invalid raw frame length")
        raw = frame[HEADER.size:-_TRAILER]
        if hashlib.sha256(raw).digest() != head.digest:
            raise CodecError("raw checksum mismatch")
        out["raw"] = np.frombuffer(raw, dtype="<u2").copy()
        return out
    if head.mode not in (MODE_RAW6, MODE_CONDITIONAL) or len(frame) != head.coded_end + _TRAILER:
        raise CodecError("invalid frame mode/length")
    packed_labels, packed_tables, main_stream, residual_stream = head.sections(frame)
    labels = _inflate_exact(packed_labels, head.rows + head.cols)
    main_bytes = head.nr * head.nc * _MAIN_VOCAB * 4
    residual_bytes = _MAIN_VOCAB * _RESIDUAL_VOCAB * 4 if head.mode == MODE_CONDITIONAL else 0
    tables = _inflate_exact(packed_tables, main_bytes + residual_bytes)
    rc = np.frombuffer(labels, dtype=np.uint8, count=head.rows).copy()
    cc = np.frombuffer(labels, dtype=np.uint8, offset=head.rows).copy()
    if (rc >= head.nr).any() or (cc >= head.nc).any():
        raise CodecError("class outside declared range")
    out.update(rows=rc, columns=cc, main_table=tables[:main_bytes], residual_table=tables[main_bytes:] if residual_bytes else None,
               main_stream=main_stream, residual_stream=residual_stream)
    return out


def decode(frame):
    """Decode a complete frame on the host and verify the source checksum; trailing data rejects."""
    f = parse(frame)
    rows, cols = f["shape"]
    if f["mode"] == MODE_WORDS:
        return f["raw"].reshape(rows, cols)
    lib = _lib()
    common = (f["rows"], f["columns"], rows, cols, f["nr"], f["nc"])
    main = _decode_kind(lib, f["main_stream"], f["main_table"], *common, 0)
    if f["mode"] == MODE_CONDITIONAL:
        residual = _decode_kind(lib, f["residual_stream"], f["residual_table"], *common, 1, main)
    else:
        residual = _unpack6(lib, f["residual_stream"], rows * cols)
    words = np.ascontiguousarray(join_words(main, residual).reshape(rows, cols))
    if hashlib.sha256(words.tobytes()).digest() != f["digest"]:
        raise CodecError("decoded checksum mismatch")
    return words
