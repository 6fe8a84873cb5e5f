"""Indexed CUDA decoding of BCTX frames and the fused linear over their resident image.

Mirrors ``context-runtime/georefine_context_runtime/bitexact_context_gpu.py``: ``checkpoints`` (:51-63),
``index_frame`` (:66-106) and ``CudaContextTensor`` (:109-168) keep their names, arguments, attributes and
errors.  The tensor gains ``linear(x, out=None)`` / ``__call__(x, y)``: the seam the reference reserves for "a
backend with a fused GEMM" (bitexact_context_serving.py:3-5).  Everything that touches the GPU goes through
the C ABI of libgeorefine_b200.so; there is no other path.
"""
from __future__ import annotations

import ctypes
import hashlib
import math

import numpy as np

from . import _native
from . import codec as base
from .resident import ResidentWeight


def _p(a, t):
    return a.ctypes.data_as(ctypes.POINTER(t))


def _walk_stream(stream, table, row_class, col_class, shape, nr, nc, stride, conditioning):
    """One serial pass of the host coder over a stream (``bcx_checkpoint``): the symbols, and the decoder's state and
    byte offset in front of every ``stride``-th symbol.  ``conditioning`` = the main symbols when the stream is the
    conditional residual stream, else None."""
    rows, cols = shape
    count = rows * cols
    blocks = -(-count // stride)
    states, offsets = np.empty(blocks, dtype=np.uint32), np.empty(blocks, dtype=np.uint32)
    symbols = np.empty(count, dtype=np.uint16)
    data = np.frombuffer(bytes(stream), dtype=np.uint8).copy() if len(stream) else np.zeros(1, dtype=np.uint8)
    table = np.ascontiguousarray(table, dtype="<u4")
    row_class = np.ascontiguousarray(row_class, dtype=np.uint8)
    col_class = np.ascontiguousarray(col_class, dtype=np.uint8)
    kind = 0 if conditioning is None else 1
    context = _native.U16P() if conditioning is None else _p(np.ascontiguousarray(conditioning, dtype=np.uint16), ctypes.c_uint16)
    status = _native.lib().bcx_checkpoint(_p(data, ctypes.c_uint8), len(stream), count, rows, cols, _p(row_class, ctypes.c_uint8),
                                          _p(col_class, ctypes.c_uint8), nr, nc, kind, context, _p(table, ctypes.c_uint32), stride,
                                          _p(states, ctypes.c_uint32), _p(offsets, ctypes.c_uint32), _p(symbols, ctypes.c_uint16))
    if status:
        raise base.CodecError(f"checkpoint validation failed ({status})")
    return states, offsets, symbols


def checkpoints(stream, freq, rows, columns, shape, nr, nc, stride, main=None):
    """(states, offsets, symbols) of one stream, under the name and argument order of the reference's helper
    (bitexact_context_gpu.py:51-63)."""
    return _walk_stream(stream, freq, rows, columns, tuple(shape), nr, nc, stride, main)


def index_frame(frame: bytes, stride: int = 1024, *, keep_words: bool = False):
    """Host index of a frame: labels, tables, streams and their restart points; the walk is bound to the
    frame's source digest.  ``keep_words`` also returns the decoded words (key ``words``)."""
    if not isinstance(stride, int) or not 1 <= stride <= 65536:
        raise base.CodecError("invalid checkpoint stride")
    if len(frame) < base.HEADER.size + 32 or hashlib.sha256(frame[:-32]).digest() != frame[-32:]:
        raise base.CodecError("invalid frame checksum/length")
    f = base.parse(frame)
    r, c = f["shape"]
    n = r * c
    out = {"shape": (r, c), "mode": f["mode"], "nr": f["nr"], "nc": f["nc"], "stride": stride,
           "source_sha256": f["digest"].hex(), "frame_sha256": hashlib.sha256(bytes(frame)).hexdigest(),
           "frame_bytes": len(frame)}
    if f["mode"] == 1:
        out["raw"] = f["raw"]
        if keep_words:
            out["words"] = f["raw"].reshape(r, c)
        return out
    nr, nc = f["nr"], f["nc"]
    sf = np.frombuffer(f["main_table"], dtype="<u4").copy().reshape(nr * nc, 1024)
    states, offsets, main = checkpoints(f["main_stream"], sf, f["rows"], f["columns"], (r, c), nr, nc, stride)
    out.update(rows=f["rows"], columns=f["columns"], main_freq=sf,
               main_stream=np.frombuffer(f["main_stream"], dtype=np.uint8).copy(), main_states=states,
               main_offsets=offsets, residual_stream=np.frombuffer(f["residual_stream"], dtype=np.uint8).copy())
    if f["mode"] == 128:
        rf = np.frombuffer(f["residual_table"], dtype="<u4").copy().reshape(1024, 64)
        rstates, roffsets, residual = checkpoints(f["residual_stream"], rf, f["rows"], f["columns"], (r, c), nr, nc,
                                                  stride, main)
        out.update(residual_freq=rf, residual_states=rstates, residual_offsets=roffsets)
    else:
        residual = base._unpack6(_native.lib(), f["residual_stream"], n)
    words = base.join_words(main, residual)
    if hashlib.sha256(words.tobytes()).digest() != f["digest"]:
        raise base.CodecError("indexed source checksum mismatch")
    if keep_words:
        out["words"] = words.reshape(r, c)
    return out


WALK_STRIDE = 128     # words per lane of the device walk when the caller's stride allows it (see CudaContextTensor)


def _lookup_tables(freq):
    """Prefix sums and the inverse index of every context, the index thinned out so that all contexts' tables together
    stay around 128 KB (they are read once per symbol on the decoder's serial chain: they have to live in L1).
    Returns (cum, bucket, log2 of the slots per bucket)."""
    nctx, vocab = freq.shape
    cum = np.empty((nctx, vocab + 1), dtype=np.uint32)
    bucket = np.empty((nctx, 4096), dtype=np.uint16)
    f = np.ascontiguousarray(freq, dtype="<u4")
    status = _native.lib().grb_bctx_build_lookup(_p(f, ctypes.c_uint32), nctx, vocab, _p(cum, ctypes.c_uint32),
                                                 _p(bucket, ctypes.c_uint16))
    if status:
        raise base.CodecError(f"invalid frequency tables ({status})")
    shift = 4
    while shift < 8 and nctx * (65536 >> shift) * 2 > 128 * 1024:
        shift += 1
    return cum, np.ascontiguousarray(bucket[:, ::1 << (shift - 4)]), shift


class CudaContextTensor:
    """A BCTX frame resident on one GPU: the unchanged streams with their restart index (for ``decode`` and
    ``gather_rows``) and, for rank-2 weights, the resident image the fused linear streams.

    ``resident_bytes`` counts every device allocation made here, the image and its scratch included.
    ``stride`` is the restart stride the caller asks for, as in the reference; the index that is actually built and
    walked on the device may be finer (``walk_stride``, by default 128 words when that divides ``stride``): a lane's walk
    is a serial chain, so the decode time is proportional to the words per lane, and eight times more lanes cost 8 bytes
    per stream and 128 words of extra index (a 4096 x 4096 frame decodes in 0.25 ms instead of 1.1 ms).  Results do not
    depend on it.  ``fused=False`` skips the image (embedding tables that are only gathered); ``layout`` picks the image's layout
    ("window4": fixed 4-bit exponent codes, the default and the fastest; "window": 3-bit codes; "rans": entropy-coded
    exponent streams, the smallest).
    """

    def __init__(self, frame: bytes, *, stride: int = 1024, device="cuda:0", fused: bool = True, max_m: int = 128,
                 layout: str | None = None, walk_stride: int | None = None):
        import torch

        if not torch.cuda.is_available():
            raise RuntimeError("CUDA is required")
        self.device = torch.device(device)
        self.stride = stride
        if not isinstance(stride, int) or not 1 <= stride <= 65536:
            raise base.CodecError("invalid checkpoint stride")
        if walk_stride is None:
            walk_stride = WALK_STRIDE if stride > WALK_STRIDE and stride % WALK_STRIDE == 0 else stride
        elif not isinstance(walk_stride, int) or walk_stride <= 0 or stride % walk_stride:
            raise ValueError("walk_stride must divide stride")
        self.walk_stride = walk_stride
        indexed = index_frame(frame, walk_stride, keep_words=fused)
        words = indexed.pop("words", None)
        # identity and geometry, as the loader checks them (bitexact_context_serving.py:560-569)
        for name in ("shape", "mode", "nr", "nc", "source_sha256", "frame_sha256", "frame_bytes"):
            setattr(self, name, indexed[name])
        self.n = math.prod(self.shape)
        # every array of the index goes to the device under its own name; coded streams get their lookup tables
        self.buffers = {name: torch.from_numpy(array).to(self.device) for name, array in indexed.items() if isinstance(array, np.ndarray)}
        self._bucket_shift = {}
        for kind in ("main", "residual"):
            table = indexed.get(kind + "_freq")
            if table is not None:
                cum, bucket, shift = _lookup_tables(table)
                self.buffers[kind + "_cum"] = torch.from_numpy(cum).to(self.device)
                self.buffers[kind + "_bucket"] = torch.from_numpy(bucket).to(self.device)
                self._bucket_shift[kind] = shift
        self.error = torch.zeros((), device=self.device, dtype=torch.int32)
        self.resident = None
        if fused and words is not None:
            self.resident = ResidentWeight.from_words(words, device=self.device, source_sha256=bytes.fromhex(self.source_sha256),
                                                      max_m=max_m, **({} if layout is None else {"layout": layout}))
        self.resident_bytes = sum(t.numel() * t.element_size() for t in self.buffers.values()) + self.error.element_size()
        if self.resident is not None:
            self.resident_bytes += self.resident.resident_bytes
        self._descriptor = None if self.mode == 1 else self._make_descriptor()

    def _make_descriptor(self):
        b = self.buffers
        t = _native.BctxTensor()
        t.n, t.rows, t.cols = self.n, self.shape[0], self.shape[1]
        t.nr, t.nc, t.mode, t.stride = self.nr, self.nc, self.mode, self.walk_stride
        t.row_class, t.col_class = b["rows"].data_ptr(), b["columns"].data_ptr()
        t.main_stream, t.main_bytes = b["main_stream"].data_ptr(), b["main_stream"].numel()
        t.main_states, t.main_offsets = b["main_states"].data_ptr(), b["main_offsets"].data_ptr()
        t.main_cum, t.main_bucket = b["main_cum"].data_ptr(), b["main_bucket"].data_ptr()
        t.main_bucket_shift = self._bucket_shift["main"]
        t.residual_stream, t.residual_bytes = b["residual_stream"].data_ptr(), b["residual_stream"].numel()
        if self.mode == 128:
            t.residual_states, t.residual_offsets = b["residual_states"].data_ptr(), b["residual_offsets"].data_ptr()
            t.residual_cum, t.residual_bucket = b["residual_cum"].data_ptr(), b["residual_bucket"].data_ptr()
            t.residual_bucket_shift = self._bucket_shift["residual"]
        return t

    def _decode_blocks(self, blocks=None, *, check=True):
        import torch

        walk = self.walk_stride                      # blocks are counted in the stride the index was built with
        if blocks is None:
            count, ids = (self.n + walk - 1) // walk, None
        else:
            blocks = blocks.to(device=self.device, dtype=torch.int64).contiguous().reshape(-1)
            count, ids = blocks.numel(), blocks.data_ptr()
        result = torch.empty(count * walk, device=self.device, dtype=torch.uint16)
        self.error.zero_()
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream().cuda_stream
            status = _native.lib().grb_bctx_decode_words(ctypes.byref(self._descriptor), ids, count, result.data_ptr(),
                                                         self.error.data_ptr(), stream)
        _native.check(status, "grb_bctx_decode_words")
        if check and self.error.item() != 0:
            raise base.CodecError("CUDA decoder checkpoint mismatch")
        return result.view(torch.bfloat16)

    def decode(self, *, check=True):
        """Dense BF16 [rows, cols], decoded from the unchanged streams (transient: the caller owns it)."""
        import torch

        if self.mode == 1:
            return self.buffers["raw"].view(torch.bfloat16).reshape(self.shape)
        return self._decode_blocks(check=check)[:self.n].reshape(self.shape)

    def gather_rows(self, ids, *, check=True):
        """Rows ``ids`` (any shape) as BF16 [..., cols].  When a row is a whole number of restart blocks only the blocks of
        the requested rows are decoded; otherwise (raw frames, strides that do not divide the row) the tensor is decoded
        once and indexed."""
        import torch

        rows, cols = self.shape
        ids = ids.to(device=self.device, dtype=torch.int64)
        if ids.numel() == 0:
            return torch.empty((*ids.shape, cols), device=self.device, dtype=torch.bfloat16)
        lowest, highest = torch.aminmax(ids)
        if int(lowest) < 0 or int(highest) >= rows:
            raise IndexError("embedding row outside tensor")
        blocks_per_row, ragged = divmod(cols, self.walk_stride)
        if self.mode == 1 or ragged:
            return self.decode(check=check)[ids]
        first_block = ids.reshape(-1, 1) * blocks_per_row
        wanted = (first_block + torch.arange(blocks_per_row, device=self.device)).reshape(-1)
        return self._decode_blocks(wanted, check=check).reshape(*ids.shape, cols)

    # -- fused linear --------------------------------------------------------------------------------
    def linear(self, x, out=None, bias=None):
        """y = x @ W.T (+ bias) with W decoded inside the kernel; x [..., cols] BF16 -> y [..., rows] BF16."""
        if self.resident is None:
            raise RuntimeError("this tensor was indexed without a resident image (fused=False)")
        return self.resident.linear(x, out=out, bias=bias)

    def __call__(self, x, y):
        self.resident(x, y)
