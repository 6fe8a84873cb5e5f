"""The resident image of a weight (layout: csrc/bxr_format.h) and the fused entry points over it.

``ResidentWeight`` follows the descriptor protocol of the reference's serving engines
(``glc_serve/fastdec.py:172-188`` ``Lin``, ``glc_serve/tbe_desc.py:127-157`` ``TBELin``,
``glc_serve/bigemm.py:468-507`` ``BILin``): attributes ``kind``, ``N``, ``K``, ``bytes``, ``coded_bytes`` and
``__call__(x[M,K], y[M,N])`` writing into a preallocated ``y`` with no allocation and no host
synchronisation, so a call can be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes
import hashlib

import numpy as np

from . import _native

GEMV_MAX_M = 8
LAYOUTS = {"rans": 0, "raw": 1, "window": 2, "window4": 3}   # bxr_format.h: BXR_MODE_CODED / _RAW / _WINDOW / _WINDOW4
DEFAULT_LAYOUT = "window4"                       # the fastest layout (12 bits/weight); "window" 11.3, "rans" 11.1 bits/weight


def sm_count(device) -> int:
    import torch

    return torch.cuda.get_device_properties(device).multi_processor_count


def default_workers(rows: int, cols: int, sms: int) -> int:
    """How many persistent CTAs an image is built for when the caller does not say: one per SM, except for small
    weights with fewer 128-row blocks than SMs, where a multiple of the row-block count is better when it costs few
    extra chunks per CTA: every row block is then cut into the same few whole CTAs (no CTA holds the tail of one row
    block and the head of the next), which shortens the partial-tile exchange at the end of a launch (measured on a
    B200: 5120 x 5120 with 120 instead of 148 CTAs 15.1 vs 16.7 us at M = 64, 17.9 vs 19.9 us at M = 128, level at M = 1;
    5120 x 17408 with 120 CTAs is slower, 30.3 vs 28.0 us: there the streaming dominates)."""
    row_blocks, chunks = -(-rows // 128), -(-cols // 128)
    if row_blocks >= sms or row_blocks == 0:
        return sms
    per_cta = row_blocks * chunks / sms
    aligned = row_blocks * (sms // row_blocks)
    if per_cta <= 16 and row_blocks * chunks / aligned - per_cta <= 5:
        return aligned
    return sms


def build_image(words, workers: int, *, threads: int = 0, layout: str = DEFAULT_LAYOUT, force_raw: bool = False,
                source_sha256: bytes | None = None):
    """Host: BF16 words [rows, cols] -> (image bytes as uint8 array, header).

    layout: "window4" (fixed 4-bit exponent codes in a 16-binade row window: 12 bits/weight, the fastest to decode,
    operand through tensor memory), "window" (fixed 3-bit codes in an 8-binade window with per-chunk exception lists:
    11.3 bits/weight), "rans" (entropy-coded exponent streams: 11.1 bits/weight) or "raw" (plain tiles).  The builder
    demotes window4 / window -> rans -> raw when a chunk does not fit its slot; the header's ``mode`` says what was
    built."""
    mode = LAYOUTS["raw"] if force_raw else LAYOUTS[layout]
    a = np.ascontiguousarray(words, dtype=np.uint16)
    if a.ndim != 2 or not all(a.shape):
        raise ValueError("expected a non-empty 2-D uint16 array")
    if source_sha256 is None:
        source_sha256 = hashlib.sha256(a.astype("<u2").tobytes()).digest()
    digest = (ctypes.c_uint8 * 32).from_buffer_copy(source_sha256)
    ptr, size = _native.U8P(), ctypes.c_uint64()
    lib = _native.lib()
    status = lib.bxr_build(a.ctypes.data_as(_native.U16P), a.shape[0], a.shape[1], int(workers), int(threads),
                           mode, digest, ctypes.byref(ptr), ctypes.byref(size))
    if status:
        raise RuntimeError(f"bxr_build failed ({status})")
    try:
        image = np.ctypeslib.as_array(ptr, shape=(size.value,)).copy()
    finally:
        lib.bxr_free(ptr)
    return image, header_of(image)


def header_of(image) -> _native.BxrHeader:
    return _native.BxrHeader.from_buffer_copy(image[:ctypes.sizeof(_native.BxrHeader)].tobytes())


def validate_image(image) -> None:
    """Structural check of an image (layout version, offsets, work partition, blob index) before anything follows an
    offset inside it; raises ValueError.  Cheap: the blobs themselves are not read."""
    a = np.ascontiguousarray(image, dtype=np.uint8)
    if _native.lib().bxr_validate(a.ctypes.data_as(_native.U8P), a.size):
        raise ValueError("resident image is malformed or was built by another version of the layout")


def decode_image_host(image) -> np.ndarray:
    """Host twin of the GPU decoder; used to bind an image to its source digest before upload."""
    h = header_of(image)
    out = np.empty((h.rows, h.cols), dtype=np.uint16)
    status = _native.lib().bxr_decode_host(image.ctypes.data_as(_native.U8P), image.size, out.ctypes.data_as(_native.U16P))
    if status:
        raise ValueError(f"resident image is malformed ({status})")
    return out


class ResidentWeight:
    kind = "bctx"

    def __init__(self, image: np.ndarray, device, *, max_m: int = 128, verify: bool = True):
        import torch

        validate_image(image)   # always: the kernels follow the image's offsets without further checks
        self.header = header_of(image)
        h = self.header
        if verify:
            words = decode_image_host(image)
            if hashlib.sha256(words.astype("<u2").tobytes()).digest() != bytes(h.source_sha256):
                raise ValueError("resident image does not reproduce its source digest")
        self.device = torch.device(device)
        self.N, self.K = int(h.rows), int(h.cols)
        self.mode = int(h.mode)
        self.image = torch.from_numpy(image).to(self.device)
        self.status = torch.zeros(1, device=self.device, dtype=torch.int32)
        self.max_m = 0
        self.workspace = None
        self.next_weight = None     # see then()
        self.reserve(max_m)

    @classmethod
    def from_words(cls, words, device, *, source_sha256=None, max_m=128, workers=None, layout=None, force_raw=False,
                   verify=True, tune=None):
        """Builds the image on the host and uploads it.  ``layout`` / ``workers`` left to None come from ``tune`` (a
        mapping {(N, K): (layout, workers)} as ``georefine_b200.tune.load_tune`` returns it) when it knows the shape,
        else from the defaults: the 4-bit window layout and ``default_workers``."""
        rows, cols = int(words.shape[0]), int(words.shape[1])
        if tune and (rows, cols) in tune:
            tuned_layout, tuned_workers = tune[(rows, cols)]
            layout = tuned_layout if layout is None else layout
            workers = tuned_workers if workers is None else workers
        layout = DEFAULT_LAYOUT if layout is None else layout
        workers = default_workers(rows, cols, sm_count(device)) if workers is None else workers
        image, _ = build_image(words, workers, layout=layout, force_raw=force_raw, source_sha256=source_sha256)
        return cls(image, device, max_m=max_m, verify=verify)

    def clone(self):
        """A second copy of the image in device memory (benchmarks rotate over copies to defeat the L2)."""
        import copy

        other = copy.copy(self)
        other.image = self.image.clone()
        other.status = self.status.clone()
        other.workspace = self.workspace.clone()
        other.next_weight = None
        return other

    # -- bookkeeping (the numerators of the roofline) ----------------------------------------------------
    @property
    def bytes(self) -> int:
        return int(self.header.total_bytes)

    @property
    def coded_bytes(self) -> int:
        """Bytes one pass of a fused kernel streams from HBM: chunk blobs, restart states, blob index."""
        return int(self.header.coded_bytes)

    @property
    def resident_bytes(self) -> int:
        ws = 0 if self.workspace is None else self.workspace.numel()
        return self.bytes + ws + 4

    def backend_identity(self):
        h = self.header
        return {"format": "BXR1", "mode": self.mode, "workers": int(h.workers), "items": int(h.items),
                "partial_slots": int(h.partial_slots), "library": str(_native.library_path().name)}

    def reserve(self, max_m: int) -> None:
        """Scratch for batches up to max_m rows (FP32 partial tiles + counters); zero-filled once."""
        import torch

        max_m = max(int(max_m), GEMV_MAX_M)
        if max_m <= self.max_m:
            return
        need = int(_native.lib().grb_bxr_workspace_bytes(ctypes.byref(self.header), max_m))
        need = max(need, int(_native.lib().grb_bxr_workspace_bytes(ctypes.byref(self.header), GEMV_MAX_M)))
        self.workspace = torch.zeros(max(need, 256), device=self.device, dtype=torch.uint8)
        self.max_m = max_m

    # -- device entry points -------------------------------------------------------------------------
    def _stream(self):
        import torch

        return torch.cuda.current_stream(self.device).cuda_stream

    def decode(self, *, check=True):
        """Dense BF16 [N, K] decoded from the image by the decode twin of the fused kernels."""
        import torch

        out = torch.empty((self.N, self.K), device=self.device, dtype=torch.bfloat16)
        self.status.zero_()
        with torch.cuda.device(self.device):
            st = _native.lib().grb_bxr_decode(self.image.data_ptr(), ctypes.byref(self.header), out.data_ptr(),
                                              self.status.data_ptr(), self._stream())
        _native.check(st, "grb_bxr_decode")
        if check and self.status.item() != 0:
            raise ValueError(f"resident decode reported status {self.status.item()}")
        return out

    def _run(self, entry, x, y, bias, extra=()):
        import torch

        if x.dim() != 2 or y.dim() != 2 or x.dtype != torch.bfloat16 or y.dtype != torch.bfloat16:
            raise ValueError("x and y must be 2-D BF16 tensors")
        m = x.shape[0]
        if x.shape[1] != self.K or y.shape != (m, self.N) or x.stride(1) != 1 or y.stride(1) != 1:
            raise ValueError("shape mismatch: x [M, K], y [M, N], unit inner stride")
        if m == 0:
            return
        if m > self.max_m and min(m, 128) > min(self.max_m, 128):
            raise ValueError(f"batch of {m} rows exceeds the reserved scratch ({self.max_m}); call reserve() first")
        args = (self.image.data_ptr(), ctypes.byref(self.header), x.data_ptr(), x.stride(0), m, y.data_ptr(), y.stride(0),
                None if bias is None else bias.data_ptr(), self.workspace.data_ptr(), self.workspace.numel(),
                self.status.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream, *extra)
        if torch.cuda.current_device() == self.device.index:   # the usual case: skip the device switch
            st = entry(*args)
        else:
            with torch.cuda.device(self.device):
                st = entry(*args)
        if st:
            _native.check(st, entry.__name__)

    def then(self, next_weight):
        """Tells this weight which one the stream multiplies by next (None: nobody).  A hint for the kernel: while a
        launch over this weight winds down, the L2 is asked for the first blobs of the next one.  Returns
        ``next_weight`` so that a layer can be chained in one line: ``qkv.then(o).then(gate_up).then(down)``."""
        self.next_weight = next_weight
        return next_weight

    def gemm(self, x, y, bias=None):
        """tcgen05 path, any M; rows of y are bitwise independent of M."""
        nxt = self.next_weight
        if nxt is None:
            self._run(_native.lib().grb_bxr_gemm, x, y, bias)
        else:
            self._run(_native.lib().grb_bxr_gemm_next, x, y, bias, extra=(nxt.image.data_ptr(), ctypes.byref(nxt.header)))

    def gemv(self, x, y, bias=None):
        """CUDA-core path, M <= 8; rows of y are bitwise independent of M within 1..8."""
        self._run(_native.lib().grb_bxr_gemv, x, y, bias)

    def __call__(self, x, y):
        self.gemm(x, y)

    def linear(self, x, out=None, bias=None):
        import torch

        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            if self.K % 8:  # the kernels want a row stride that is a multiple of 16 bytes
                padded = torch.zeros((x2.shape[0], (self.K + 7) // 8 * 8), device=self.device, dtype=torch.bfloat16)
                padded[:, :self.K] = x2
                x2 = padded[:, :self.K]
            else:
                x2 = x2.contiguous()
        y = torch.empty((x2.shape[0], self.N), device=self.device, dtype=torch.bfloat16) if out is None else out.reshape(-1, self.N)
        if x2.shape[0] > self.max_m:
            self.reserve(x2.shape[0])
        self.gemm(x2, y, bias)
        return y.reshape(*lead, self.N)

    def check_status(self) -> int:
        """Host read of the device status word (synchronises); 0 means every call since the last reset was clean."""
        return int(self.status.item())
