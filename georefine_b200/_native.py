"""ctypes binding of libgeorefine_b200.so (declarations: include/georefine_b200.h).

There is no fallback: if the library is missing and cannot be built, importing a symbol raises.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

from . import build as _build

_LOCK = threading.Lock()
_LIB = None

U8P = ctypes.POINTER(ctypes.c_uint8)
U16P = ctypes.POINTER(ctypes.c_uint16)
U32P = ctypes.POINTER(ctypes.c_uint32)
I64P = ctypes.POINTER(ctypes.c_int64)
VOIDP = ctypes.c_void_p

EXPORTS = (
    "bcx_encode", "bcx_frequencies", "bcx_decode", "bcx_decode_compact", "bcx_free", "bcx_pack6", "bcx_unpack6",
    "bcx_checkpoint", "grb_bctx_build_lookup", "grb_bctx_decode_words", "bxr_build", "bxr_free", "bxr_decode_host",
    "bxr_validate", "bxr_layout_version", "grb_bxr_workspace_bytes", "grb_bxr_decode", "grb_bxr_gemm", "grb_bxr_gemv", "grb_bxr_gemm_next", "grb_kernel_attributes",
    "grb_static_scratch_bytes", "grb_bxr_gemv_static", "grb_dense_gemv_bf16", "grb_peer_control_bytes", "grb_peer_enable", "grb_peer_allreduce_bf16",
    "grb_peer_alloc", "grb_peer_free", "grb_peer_open", "grb_peer_close",
    "grb_rmsnorm_bf16", "grb_silu_mul_bf16", "grb_argmax_bf16", "grb_attn_decode_bf16",
)


class BxrItem(ctypes.Structure):
    _fields_ = [("row_block", ctypes.c_uint32), ("chunk_begin", ctypes.c_uint32), ("chunk_end", ctypes.c_uint32),
                ("part", ctypes.c_uint32), ("parts", ctypes.c_uint32), ("slot", ctypes.c_uint32),
                ("reserved", ctypes.c_uint32 * 2)]


class BxrHeader(ctypes.Structure):
    _fields_ = [("magic", ctypes.c_uint32), ("mode", ctypes.c_uint32), ("rows", ctypes.c_uint32),
                ("cols", ctypes.c_uint32), ("row_blocks", ctypes.c_uint32), ("chunks", ctypes.c_uint32),
                ("workers", ctypes.c_uint32), ("items", ctypes.c_uint32), ("partial_slots", ctypes.c_uint32),
                ("blob_stride16", ctypes.c_uint32), ("layout_version", ctypes.c_uint32),
                ("reserved0", ctypes.c_uint32), ("lut_at", ctypes.c_uint64), ("base_at", ctypes.c_uint64),
                ("items_at", ctypes.c_uint64), ("worker_items_at", ctypes.c_uint64), ("states_at", ctypes.c_uint64),
                ("blob_index_at", ctypes.c_uint64), ("blobs_at", ctypes.c_uint64), ("total_bytes", ctypes.c_uint64),
                ("coded_bytes", ctypes.c_uint64), ("source_sha256", ctypes.c_uint8 * 32)]


class BctxTensor(ctypes.Structure):
    _fields_ = [("n", ctypes.c_uint64), ("rows", ctypes.c_uint32), ("cols", ctypes.c_uint32), ("nr", ctypes.c_uint32),
                ("nc", ctypes.c_uint32), ("mode", ctypes.c_uint32), ("stride", ctypes.c_uint32),
                ("row_class", VOIDP), ("col_class", VOIDP), ("main_stream", VOIDP), ("main_bytes", ctypes.c_uint64),
                ("main_states", VOIDP), ("main_offsets", VOIDP), ("main_cum", VOIDP), ("main_bucket", VOIDP),
                ("residual_stream", VOIDP), ("residual_bytes", ctypes.c_uint64), ("residual_states", VOIDP),
                ("residual_offsets", VOIDP), ("residual_cum", VOIDP), ("residual_bucket", VOIDP),
                ("main_bucket_shift", ctypes.c_uint32), ("residual_bucket_shift", ctypes.c_uint32)]


class AttnStep(ctypes.Structure):
    _fields_ = [("qkv", VOIDP), ("ldq", ctypes.c_int64), ("cos_table", VOIDP), ("sin_table", VOIDP), ("row_seq", VOIDP),
                ("row_pos", VOIDP), ("page_table", VOIDP), ("max_pages", ctypes.c_uint32), ("k_pages", VOIDP), ("v_pages", VOIDP),
                ("q", VOIDP), ("part_acc", VOIDP), ("part_ml", VOIDP), ("out", VOIDP), ("rows", ctypes.c_uint32),
                ("nq", ctypes.c_uint32), ("nkv", ctypes.c_uint32), ("head_dim", ctypes.c_uint32), ("max_splits", ctypes.c_uint32),
                ("scaling", ctypes.c_float)]


def _declare(lib):
    u32, u64, sz, ci = ctypes.c_uint32, ctypes.c_uint64, ctypes.c_size_t, ctypes.c_int
    lib.bcx_encode.argtypes = [U16P, u64, u32, u32, U8P, U8P, u32, u32, u32, U32P, ctypes.POINTER(U8P), ctypes.POINTER(sz)]
    lib.bcx_frequencies.argtypes = [U16P, u64, u32, u32, U8P, U8P, u32, u32, u32, U32P]
    lib.bcx_decode.argtypes = [U8P, sz, u64, u32, u32, U8P, U8P, u32, u32, u32, U16P, U32P, U16P]
    lib.bcx_decode_compact.argtypes = lib.bcx_decode.argtypes
    lib.bcx_free.argtypes = [VOIDP]
    lib.bcx_free.restype = None
    lib.bcx_pack6.argtypes = [U16P, u64, ctypes.POINTER(U8P), ctypes.POINTER(sz)]
    lib.bcx_unpack6.argtypes = [U8P, sz, u64, U16P]
    lib.bcx_checkpoint.argtypes = [U8P, sz, u64, u32, u32, U8P, U8P, u32, u32, u32, U16P, U32P, u32, U32P, U32P, U16P]
    lib.grb_bctx_build_lookup.argtypes = [U32P, u32, u32, U32P, U16P]
    lib.grb_bctx_decode_words.argtypes = [ctypes.POINTER(BctxTensor), VOIDP, u64, VOIDP, VOIDP, VOIDP]
    lib.bxr_build.argtypes = [U16P, u32, u32, u32, u32, u32, U8P, ctypes.POINTER(U8P), ctypes.POINTER(u64)]
    lib.bxr_free.argtypes = [VOIDP]
    lib.bxr_free.restype = None
    lib.bxr_decode_host.argtypes = [U8P, u64, U16P]
    lib.bxr_validate.argtypes = [U8P, u64]
    lib.bxr_layout_version.argtypes = []
    lib.bxr_layout_version.restype = u32
    lib.grb_bxr_workspace_bytes.argtypes = [ctypes.POINTER(BxrHeader), u32]
    lib.grb_bxr_workspace_bytes.restype = u64
    lib.grb_bxr_decode.argtypes = [VOIDP, ctypes.POINTER(BxrHeader), VOIDP, VOIDP, VOIDP]
    linear = [VOIDP, ctypes.POINTER(BxrHeader), VOIDP, ctypes.c_int64, u32, VOIDP, ctypes.c_int64, VOIDP, VOIDP, u64,
              VOIDP, VOIDP]
    lib.grb_bxr_gemm.argtypes = linear
    lib.grb_bxr_gemv.argtypes = linear
    lib.grb_bxr_gemm_next.argtypes = linear + [VOIDP, ctypes.POINTER(BxrHeader)]
    lib.grb_kernel_attributes.argtypes = [ci, ctypes.POINTER(ci * 5)]
    lib.grb_static_scratch_bytes.argtypes = []
    lib.grb_static_scratch_bytes.restype = u64
    lib.grb_bxr_gemv_static.argtypes = [VOIDP, ctypes.POINTER(BxrHeader), VOIDP, ctypes.c_int64, u32, VOIDP, ctypes.c_int64,
                                        VOIDP, VOIDP, VOIDP]
    lib.grb_dense_gemv_bf16.argtypes = [VOIDP, ctypes.c_int64, u32, u32, VOIDP, ctypes.c_int64, u32, VOIDP, ctypes.c_int64,
                                        VOIDP, VOIDP]
    lib.grb_rmsnorm_bf16.argtypes = [VOIDP, ctypes.c_int64, VOIDP, ctypes.c_int64, VOIDP, VOIDP, ctypes.c_int64, u32, u32,
                                     ctypes.c_float, ci, VOIDP]
    lib.grb_silu_mul_bf16.argtypes = [VOIDP, ctypes.c_int64, VOIDP, ctypes.c_int64, u32, u32, VOIDP]
    lib.grb_argmax_bf16.argtypes = [VOIDP, ctypes.c_int64, u32, u32, VOIDP, VOIDP]
    lib.grb_attn_decode_bf16.argtypes = [ctypes.POINTER(AttnStep), VOIDP]
    lib.grb_peer_control_bytes.argtypes = []
    lib.grb_peer_control_bytes.restype = u64
    lib.grb_peer_enable.argtypes = [ci]
    lib.grb_peer_alloc.argtypes = [u64, ctypes.POINTER(VOIDP), U8P]
    lib.grb_peer_free.argtypes = [VOIDP]
    lib.grb_peer_open.argtypes = [U8P, ctypes.POINTER(VOIDP)]
    lib.grb_peer_close.argtypes = [VOIDP]
    lib.grb_peer_allreduce_bf16.argtypes = [VOIDP, ctypes.POINTER(VOIDP), ctypes.POINTER(VOIDP), u64, u32, u32, VOIDP, u64, u64, VOIDP, VOIDP]
    for name in EXPORTS:
        if name not in ("bcx_free", "bxr_free", "grb_bxr_workspace_bytes", "grb_static_scratch_bytes", "grb_peer_control_bytes",
                        "bxr_layout_version"):
            getattr(lib, name).restype = ci


def library_path() -> Path:
    override = os.environ.get("GEOREFINE_B200_LIBRARY")
    return Path(override) if override else _build.OUT


def lib():
    """The loaded library; builds it first when sources are newer (needs nvcc)."""
    global _LIB
    with _LOCK:
        if _LIB is None:
            override = os.environ.get("GEOREFINE_B200_LIBRARY")
            path = Path(override) if override else _build.OUT
            if not override and _build.needs_build():
                try:
                    path = _build.build()
                except RuntimeError:
                    if not path.exists():
                        raise
            handle = ctypes.CDLL(str(path))
            _declare(handle)
            _LIB = handle
        return _LIB


def check(status: int, what: str) -> None:
    if status:
        detail = f"CUDA error {status - 100}" if status >= 100 else {1: "bad argument", 2: "unsupported", 3: "workspace too small"}.get(status, "failure")
        raise RuntimeError(f"{what}: {detail} (status {status})")
