"""The kernels of a batched decode step other than the linears, as calls on torch tensors.

Thin wrappers over the C ABI (``grb_rmsnorm_bf16``, ``grb_silu_mul_bf16``, ``grb_argmax_bf16``,
``grb_attn_decode_bf16``; kernels in ``csrc/decode_ops.cuh``): every call writes into a tensor the caller provides, on
the current stream, without allocating or synchronising, so a whole step can be captured in a CUDA graph.  They take the
place of the reference's step kernels (``glc_serve/fastdec_kernels.cu:83-110,324-488``) for a plain grouped-query
decoder with head dimension 128.
"""
from __future__ import annotations

import ctypes
import math

from . import _native

PAGE = 256        # positions per KV page
PART = 128        # positions per attention CTA pass: two parts per page
HEAD_DIM = 128


def _stream(t):
    import torch

    return torch.cuda.current_stream(t.device).cuda_stream


def rmsnorm(h, weight, out, *, delta=None, eps=1e-6, unit_offset=False):
    """out = bf16(h * rsqrt(mean(h^2) + eps) * weight); with ``delta`` the residual add h = bf16(h + delta) happens first
    and is written back into ``h``.  ``unit_offset``: the weight is stored as an offset from one."""
    rows, hidden = h.shape
    st = _native.lib().grb_rmsnorm_bf16(h.data_ptr(), h.stride(0), None if delta is None else delta.data_ptr(),
                                        0 if delta is None else delta.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0),
                                        rows, hidden, float(eps), int(bool(unit_offset)), _stream(h))
    _native.check(st, "grb_rmsnorm_bf16")


def silu_mul(gate_up, out):
    """out[r, i] = bf16(bf16(silu(gate_up[r, i])) * gate_up[r, f + i]) with f = out.shape[1]."""
    rows, f = out.shape
    st = _native.lib().grb_silu_mul_bf16(gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), out.stride(0), rows, f, _stream(out))
    _native.check(st, "grb_silu_mul_bf16")


def argmax(logits, out):
    """out[r] (int32) = index of the first maximum of row r."""
    rows, vocab = logits.shape
    st = _native.lib().grb_argmax_bf16(logits.data_ptr(), logits.stride(0), rows, vocab, out.data_ptr(), _stream(logits))
    _native.check(st, "grb_argmax_bf16")


def rope_tables(positions: int, theta: float = 1e6, device="cuda:0"):
    """BF16 cos / sin tables [positions, 128] in the rotate-half convention (the second half repeats the first)."""
    import torch

    inv = 1.0 / (theta ** (torch.arange(0, HEAD_DIM, 2, dtype=torch.float32) / HEAD_DIM))
    angle = torch.arange(positions, dtype=torch.float32)[:, None] * inv[None, :]
    angle = torch.cat([angle, angle], dim=1)
    return angle.cos().to(torch.bfloat16).to(device), angle.sin().to(torch.bfloat16).to(device)


class PagedAttention:
    """Scratch and geometry of the attention call for up to ``max_rows`` rows per step and ``max_pages`` pages per
    sequence; ``__call__`` runs rotary embedding + KV append + decode attention for one layer."""

    def __init__(self, nq: int, nkv: int, max_rows: int, max_pages: int, device):
        import torch

        if nq % nkv or nq // nkv not in (1, 2, 4, 5, 8):
            raise ValueError("query heads per kv head must be 1, 2, 4, 5 or 8")
        self.nq, self.nkv, self.max_rows, self.max_pages = nq, nkv, max_rows, max_pages
        self.q = torch.empty(max_rows, nq, HEAD_DIM, device=device, dtype=torch.bfloat16)
        self.max_parts = max_pages * (PAGE // PART)
        self.part_acc = torch.empty(max_rows, nq, self.max_parts, HEAD_DIM, device=device, dtype=torch.float32)
        self.part_ml = torch.empty(max_rows, nq, self.max_parts, 2, device=device, dtype=torch.float32)
        self.scratch_bytes = sum(t.numel() * t.element_size() for t in (self.q, self.part_acc, self.part_ml))

    def __call__(self, qkv, cos, sin, row_seq, row_pos, page_table, k_pages, v_pages, out, *, max_splits=None):
        rows = qkv.shape[0]
        if rows > self.max_rows:
            raise ValueError("more rows than the attention scratch was sized for")
        step = _native.AttnStep()
        step.qkv, step.ldq = qkv.data_ptr(), qkv.stride(0)
        step.cos_table, step.sin_table = cos.data_ptr(), sin.data_ptr()
        step.row_seq, step.row_pos, step.page_table = row_seq.data_ptr(), row_pos.data_ptr(), page_table.data_ptr()
        step.max_pages = page_table.shape[1]
        step.k_pages, step.v_pages = k_pages.data_ptr(), v_pages.data_ptr()
        step.q, step.part_acc, step.part_ml, step.out = self.q.data_ptr(), self.part_acc.data_ptr(), self.part_ml.data_ptr(), out.data_ptr()
        step.rows, step.nq, step.nkv, step.head_dim = rows, self.nq, self.nkv, HEAD_DIM
        # parts (128 positions each) launched per (row group, kv head) = the stride of the partial buffers in this call;
        # rows shorter than that leave their surplus CTAs at once.  A caller that knows every row is short passes fewer.
        step.max_splits = min(self.max_parts, page_table.shape[1] * (PAGE // PART)) if max_splits is None else int(max_splits)
        if not 1 <= step.max_splits <= self.max_parts:
            raise ValueError("max_splits outside the scratch that was allocated")
        step.scaling = 1.0 / math.sqrt(HEAD_DIM)
        st = _native.lib().grb_attn_decode_bf16(ctypes.byref(step), _stream(qkv))
        _native.check(st, "grb_attn_decode_bf16")
