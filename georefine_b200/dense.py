"""Dense BF16 linear for small batches: the library's own GEMV over an uncompressed weight.

``DenseLinear`` follows the descriptor protocol of the reference's serving engine (``Lin``,
``glc_serve/fastdec.py:172-188``: ``kind``, ``N``, ``K``, ``bytes``, ``__call__(x, y)`` into a preallocated ``y``, no
allocation, no host synchronisation) and the numerical contract of its M-invariant GEMV
(``glc_serve/miv_gemv.py:103-191``): rows of ``y`` are bitwise the same for every batch size from 1 to 8.  It is what
the fused decode-GEMV is compared with ("effective bandwidth versus a dense BF16 GEMV on the same GPU") and what serves
weights that are kept uncompressed.  Kernel: ``csrc/dense_gemv.cuh``; entry point ``grb_dense_gemv_bf16``.
"""
from __future__ import annotations

from . import _native

DENSE_MAX_M = 8


def dense_gemv(weight, x, y, bias=None) -> None:
    """y[M, N] = bf16(x[M, K] @ weight[N, K].T (+ bias)), FP32 accumulation, M <= 8, on the current stream."""
    import torch

    if weight.dim() != 2 or x.dim() != 2 or y.dim() != 2 or not (weight.dtype == x.dtype == y.dtype == torch.bfloat16):
        raise ValueError("weight, x and y must be 2-D BF16 tensors")
    n, k = weight.shape
    m = x.shape[0]
    if x.shape[1] != k or tuple(y.shape) != (m, n) or weight.stride(1) != 1 or x.stride(1) != 1 or y.stride(1) != 1:
        raise ValueError("shape mismatch: weight [N, K], x [M, K], y [M, N], unit inner strides")
    if m == 0:
        return
    status = _native.lib().grb_dense_gemv_bf16(weight.data_ptr(), weight.stride(0), n, k, x.data_ptr(), x.stride(0), m,
                                               y.data_ptr(), y.stride(0), None if bias is None else bias.data_ptr(),
                                               torch.cuda.current_stream(weight.device).cuda_stream)
    _native.check(status, "grb_dense_gemv_bf16")


class DenseLinear:
    """An uncompressed BF16 weight [N, K] on one GPU, called like the compressed descriptors."""

    kind = "dense"

    def __init__(self, weight, bias=None):
        import torch

        if weight.dim() != 2 or weight.dtype != torch.bfloat16 or not weight.is_cuda:
            raise ValueError("expected a 2-D BF16 CUDA tensor")
        self.weight = weight.contiguous()
        self.bias = bias
        self.N, self.K = map(int, weight.shape)
        self.device = weight.device

    @property
    def bytes(self) -> int:
        return 2 * self.N * self.K

    coded_bytes = bytes

    def __call__(self, x, y):
        dense_gemv(self.weight, x, y, self.bias)

    def linear(self, x, out=None):
        import torch

        x2 = x.reshape(-1, self.K)
        y = torch.empty((x2.shape[0], self.N), device=self.device, dtype=torch.bfloat16) if out is None else out.reshape(-1, self.N)
        for lo in range(0, x2.shape[0], DENSE_MAX_M):
            dense_gemv(self.weight, x2[lo:lo + DENSE_MAX_M], y[lo:lo + DENSE_MAX_M], self.bias)
        return y.reshape(*x.shape[:-1], self.N)


class Stats:
    """How often ``linear`` took the GEMV (by batch rows) and why it did not (by reason), as the reference counts them
    (``glc_serve/miv_gemv.py`` ``STATS``)."""

    def __init__(self):
        self.reset()

    def reset(self):
        self.gemv_by_m, self.fallback_by_reason = {}, {}


STATS = Stats()
_ENABLED = True


def enable(on: bool = True) -> None:
    """Switches the GEMV route of ``linear`` on or off for the process (off: every call is ``F.linear``)."""
    global _ENABLED
    _ENABLED = bool(on)


def ineligible(x, weight):
    """Why ``linear`` cannot hand this product to the GEMV (a short reason), or None when it can."""
    import torch

    if not (weight.is_cuda and x.is_cuda):
        return "not_cuda"
    if weight.dtype != torch.bfloat16 or weight.dim() != 2:
        return "weight_not_bf16_matrix"
    if x.dtype != torch.bfloat16:
        return "x_not_bf16"
    k = int(weight.shape[1])
    if x.shape[-1] != k:
        return "shape_mismatch"
    if k % 8:
        return "k_not_multiple_of_8"
    m = x.numel() // max(1, k)
    if not 1 <= m <= DENSE_MAX_M:
        return "m_gt8" if m > DENSE_MAX_M else "m_lt1"
    if weight.stride(1) != 1 or weight.stride(0) % 8 or weight.data_ptr() % 16:
        return "weight_layout"
    return None


def linear(x, weight, bias=None):
    """``F.linear`` semantics over a dense BF16 weight: the library's M-invariant GEMV when the call has 1 to 8 rows and the
    operands meet its layout rules, else ``F.linear`` (counted in ``STATS`` with the reason) - the role of the reference's
    ``miv_gemv.linear`` (``glc_serve/miv_gemv.py:916-941``)."""
    import torch
    import torch.nn.functional as F

    why = "disabled" if not _ENABLED else ineligible(x, weight)
    if why is not None:
        STATS.fallback_by_reason[why] = STATS.fallback_by_reason.get(why, 0) + 1
        return F.linear(x, weight, bias)
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    b = None
    if bias is not None:
        b = bias if (bias.dtype == torch.bfloat16 and bias.is_contiguous()) else bias.to(torch.bfloat16).contiguous()
    m = int(x2.shape[0])
    STATS.gemv_by_m[m] = STATS.gemv_by_m.get(m, 0) + 1
    y = torch.empty((m, weight.shape[0]), device=weight.device, dtype=torch.bfloat16)
    dense_gemv(weight, x2, y, b)
    return y.reshape(*x.shape[:-1], weight.shape[0])


def install_dense(root, *, prefix_filter=None) -> int:
    """Routes the forward of every plain ``nn.Linear`` under ``root`` through ``linear`` (``prefix_filter``: only modules
    whose qualified name starts with one of the prefixes).  Returns how many were wrapped; a module is wrapped once
    (the reference's ``install_dense``, ``glc_serve/miv_gemv.py:944-969``)."""
    from torch import nn

    prefixes = tuple(prefix_filter) if prefix_filter else None
    count = 0
    for name, module in root.named_modules():
        if type(module) is not nn.Linear or getattr(module, "_dense_gemv_installed", False):
            continue
        if prefixes and not name.startswith(prefixes):
            continue
        module.forward = (lambda x, _m=module: linear(x, _m.weight, _m.bias))
        module._dense_gemv_installed = True
        count += 1
    return count
