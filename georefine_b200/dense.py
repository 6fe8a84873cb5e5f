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
