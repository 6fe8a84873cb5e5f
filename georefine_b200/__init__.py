"""B200-native BCTX path: host codec, CUDA decode of indexed frames, fused decode-GEMV/GEMM.

Public surface (names follow the reference's context runtime):
  codec.encode / codec.decode / codec.CodecError      frame codec (host)
  gpu.index_frame / gpu.CudaContextTensor             indexed frame on a GPU: decode, gather_rows, linear
  resident.ResidentWeight                             weight descriptor: __call__(x, y), gemm, gemv, decode
  serving.BctxLinear / serving.BctxEmbedding          nn.Module adapters
  tp.ColumnParallelLinear / tp.RowParallelLinear      tensor-parallel shards of a weight
"""
from .codec import CodecError, decode, encode  # noqa: F401

__all__ = ["encode", "decode", "CodecError"]
