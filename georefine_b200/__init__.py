"""B200-native BCTX path: host codec, CUDA decode of indexed frames, fused decode-GEMV/GEMM.

Public surface (names follow the reference's context runtime):
  codec.encode / codec.decode / codec.CodecError      frame codec (host)
  gpu.index_frame / gpu.CudaContextTensor             indexed frame on a GPU: decode, gather_rows, linear
  resident.ResidentWeight                             weight descriptor: __call__(x, y), gemm, gemv, decode
  serving.BctxLinear / serving.BctxEmbedding          nn.Module adapters; serving.load_bctx_model
  package.build / verify / restore / decode_check     BCTX packages of safetensors checkpoints
  tp.ColumnParallelLinear / tp.RowParallelLinear      tensor-parallel shards of a weight
  serve.BatchDecoder / Batcher / FastSession / MTPSpeculator   the decode engine over compressed weights
  checkpoint.load_decoder_weights / load_mtp_head     the engine's weights from a package's frames
  sampling.Sampler                                    temperature / top-p sampling, speculative acceptance
  dense.DenseLinear / dense.linear / install_dense    the dense BF16 GEMV for weights kept uncompressed
  image_cache.ImageCache, tune, tbe                   cached resident images, per-shape tuning, TBE container reader
"""
from .codec import CodecError, decode, encode  # noqa: F401

__all__ = ["encode", "decode", "CodecError"]
