// extern "C" device entry points: argument validation, launch geometry, the activation tensor map.
// No allocation and no host synchronisation happen here; errors are returned, never thrown.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstring>
#include <mutex>

#include "../../include/georefine_b200.h"
#include "bctx_decode.cuh"
#include "bxr_kernels.cuh"
#include "bxw_kernels.cuh"
#include "bxq_kernels.cuh"
#include "peer_reduce.cuh"
#include "dense_gemv.cuh"
#include "decode_ops.cuh"

namespace {

using namespace grb;

int cuda_status(cudaError_t e) { return e == cudaSuccess ? GRB_OK : GRB_ERR_CUDA + int(e); }

uint32_t batch_tile(uint32_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : 128; }

uint64_t counter_bytes(const bxr_header* h) { return (uint64_t(h->row_blocks) * 4 + 255) & ~uint64_t(255); }

bool header_ok(const bxr_header* h) {
  return h && h->magic == BXR_MAGIC && h->layout_version == BXR_LAYOUT_VERSION && h->rows && h->cols && h->workers && h->mode <= BXR_MODE_WINDOW4 &&
         h->row_blocks == (h->rows + BXR_ROWS - 1) / BXR_ROWS && h->chunks == (h->cols + BXR_COLS - 1) / BXR_COLS;
}

BxrArgs view_of(const void* image, const bxr_header* h) {
  const auto* p = static_cast<const uint8_t*>(image);
  BxrArgs a{};
  a.lut = reinterpret_cast<const uint32_t*>(p + h->lut_at);
  a.k = BxrPowers{128u, 1u << 16};
  a.kw = BxwPowers{1u, 8u, 64u, 128u, 256u, 512u};
  a.base = p + h->base_at;
  a.items = reinterpret_cast<const bxr_item*>(p + h->items_at);
  a.worker_items = reinterpret_cast<const uint32_t*>(p + h->worker_items_at);
  a.states = reinterpret_cast<const uint32_t*>(p + h->states_at);
  a.blob_index = reinterpret_cast<const uint32_t*>(p + h->blob_index_at);
  a.blobs = p + h->blobs_at;
  a.blob_stride16 = h->blob_stride16;
  a.rows = h->rows;
  a.cols = h->cols;
  a.row_blocks = h->row_blocks;
  a.chunks = h->chunks;
  a.workers = h->workers;
  a.raw = h->mode == BXR_MODE_RAW;
  a.window = h->mode == BXR_MODE_WINDOW;
  a.window4 = h->mode == BXR_MODE_WINDOW4;
  return a;
}

// One launcher for the three fused kernels (bxr_, bxw_, bxq_kernel): opts the instantiation into its dynamic shared
// memory once per process and device, then launches one persistent CTA per worker.
// Programmatic stream serialisation: the kernel may begin (table and blob loads, decoding) while the tail of the
// previous kernel in the stream is still running; it waits in-kernel before touching x, y or the scratch.
template <auto Kernel, uint32_t kSmemBytes, int kThreads>
int launch_fused(const BxrArgs& a, const CUtensorMap& tmap, cudaStream_t stream, uint32_t cluster = 1) {
  static std::mutex mu;
  static bool done[64] = {false};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !done[dev]) {
      e = cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kSmemBytes));
      if (e != cudaSuccess) return cuda_status(e);
      if (dev >= 0 && dev < 64) done[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(a.workers);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cluster > 1) {  // consecutive CTAs form a thread-block cluster (the grid is a multiple of it)
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  return cuda_status(cudaLaunchKernelEx(&cfg, Kernel, a, tmap));
}

// Aligned partitions - workers = row blocks x P with 2 <= P <= 8 - run the 4-bit window kernel as one thread-block
// cluster of P CTAs per row block: the K parts of a row block are then added over distributed shared memory.
uint32_t cluster_of(const BxrArgs& a) {
  if (!a.window4 || a.workers % a.row_blocks) return 1;
  const uint32_t p = a.workers / a.row_blocks;
  return (p >= 2 && p <= 8 && a.chunks >= p) ? p : 1;
}

template <int MODE>
constexpr int kFusedThreads = MODE == kUmma ? kThreadsUmma : kThreadsSimt;

template <int MODE, int NB>
int launch(const BxrArgs& a, const CUtensorMap& tmap, cudaStream_t stream) {  // entropy-coded and raw images
  return launch_fused<bxr_kernel<MODE, NB>, BxrSmem<MODE, NB>::alloc, kFusedThreads<MODE>>(a, tmap, stream);
}
template <int MODE, int NB>
int launch_window(const BxrArgs& a, const CUtensorMap& tmap, cudaStream_t stream) {  // 3-bit window images
  return launch_fused<bxw_kernel<MODE, NB>, BxwSmem<MODE, NB>::alloc, kFusedThreads<MODE>>(a, tmap, stream);
}
template <int MODE, int NB>
int launch_wide(BxrArgs a, const CUtensorMap& tmap, cudaStream_t stream) {  // 4-bit window images
  a.cluster = MODE == kUmma ? cluster_of(a) : 1;
  return launch_fused<bxq_kernel<MODE, NB>, BxqSmem<MODE, NB>::alloc, kFusedThreads<MODE>>(a, tmap, stream, a.cluster);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// x viewed as [m rows][cols] BF16 with row stride ldx; box = 64 columns x tile rows, 128-byte swizzle, zeros
// outside the tensor (rows beyond m and columns beyond cols contribute nothing).
int make_x_map(CUtensorMap* map, const void* x, int64_t ldx, uint32_t m, uint32_t cols, uint32_t tile) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return GRB_ERR_UNSUPPORTED;
  const cuuint64_t dims[2] = {cols, m};
  const cuuint64_t strides[1] = {cuuint64_t(ldx) * 2};
  const cuuint32_t box[2] = {64, tile};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims, strides, box, elem,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? GRB_OK : GRB_ERR_ARGUMENT;
}

// Raw-mode image -> dense words: undo the operand-order tiling (two 64-column atoms per 128x128 tile, 16-byte
// pieces XOR-swizzled by row).  One thread per 16-byte piece.
__global__ void bxr_raw_decode_kernel(const uint8_t* blobs, uint32_t rows, uint32_t cols, uint32_t chunks, uint64_t pieces,
                                      uint16_t* out) {
  const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= pieces) return;
  const uint32_t j = uint32_t(i & 7), r = uint32_t(i >> 3) & 127, a = uint32_t(i >> 10) & 1;
  const uint64_t tile = i >> 11;
  const uint32_t rb = uint32_t(tile / chunks), c = uint32_t(tile % chunks);
  const uint32_t row = rb * BXR_ROWS + r, col = c * BXR_COLS + a * 64 + j * 8;
  if (row >= rows) return;
  const uint4 v = *reinterpret_cast<const uint4*>(blobs + tile * BXR_RAW_TILE_BYTES + a * 16384 + r * 128 + ((j ^ (r & 7)) * 16));
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  for (int e = 0; e < 8; ++e)
    if (col + e < cols) out[size_t(row) * cols + col + e] = uint16_t(w[e >> 1] >> (16 * (e & 1)));
}

template <int NB>
int gemm_tile(BxrArgs a, const void* x, int64_t ldx, cudaStream_t stream) {
  CUtensorMap map;
  const int st = make_x_map(&map, x, ldx, a.m, a.cols, NB);
  if (st) return st;
  if (a.window4) return launch_wide<kUmma, NB>(a, map, stream);
  return a.window ? launch_window<kUmma, NB>(a, map, stream) : launch<kUmma, NB>(a, map, stream);
}

template <int M>
int gemv_m(const BxrArgs& a, cudaStream_t stream) {
  CUtensorMap none{};
  return launch<kGemv, M>(a, none, stream);
}

template <int M, bool WIDE>
int dense_launch_as(const DenseArgs& a, uint32_t groups, uint32_t sms, cudaStream_t stream) {
  // whole waves of resident CTAs; the CTAs walk the remaining row groups with a grid stride
  static int resident = 0;   // per SM; the same on every device of a process (one architecture)
  if (!resident) {
    int n = 0;
    const cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, dense_gemv_kernel<M, WIDE>, kDenseThreads, 0);
    if (e != cudaSuccess) return cuda_status(e);
    resident = n > 0 ? n : 1;
  }
  const uint32_t ctas = std::min<uint32_t>(groups, sms * uint32_t(resident));
  dense_gemv_kernel<M, WIDE><<<ctas, kDenseThreads, 0, stream>>>(a);
  return cuda_status(cudaGetLastError());
}

template <int M>
int dense_launch(const DenseArgs& a, uint32_t groups, uint32_t sms, cudaStream_t stream) {
  // 256-bit loads need rows that start on 32-byte boundaries and a whole number of 32-byte pieces per row
  const bool wide = (reinterpret_cast<uintptr_t>(a.w) & 31) == 0 && (a.ldw & 15) == 0 && (a.cols & 15) == 0;
  return wide ? dense_launch_as<M, true>(a, groups, sms, stream) : dense_launch_as<M, false>(a, groups, sms, stream);
}

// Launch of a decode-step kernel with programmatic stream serialisation: the kernel calls
// griddepcontrol.launch_dependents and griddepcontrol.wait before anything else, so the kernel after it in the stream
// (a fused linear, mostly) is set up and already streams its first weights on the SMs this one leaves idle, and every
// kernel still sees the complete output of the one before it.
template <class... Params, class... Args>
int launch_step(void (*kernel)(Params...), dim3 grid, dim3 block, uint32_t smem_bytes, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cuda_status(cudaLaunchKernelEx(&cfg, kernel, Params(args)...));
}

// SM count of a device, looked up once.
int device_sm_count(int dev) {
  static std::mutex mu;
  static int sms[64] = {0};
  if (dev < 0 || dev >= 64) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (!sms[dev] && cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) sms[dev] = 0;
  return sms[dev];
}

template <int G>
int attn_part_launch(const AttnArgs& a, cudaStream_t stream) {
  static std::once_flag once[64];
  static int prepared[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return GRB_ERR_CUDA;
  std::call_once(once[dev], [&] {
    prepared[dev] = cuda_status(cudaFuncSetAttribute(attn_part_kernel<G>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kAttnPartSmem)));
  });
  if (prepared[dev]) return prepared[dev];
  constexpr uint32_t kRowsPerGroup = 16 / G;
  const uint32_t columns = (a.max_splits + kAttnPartsPerCta - 1) / kAttnPartsPerCta;
  return launch_step(attn_part_kernel<G>, dim3(columns, a.nkv, (a.rows + kRowsPerGroup - 1) / kRowsPerGroup), dim3(kAttnPartThreads),
                     kAttnPartSmem, stream, a);
}

}  // namespace

extern "C" {

uint64_t grb_bxr_workspace_bytes(const bxr_header* h, uint32_t max_m) {
  if (!header_ok(h) || !max_m) return 0;
  const uint64_t tile = batch_tile(max_m > 128 ? 128 : max_m);
  return counter_bytes(h) + uint64_t(h->partial_slots) * tile * BXR_ROWS * 4;
}

int grb_bctx_decode_words(const grb_bctx_tensor* t, const int64_t* block_ids, uint64_t count, uint16_t* out,
                          uint32_t* status, void* cuda_stream) {
  if (!t || !out || !status || !t->row_class || !t->col_class || !t->main_stream || !t->main_states || !t->main_offsets ||
      !t->main_cum || !t->main_bucket || !t->residual_stream || !t->stride || !t->cols || !t->rows ||
      t->n != uint64_t(t->rows) * t->cols || (t->mode != 0 && t->mode != 128))
    return GRB_ERR_ARGUMENT;
  if (t->mode == 128 && (!t->residual_states || !t->residual_offsets || !t->residual_cum || !t->residual_bucket))
    return GRB_ERR_ARGUMENT;
  if (count == 0) return GRB_OK;
  if (count > (uint64_t(1) << 37)) return GRB_ERR_ARGUMENT;
  BctxArgs a{};
  const uint32_t main_shift = t->main_bucket_shift ? t->main_bucket_shift : 4, resid_shift = t->residual_bucket_shift ? t->residual_bucket_shift : 4;
  if (main_shift > 16 || resid_shift > 16) return GRB_ERR_ARGUMENT;
  a.main_s = {t->main_stream, t->main_bytes, t->main_states, t->main_offsets, t->main_cum, t->main_bucket, main_shift};
  a.resid_s = {t->residual_stream, t->residual_bytes, t->residual_states, t->residual_offsets, t->residual_cum,
               t->residual_bucket, resid_shift};
  a.row_class = t->row_class;
  a.col_class = t->col_class;
  a.n = t->n;
  a.cols = t->cols;
  a.nc = t->nc;
  a.stride = t->stride;
  a.raw6 = t->mode == 0;
  a.main_contexts = t->nr * t->nc;
  a.block_ids = reinterpret_cast<const long long*>(block_ids);
  a.count = count;
  a.out = out;
  a.status = status;
  const auto stream = static_cast<cudaStream_t>(cuda_stream);
  const unsigned grid = unsigned((count + 63) / 64);
  bctx_decode_kernel<<<grid, 64, 0, stream>>>(a);
  return cuda_status(cudaGetLastError());
}

int grb_bxr_decode(const void* image, const bxr_header* h, uint16_t* out, uint32_t* status, void* cuda_stream) {
  if (!image || !header_ok(h) || !out || !status) return GRB_ERR_ARGUMENT;
  if (h->mode == BXR_MODE_RAW) {
    const uint64_t pieces = uint64_t(h->row_blocks) * h->chunks * 2048;
    bxr_raw_decode_kernel<<<unsigned((pieces + 255) / 256), 256, 0, static_cast<cudaStream_t>(cuda_stream)>>>(
        static_cast<const uint8_t*>(image) + h->blobs_at, h->rows, h->cols, h->chunks, pieces, out);
    return cuda_status(cudaGetLastError());
  }
  BxrArgs a = view_of(image, h);
  a.dense = out;
  a.status = status;
  CUtensorMap none{};
  if (a.window4) return launch_wide<kDense, 8>(a, none, static_cast<cudaStream_t>(cuda_stream));
  if (a.window) return launch_window<kDense, 8>(a, none, static_cast<cudaStream_t>(cuda_stream));
  return launch<kDense, 8>(a, none, static_cast<cudaStream_t>(cuda_stream));
}

static int check_linear(const void* image, const bxr_header* h, const void* x, int64_t ldx, uint32_t m, void* y, int64_t ldy,
                        void* ws, uint64_t ws_bytes, uint32_t* status, uint32_t tile_m) {
  if (!image || !header_ok(h) || !x || !y || !status || !m) return GRB_ERR_ARGUMENT;
  if (ldx < int64_t(h->cols) || ldy < int64_t(h->rows) || (ldx & 7) || (reinterpret_cast<uintptr_t>(x) & 15))
    return GRB_ERR_ARGUMENT;
  const uint64_t need = counter_bytes(h) + uint64_t(h->partial_slots) * tile_m * BXR_ROWS * 4;
  if (!ws || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 15)) return GRB_ERR_WORKSPACE;
  return GRB_OK;
}

int grb_bxr_gemm(const void* image, const bxr_header* h, const void* x, int64_t ldx, uint32_t m, void* y, int64_t ldy,
                 const void* bias, void* ws, uint64_t ws_bytes, uint32_t* status, void* cuda_stream) {
  return grb_bxr_gemm_next(image, h, x, ldx, m, y, ldy, bias, ws, ws_bytes, status, cuda_stream, nullptr, nullptr);
}

int grb_bxr_gemm_next(const void* image, const bxr_header* h, const void* x, int64_t ldx, uint32_t m, void* y, int64_t ldy,
                      const void* bias, void* ws, uint64_t ws_bytes, uint32_t* status, void* cuda_stream, const void* next_image,
                      const bxr_header* next_header) {
  const uint32_t tile = batch_tile(m > 128 ? 128 : m);
  int st = check_linear(image, h, x, ldx, m, y, ldy, ws, ws_bytes, status, tile);
  if (st) return st;
  const auto stream = static_cast<cudaStream_t>(cuda_stream);
  BxrArgs a = view_of(image, h);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.counters = static_cast<uint32_t*>(ws);
  a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + counter_bytes(h));
  a.status = status;
  a.ldx = ldx;
  a.ldy = ldy;
  // The hint is used where it is cheap to follow: both images in the 4-bit window layout with blobs of one size.
  if (next_image && header_ok(next_header) && a.window4 && next_header->mode == BXR_MODE_WINDOW4 && next_header->blob_stride16) {
    a.next_blobs = static_cast<const uint8_t*>(next_image) + next_header->blobs_at;
    a.next_blob_bytes = next_header->blob_stride16 << 4;
    a.next_units = next_header->row_blocks * next_header->chunks;
    a.next_workers = next_header->workers;
  }
  // Batches above one tile are processed as consecutive tiles: one pass over the weights per 128 rows.
  for (uint32_t m0 = 0; m0 < m; m0 += 128) {
    a.m = m - m0 < 128 ? m - m0 : 128;
    const auto* xt = static_cast<const __nv_bfloat16*>(x) + size_t(m0) * ldx;
    a.y = static_cast<__nv_bfloat16*>(y) + size_t(m0) * ldy;
    switch (batch_tile(a.m)) {
      case 16: st = gemm_tile<16>(a, xt, ldx, stream); break;
      case 32: st = gemm_tile<32>(a, xt, ldx, stream); break;
      case 64: st = gemm_tile<64>(a, xt, ldx, stream); break;
      default: st = gemm_tile<128>(a, xt, ldx, stream); break;
    }
    if (st) return st;
  }
  return GRB_OK;
}

int grb_bxr_gemv(const void* image, const bxr_header* h, const void* x, int64_t ldx, uint32_t m, void* y, int64_t ldy,
                 const void* bias, void* ws, uint64_t ws_bytes, uint32_t* status, void* cuda_stream) {
  if (m > uint32_t(kGemvMaxM)) return GRB_ERR_UNSUPPORTED;
  // A raw-mode image has nothing to decode and a window-mode image decodes cheaply enough for the tensor-core
  // pipeline to stay memory-bound at any batch size: both are served by that path.
  if (header_ok(h) && h->mode != BXR_MODE_CODED) return grb_bxr_gemm(image, h, x, ldx, m, y, ldy, bias, ws, ws_bytes, status, cuda_stream);
  int st = check_linear(image, h, x, ldx, m, y, ldy, ws, ws_bytes, status, kGemvMaxM);
  if (st) return st;
  BxrArgs a = view_of(image, h);
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.ldx = ldx;
  a.y = static_cast<__nv_bfloat16*>(y);
  a.ldy = ldy;
  a.m = m;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.counters = static_cast<uint32_t*>(ws);
  a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + counter_bytes(h));
  a.status = status;
  const auto stream = static_cast<cudaStream_t>(cuda_stream);
  switch (m) {
    case 1: return gemv_m<1>(a, stream);
    case 2: return gemv_m<2>(a, stream);
    case 3: return gemv_m<3>(a, stream);
    case 4: return gemv_m<4>(a, stream);
    case 5: return gemv_m<5>(a, stream);
    case 6: return gemv_m<6>(a, stream);
    case 7: return gemv_m<7>(a, stream);
    default: return gemv_m<8>(a, stream);
  }
}

// ---- dense BF16 GEMV --------------------------------------------------------------------------------
int grb_dense_gemv_bf16(const void* w, int64_t ldw, uint32_t rows, uint32_t cols, const void* x, int64_t ldx, uint32_t m, void* y,
                        int64_t ldy, const void* bias, void* cuda_stream) {
  if (!w || !x || !y || !rows || !cols || !m) return GRB_ERR_ARGUMENT;
  if (m > 8) return GRB_ERR_UNSUPPORTED;
  if ((cols & 7) || ldw < int64_t(cols) || ldx < int64_t(cols) || ldy < int64_t(rows) || (ldw & 7) || (ldx & 7) ||
      (reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 15))
    return GRB_ERR_ARGUMENT;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e);
  if (dev < 0 || dev >= 64) return GRB_ERR_UNSUPPORTED;
  const int sm_count = device_sm_count(dev);
  if (sm_count <= 0) return GRB_ERR_CUDA;
  DenseArgs a{};
  a.w = static_cast<const __nv_bfloat16*>(w);
  a.x = static_cast<const __nv_bfloat16*>(x);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.y = static_cast<__nv_bfloat16*>(y);
  a.ldw = ldw;
  a.ldx = ldx;
  a.ldy = ldy;
  a.rows = rows;
  a.cols = cols;
  a.slices = dense_slices(rows, cols, uint32_t(sm_count));
  const uint32_t groups = (rows + kDenseWarps / a.slices - 1) / (kDenseWarps / a.slices);
  const uint32_t ctas = uint32_t(sm_count);
  const auto stream = static_cast<cudaStream_t>(cuda_stream);
  switch (m) {
    case 1: return dense_launch<1>(a, groups, ctas, stream);
    case 2: return dense_launch<2>(a, groups, ctas, stream);
    case 3: return dense_launch<3>(a, groups, ctas, stream);
    case 4: return dense_launch<4>(a, groups, ctas, stream);
    case 5: return dense_launch<5>(a, groups, ctas, stream);
    case 6: return dense_launch<6>(a, groups, ctas, stream);
    case 7: return dense_launch<7>(a, groups, ctas, stream);
    default: return dense_launch<8>(a, groups, ctas, stream);
  }
}

// ---- decode-step kernels around the fused linears --------------------------------------------------------
int grb_rmsnorm_bf16(void* h, int64_t ldh, const void* delta, int64_t ldd, const void* weight, void* out, int64_t ldo, uint32_t rows,
                     uint32_t hidden, float eps, int unit_offset, void* cuda_stream) {
  if (!h || !weight || !out || !rows || !hidden) return GRB_ERR_ARGUMENT;
  if ((hidden & 7) || hidden > uint32_t(kRmsThreads * kRmsVectors * 8) || ldh < int64_t(hidden) || ldo < int64_t(hidden) || (ldh & 7) ||
      (ldo & 7) || (delta && (ldd < int64_t(hidden) || (ldd & 7))))
    return GRB_ERR_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(delta)) & 15)
    return GRB_ERR_ARGUMENT;
  return launch_step(rmsnorm_kernel, dim3(rows), dim3(kRmsThreads), 0, static_cast<cudaStream_t>(cuda_stream),
                     static_cast<__nv_bfloat16*>(h), ldh, static_cast<const __nv_bfloat16*>(delta), ldd,
                     static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), ldo, hidden, eps, unit_offset);
}

int grb_silu_mul_bf16(const void* gate_up, int64_t ldg, void* out, int64_t ldo, uint32_t rows, uint32_t f, void* cuda_stream) {
  if (!gate_up || !out || !rows || !f || (f & 7) || ldg < 2 * int64_t(f) || ldo < int64_t(f) || (ldg & 7) || (ldo & 7)) return GRB_ERR_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(gate_up) | reinterpret_cast<uintptr_t>(out)) & 15) return GRB_ERR_ARGUMENT;
  if (rows > 65535) return GRB_ERR_UNSUPPORTED;
  return launch_step(silu_mul_kernel, dim3(((f >> 3) + 255) / 256, rows), dim3(256), 0, static_cast<cudaStream_t>(cuda_stream),
                     static_cast<const __nv_bfloat16*>(gate_up), ldg, static_cast<__nv_bfloat16*>(out), ldo, f);
}

int grb_argmax_bf16(const void* logits, int64_t ld, uint32_t rows, uint32_t vocab, int32_t* out, void* cuda_stream) {
  if (!logits || !out || !rows || !vocab || ld < int64_t(vocab) || (ld & 7) || (reinterpret_cast<uintptr_t>(logits) & 15)) return GRB_ERR_ARGUMENT;
  return launch_step(argmax_kernel, dim3(rows), dim3(kArgmaxThreads), 0, static_cast<cudaStream_t>(cuda_stream),
                     static_cast<const __nv_bfloat16*>(logits), ld, vocab, out);
}

int grb_attn_decode_bf16(const grb_attn_step* s, void* cuda_stream) {
  if (!s || !s->qkv || !s->cos_table || !s->sin_table || !s->row_seq || !s->row_pos || !s->page_table || !s->k_pages || !s->v_pages ||
      !s->q || !s->part_acc || !s->part_ml || !s->out)
    return GRB_ERR_ARGUMENT;
  if (!s->rows || !s->nq || !s->nkv || !s->max_pages || !s->max_splits || s->nq % s->nkv || s->head_dim != uint32_t(kAttnDim))
    return GRB_ERR_ARGUMENT;
  if (s->ldq < int64_t(s->nq + 2 * s->nkv) * kAttnDim || (s->ldq & 7) ||
      ((reinterpret_cast<uintptr_t>(s->qkv) | reinterpret_cast<uintptr_t>(s->q) | reinterpret_cast<uintptr_t>(s->k_pages) |
        reinterpret_cast<uintptr_t>(s->v_pages) | reinterpret_cast<uintptr_t>(s->part_acc)) & 15))
    return GRB_ERR_ARGUMENT;
  if (s->rows > 65535 || s->nq + 2 * s->nkv > 65535 || s->max_splits > 2 * s->max_pages) return GRB_ERR_UNSUPPORTED;
  AttnArgs a{};
  a.qkv = static_cast<const __nv_bfloat16*>(s->qkv);
  a.ldq = s->ldq;
  a.cos_table = static_cast<const __nv_bfloat16*>(s->cos_table);
  a.sin_table = static_cast<const __nv_bfloat16*>(s->sin_table);
  a.row_seq = s->row_seq;
  a.row_pos = s->row_pos;
  a.page_table = s->page_table;
  a.max_pages = s->max_pages;
  a.k_pages = static_cast<__nv_bfloat16*>(s->k_pages);
  a.v_pages = static_cast<__nv_bfloat16*>(s->v_pages);
  a.q = static_cast<__nv_bfloat16*>(s->q);
  a.part_acc = s->part_acc;
  a.part_ml = s->part_ml;
  a.out = static_cast<__nv_bfloat16*>(s->out);
  a.rows = s->rows;
  a.nq = s->nq;
  a.nkv = s->nkv;
  a.max_splits = s->max_splits;
  a.scaling = s->scaling;
  const auto stream = static_cast<cudaStream_t>(cuda_stream);
  int st = launch_step(attn_prep_kernel, dim3(a.rows, (a.nq + 2 * a.nkv + kPrepHeadsPerCta - 1) / kPrepHeadsPerCta), dim3(kAttnDim), 0, stream, a);
  if (st) return st;
  switch (a.nq / a.nkv) {
    case 1: st = attn_part_launch<1>(a, stream); break;
    case 2: st = attn_part_launch<2>(a, stream); break;
    case 4: st = attn_part_launch<4>(a, stream); break;
    case 5: st = attn_part_launch<5>(a, stream); break;
    case 8: st = attn_part_launch<8>(a, stream); break;
    default: return GRB_ERR_UNSUPPORTED;
  }
  if (st) return st;
  return launch_step(attn_combine_kernel, dim3(a.rows * a.nq), dim3(kCombineWarps * 32), 0, stream, a);
}

// ---- allocation-free variant ----------------------------------------------------------------------
// Scratch for grb_bxr_gemv_static: one array per GPU that loads this library, held until the process exits.
// In host code the name below is only a handle; the device address comes from cudaGetSymbolAddress.
constexpr uint64_t kStaticScratchBytes = 4ull << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

uint64_t grb_static_scratch_bytes(void) { return kStaticScratchBytes; }

// Device address of the array on the current device, looked up once per device.
static int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* address[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e);
  if (dev < 0 || dev >= 64) return GRB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (!address[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess) return cuda_status(e);
    if (!p) return GRB_ERR_UNSUPPORTED;
    address[dev] = p;
  }
  *out = address[dev];
  return GRB_OK;
}

int grb_bxr_gemv_static(const void* image, const bxr_header* h, const void* x, int64_t ldx, uint32_t m, void* y, int64_t ldy,
                        const void* bias, uint32_t* status, void* cuda_stream) {
  if (!header_ok(h)) return GRB_ERR_ARGUMENT;
  // coded images run the CUDA-core GEMV (8 batch rows of partial sums); the others the narrowest tensor-core tile
  const uint64_t tile_rows = h->mode == BXR_MODE_CODED ? kGemvMaxM : 16;
  const uint64_t need = counter_bytes(h) + uint64_t(h->partial_slots) * tile_rows * BXR_ROWS * 4;
  if (need > kStaticScratchBytes) return GRB_ERR_STATIC_LIMIT;
  if (m > uint32_t(kGemvMaxM)) return GRB_ERR_UNSUPPORTED;
  void* scratch = nullptr;
  int st = static_scratch_address(&scratch);
  if (st) return st;
  // Every argument is checked before the first thing goes onto the stream: a refused call leaves the stream, the
  // output and the shared array exactly as they were.
  st = check_linear(image, h, x, ldx, m, y, ldy, scratch, kStaticScratchBytes, status, uint32_t(tile_rows));
  if (st) return st;
  // The array keeps whatever the previous call left: the per-row-block counters must start at zero.
  const cudaError_t e = cudaMemsetAsync(scratch, 0, counter_bytes(h), static_cast<cudaStream_t>(cuda_stream));
  if (e != cudaSuccess) return cuda_status(e);
  return grb_bxr_gemv(image, h, x, ldx, m, y, ldy, bias, scratch, kStaticScratchBytes, status, cuda_stream);
}

int grb_kernel_attributes(int which, int out[5]) {
  if (!out) return GRB_ERR_ARGUMENT;
  cudaFuncAttributes fa{};
  cudaError_t e;
  switch (which) {
    case 0: e = cudaFuncGetAttributes(&fa, bctx_decode_kernel); break;
    case 1: e = cudaFuncGetAttributes(&fa, bxr_kernel<kDense, 8>); break;
    case 2: e = cudaFuncGetAttributes(&fa, bxr_kernel<kGemv, 1>); break;
    case 3: e = cudaFuncGetAttributes(&fa, bxr_kernel<kUmma, 16>); break;
    case 4: e = cudaFuncGetAttributes(&fa, bxr_kernel<kUmma, 128>); break;
    case 5: e = cudaFuncGetAttributes(&fa, bxw_kernel<kDense, 8>); break;
    case 6: e = cudaFuncGetAttributes(&fa, bxw_kernel<kUmma, 16>); break;
    case 7: e = cudaFuncGetAttributes(&fa, bxw_kernel<kUmma, 128>); break;
    case 8: e = cudaFuncGetAttributes(&fa, bxq_kernel<kDense, 8>); break;
    case 9: e = cudaFuncGetAttributes(&fa, bxq_kernel<kUmma, 16>); break;
    case 10: e = cudaFuncGetAttributes(&fa, bxq_kernel<kUmma, 128>); break;
    default: return GRB_ERR_ARGUMENT;
  }
  if (e != cudaSuccess) return cuda_status(e);
  out[0] = fa.numRegs;
  out[1] = int(fa.localSizeBytes);
  out[2] = int(fa.sharedSizeBytes);
  out[3] = fa.maxDynamicSharedSizeBytes;
  out[4] = fa.maxThreadsPerBlock;
  return GRB_OK;
}

uint64_t grb_peer_control_bytes(void) { return uint64_t(kPeerControlWords) * 4; }

// A buffer other processes of the node can map: its own cudaMalloc allocation (an IPC handle names a whole
// allocation), zeroed; `handle` receives the 64 bytes a peer passes to grb_peer_open.
int grb_peer_alloc(uint64_t bytes, void** ptr, uint8_t handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (!ptr || !handle || bytes == 0) return GRB_ERR_ARGUMENT;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return cuda_status(e);
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_status(e);
  }
  memcpy(handle, &h, 64);
  *ptr = p;
  return GRB_OK;
}
int grb_peer_free(void* ptr) { return cuda_status(cudaFree(ptr)); }
// Maps a peer's buffer into this process for the CURRENT device (peer access is enabled by the runtime as needed).
int grb_peer_open(const uint8_t handle[64], void** ptr) {
  if (!ptr || !handle) return GRB_ERR_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return cuda_status(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
int grb_peer_close(void* ptr) { return cuda_status(cudaIpcCloseMemHandle(ptr)); }

int grb_peer_enable(int peer_device) {
  int current = 0;
  cudaError_t e = cudaGetDevice(&current);
  if (e != cudaSuccess) return cuda_status(e);
  if (peer_device == current) return GRB_OK;
  int can = 0;
  e = cudaDeviceCanAccessPeer(&can, current, peer_device);
  if (e != cudaSuccess) return cuda_status(e);
  if (!can) return GRB_ERR_UNSUPPORTED;
  e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    return GRB_OK;
  }
  return e == cudaSuccess ? GRB_OK : cuda_status(e);
}

int grb_peer_allreduce_bf16(const void* partial, void* const* receives, void* const* controls, uint64_t block_bytes, uint32_t rank,
                            uint32_t world, void* out, uint64_t elems, uint64_t wait_limit_ns, uint32_t* status, void* cuda_stream) {
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  if (!partial || !receives || !controls || !out || !status || world < 1 || world > uint32_t(kPeerMaxRanks) || rank >= world) return GRB_ERR_ARGUMENT;
  if (elems == 0 || (elems & 7u) || elems > 0xFFFFFFF8ull || block_bytes < 2 * elems || (block_bytes & 15u)) return GRB_ERR_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(out) & 15u) || (reinterpret_cast<uintptr_t>(partial) & 15u) || out == partial) return GRB_ERR_ARGUMENT;
  PeerArgs a{};
  for (uint32_t r = 0; r < world; ++r) {
    if (!receives[r] || !controls[r] || (reinterpret_cast<uintptr_t>(receives[r]) & 15u) || (reinterpret_cast<uintptr_t>(controls[r]) & 127u))
      return GRB_ERR_ARGUMENT;
    a.receive[r] = static_cast<uint8_t*>(receives[r]);
    a.control[r] = static_cast<uint32_t*>(controls[r]);
  }
  a.partial = static_cast<const __nv_bfloat16*>(partial);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.block_bytes = block_bytes;
  a.elems = uint32_t(elems);
  a.rank = rank;
  a.world = world;
  a.status = status;
  a.wait_limit_ns = wait_limit_ns ? wait_limit_ns : kWaitLimitNs;
  const uint64_t vectors = elems >> 3;
  // a small message stays in one CTA (no wait for other CTAs' pushes); a large one spreads over up to kPeerMaxCtas
  const uint32_t ctas = vectors <= 8 * kPeerThreads ? 1u : uint32_t(std::min<uint64_t>(kPeerMaxCtas, (vectors + 2 * kPeerThreads - 1) / (2 * kPeerThreads)));
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(kPeerThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cuda_status(cudaLaunchKernelEx(&cfg, peer_allreduce_kernel, a));
}

}  // extern "C"
