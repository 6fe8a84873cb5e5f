// The element-wise and attention kernels of a batched decode step, around the fused linears: RMSNorm with the residual
// add folded in, rotary embedding + paged KV append, decode attention over a paged KV cache (fixed 128-position parts,
// merged in part order), SwiGLU and arg-max.  Counterparts of the reference's step kernels
// (glc_serve/fastdec_kernels.cu:83-110 rmsnorm, :324-359 attn_prep, :365-423 attn_split, :426-448 attn_combine, :451-459
// silu_mul, :462-488 argmax) and of their batched twins with a page table (glc_serve/bidec.py:71-81), for a plain
// grouped-query decoder: no per-head q/k norm, no output gate, full-width rotary embedding, head dimension 128.
//
// Numerical contract (what makes a row of the step independent of the batch it is in): every row is computed by CTAs of
// its own, with a fixed order of additions; every intermediate that the BF16 model rounds is rounded here (norm output,
// rotary products and their sum, attention weights, attention output, SiLU before the product).  A KV page holds 256
// positions of one sequence as [kv head][position][128] BF16, so an attention part (128 positions) streams one
// contiguous 32 KB run per kv head for K and one for V, once for all the query heads of the group and for all the rows
// of the step that belong to the same sequence and share the CTA.
//
// These are HBM-bound streaming kernels: coalesced 128-bit loads, several CTAs resident per SM, grids far larger than
// 148 so that the tail does not matter.  Only the attention has products to form (scores and weighted values of up to
// 16 query rows per part); it uses the warp-level MMA, see attn_part_kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_utils.cuh"

namespace grb {

constexpr int kAttnDim = 128;     // head dimension the attention kernels are written for
constexpr int kAttnSplit = 256;   // positions per KV page

__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
__device__ __forceinline__ float round_bf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// First thing in every kernel of this file (they are launched with programmatic stream serialisation): let the next
// kernel of the stream begin its set-up, then wait until the kernel before this one has finished and its writes are
// visible.
__device__ __forceinline__ void step_kernel_entry() {
  grid_dependents_may_launch();
  grid_dependency_wait();
}

// Sum over the CTA in a fixed order: lanes by xor butterfly, then the warps' sums in warp order.  Every thread gets it.
template <int THREADS>
__device__ __forceinline__ float cta_sum(float v, float* scratch /* THREADS / 32 floats */) {
#pragma unroll
  for (int off = 16; off; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xFFFFFFFFu, v, off));
  __syncthreads();  // scratch may still be read from a previous call
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float total = scratch[0];
#pragma unroll
  for (int w = 1; w < THREADS / 32; ++w) total = __fadd_rn(total, scratch[w]);
  return total;
}

// ---- RMSNorm (+ residual add) -----------------------------------------------------------------------
// if delta: h = bf16(h + delta), written back.  out = bf16((h * rsqrt(mean(h^2) + eps)) * (unit_offset ? 1 + w : w)).
// One CTA per row; a thread keeps its (at most kRmsVectors) 16-byte vectors in registers between the two passes.
constexpr int kRmsThreads = 256;
constexpr int kRmsVectors = 8;  // hidden <= 256 * 8 * 8 = 16384

__global__ void __launch_bounds__(kRmsThreads)
rmsnorm_kernel(__nv_bfloat16* h, int64_t ldh, const __nv_bfloat16* delta, int64_t ldd, const __nv_bfloat16* w, __nv_bfloat16* out,
               int64_t ldo, uint32_t hidden, float eps, int unit_offset) {
  step_kernel_entry();
  __shared__ float scratch[kRmsThreads / 32];
  const uint32_t row = blockIdx.x, vectors = hidden >> 3;
  uint4* hr = reinterpret_cast<uint4*>(h + row * ldh);
  const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + row * ldd) : nullptr;
  float x[kRmsVectors][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kRmsVectors; ++j) {
    const uint32_t v = threadIdx.x + j * kRmsThreads;
    if (v >= vectors) break;
    uint4 a = hr[v];
    uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    if (dr) {
      const uint4 d = dr[v];
      const uint32_t dw[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) aw[i] = pack_bf(__fadd_rn(bf_lo(aw[i]), bf_lo(dw[i])), __fadd_rn(bf_hi(aw[i]), bf_hi(dw[i])));
      hr[v] = make_uint4(aw[0], aw[1], aw[2], aw[3]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      x[j][2 * i] = bf_lo(aw[i]);
      x[j][2 * i + 1] = bf_hi(aw[i]);
      ss = __fmaf_rn(x[j][2 * i], x[j][2 * i], ss);
      ss = __fmaf_rn(x[j][2 * i + 1], x[j][2 * i + 1], ss);
    }
  }
  const float total = cta_sum<kRmsThreads>(ss, scratch);
  const float r = rsqrtf(__fadd_rn(__fdiv_rn(total, float(hidden)), eps));
  uint4* orow = reinterpret_cast<uint4*>(out + row * ldo);
#pragma unroll
  for (int j = 0; j < kRmsVectors; ++j) {
    const uint32_t v = threadIdx.x + j * kRmsThreads;
    if (v >= vectors) break;
    const uint4 wv = reinterpret_cast<const uint4*>(w)[v];
    const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float s0 = bf_lo(ww[i]), s1 = bf_hi(ww[i]);
      if (unit_offset) { s0 = __fadd_rn(1.f, s0); s1 = __fadd_rn(1.f, s1); }
      o[i] = pack_bf(__fmul_rn(__fmul_rn(x[j][2 * i], r), s0), __fmul_rn(__fmul_rn(x[j][2 * i + 1], r), s1));
    }
    orow[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---- SwiGLU: out = bf16(bf16(silu(gate)) * up), gate|up side by side in one row --------------------------
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __nv_bfloat16* gu, int64_t ldg, __nv_bfloat16* out, int64_t ldo, uint32_t f) {
  step_kernel_entry();
  const uint32_t row = blockIdx.y, v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= (f >> 3)) return;
  const uint4 g = reinterpret_cast<const uint4*>(gu + row * ldg)[v];
  const uint4 u = reinterpret_cast<const uint4*>(gu + row * ldg + f)[v];
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float g0 = bf_lo(gw[i]), g1 = bf_hi(gw[i]);
    const float a0 = round_bf(__fdiv_rn(g0, __fadd_rn(1.f, expf(-g0)))), a1 = round_bf(__fdiv_rn(g1, __fadd_rn(1.f, expf(-g1))));
    o[i] = pack_bf(__fmul_rn(a0, bf_lo(uw[i])), __fmul_rn(a1, bf_hi(uw[i])));
  }
  reinterpret_cast<uint4*>(out + row * ldo)[v] = make_uint4(o[0], o[1], o[2], o[3]);
}

// ---- arg-max of a row of logits, first maximum wins -----------------------------------------------------
constexpr int kArgmaxThreads = 1024;
__global__ void __launch_bounds__(kArgmaxThreads)
argmax_kernel(const __nv_bfloat16* logits, int64_t ld, uint32_t vocab, int32_t* out) {
  step_kernel_entry();
  __shared__ float best_v[kArgmaxThreads / 32];
  __shared__ int best_i[kArgmaxThreads / 32];
  const __nv_bfloat16* r = logits + blockIdx.x * ld;
  float bv = -INFINITY;
  int bi = 0x7FFFFFFF;
  auto take = [&](float v, int i) {
    if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
  };
  const uint32_t vectors = vocab >> 3;
  for (uint32_t v = threadIdx.x; v < vectors; v += kArgmaxThreads) {
    const uint4 a = reinterpret_cast<const uint4*>(r)[v];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      take(bf_lo(aw[i]), int(v * 8 + 2 * i));
      take(bf_hi(aw[i]), int(v * 8 + 2 * i + 1));
    }
  }
  for (uint32_t i = (vectors << 3) + threadIdx.x; i < vocab; i += kArgmaxThreads) take(__bfloat162float(r[i]), int(i));
#pragma unroll
  for (int off = 16; off; off >>= 1) {
    const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
    const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
    take(ov, oi);
  }
  if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < kArgmaxThreads / 32; ++w) take(best_v[w], best_i[w]);
    out[blockIdx.x] = bi;
  }
}

// ---- attention ---------------------------------------------------------------------------------------------
// Rows of a step: row r belongs to sequence slot row_seq[r] and sits at position row_pos[r] of it.  The sequence's
// pages: page_table[slot * max_pages + p / 256]; page g of a layer's cache: [kv head][256][128] BF16.
struct AttnArgs {
  const __nv_bfloat16* qkv;   // [rows][ldq]: nq query heads | nkv key heads | nkv value heads, 128 each
  int64_t ldq;
  const __nv_bfloat16* cos_table;  // [positions][128]
  const __nv_bfloat16* sin_table;
  const int32_t* row_seq;     // [rows]
  const int32_t* row_pos;     // [rows]
  const int32_t* page_table;  // [slots][max_pages]
  uint32_t max_pages;
  __nv_bfloat16* k_pages;     // [pages][nkv][256][128]
  __nv_bfloat16* v_pages;
  __nv_bfloat16* q;           // [rows][nq][128]: rotated queries
  float* part_acc;            // [rows][nq][max_splits][128]
  float* part_ml;             // [rows][nq][max_splits][2]: split maximum, split sum
  __nv_bfloat16* out;         // [rows][nq * 128]
  uint32_t rows, nq, nkv, max_splits;
  float scaling;
};

// Rotary embedding of the query and key heads (rotate-half convention, each product and the sum rounded to BF16 as
// the BF16 model does), queries to `q`, keys and values appended to the row's page at its position.
// grid (rows, ceil((nq + 2 nkv) / 2)), 128 threads: 64 threads per head (a thread owns dimensions d and d + 64, the two
// that the rotation pairs), two heads per CTA (more per CTA was measured slower on a one-row step).
constexpr int kPrepHeadsPerCta = 2;
__global__ void __launch_bounds__(kAttnDim)
attn_prep_kernel(const AttnArgs a) {
  step_kernel_entry();
  const uint32_t row = blockIdx.x, d = threadIdx.x & 63u;
  const int32_t pos = a.row_pos[row], slot = a.row_seq[row];
  const int32_t page = a.page_table[size_t(slot) * a.max_pages + uint32_t(pos) / kAttnSplit];
  const size_t in_page = size_t(uint32_t(pos) % kAttnSplit) * kAttnDim;
  const float c0 = __bfloat162float(a.cos_table[size_t(pos) * kAttnDim + d]), c1 = __bfloat162float(a.cos_table[size_t(pos) * kAttnDim + d + 64]);
  const float s0 = __bfloat162float(a.sin_table[size_t(pos) * kAttnDim + d]), s1 = __bfloat162float(a.sin_table[size_t(pos) * kAttnDim + d + 64]);
  const uint32_t heads = a.nq + 2 * a.nkv;
#pragma unroll
  for (int i = 0; i < kPrepHeadsPerCta / 2; ++i) {
    const uint32_t head = blockIdx.y * kPrepHeadsPerCta + 2 * i + (threadIdx.x >> 6);
    if (head >= heads) break;
    const __nv_bfloat16* src = a.qkv + row * a.ldq + size_t(head) * kAttnDim;
    const __nv_bfloat16 lo = src[d], hi = src[d + 64];
    if (head >= a.nq + a.nkv) {  // value head: copy
      __nv_bfloat16* dst = a.v_pages + (size_t(page) * a.nkv + (head - a.nq - a.nkv)) * kAttnSplit * kAttnDim + in_page;
      dst[d] = lo;
      dst[d + 64] = hi;
      continue;
    }
    const float x0 = __bfloat162float(lo), x1 = __bfloat162float(hi);
    // out[d] = x[d] cos[d] - x[d + 64] sin[d];  out[d + 64] = x[d + 64] cos[d + 64] + x[d] sin[d + 64]
    const __nv_bfloat16 o0 = __float2bfloat16_rn(__fadd_rn(round_bf(__fmul_rn(x0, c0)), round_bf(__fmul_rn(-x1, s0))));
    const __nv_bfloat16 o1 = __float2bfloat16_rn(__fadd_rn(round_bf(__fmul_rn(x1, c1)), round_bf(__fmul_rn(x0, s1))));
    __nv_bfloat16* dst = head < a.nq ? a.q + (size_t(row) * a.nq + head) * kAttnDim
                                     : a.k_pages + (size_t(page) * a.nkv + (head - a.nq)) * kAttnSplit * kAttnDim + in_page;
    dst[d] = o0;
    dst[d + 64] = o1;
  }
}

// ---- one part (128 positions) of the context, for one kv head and a group of rows ----------------------------
// grid (parts, kv heads, row groups), 128 threads, 64 KB of dynamic shared memory, three CTAs per SM.
//
// A row group is R = 16 / G consecutive rows of the step (G = query heads per kv head).  Inside a group, each run of
// rows that belong to one sequence - the k + 1 rows of a speculative verify, the rows of a prompt chunk, or a single
// row of a plain decode step - shares its passes: a pass brings the 32 KB of K and the 32 KB of V of one part into
// shared memory once (16-byte asynchronous copies, the 16-byte pieces of a row permuted by the row's low bits so that
// the matrix loads below are conflict-free) for all the run's rows and all G query heads: the M = 16 rows of a
// warp-level MMA are (row of the run, query head).
//   scores  S[16 x 32 per warp] = Q[16 x 128] K^T   mma.m16n8k16, K fragments by ldmatrix
//   soft-max partials per warp over its 32 positions (each row of the MMA masked by its own context length)
//   values  O[16 x 128] += P[16 x 32] V[32 x 128]   P from the score registers rounded to BF16, V by ldmatrix.trans
//   the four warps' (maximum, sum, O) merged in warp order under their common maximum -> part_acc, part_ml.
// The CTA's passes (one per run that sees the part) are listed up front and software-pipelined: the K tile of the next
// pass is requested as soon as the scores of this one are done, its V tile as soon as the merge (which borrows the V
// tile's place) is, so the memory system always has the next 32 KB in flight while the SM computes.
// Five query rows would fill 5 of the 64 rows that a tcgen05 instruction computes at least; the warp-level MMA has 16,
// and the kernel is bound by HBM either way (8 flops per byte of K and V).  Every output element depends on its own
// row's operands only, so a row's bits do not depend on what shares the MMA with it.
constexpr int kAttnPart = 128;          // positions per pass; two parts per 256-position page
constexpr int kAttnPartsPerCta = 1;     // parts per CTA (x its runs = its passes)
constexpr int kAttnPartThreads = 128;
constexpr int kAttnTileBytes = kAttnPart * kAttnDim * 2;   // 32 KB: K or V of one part
constexpr uint32_t kAttnPartSmem = 2 * kAttnTileBytes;

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// D (16 x 8, FP32) += A (16 x 16, BF16, row) * B (16 x 8, BF16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float exp2_approx(float v) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
// Byte offset of 16-byte piece `piece` (0..15) of tile row `row` (256 bytes per row).
__device__ __forceinline__ uint32_t attn_tile_offset(uint32_t row, uint32_t piece) {
  return row * 256u + ((((piece ^ row) & 7u) | (piece & 8u)) << 4);
}
// Float index of (MMA row m, dimension d) in a warp's 16 x 128 block of the merge buffer: the columns of a row are
// permuted by the row's low bits, which spreads a warp's accumulator stores (eight rows, same columns) over the banks.
__device__ __forceinline__ uint32_t attn_merge_index(uint32_t m, uint32_t d) { return m * kAttnDim + (d ^ ((m & 7u) << 2)); }

struct AttnPass {
  const __nv_bfloat16* k;   // the part's K tile: [128][128]
  const __nv_bfloat16* v;
  uint32_t run_first;       // first row of the run in the step
  uint32_t run_rows;
  int32_t start;            // first position of the part
  uint32_t npos;            // positions of the part that the run's longest row sees
  uint32_t part;
};

// One tile (K or V) of a pass into shared memory: 2048 pieces of 16 bytes, rows beyond the context zero-filled.
__device__ __forceinline__ void attn_request_tile(uint32_t dst, const __nv_bfloat16* src, uint32_t npos, uint32_t tid) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t c = tid + i * kAttnPartThreads, r = c >> 4, piece = c & 15u;
    cp_async_16(dst + attn_tile_offset(r, piece), src + r * kAttnDim + piece * 8, r < npos ? 16u : 0u);
  }
  cp_async_commit();
}

template <int G>
__global__ void __launch_bounds__(kAttnPartThreads, 3)
attn_part_kernel(const AttnArgs a) {
  step_kernel_entry();
  constexpr int R = 16 / G;              // rows of the step per group
  constexpr int kMaxPasses = R * kAttnPartsPerCta;
  extern __shared__ __align__(128) unsigned char attn_smem[];
  __shared__ float ml_sm[kAttnPartThreads / 32][16][2];
  __shared__ AttnPass passes[kMaxPasses];
  __shared__ uint32_t pass_count;
  const uint32_t ks = smem_u32(attn_smem), vs = ks + kAttnTileBytes;
  float* const merge = reinterpret_cast<float*>(attn_smem + kAttnTileBytes);   // [4][16][128], in the V tile's place once it is used up
  const uint32_t part0 = blockIdx.x * kAttnPartsPerCta, kvh = blockIdx.y, row0 = blockIdx.z * R;
  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t m0 = lane >> 2, m1 = m0 + 8;      // the two MMA rows whose scores and outputs this lane holds
  const float scale2 = __fmul_rn(a.scaling, 1.4426950408889634f);   // scores in units of log 2: exponentials are one ex2 each
  if (tid == 0) {                                  // the CTA's passes: every run of the group x the page's parts it sees
    const uint32_t group_rows = min(uint32_t(R), a.rows - row0);
    uint32_t n = 0;
    for (uint32_t run_begin = 0; run_begin < group_rows;) {
      const int32_t seq = a.row_seq[row0 + run_begin];
      uint32_t run_end = run_begin + 1;
      int32_t longest = a.row_pos[row0 + run_begin] + 1;
      while (run_end < group_rows && a.row_seq[row0 + run_end] == seq) {
        longest = max(longest, a.row_pos[row0 + run_end] + 1);
        ++run_end;
      }
      for (uint32_t h = 0; h < uint32_t(kAttnPartsPerCta); ++h) {
        const uint32_t part = part0 + h;
        const int32_t start = int32_t(part) * kAttnPart;
        if (start >= longest || part >= a.max_splits) break;
        const int32_t page = a.page_table[size_t(seq) * a.max_pages + part / (kAttnSplit / kAttnPart)];
        const size_t tile_at = ((size_t(page) * a.nkv + kvh) * kAttnSplit + (part % (kAttnSplit / kAttnPart)) * kAttnPart) * kAttnDim;
        AttnPass& p = passes[n++];
        p.k = a.k_pages + tile_at;
        p.v = a.v_pages + tile_at;
        p.run_first = row0 + run_begin;
        p.run_rows = run_end - run_begin;
        p.start = start;
        p.npos = uint32_t(min(kAttnPart, longest - start));
        p.part = part;
      }
      run_begin = run_end;
    }
    pass_count = n;
  }
  __syncthreads();
  const uint32_t n_passes = pass_count;
  if (n_passes == 0) return;
  attn_request_tile(ks, passes[0].k, passes[0].npos, tid);
  attn_request_tile(vs, passes[0].v, passes[0].npos, tid);
  for (uint32_t ip = 0; ip < n_passes; ++ip) {
    const AttnPass pass = passes[ip];
    const uint32_t run_first = pass.run_first, run_rows = pass.run_rows, part = pass.part;
    const int32_t start = pass.start;
    // the queries as A fragments: MMA row m = (row of the run) * G + (query head of the group)
    uint32_t qa[8][4];
    int32_t n0 = 0, n1 = 0;                         // positions of this part that MMA rows m0 and m1 may see
    {
      const uint32_t rl0 = m0 / G, rl1 = m1 / G;
      const bool ok0 = rl0 < run_rows, ok1 = rl1 < run_rows;
      const __nv_bfloat16* q0 = a.q + (size_t(run_first + (ok0 ? rl0 : 0)) * a.nq + kvh * G + m0 % G) * kAttnDim + (lane & 3u) * 2;
      const __nv_bfloat16* q1 = a.q + (size_t(run_first + (ok1 ? rl1 : 0)) * a.nq + kvh * G + m1 % G) * kAttnDim + (lane & 3u) * 2;
      if (ok0) n0 = min(kAttnPart, a.row_pos[run_first + rl0] + 1 - start);
      if (ok1) n1 = min(kAttnPart, a.row_pos[run_first + rl1] + 1 - start);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        qa[k][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + 16 * k) : 0u;
        qa[k][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + 16 * k) : 0u;
        qa[k][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + 16 * k + 8) : 0u;
        qa[k][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + 16 * k + 8) : 0u;
      }
    }
    cp_async_wait<1>();                             // all but the newest request: this pass's K
    __syncthreads();
    const uint32_t p_warp = warp * 32;              // this warp's 32 positions of the part
    float sc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) sc[nt][e] = 0.f;
#pragma unroll
    for (int kq = 0; kq < 4; ++kq) {                // 32 dimensions per step; the four position tiles are independent chains
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        uint32_t b[4];
        ldsm_x4(ks + attn_tile_offset(p_warp + 8 * nt + (lane & 7u), 4 * kq + (lane >> 3)), b);
        mma_bf16_16816(sc[nt], qa[2 * kq], b[0], b[1]);
        mma_bf16_16816(sc[nt], qa[2 * kq + 1], b[2], b[3]);
      }
    }
    // soft-max partials of the warp's 32 positions, per MMA row
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int32_t pos = int32_t(p_warp) + 8 * nt + int32_t(lane & 3u) * 2 + j;
        sc[nt][j] = pos < n0 ? __fmul_rn(sc[nt][j], scale2) : -INFINITY;
        sc[nt][2 + j] = pos < n1 ? __fmul_rn(sc[nt][2 + j], scale2) : -INFINITY;
        mx0 = fmaxf(mx0, sc[nt][j]);
        mx1 = fmaxf(mx1, sc[nt][2 + j]);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, 2));
    const float base0 = mx0 == -INFINITY ? 0.f : mx0, base1 = mx1 == -INFINITY ? 0.f : mx1;
    float l0 = 0.f, l1 = 0.f;
    uint32_t pa[2][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      // the weights as the MMA will see them (BF16); the sums are taken over these, so numerator and denominator agree
      const float p00 = round_bf(exp2_approx(__fsub_rn(sc[nt][0], base0))), p01 = round_bf(exp2_approx(__fsub_rn(sc[nt][1], base0)));
      const float p10 = round_bf(exp2_approx(__fsub_rn(sc[nt][2], base1))), p11 = round_bf(exp2_approx(__fsub_rn(sc[nt][3], base1)));
      l0 = __fadd_rn(l0, __fadd_rn(p00, p01));
      l1 = __fadd_rn(l1, __fadd_rn(p10, p11));
      pa[nt >> 1][(nt & 1) * 2] = pack_bf(p00, p01);
      pa[nt >> 1][(nt & 1) * 2 + 1] = pack_bf(p10, p11);
    }
    l0 = __fadd_rn(l0, __shfl_xor_sync(0xFFFFFFFFu, l0, 1));
    l0 = __fadd_rn(l0, __shfl_xor_sync(0xFFFFFFFFu, l0, 2));
    l1 = __fadd_rn(l1, __shfl_xor_sync(0xFFFFFFFFu, l1, 1));
    l1 = __fadd_rn(l1, __shfl_xor_sync(0xFFFFFFFFu, l1, 2));
    cp_async_wait<0>();
    __syncthreads();                                // V is in shared memory, and every warp is done with K
    const bool more = ip + 1 < n_passes;
    if (more) attn_request_tile(ks, passes[ip + 1].k, passes[ip + 1].npos, tid);
    float o[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) o[nt][e] = 0.f;
#pragma unroll
    for (int t = 0; t < 2; ++t) {                   // 16 positions per step
      const uint32_t vrow = p_warp + 16 * t + ((lane >> 3) & 1u) * 8 + (lane & 7u);
#pragma unroll
      for (int dn = 0; dn < 8; ++dn) {              // 16 dimensions per step
        uint32_t b[4];
        ldsm_x4_trans(vs + attn_tile_offset(vrow, 2 * dn + (lane >> 4)), b);
        mma_bf16_16816(o[2 * dn], pa[t], b[0], b[1]);
        mma_bf16_16816(o[2 * dn + 1], pa[t], b[2], b[3]);
      }
    }
    __syncthreads();                                // every warp is done with V: the merge buffer takes its place
    {
      float* mine = merge + size_t(warp) * 16 * kAttnDim;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) {
        const uint32_t col = 8 * nt + (lane & 3u) * 2;
        *reinterpret_cast<float2*>(mine + attn_merge_index(m0, col)) = make_float2(o[nt][0], o[nt][1]);
        *reinterpret_cast<float2*>(mine + attn_merge_index(m1, col)) = make_float2(o[nt][2], o[nt][3]);
      }
      if ((lane & 3u) == 0) {
        ml_sm[warp][m0][0] = mx0; ml_sm[warp][m0][1] = l0;
        ml_sm[warp][m1][0] = mx1; ml_sm[warp][m1][1] = l1;
      }
    }
    __syncthreads();
    // warp w merges MMA rows w, w + 4, ... (a lane: four dimensions), the four warps' shares in warp order under their
    // common maximum (maxima and sums are in units of log 2 here and in part_ml)
    for (uint32_t m = warp; m < run_rows * G; m += kAttnPartThreads / 32) {
      float wm[kAttnPartThreads / 32];
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < kAttnPartThreads / 32; ++w) { wm[w] = ml_sm[w][m][0]; mx = fmaxf(mx, wm[w]); }
      if (mx == -INFINITY) continue;                // this row's context ends before this part
      float den = 0.f;
      float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < kAttnPartThreads / 32; ++w) {
        const float e = wm[w] == -INFINITY ? 0.f : exp2_approx(__fsub_rn(wm[w], mx));
        den = __fmaf_rn(e, ml_sm[w][m][1], den);
        const float4 v = *reinterpret_cast<const float4*>(merge + size_t(w) * 16 * kAttnDim + attn_merge_index(m, lane * 4));
        num.x = __fmaf_rn(e, v.x, num.x);
        num.y = __fmaf_rn(e, v.y, num.y);
        num.z = __fmaf_rn(e, v.z, num.z);
        num.w = __fmaf_rn(e, v.w, num.w);
      }
      const size_t base = (size_t(run_first + m / G) * a.nq + kvh * G + m % G) * a.max_splits + part;
      *reinterpret_cast<float4*>(a.part_acc + base * kAttnDim + lane * 4) = num;
      if (lane == 0) { a.part_ml[base * 2] = mx; a.part_ml[base * 2 + 1] = den; }
    }
    if (more) {
      __syncthreads();                              // the merge buffer has been read: V of the next pass may land there
      attn_request_tile(vs, passes[ip + 1].v, passes[ip + 1].npos, tid);
    }
  }
}

// The parts of a (row, query head) merged under their common maximum, one division, BF16 out.
// One CTA of four warps per (row, query head); a lane owns four dimensions.  The parts are cut into four runs of
// consecutive parts, one per warp, each added up in part order (all of a run's loads are in flight together: on a
// one-row step this kernel is one L2 round trip long, not one per part); the four sums are then added in warp order.
// The cut depends on the row's own context length only.
constexpr int kCombineWarps = 4;
constexpr int kCombineUnroll = 8;
__global__ void __launch_bounds__(kCombineWarps * 32)
attn_combine_kernel(const AttnArgs a) {
  step_kernel_entry();
  __shared__ float4 sums[kCombineWarps - 1][32];
  __shared__ float dens[kCombineWarps - 1];
  const uint32_t pair = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
  const uint32_t row = pair / a.nq;
  const uint32_t ns = (uint32_t(a.row_pos[row]) + kAttnPart) / kAttnPart;   // ceil((pos + 1) / 128)
  const size_t base = size_t(pair) * a.max_splits;
  float mx = -INFINITY;
  for (uint32_t s = lane; s < ns; s += 32) mx = fmaxf(mx, a.part_ml[(base + s) * 2]);
#pragma unroll
  for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
  const uint32_t per = (ns + kCombineWarps - 1) / kCombineWarps;
  const uint32_t first = min(ns, warp * per), last = min(ns, first + per);
  float den = 0.f;
  float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
  for (uint32_t s0 = first; s0 < last; s0 += kCombineUnroll) {
    float4 v[kCombineUnroll];
    float2 ml[kCombineUnroll];
#pragma unroll
    for (int j = 0; j < kCombineUnroll; ++j) {
      const bool in = s0 + j < last;
      v[j] = in ? *(reinterpret_cast<const float4*>(a.part_acc + (base + s0 + j) * kAttnDim) + lane) : make_float4(0.f, 0.f, 0.f, 0.f);
      ml[j] = in ? *reinterpret_cast<const float2*>(a.part_ml + (base + s0 + j) * 2) : make_float2(-INFINITY, 0.f);
    }
#pragma unroll
    for (int j = 0; j < kCombineUnroll; ++j) {
      if (s0 + j < last) {
        const float e = exp2f(__fsub_rn(ml[j].x, mx));   // the parts' maxima are in units of log 2
        den = __fmaf_rn(e, ml[j].y, den);
        num.x = __fmaf_rn(e, v[j].x, num.x);
        num.y = __fmaf_rn(e, v[j].y, num.y);
        num.z = __fmaf_rn(e, v[j].z, num.z);
        num.w = __fmaf_rn(e, v[j].w, num.w);
      }
    }
  }
  if (warp) {
    sums[warp - 1][lane] = num;
    if (lane == 0) dens[warp - 1] = den;
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int w = 0; w < kCombineWarps - 1; ++w) {
      const float4 o = sums[w][lane];
      den = __fadd_rn(den, dens[w]);
      num.x = __fadd_rn(num.x, o.x);
      num.y = __fadd_rn(num.y, o.y);
      num.z = __fadd_rn(num.z, o.z);
      num.w = __fadd_rn(num.w, o.w);
    }
    const uint32_t lo = pack_bf(__fdiv_rn(num.x, den), __fdiv_rn(num.y, den)), hi = pack_bf(__fdiv_rn(num.z, den), __fdiv_rn(num.w, den));
    *reinterpret_cast<uint2*>(a.out + size_t(pair) * kAttnDim + lane * 4) = make_uint2(lo, hi);
  }
}

}  // namespace grb
