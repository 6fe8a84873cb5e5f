// The element-wise and attention kernels of a batched decode step, around the fused linears: RMSNorm with the residual
// add folded in, rotary embedding + paged KV append, decode attention over a paged KV cache (fixed 256-position splits,
// merged in split order), SwiGLU and arg-max.  Counterparts of the reference's step kernels
// (glc_serve/fastdec_kernels.cu:83-110 rmsnorm, :324-359 attn_prep, :365-423 attn_split, :426-448 attn_combine, :451-459
// silu_mul, :462-488 argmax) and of their batched twins with a page table (glc_serve/bidec.py:71-81), for a plain
// grouped-query decoder: no per-head q/k norm, no output gate, full-width rotary embedding, head dimension 128.
//
// Numerical contract (what makes a row of the step independent of the batch it is in): every row is computed by CTAs of
// its own, with a fixed order of additions; every intermediate that the BF16 model rounds is rounded here (norm output,
// rotary products and their sum, attention output, SiLU before the product).  A KV page holds 256 positions of one
// sequence - exactly one attention split - as [kv head][position][128] BF16, so a split streams one contiguous 64 KB
// run per kv head for K and one for V, once for all the query heads of the group.
//
// These are HBM-bound streaming kernels: coalesced 128-bit loads, several CTAs resident per SM, grids far larger than
// 148 so that the tail does not matter; nothing here is GEMM-shaped (a decode query is one row), so no tensor cores.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace grb {

constexpr int kAttnDim = 128;     // head dimension the attention kernels are written for
constexpr int kAttnSplit = 256;   // positions per split = positions per KV page
constexpr int kAttnThreads = 256;
constexpr int kAttnMaxGroup = 8;  // query heads per kv head

__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }
__device__ __forceinline__ float round_bf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint32_t pack_bf(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
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
// grid (rows, nq + 2 nkv), 128 threads.
__global__ void __launch_bounds__(kAttnDim)
attn_prep_kernel(const AttnArgs a) {
  __shared__ float xs[kAttnDim];
  const uint32_t row = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const int32_t pos = a.row_pos[row], slot = a.row_seq[row];
  const __nv_bfloat16* src = a.qkv + row * a.ldq + size_t(head) * kAttnDim;
  const int32_t page = a.page_table[size_t(slot) * a.max_pages + uint32_t(pos) / kAttnSplit];
  const size_t in_page = size_t(uint32_t(pos) % kAttnSplit) * kAttnDim + d;
  if (head >= a.nq + a.nkv) {  // value head: copy
    const uint32_t vh = head - a.nq - a.nkv;
    a.v_pages[(size_t(page) * a.nkv + vh) * kAttnSplit * kAttnDim + in_page] = src[d];
    return;
  }
  const float x = __bfloat162float(src[d]);
  xs[d] = x;
  __syncthreads();
  const float c = __bfloat162float(a.cos_table[size_t(pos) * kAttnDim + d]), s = __bfloat162float(a.sin_table[size_t(pos) * kAttnDim + d]);
  const float rot = d < kAttnDim / 2 ? -xs[d + kAttnDim / 2] : xs[d - kAttnDim / 2];
  const __nv_bfloat16 o = __float2bfloat16_rn(__fadd_rn(round_bf(__fmul_rn(x, c)), round_bf(__fmul_rn(rot, s))));
  if (head < a.nq) a.q[(size_t(row) * a.nq + head) * kAttnDim + d] = o;
  else a.k_pages[(size_t(page) * a.nkv + (head - a.nq)) * kAttnSplit * kAttnDim + in_page] = o;
}

// One split of one row for one kv head and ALL the query heads of its group: the 64 KB of K and of V of the split are
// read once.  grid (max_splits, nkv, rows), 256 threads.
//   scores: half a warp per position (16 lanes x 16 bytes = one K row), G dot products per position, xor butterfly over
//           the 16 lanes; a warp handles two positions per step, eight steps in flight;
//   soft-max partials per query head: maximum, exponentials, sum (fixed order);
//   values: half a warp per position too (16 lanes x 16 bytes = one V row): acc += p[i] * V[i][d]; the sixteen
//           position groups are added in a fixed order (the halves of a warp by shuffle, the warps in warp order).
template <int G>
__global__ void __launch_bounds__(kAttnThreads, G <= 5 ? 3 : 2)
attn_split_kernel(const AttnArgs a) {
  __shared__ float score[G][kAttnSplit];
  __shared__ float red[kAttnThreads / 32];
  __shared__ float acc_sm[kAttnThreads / 32 - 1][G][kAttnDim];
  const uint32_t split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
  const int32_t nk = a.row_pos[row] + 1;
  const int32_t start = int32_t(split) * kAttnSplit;
  if (start >= nk) return;
  const uint32_t n = uint32_t(min(kAttnSplit, nk - start));
  const int32_t page = a.page_table[size_t(a.row_seq[row]) * a.max_pages + split];
  const __nv_bfloat16* kp = a.k_pages + (size_t(page) * a.nkv + kvh) * kAttnSplit * kAttnDim;
  const __nv_bfloat16* vp = a.v_pages + (size_t(page) * a.nkv + kvh) * kAttnSplit * kAttnDim;
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, half = lane >> 4, l16 = lane & 15;
  const uint32_t hq0 = kvh * G;
  // the group's queries: this lane's eight dimensions of each head
  float q[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 u = *reinterpret_cast<const uint4*>(a.q + (size_t(row) * a.nq + hq0 + g) * kAttnDim + l16 * 8);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { q[g][2 * i] = bf_lo(w[i]); q[g][2 * i + 1] = bf_hi(w[i]); }
  }
  // scores
  constexpr int kFlight = 4;     // value rows in flight per lane
  constexpr int kKeyFlight = 8;  // key rows in flight per lane
  for (uint32_t i0 = warp * 2 * kKeyFlight; i0 < n; i0 += (kAttnThreads / 32) * 2 * kKeyFlight) {
    uint4 kv[kKeyFlight];
#pragma unroll
    for (int f = 0; f < kKeyFlight; ++f) {
      const uint32_t i = i0 + 2 * f + half;
      kv[f] = i < n ? *reinterpret_cast<const uint4*>(kp + size_t(i) * kAttnDim + l16 * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int f = 0; f < kKeyFlight; ++f) {
      const uint32_t i = i0 + 2 * f + half;
      const uint32_t w[4] = {kv[f].x, kv[f].y, kv[f].z, kv[f].w};
      float dot[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float s = 0.f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s = __fmaf_rn(q[g][2 * e], bf_lo(w[e]), s);
          s = __fmaf_rn(q[g][2 * e + 1], bf_hi(w[e]), s);
        }
        dot[g] = s;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int off = 8; off; off >>= 1) dot[g] = __fadd_rn(dot[g], __shfl_xor_sync(0xFFFFFFFFu, dot[g], off));
        if (l16 == 0 && i < n) score[g][i] = __fmul_rn(dot[g], a.scaling);
      }
    }
  }
  __syncthreads();
  // soft-max partials: thread t looks at position t of every head
  const uint32_t t = threadIdx.x;
  float mx[G], sum[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float m = t < n ? score[g][t] : -INFINITY;
#pragma unroll
    for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
    __syncthreads();
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int w = 1; w < kAttnThreads / 32; ++w) m = fmaxf(m, red[w]);
    mx[g] = m;
    const float p = t < n ? expf(__fsub_rn(score[g][t], m)) : 0.f;
    sum[g] = cta_sum<kAttnThreads>(p, red);
    if (t < n) score[g][t] = p;
  }
  __syncthreads();
  // values: half a warp per position again (16 lanes x 16 bytes = one V row, eight dimensions per lane); half-warp hw of
  // the 16 takes positions hw, hw + 16, ..., four rows in flight per lane.  The two halves of a warp are added by one
  // shuffle, the eight warps through shared memory in warp order.
  const uint32_t hw = t >> 4;
  float acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = 0.f;
  for (uint32_t i0 = hw; i0 < n; i0 += 16 * kFlight) {
    uint4 vv[kFlight];
#pragma unroll
    for (int f = 0; f < kFlight; ++f) {
      const uint32_t i = i0 + 16 * f;
      vv[f] = i < n ? *reinterpret_cast<const uint4*>(vp + size_t(i) * kAttnDim + l16 * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int f = 0; f < kFlight; ++f) {
      const uint32_t i = i0 + 16 * f;
      if (i < n) {
        const uint32_t w[4] = {vv[f].x, vv[f].y, vv[f].z, vv[f].w};
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float p = score[g][i];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[g][2 * e] = __fmaf_rn(p, bf_lo(w[e]), acc[g][2 * e]);
            acc[g][2 * e + 1] = __fmaf_rn(p, bf_hi(w[e]), acc[g][2 * e + 1]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < G; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[g][e] = __fadd_rn(acc[g][e], __shfl_xor_sync(0xFFFFFFFFu, acc[g][e], 16));
  if (warp && half == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc_sm[warp - 1][g][l16 * 8 + e] = acc[g][e];
  }
  __syncthreads();
  if (warp == 0 && half == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        o[e] = acc[g][e];
#pragma unroll
        for (int k = 0; k < kAttnThreads / 32 - 1; ++k) o[e] = __fadd_rn(o[e], acc_sm[k][g][l16 * 8 + e]);
      }
      const size_t base = (size_t(row) * a.nq + hq0 + g) * a.max_splits + split;
      float4* dst = reinterpret_cast<float4*>(a.part_acc + base * kAttnDim + l16 * 8);
      dst[0] = make_float4(o[0], o[1], o[2], o[3]);
      dst[1] = make_float4(o[4], o[5], o[6], o[7]);
      if (l16 == 0) { a.part_ml[base * 2] = mx[g]; a.part_ml[base * 2 + 1] = sum[g]; }
    }
  }
}

// The splits of a (row, query head) merged in split order under their common maximum, one division, BF16 out.
// grid (rows, nq), 128 threads.
__global__ void __launch_bounds__(kAttnDim)
attn_combine_kernel(const AttnArgs a) {
  const uint32_t row = blockIdx.x, hq = blockIdx.y, d = threadIdx.x;
  const uint32_t ns = (uint32_t(a.row_pos[row]) + kAttnSplit) / kAttnSplit;   // ceil((pos + 1) / 256)
  const size_t base = (size_t(row) * a.nq + hq) * a.max_splits;
  float mx = a.part_ml[base * 2];
  for (uint32_t s = 1; s < ns; ++s) mx = fmaxf(mx, a.part_ml[(base + s) * 2]);
  float den = 0.f, num = 0.f;
  for (uint32_t s = 0; s < ns; ++s) {
    const float e = expf(__fsub_rn(a.part_ml[(base + s) * 2], mx));
    den = __fmaf_rn(e, a.part_ml[(base + s) * 2 + 1], den);
    num = __fmaf_rn(e, a.part_acc[(base + s) * kAttnDim + d], num);
  }
  a.out[(size_t(row) * a.nq + hq) * kAttnDim + d] = __float2bfloat16_rn(__fdiv_rn(num, den));
}

}  // namespace grb
