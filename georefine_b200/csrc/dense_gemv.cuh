// Dense BF16 GEMV for small batches (M <= 8) over an uncompressed weight: the yardstick the fused kernels are measured
// against ("effective bandwidth versus a dense BF16 GEMV on the same GPU"), and the linear for tensors that are kept
// dense (norm-sized or incompressible ones).  Same numerical contract as the reference's M-invariant GEMV
// (glc_serve/miv_gemv.py:103-191): a lane walks the pieces lane, lane + 32, ... of its K slice in increasing order,
// eight FMAs per 16-byte vector in element order, xor butterfly 16..1, slice partials added in slice order by one
// thread, bias added in FP32, one rounding to BF16 - so a row of y does not depend on M (1..8).
//
// B200 shape of it: HBM-bound streaming of W, so the grid is a whole number of waves of 148 SMs x 8 CTAs of 256
// threads, every CTA loops over (row, slice) items with a grid stride, and a lane keeps 128 bytes of loads in flight
// (256-bit loads where the rows are 32-byte aligned; L1 bypassed, L2 evict-first: a weight is read once per call).  x is read through the read-only path (it
// stays in L1: at most 8 x K x 2 bytes).  The number of K slices per row depends on the shape only, never on M.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace grb {

constexpr int kDenseThreads = 256;
constexpr int kDenseWarps = kDenseThreads / 32;
constexpr int kDenseUnroll = 8;
constexpr int kDenseMaxSlices = 8;

struct DenseArgs {
  const __nv_bfloat16* w;   // [rows, ldw]
  const __nv_bfloat16* x;   // [m, ldx]
  const __nv_bfloat16* bias;
  __nv_bfloat16* y;         // [m, ldy]
  int64_t ldw, ldx, ldy;
  uint32_t rows, cols;      // cols % 8 == 0
  uint32_t slices;          // K slices per row, 1..8, divides kDenseWarps
};

// A weight is read once per call: past the L1, first out of the L2.  sm_100 has 256-bit global loads; the wide kernel
// uses them (32-byte aligned rows), the narrow one is the same walk in 16-byte steps for any other alignment.
__device__ __forceinline__ void dense_load_once(const void* p, uint4& lo, uint4& hi) {
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
               : "l"(p));
}
__device__ __forceinline__ uint4 dense_load_once(const void* p, uint64_t policy) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p), "l"(policy));
  return r;
}

// Eight weights (one 16-byte vector, columns col..col+7) folded into the M running sums, element order 0..7, one FMA each.
template <int M>
__device__ __forceinline__ void dense_fold(float (&acc)[M], const uint4& w, const __nv_bfloat16* x, int64_t ldx, uint32_t col) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int m = 0; m < M; ++m) {
    const uint4 xv = __ldg(reinterpret_cast<const uint4*>(x + m * ldx + col));
    const uint32_t xx[4] = {xv.x, xv.y, xv.z, xv.w};
    float a = acc[m];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a = __fmaf_rn(__uint_as_float(xx[i] << 16), __uint_as_float(ww[i] << 16), a);
      a = __fmaf_rn(__uint_as_float(xx[i] & 0xFFFF0000u), __uint_as_float(ww[i] & 0xFFFF0000u), a);
    }
    acc[m] = a;
  }
}

// The walk of one lane over its slice: pieces of kPiece 16-byte vectors at lane, lane + 32, ... in increasing k.  The
// order of additions depends on (cols, slices, kPiece) only, never on M.
template <int M, bool WIDE>
__device__ __forceinline__ void dense_walk(float (&acc)[M], const DenseArgs& a, const __nv_bfloat16* wrow, uint32_t s, uint32_t lane) {
  constexpr uint32_t kPiece = WIDE ? 2 : 1;             // 16-byte vectors per load
  constexpr int kUnroll = WIDE ? kDenseUnroll / 2 : kDenseUnroll;
  const uint32_t pieces = (a.cols >> 3) / kPiece;
  const uint32_t p0 = uint32_t(uint64_t(s) * pieces / a.slices), p1 = uint32_t(uint64_t(s + 1) * pieces / a.slices);
  uint64_t policy = 0;
  if (!WIDE) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  uint32_t p = p0 + lane;
  for (; p + 32 * (kUnroll - 1) < p1; p += 32 * kUnroll) {
    uint4 lo[kUnroll], hi[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const __nv_bfloat16* src = wrow + size_t(p + 32 * u) * 8 * kPiece;
      if (WIDE) dense_load_once(src, lo[u], hi[u]);
      else lo[u] = dense_load_once(src, policy);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const uint32_t col = (p + 32 * u) * 8 * kPiece;
      dense_fold<M>(acc, lo[u], a.x, a.ldx, col);
      if (WIDE) dense_fold<M>(acc, hi[u], a.x, a.ldx, col + 8);
    }
  }
  for (; p < p1; p += 32) {
    uint4 lo, hi;
    const __nv_bfloat16* src = wrow + size_t(p) * 8 * kPiece;
    if (WIDE) dense_load_once(src, lo, hi);
    else lo = dense_load_once(src, policy);
    dense_fold<M>(acc, lo, a.x, a.ldx, p * 8 * kPiece);
    if (WIDE) dense_fold<M>(acc, hi, a.x, a.ldx, p * 8 * kPiece + 8);
  }
}

template <int M, bool WIDE>
__global__ void __launch_bounds__(kDenseThreads) dense_gemv_kernel(const DenseArgs a) {
  __shared__ float part[kDenseWarps][M];
  const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rows_per_cta = kDenseWarps / a.slices;
  const uint32_t groups = (a.rows + rows_per_cta - 1) / rows_per_cta;
  for (uint32_t g = blockIdx.x; g < groups; g += gridDim.x) {   // uniform per CTA: the barriers below are safe
    const uint32_t local = warp / a.slices, s = warp % a.slices;
    const uint32_t row = g * rows_per_cta + local;
    float acc[M];
#pragma unroll
    for (int m = 0; m < M; ++m) acc[m] = 0.f;
    if (row < a.rows) dense_walk<M, WIDE>(acc, a, a.w + int64_t(row) * a.ldw, s, lane);
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int off = 16; off; off >>= 1) acc[m] = __fadd_rn(acc[m], __shfl_xor_sync(0xFFFFFFFFu, acc[m], off));
    if (lane == 0)
#pragma unroll
      for (int m = 0; m < M; ++m) part[warp][m] = acc[m];
    __syncthreads();
    if (threadIdx.x < rows_per_cta * M) {
      const uint32_t r = threadIdx.x / M, m = threadIdx.x % M, out = g * rows_per_cta + r;
      if (out < a.rows) {
        float t = part[r * a.slices][m];
        for (uint32_t j = 1; j < a.slices; ++j) t = __fadd_rn(t, part[r * a.slices + j][m]);
        if (a.bias) t = __fadd_rn(t, __bfloat162float(a.bias[out]));
        a.y[int64_t(m) * a.ldy + out] = __float2bfloat16_rn(t);
      }
    }
    __syncthreads();
  }
}

// K slices per row for a shape: enough (row, slice) items to fill the GPU several times over, at least four loads per
// lane and slice, a divisor of the 8 warps of a CTA.  A function of the shape and the SM count alone.
inline uint32_t dense_slices(uint32_t rows, uint32_t cols, uint32_t sms) {
  uint32_t s = 1;
  while (s < uint32_t(kDenseMaxSlices) && uint64_t(rows) * s < uint64_t(sms) * 64 * 2 && (cols >> 3) / (2 * s) >= 32 * 4) s *= 2;
  return s;
}

}  // namespace grb
