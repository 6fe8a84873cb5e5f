// Indexed decode of UNCHANGED BCTX streams: every thread resumes the serial rANS stream at one restart
// point (state, byte offset) and decodes `stride` words.  This is the CUDA counterpart of the reference's
// Triton kernel decode_words (context-runtime/georefine_context_runtime/bitexact_context_gpu_kernels.py:
// 114-169): same inputs, same output order (count * stride words, block-major), same end-of-block check
// against the next restart point, with the status bits split by cause.
//
// Differences in method: the symbol is found through a 4096-bucket inverse index plus a short forward scan
// of the prefix sums (two or three dependent loads, served by L1/L2) instead of an 11-probe bisection, and
// a block never touches memory outside [0, bytes) of its stream: overruns set a status bit and stop.
#pragma once
#include "device_utils.cuh"

namespace grb {

struct BctxStream {
  const uint8_t* bytes;
  uint64_t size;
  const uint32_t* states;
  const uint32_t* offsets;
  const uint32_t* cum;      // [nctx][vocab + 1]
  const uint16_t* bucket;   // [nctx][4096]
};

struct BctxArgs {
  BctxStream main_s, resid_s;  // resid_s: conditional residual stream (mode 128) or raw6 bytes (mode 0)
  const uint8_t* row_class;
  const uint8_t* col_class;
  uint64_t n;
  uint32_t cols, nc, stride, raw6;
  uint32_t main_contexts;
  const long long* block_ids;  // nullptr: blocks 0..count-1
  uint64_t count;
  uint16_t* out;
  uint32_t* status;
};

template <uint32_t VOCAB>
__device__ __forceinline__ uint32_t bctx_symbol(const BctxStream& st, uint32_t ctx, uint32_t& x, uint64_t& ip, uint32_t& bad) {
  const uint32_t slot = x & 0xFFFFu;
  const uint32_t* cum = st.cum + size_t(ctx) * (VOCAB + 1);
  uint32_t s = __ldg(st.bucket + size_t(ctx) * 4096 + (slot >> 4));
  uint32_t lo = __ldg(cum + s), hi = __ldg(cum + s + 1);
  while (hi <= slot && s + 1 < VOCAB) {  // bounded by the vocabulary
    ++s;
    lo = hi;
    hi = __ldg(cum + s + 1);
  }
  const uint32_t f = hi - lo;
  if (f == 0 || slot < lo || slot - lo >= f) {
    bad |= kStatusBadSymbol;
    return 0;
  }
  x = f * (x >> 16) + (slot - lo);
#pragma unroll
  for (int k = 0; k < 3; ++k)
    if (x < (1u << 23)) {
      if (ip < st.size) {
        x = (x << 8) | __ldg(st.bytes + ip);
        ++ip;
      } else {
        bad |= kStatusOverrun;
      }
    }
  if (x < (1u << 23)) bad |= kStatusLowState;
  return s;
}

__global__ void __launch_bounds__(64) bctx_decode_kernel(const BctxArgs a) {
  const uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= a.count) return;
  const uint64_t block = a.block_ids ? uint64_t(a.block_ids[i]) : i;
  const uint64_t blocks_total = (a.n + a.stride - 1) / a.stride;
  uint32_t bad = 0;
  if (block >= blocks_total) {
    atomicOr(a.status, kStatusBadArgument);
    return;
  }
  const uint64_t start = block * a.stride;
  uint32_t row = uint32_t(start / a.cols), col = uint32_t(start % a.cols);
  uint32_t x = a.main_s.states[block];
  uint64_t ip = a.main_s.offsets[block];
  uint32_t rx = 0;
  uint64_t rip = 0;
  if (!a.raw6) {
    rx = a.resid_s.states[block];
    rip = a.resid_s.offsets[block];
  }
  uint16_t* out = a.out + i * a.stride;
  const uint32_t steps = uint32_t(min(uint64_t(a.stride), a.n - start));
  // A lane's words go out eight at a time as one 16-byte store (its run of the output is contiguous); with 2-byte
  // stores the 32 lanes of a warp, 2 * stride bytes apart, would issue sixteen times as many store instructions, each
  // touching 32 sectors.  Needs runs that start on 16-byte boundaries; any other stride keeps the plain stores.
  const bool wide = (a.stride & 7u) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
  uint32_t packed[4] = {0, 0, 0, 0};
  for (uint32_t step = 0; step < steps && !bad; ++step) {
    const uint32_t ctx = uint32_t(__ldg(a.row_class + row)) * a.nc + __ldg(a.col_class + col);
    uint32_t sym = 0, res = 0;
    if (ctx >= a.main_contexts) {
      bad |= kStatusBadSymbol;
    } else {
      sym = bctx_symbol<1024>(a.main_s, ctx, x, ip, bad);
      if (a.raw6) {
        const uint64_t bit = (start + step) * 6, byte = bit >> 3;
        const uint32_t hi = byte < a.resid_s.size ? __ldg(a.resid_s.bytes + byte) : 0u;
        const uint32_t lo = byte + 1 < a.resid_s.size ? __ldg(a.resid_s.bytes + byte + 1) : 0u;
        res = (((hi << 8) | lo) >> (10 - uint32_t(bit & 7))) & 63u;
      } else {
        res = bctx_symbol<64>(a.resid_s, sym, rx, rip, bad);
      }
    }
    const uint32_t word = ((sym << 5) | (res & 31u) | ((res & 32u) << 10)) & 0xFFFFu;
    if (wide) {
      const uint32_t k = step & 7u;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (uint32_t(j) == (k >> 1)) packed[j] = (k & 1u) ? (packed[j] | word << 16) : word;
      if (k == 7u) *reinterpret_cast<uint4*>(out + step - 7) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      else if (step + 1 == steps) {  // a ragged last block: what has been gathered so far
        for (uint32_t e = 0; e <= k; ++e) out[step - k + e] = uint16_t(packed[e >> 1] >> (16 * (e & 1)));
      }
    } else {
      out[step] = uint16_t(word);
    }
    if (++col == a.cols) {
      col = 0;
      ++row;
    }
  }
  // The block must end exactly where the next one starts (or at the canonical end of the stream).
  const bool has_next = block + 1 < blocks_total;
  if (!bad) {
    const uint32_t want_x = has_next ? a.main_s.states[block + 1] : (1u << 23);
    const uint64_t want_ip = has_next ? uint64_t(a.main_s.offsets[block + 1]) : a.main_s.size;
    if (x != want_x || ip != want_ip) bad |= kStatusCheckpoint;
    if (!a.raw6) {
      const uint32_t want_rx = has_next ? a.resid_s.states[block + 1] : (1u << 23);
      const uint64_t want_rip = has_next ? uint64_t(a.resid_s.offsets[block + 1]) : a.resid_s.size;
      if (rx != want_rx || rip != want_rip) bad |= kStatusCheckpoint;
    }
  }
  if (bad) atomicOr(a.status, bad);
}

}  // namespace grb
