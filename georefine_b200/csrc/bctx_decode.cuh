// Indexed decode of UNCHANGED BCTX streams: every thread resumes the serial rANS stream at one restart
// point (state, byte offset) and decodes `stride` words.  This is the CUDA counterpart of the reference's
// Triton kernel decode_words (context-runtime/georefine_context_runtime/bitexact_context_gpu_kernels.py:
// 114-169): same inputs, same output order (count * stride words, block-major), same end-of-block check
// against the next restart point, with the status bits split by cause.
//
// Differences in method.  A lane's walk is one serial chain - symbol k+1 cannot start before symbol k has
// renormalised the state - so the kernel's time is (symbols per block) x (latency of one step), whatever the
// number of blocks; everything below shortens the step:
//  * the symbol is found through an inverse index (one 2-byte entry per bucket of 2^shift slots; the caller
//    picks the shift so that the tables of all contexts stay in L1) plus a short forward scan of the prefix
//    sums, instead of an 11-probe bisection;
//  * the stream is read through a 12-byte look-ahead window of aligned 32-bit words, refilled two symbols
//    before the bytes are needed, so no load of stream bytes sits on the chain; the number of bytes a
//    renormalisation takes (0, 1 or 2: the state after a step is at least 2^7) comes from a leading-zero
//    count, the bytes from one funnel shift;
//  * eight symbols at a time: their contexts and their six bytes of raw residuals are loaded up front, the
//    eight words leave as one 16-byte store.
// Blocks that cannot take that path (a stride that is not a multiple of 8, rows shorter than 8, unaligned
// buffers, the ragged end of the tensor) take a plain symbol-by-symbol loop.  No path touches memory
// outside its streams: the window clamps at the stream's last word, an overrun sets a status bit.
#pragma once
#include "device_utils.cuh"

namespace grb {

struct BctxStream {
  const uint8_t* bytes;
  uint64_t size;
  const uint32_t* states;
  const uint32_t* offsets;
  const uint32_t* cum;      // [nctx][vocab + 1]
  const uint16_t* bucket;   // [nctx][65536 >> shift]: the symbol that owns the first slot of each bucket
  uint32_t shift;           // log2 of the slots per bucket
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
  uint32_t s = min(uint32_t(__ldg(st.bucket + (size_t(ctx) << (16 - st.shift)) + (slot >> st.shift))), VOCAB - 1);
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

// Big-endian look-ahead over a byte stream: w0, w1 hold the eight bytes from `base` (a multiple of 4, counted
// from the stream's address rounded down to 4 bytes), w2 the four after them, already on their way.
struct ByteWindow {
  const uint32_t* words;
  uint32_t limit;   // bytes from `words` to the end of the stream's last word
  uint32_t base, w0, w1, w2;
  __device__ __forceinline__ uint32_t fetch(uint32_t off) const {
    return off < limit ? __byte_perm(__ldg(words + (off >> 2)), 0, 0x0123) : 0u;
  }
  // Returns the position of stream byte `at` in the window's own count (the stream's misalignment added).
  __device__ __forceinline__ uint32_t open(const uint8_t* bytes, uint64_t size, uint32_t at) {
    const uint32_t skew = uint32_t(reinterpret_cast<uintptr_t>(bytes) & 3u);
    words = reinterpret_cast<const uint32_t*>(bytes - skew);
    limit = uint32_t(min(uint64_t(0xFFFFFFF0u), (size + skew + 3) & ~uint64_t(3)));
    const uint32_t ip = at + skew;
    base = ip & ~3u;
    w0 = fetch(base);
    w1 = fetch(base + 4);
    w2 = fetch(base + 8);
    return ip;
  }
  // The state takes n (0..2) bytes from position ip.
  __device__ __forceinline__ void feed(uint32_t& x, uint32_t& ip, uint32_t n) {
    const uint32_t top = __funnelshift_l(w1, w0, (ip - base) * 8);
    x = __funnelshift_l(top, x, n * 8);
    ip += n;
    if (ip - base >= 4) {
      w0 = w1;
      w1 = w2;
      base += 4;
      w2 = fetch(base + 8);
    }
  }
};

// One decoding step on the look-ahead window, on one context's tables: prefix sums `cum` (vocab + 1 entries) and the
// inverse index `bucket` (65536 >> shift entries).  The scan ends at the latest on the table's last entry (65536).
// (Measured alternatives that did not pay: a bisection between the owners of this bucket's and the next bucket's first
// slots - the warp waits for its slowest lane either way, and the common case got longer - and a copy of the tables in
// shared memory: the step is bound by its chain of dependent instructions, not by where the tables live.)
template <uint32_t VOCAB>
__device__ __forceinline__ uint32_t bctx_symbol_fast(const uint32_t* cum, const uint16_t* bucket, uint32_t shift, uint32_t& x,
                                                     ByteWindow& w, uint32_t& ip) {
  const uint32_t slot = x & 0xFFFFu;
  uint32_t s = min(uint32_t(__ldg(bucket + (slot >> shift))), VOCAB - 1);
  uint32_t lo = __ldg(cum + s), hi = __ldg(cum + s + 1);
  while (hi <= slot && s + 1 < VOCAB) {
    ++s;
    lo = hi;
    hi = __ldg(cum + s + 1);
  }
  x = (hi - lo) * (x >> 16) + (slot - lo);
  w.feed(x, ip, min(2u, (uint32_t(__clz(int(x | 1u))) - 1u) >> 3));
  return s;
}

// `groups` runs of eight symbols from (row, col) on; leaves x, ip (and rx, rip) where the plain loop can carry on.
template <bool RAW6>
__device__ __forceinline__ void bctx_block_fast(const BctxArgs& a, uint32_t groups, uint64_t start, uint32_t& row, uint32_t& col,
                                                uint32_t& x, uint64_t& ip64, uint32_t& rx, uint64_t& rip64, uint16_t* out, uint32_t& bad) {
  ByteWindow mw, rw;
  uint32_t ip = mw.open(a.main_s.bytes, a.main_s.size, uint32_t(ip64));
  const uint32_t skew = ip - uint32_t(ip64);
  uint32_t rip = 0, rskew = 0;
  if (!RAW6) {
    rip = rw.open(a.resid_s.bytes, a.resid_s.size, uint32_t(rip64));
    rskew = rip - uint32_t(rip64);
  }
  const uint32_t cols = a.cols, nc = a.nc, top_ctx = a.main_contexts - 1;
  const uint32_t mshift = a.main_s.shift, rshift = a.resid_s.shift;
  const uint32_t* const mcum = a.main_s.cum;
  const uint16_t* const mbucket = a.main_s.bucket;
  const uint16_t* raw = reinterpret_cast<const uint16_t*>(a.resid_s.bytes + (start >> 2) * 3);   // 6 bytes per group
  for (uint32_t g = 0; g < groups; ++g) {
    // the eight contexts and the eight raw residuals first: nothing of this depends on the decoder's state
    const uint32_t here = uint32_t(__ldg(a.row_class + row)) * nc;
    const uint32_t below = col + 7 >= cols ? uint32_t(__ldg(a.row_class + row + 1)) * nc : here;   // a group crosses at most one row end (cols >= 8)
    uint32_t ctx[8], worst = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t c = col + j;
      const bool wrapped = c >= cols;
      ctx[j] = (wrapped ? below : here) + __ldg(a.col_class + (wrapped ? c - cols : c));
      worst = max(worst, ctx[j]);
    }
    if (worst > top_ctx) {          // labels outside the model: flag, and stay inside the tables
      bad |= kStatusBadSymbol;
#pragma unroll
      for (int j = 0; j < 8; ++j) ctx[j] = min(ctx[j], top_ctx);
    }
    uint32_t r32 = 0, r16 = 0;
    if (RAW6) {
      const uint32_t h0 = __ldg(raw + 3 * g), h1 = __ldg(raw + 3 * g + 1), h2 = __ldg(raw + 3 * g + 2);
      r32 = __byte_perm(h0 | (h1 << 16), 0, 0x0123);     // the first four bytes, most significant first
      r16 = __byte_perm(h2, 0, 0x4401);                  // the last two
    }
    uint32_t packed[4];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t sym = bctx_symbol_fast<1024>(mcum + ctx[j] * 1025u, mbucket + (size_t(ctx[j]) << (16 - mshift)), mshift, x, mw, ip);
      uint32_t res;
      if (RAW6) {
        res = j < 5 ? (r32 >> (26 - 6 * j)) & 63u : j == 5 ? ((r32 & 3u) << 4) | (r16 >> 12) : j == 6 ? (r16 >> 6) & 63u : r16 & 63u;
      } else {
        res = bctx_symbol_fast<64>(a.resid_s.cum + sym * 65u, a.resid_s.bucket + (size_t(sym) << (16 - rshift)), rshift, rx, rw, rip);
      }
      const uint32_t word = ((sym << 5) | (res & 31u) | ((res & 32u) << 10)) & 0xFFFFu;
      if (j & 1) packed[j >> 1] |= word << 16;
      else packed[j >> 1] = word;
    }
    *reinterpret_cast<uint4*>(out + 8 * g) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    col += 8;
    if (col >= cols) { col -= cols; ++row; }
  }
  ip64 = ip - skew;
  if (ip64 > a.main_s.size) bad |= kStatusOverrun;
  if (!RAW6) {
    rip64 = rip - rskew;
    if (rip64 > a.resid_s.size) bad |= kStatusOverrun;
  }
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
  // Runs of eight symbols on the look-ahead path (16-byte stores: needs runs that start on 16-byte boundaries), what
  // is left - at most seven symbols of a ragged last block, or everything when the path does not apply - step by step.
  const bool wide = (a.stride & 7u) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 15u) == 0;
  uint32_t done = 0;
  if (wide && a.cols >= 8 && (reinterpret_cast<uintptr_t>(a.resid_s.bytes) & 1u) == 0 && a.main_s.size < 0xFFFFFF00ull &&
      a.resid_s.size < 0xFFFFFF00ull) {
    const uint32_t groups = steps >> 3;
    if (a.raw6) bctx_block_fast<true>(a, groups, start, row, col, x, ip, rx, rip, out, bad);
    else bctx_block_fast<false>(a, groups, start, row, col, x, ip, rx, rip, out, bad);
    done = groups << 3;
  }
  for (uint32_t step = done; step < steps && !bad; ++step) {
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
    out[step] = uint16_t(word);
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
