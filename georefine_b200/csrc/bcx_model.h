// Static probability model of one BCTX stream kind: per context, validated prefix sums of the 16-bit
// frequencies and an inverse index from slot to symbol.  Shared by the host walker and (through its
// exported tables) by the CUDA decoder of unchanged streams.
//
// Word split (reference: context-runtime/georefine_context_runtime/bitexact_context_ans.cpp:9-12):
//   main     = exponent(8) << 2 | mantissa[6:5]      10 bits, vocabulary 1024
//   residual = sign << 5 | mantissa[4:0]              6 bits, vocabulary 64
#pragma once
#include <cstdint>
#include <vector>

namespace grb {

inline uint32_t main_symbol(uint16_t w) { return (uint32_t(w) >> 5) & 0x3FFu; }
inline uint32_t residual_symbol(uint16_t w) { return ((uint32_t(w) >> 10) & 32u) | (w & 31u); }
inline uint16_t join_word(uint32_t main, uint32_t residual) {
  return uint16_t((main << 5) | (residual & 31u) | ((residual & 32u) << 10));
}

constexpr uint32_t kBucketShift = 4;                   // 16 slots per bucket
constexpr uint32_t kBuckets = 65536u >> kBucketShift;  // 4096 buckets per context

class Model {
 public:
  // False when a frequency exceeds 2^16, or a context's sum is neither 0 nor 2^16.
  bool load(const uint32_t* freq, uint32_t nctx, uint32_t vocab) {
    nctx_ = nctx;
    vocab_ = vocab;
    cum_.assign(size_t(nctx) * (vocab + 1), 0);
    bucket_.assign(size_t(nctx) * kBuckets, 0);
    live_.assign(nctx, 0);
    for (uint32_t cx = 0; cx < nctx; ++cx) {
      uint32_t* c = &cum_[size_t(cx) * (vocab + 1)];
      uint64_t run = 0;
      for (uint32_t s = 0; s < vocab; ++s) {
        const uint32_t f = freq[size_t(cx) * vocab + s];
        c[s] = uint32_t(run);
        if (f > 65536u || run + f > 65536u) return false;
        run += f;
      }
      c[vocab] = uint32_t(run);
      if (run != 0 && run != 65536u) return false;
      live_[cx] = run == 65536u;
      if (!live_[cx]) continue;
      uint16_t* b = &bucket_[size_t(cx) * kBuckets];
      uint32_t s = 0;
      for (uint32_t k = 0; k < kBuckets; ++k) {
        const uint32_t slot = k << kBucketShift;
        while (c[s + 1] <= slot) ++s;
        b[k] = uint16_t(s);
      }
    }
    return true;
  }
  bool live(uint32_t cx) const { return live_[cx] != 0; }
  uint32_t start(uint32_t cx, uint32_t s) const { return cum_[size_t(cx) * (vocab_ + 1) + s]; }
  // The symbol whose slot range contains `slot` (context must be live).
  uint32_t find(uint32_t cx, uint32_t slot) const {
    const uint32_t* c = &cum_[size_t(cx) * (vocab_ + 1)];
    uint32_t s = bucket_[size_t(cx) * kBuckets + (slot >> kBucketShift)];
    while (c[s + 1] <= slot) ++s;
    return s;
  }
  void export_tables(uint32_t* cum, uint16_t* bucket) const {
    std::copy(cum_.begin(), cum_.end(), cum);
    std::copy(bucket_.begin(), bucket_.end(), bucket);
  }

 private:
  uint32_t nctx_ = 0, vocab_ = 0;
  std::vector<uint32_t> cum_;
  std::vector<uint16_t> bucket_;
  std::vector<uint8_t> live_;
};

}  // namespace grb
