// Host side of the BCTX v1 context codec: static rANS models per (row class x column class) for the
// 10-bit exponent-side symbol, an optional conditional model for the 6-bit residual, MSB-first 6-bit
// packing, and the restart index that lets a GPU resume the unchanged stream every `stride` symbols.
//
// The exported names, argument lists, status codes and ownership rules are those of the reference's
// ctypes ABI (context-runtime/georefine_context_runtime/bitexact_context_ans.cpp:235-359 and
// bitexact_context_gpu_index.cpp:21-137), so a caller written against that ABI binds to this library
// unchanged.  The implementation is organised around one Model class (validated prefix sums + a
// 4096-bucket inverse index) that the CUDA decoder shares through grb_bctx_build_lookup.
//
// Nothing here throws across the ABI; outputs are written only when a call succeeds.
#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <memory>
#include <new>
#include <numeric>
#include <vector>

#include "bcx_model.h"

namespace grb {

namespace {

constexpr uint32_t kProbBits = 16;
constexpr uint32_t kProbTotal = 1u << kProbBits;
constexpr uint32_t kStateLow = 1u << 23;

struct Geometry {
  uint32_t cols, nc;
  const uint8_t* row_class;
  const uint8_t* col_class;
};

// Walks (row, col) alongside a linear element index without dividing per element.
struct Cursor {
  uint32_t row = 0, col = 0;
  void seek(uint64_t i, uint32_t cols) { row = uint32_t(i / cols); col = uint32_t(i % cols); }
  void next(uint32_t cols) { if (++col == cols) { col = 0; ++row; } }
  void prev(uint32_t cols) { if (col == 0) { col = cols - 1; --row; } else --col; }
};

inline uint32_t context_of(const Geometry& g, const Cursor& c) {
  return uint32_t(g.row_class[c.row]) * g.nc + g.col_class[c.col];
}

// Counts -> integer frequencies with sum 2^16.  Every symbol that occurs keeps at least one slot; the
// rounding surplus or deficit goes to the symbols with the largest (smallest) division remainders,
// ties resolved by symbol index, cycling if one pass is not enough.
void quantise_counts(const uint64_t* counts, uint32_t vocab, uint32_t* freq) {
  const uint64_t total = std::accumulate(counts, counts + vocab, uint64_t(0));
  if (total == 0) return;  // an unused context keeps an all-zero row
  std::vector<uint32_t> seen;
  std::vector<uint64_t> rem(vocab, 0);
  int64_t sum = 0;
  for (uint32_t s = 0; s < vocab; ++s) {
    if (counts[s] == 0) { freq[s] = 0; continue; }
    const uint64_t scaled = counts[s] << kProbBits;
    freq[s] = std::max<uint32_t>(1u, uint32_t(scaled / total));
    rem[s] = scaled % total;
    sum += freq[s];
    seen.push_back(s);
  }
  if (sum < int64_t(kProbTotal)) {
    std::sort(seen.begin(), seen.end(), [&](uint32_t a, uint32_t b) { return rem[a] != rem[b] ? rem[a] > rem[b] : a < b; });
    uint32_t lack = kProbTotal - uint32_t(sum);
    for (size_t j = 0; lack; j = (j + 1) % seen.size(), --lack) ++freq[seen[j]];
  } else if (sum > int64_t(kProbTotal)) {
    std::sort(seen.begin(), seen.end(), [&](uint32_t a, uint32_t b) { return rem[a] != rem[b] ? rem[a] < rem[b] : a > b; });
    uint32_t extra = uint32_t(sum) - kProbTotal;
    for (size_t j = 0; extra; j = (j + 1) % seen.size())
      if (freq[seen[j]] > 1) { --freq[seen[j]]; --extra; }
  }
}

struct StreamKind {
  uint32_t kind, vocab, nctx;
  StreamKind(uint32_t k, uint32_t nr, uint32_t nc) : kind(k), vocab(k ? 64u : 1024u), nctx(k ? 1024u : nr * nc) {}
};

void tally(const uint16_t* w, uint64_t n, const Geometry& g, const StreamKind& k, uint32_t* freq) {
  std::vector<uint64_t> counts(size_t(k.nctx) * k.vocab, 0);
  Cursor c;
  for (uint64_t i = 0; i < n; ++i, c.next(g.cols)) {
    const uint32_t m = main_symbol(w[i]);
    if (k.kind) ++counts[size_t(m) * k.vocab + residual_symbol(w[i])];
    else ++counts[size_t(context_of(g, c)) * k.vocab + m];
  }
  for (uint32_t cx = 0; cx < k.nctx; ++cx) quantise_counts(&counts[size_t(cx) * k.vocab], k.vocab, freq + size_t(cx) * k.vocab);
}

// Emits the stream in decode order: 4-byte little-endian state the decoder starts from, then the
// renormalisation bytes.  Coding runs from the last symbol to the first.
bool emit_stream(const uint16_t* w, uint64_t n, const Geometry& g, const StreamKind& k, const uint32_t* freq,
                 std::vector<uint8_t>& out) {
  std::vector<uint32_t> start(size_t(k.nctx) * k.vocab);
  for (uint32_t cx = 0; cx < k.nctx; ++cx) {
    uint32_t run = 0;
    for (uint32_t s = 0; s < k.vocab; ++s) { start[size_t(cx) * k.vocab + s] = run; run += freq[size_t(cx) * k.vocab + s]; }
  }
  std::vector<uint8_t> tail;
  tail.reserve(size_t(n / 2) + 16);
  uint32_t x = kStateLow;
  Cursor c;
  if (n) c.seek(n - 1, g.cols);
  for (uint64_t i = n; i-- > 0;) {
    const uint32_t m = main_symbol(w[i]);
    const size_t at = k.kind ? size_t(m) * k.vocab + residual_symbol(w[i]) : size_t(context_of(g, c)) * k.vocab + m;
    const uint32_t f = freq[at];
    if (f == 0) return false;
    const uint64_t ceiling = (uint64_t(kStateLow >> kProbBits) << 8) * f;
    while (x >= ceiling) { tail.push_back(uint8_t(x)); x >>= 8; }
    x = ((x / f) << kProbBits) + (x % f) + start[at];
    if (i) c.prev(g.cols);
  }
  out.resize(tail.size() + 4);
  for (int b = 0; b < 4; ++b) out[b] = uint8_t(x >> (8 * b));
  std::reverse_copy(tail.begin(), tail.end(), out.begin() + 4);
  return true;
}

enum WalkStatus { kOk = 0, kBadTables = 2, kBadStream = 3, kOffsetOverflow = 4 };

// One forward pass over a stream.  Optionally records (state, byte offset) before every stride-th symbol.
// Symbols go to `sym`; nothing outside the local vectors is touched on failure.
WalkStatus walk(const uint8_t* stream, size_t bytes, uint64_t n, const Geometry& g, const StreamKind& k,
                const uint16_t* resctx, const uint32_t* freq, uint32_t stride, std::vector<uint16_t>& sym,
                std::vector<uint32_t>* states, std::vector<uint32_t>* offsets) {
  Model model;
  if (!model.load(freq, k.nctx, k.vocab)) return kBadTables;
  if (bytes < 4) return kBadStream;
  uint32_t x = uint32_t(stream[0]) | uint32_t(stream[1]) << 8 | uint32_t(stream[2]) << 16 | uint32_t(stream[3]) << 24;
  if (x < kStateLow) return kBadStream;
  size_t ip = 4;
  sym.resize(size_t(n));
  uint64_t next_mark = 0;
  Cursor c;
  for (uint64_t i = 0; i < n; ++i, c.next(g.cols)) {
    if (states && i == next_mark) {
      if (ip > std::numeric_limits<uint32_t>::max()) return kOffsetOverflow;
      states->push_back(x);
      offsets->push_back(uint32_t(ip));
      next_mark += stride;
    }
    const uint32_t cx = k.kind ? resctx[i] : context_of(g, c);
    if (cx >= k.nctx || !model.live(cx)) return kBadTables;
    const uint32_t slot = x & (kProbTotal - 1);
    const uint32_t s = model.find(cx, slot);
    const uint32_t lo = model.start(cx, s), f = model.start(cx, s + 1) - lo;
    if (f == 0 || slot - lo >= f) return kBadTables;
    sym[size_t(i)] = uint16_t(s);
    const uint64_t nx = uint64_t(f) * (x >> kProbBits) + (slot - lo);
    if (nx > std::numeric_limits<uint32_t>::max()) return kBadStream;
    x = uint32_t(nx);
    while (x < kStateLow) {
      if (ip >= bytes) return kBadStream;
      x = (x << 8) | stream[ip++];
    }
  }
  return (ip == bytes && x == kStateLow) ? kOk : kBadStream;
}

bool decode_args_ok(const uint8_t* stream, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* rc, const uint8_t* cc,
                    uint32_t nr, uint32_t nc, uint32_t kind, const uint16_t* resctx, const uint32_t* freq, const void* out) {
  return stream && rc && cc && freq && out && rows && cols && kind <= 1 && nr && nc && nr <= 64 && nc <= 16 &&
         !(kind && !resctx) && n == uint64_t(rows) * cols;
}

int decode_common(const uint8_t* stream, size_t bytes, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* rc,
                  const uint8_t* cc, uint32_t nr, uint32_t nc, uint32_t kind, const uint16_t* resctx, const uint32_t* freq,
                  uint16_t* out) {
  if (!decode_args_ok(stream, n, rows, cols, rc, cc, nr, nc, kind, resctx, freq, out)) return 1;
  // Labels index the tables, so a label outside the declared class count is a malformed stream here.
  if (!kind) {
    for (uint32_t r = 0; r < rows; ++r) if (rc[r] >= nr) return 2;
    for (uint32_t c = 0; c < cols; ++c) if (cc[c] >= nc) return 2;
  }
  const Geometry g{cols, nc, rc, cc};
  const StreamKind k(kind, nr, nc);
  std::vector<uint16_t> sym;
  if (walk(stream, bytes, n, g, k, resctx, freq, 0, sym, nullptr, nullptr) != kOk) return 2;
  std::copy(sym.begin(), sym.end(), out);
  return 0;
}

}  // namespace
}  // namespace grb

extern "C" {

using namespace grb;

int bcx_frequencies(const uint16_t* w, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* rc, const uint8_t* cc,
                    uint32_t nr, uint32_t nc, uint32_t kind, uint32_t* freq) {
  try {
    if (!w || !rc || !cc || !freq || n != uint64_t(rows) * cols) return 1;
    tally(w, n, Geometry{cols, nc, rc, cc}, StreamKind(kind, nr, nc), freq);
    return 0;
  } catch (...) {
    return 3;
  }
}

int bcx_encode(const uint16_t* w, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* rc, const uint8_t* cc,
               uint32_t nr, uint32_t nc, uint32_t kind, uint32_t* freq, uint8_t** stream, size_t* stream_n) {
  try {
    if (!w || !rc || !cc || !freq || !stream || !stream_n || n != uint64_t(rows) * cols) return 1;
    const Geometry g{cols, nc, rc, cc};
    const StreamKind k(kind, nr, nc);
    tally(w, n, g, k, freq);
    std::vector<uint8_t> bytes;
    if (!emit_stream(w, n, g, k, freq, bytes)) return 3;
    auto* p = static_cast<uint8_t*>(std::malloc(bytes.size()));
    if (!p) return 2;
    std::memcpy(p, bytes.data(), bytes.size());
    *stream = p;
    *stream_n = bytes.size();
    return 0;
  } catch (...) {
    return 3;
  }
}

int bcx_decode(const uint8_t* stream, size_t bytes, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* rc,
               const uint8_t* cc, uint32_t nr, uint32_t nc, uint32_t kind, const uint16_t* resctx, const uint32_t* freq,
               uint16_t* out) {
  try {
    return decode_common(stream, bytes, n, rows, cols, rc, cc, nr, nc, kind, resctx, freq, out);
  } catch (...) {
    return 3;
  }
}

// The reference offers a second decoder with a smaller inverse table behind the same signature; this
// library has a single compact model, so both names resolve to it.
int bcx_decode_compact(const uint8_t* stream, size_t bytes, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* rc,
                       const uint8_t* cc, uint32_t nr, uint32_t nc, uint32_t kind, const uint16_t* resctx,
                       const uint32_t* freq, uint16_t* out) {
  return bcx_decode(stream, bytes, n, rows, cols, rc, cc, nr, nc, kind, resctx, freq, out);
}

void bcx_free(void* p) { std::free(p); }

int bcx_pack6(const uint16_t* w, uint64_t n, uint8_t** out, size_t* bytes) {
  if (!w || !out || !bytes) return 1;
  const size_t z = size_t((n * 6 + 7) / 8);
  auto* p = static_cast<uint8_t*>(std::calloc(z ? z : 1, 1));
  if (!p) return 2;
  // Four residuals fill three bytes exactly: aaaaaabb bbbbcccc ccdddddd.
  uint64_t i = 0;
  size_t o = 0;
  for (; i + 4 <= n; i += 4, o += 3) {
    const uint32_t a = residual_symbol(w[i]), b = residual_symbol(w[i + 1]), c = residual_symbol(w[i + 2]),
                   d = residual_symbol(w[i + 3]);
    const uint32_t v = a << 18 | b << 12 | c << 6 | d;
    p[o] = uint8_t(v >> 16); p[o + 1] = uint8_t(v >> 8); p[o + 2] = uint8_t(v);
  }
  uint32_t v = 0;
  const uint32_t left = uint32_t(n - i);
  for (uint32_t j = 0; j < left; ++j) v |= residual_symbol(w[i + j]) << (18 - 6 * j);
  for (uint32_t j = 0; o + j < z; ++j) p[o + j] = uint8_t(v >> (16 - 8 * j));
  *out = p;
  *bytes = z;
  return 0;
}

int bcx_unpack6(const uint8_t* in, size_t bytes, uint64_t n, uint16_t* out) {
  if (!in || !out || bytes != size_t((n * 6 + 7) / 8)) return 1;
  const uint32_t used = uint32_t(n * 6 % 8);
  if (used && (in[bytes - 1] & (0xFFu >> used))) return 2;
  for (uint64_t i = 0; i < n; ++i) {
    const uint64_t bit = i * 6;
    const size_t b = size_t(bit >> 3);
    const uint32_t window = uint32_t(in[b]) << 8 | (b + 1 < bytes ? in[b + 1] : 0u);
    out[i] = uint16_t((window >> (10 - uint32_t(bit & 7))) & 63u);
  }
  return 0;
}

int bcx_checkpoint(const uint8_t* stream, size_t bytes, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* rc,
                   const uint8_t* cc, uint32_t nr, uint32_t nc, uint32_t kind, const uint16_t* resctx,
                   const uint32_t* freq, uint32_t stride, uint32_t* states, uint32_t* offsets, uint16_t* out) {
  try {
    if (!stream || !rc || !cc || !freq || !states || !offsets || !out || !rows || !cols || !nr || !nc || nr > 64 ||
        nc > 16 || !stride || kind > 1 || (kind == 1 && !resctx) || n != uint64_t(rows) * cols || !n || bytes < 4 ||
        bytes > std::numeric_limits<uint32_t>::max())
      return 1;
    for (uint32_t r = 0; r < rows; ++r) if (rc[r] >= nr) return 1;
    for (uint32_t c = 0; c < cols; ++c) if (cc[c] >= nc) return 1;
    if (kind == 1)
      for (uint64_t i = 0; i < n; ++i) if (resctx[i] >= 1024u) return 1;
    const Geometry g{cols, nc, rc, cc};
    const StreamKind k(kind, nr, nc);
    std::vector<uint16_t> sym;
    std::vector<uint32_t> st, of;
    const uint64_t marks = (n - 1) / stride + 1;
    st.reserve(size_t(marks));
    of.reserve(size_t(marks));
    const WalkStatus ws = walk(stream, bytes, n, g, k, resctx, freq, stride, sym, &st, &of);
    if (ws != kOk) return int(ws);
    std::copy(st.begin(), st.end(), states);
    std::copy(of.begin(), of.end(), offsets);
    std::copy(sym.begin(), sym.end(), out);
    return 0;
  } catch (const std::bad_alloc&) {
    return 5;
  } catch (...) {
    return 6;
  }
}

// Tables the CUDA decoder of unchanged BCTX streams reads: for every context the 1025 prefix sums
// (`cum`, u32) and a 4096-bucket inverse index (`bucket`, u16: the symbol that owns the first slot of each
// 16-slot bucket).  Returns 0, 1 on bad arguments, 2 if a context neither is empty nor sums to 2^16.
int grb_bctx_build_lookup(const uint32_t* freq, uint32_t nctx, uint32_t vocab, uint32_t* cum, uint16_t* bucket) {
  try {
    if (!freq || !cum || !bucket || !nctx || (vocab != 1024 && vocab != 64)) return 1;
    Model model;
    if (!model.load(freq, nctx, vocab)) return 2;
    model.export_tables(cum, bucket);
    return 0;
  } catch (...) {
    return 3;
  }
}

}  // extern "C"
