// Host builder and host twin of the BXR1 resident layout (see bxr_format.h for the layout itself).
//
// bxr_build re-codes decoded BF16 words (the output of the BCTX index walk) into the image the fused
// kernels stream; bxr_decode_host walks an image exactly the way a GPU lane does (slot records, forward
// and backward segment cursors, exception list) and returns the words, so a loader can bind the image to
// the frame's source digest before it is uploaded.  This plays the role of the load-time transcode the
// reference performs for its other resident formats (glc_serve/bctx_v21_transcode.py) and of the digest
// check in bitexact_context_gpu.py:104-105.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <memory>
#include <new>
#include <thread>
#include <vector>

#include "bxr_format.h"

namespace {

inline uint32_t exponent_of(uint16_t w) { return (w >> 7) & 0xFFu; }
inline uint8_t raw_byte_of(uint16_t w) { return uint8_t((w & 0x7Fu) | ((w >> 8) & 0x80u)); }

struct Plan {
  uint32_t rows, cols, row_blocks, chunks, workers;
  std::vector<bxr_item> items;
  std::vector<uint32_t> worker_items;  // workers + 1
  uint32_t partial_slots = 0;
};

// Equal shares of the (row block, chunk) sequence; a share is cut at row-block boundaries into items.
Plan make_plan(uint32_t rows, uint32_t cols, uint32_t workers) {
  Plan p;
  p.rows = rows;
  p.cols = cols;
  p.row_blocks = (rows + BXR_ROWS - 1) / BXR_ROWS;
  p.chunks = (cols + BXR_COLS - 1) / BXR_COLS;
  p.workers = workers;
  const uint64_t units = uint64_t(p.row_blocks) * p.chunks;
  p.worker_items.assign(workers + 1, 0);
  std::vector<uint32_t> parts(p.row_blocks, 0);
  for (uint32_t w = 0; w < workers; ++w) {
    uint64_t u = units * w / workers;
    const uint64_t end = units * (w + 1) / workers;
    p.worker_items[w] = uint32_t(p.items.size());
    while (u < end) {
      const uint32_t rb = uint32_t(u / p.chunks), c0 = uint32_t(u % p.chunks);
      const uint32_t c1 = uint32_t(std::min<uint64_t>(p.chunks, c0 + (end - u)));
      bxr_item it{};
      it.row_block = rb;
      it.chunk_begin = c0;
      it.chunk_end = c1;
      it.part = parts[rb]++;
      p.items.push_back(it);
      u += c1 - c0;
    }
  }
  p.worker_items[workers] = uint32_t(p.items.size());
  for (auto& it : p.items) {
    it.parts = parts[it.row_block];
    it.slot = 0;
  }
  // Partial tiles of one row block occupy consecutive slots in item (= K) order.
  std::vector<uint32_t> first(p.row_blocks, 0);
  uint32_t next = 0;
  for (uint32_t rb = 0; rb < p.row_blocks; ++rb)
    if (parts[rb] > 1) { first[rb] = next; next += parts[rb]; }
  for (auto& it : p.items)
    if (it.parts > 1) it.slot = first[it.row_block] + it.part;
  p.partial_slots = next;
  return p;
}

struct Source {
  const uint16_t* words;
  uint32_t rows, cols;
  // Padded rows repeat the last row (keeps the statistics).  Padded columns never reach an output (the
  // activation tile is zero there), so they carry whatever finite word is cheapest to code.
  uint16_t at(uint32_t r, uint32_t c) const { return words[size_t(std::min(r, rows - 1)) * cols + c]; }
  uint16_t padded(uint32_t r, uint32_t c, const uint8_t* base) const {
    return c < cols ? at(r, c) : uint16_t((uint32_t(base[r]) + 12u) << 7);
  }
};

void parallel_for(uint32_t n, uint32_t threads, const std::function<void(uint32_t)>& fn) {
  threads = std::max(1u, std::min(threads, n));
  if (threads == 1) {
    for (uint32_t i = 0; i < n; ++i) fn(i);
    return;
  }
  std::atomic<uint32_t> next{0};
  std::vector<std::thread> pool;
  for (uint32_t t = 0; t < threads; ++t)
    pool.emplace_back([&] {
      for (uint32_t i = next.fetch_add(1); i < n; i = next.fetch_add(1)) fn(i);
    });
  for (auto& th : pool) th.join();
}

// Chooses the exponent window of every row: start from the row's most frequent exponent, then move the
// window by a few binades if that lowers the row's cost under the tensor-wide nibble statistics.
std::vector<uint8_t> choose_bases(const Source& src, uint32_t rows_pad, uint32_t threads) {
  std::vector<uint32_t> hist(size_t(rows_pad) * 256, 0);
  parallel_for(rows_pad, threads, [&](uint32_t r) {
    uint32_t* h = &hist[size_t(r) * 256];
    for (uint32_t c = 0; c < src.cols; ++c) ++h[exponent_of(src.at(r, c))];
  });
  std::vector<uint8_t> base(rows_pad);
  for (uint32_t r = 0; r < rows_pad; ++r) {
    const uint32_t* h = &hist[size_t(r) * 256];
    const uint32_t mode = uint32_t(std::max_element(h, h + 256) - h);
    // most frequent exponent at code 12: two binades of headroom above it, twelve below (the long tail)
    base[r] = uint8_t(std::min<int>(241, std::max<int>(0, int(mode) - 12)));
  }
  for (int round = 0; round < 2; ++round) {
    double cnt[16] = {0};
    for (uint32_t r = 0; r < rows_pad; ++r) {
      const uint32_t* h = &hist[size_t(r) * 256];
      for (uint32_t e = 0; e < 256; ++e) {
        if (!h[e]) continue;
        const int n = int(e) - int(base[r]);
        cnt[(n >= 0 && n <= 14) ? n : 15] += h[e];
      }
    }
    double total = 0;
    for (double c : cnt) total += c;
    double cost[16];
    for (int n = 0; n < 16; ++n) cost[n] = -std::log2((cnt[n] + 0.5) / (total + 8.0));
    // 32 bits for the list entry, plus a penalty: an exception costs the decoding warp a divergent patch, so the
    // window is pushed towards the side where exceptions are rarest even when the size gain is negligible
    cost[15] += 8.0 + 24.0;
    for (uint32_t r = 0; r < rows_pad; ++r) {
      const uint32_t* h = &hist[size_t(r) * 256];
      double best = 0;
      int best_base = -1;
      for (int cand = std::max(0, int(base[r]) - 3); cand <= std::min(241, int(base[r]) + 3); ++cand) {
        double bits = 0;
        for (uint32_t e = 0; e < 256; ++e) {
          if (!h[e]) continue;
          const int n = int(e) - cand;
          bits += h[e] * cost[(n >= 0 && n <= 14) ? n : 15];
        }
        if (best_base < 0 || bits < best) { best = bits; best_base = cand; }
      }
      base[r] = uint8_t(best_base);
    }
  }
  return base;
}

inline uint32_t nibble_of(uint32_t e, uint32_t base) {
  const uint32_t n = e - base;  // wraps for e < base
  return n <= 14 ? n : uint32_t(BXR_ESCAPE);
}

// Pair counts -> frequencies with sum 4096, at least 1 for every pair that occurs.
void quantise_pairs(const std::vector<uint64_t>& counts, uint32_t* freq) {
  uint64_t total = 0;
  for (uint64_t c : counts) total += c;
  std::vector<uint32_t> seen;
  std::vector<uint64_t> rem(256, 0);
  int64_t sum = 0;
  for (uint32_t s = 0; s < 256; ++s) {
    freq[s] = 0;
    if (!counts[s]) continue;
    const uint64_t scaled = counts[s] * uint64_t(BXR_PROB_TOTAL);
    freq[s] = std::max<uint32_t>(1u, uint32_t(scaled / total));
    rem[s] = scaled % total;
    sum += freq[s];
    seen.push_back(s);
  }
  if (seen.empty()) { freq[0] = BXR_PROB_TOTAL; return; }
  if (sum < BXR_PROB_TOTAL) {
    std::sort(seen.begin(), seen.end(), [&](uint32_t a, uint32_t b) { return rem[a] != rem[b] ? rem[a] > rem[b] : a < b; });
    uint32_t lack = uint32_t(BXR_PROB_TOTAL - sum);
    for (size_t j = 0; lack; j = (j + 1) % seen.size(), --lack) ++freq[seen[j]];
  } else if (sum > BXR_PROB_TOTAL) {
    // take from the largest frequencies first: they lose the least precision
    std::sort(seen.begin(), seen.end(), [&](uint32_t a, uint32_t b) { return freq[a] != freq[b] ? freq[a] > freq[b] : a < b; });
    uint32_t extra = uint32_t(sum - BXR_PROB_TOTAL);
    for (size_t j = 0; extra; j = (j + 1) % seen.size())
      if (freq[seen[j]] > 1) { --freq[seen[j]]; --extra; }
  }
}

struct StreamCoder {
  uint32_t x = BXR_STATE_LOW;
  std::vector<uint16_t>* out;
  void renorm(uint64_t ceiling) {
    if (x >= ceiling) { out->push_back(uint16_t(x)); x >>= 16; }
  }
  void put_symbol(uint32_t f, uint32_t cum) {
    renorm(uint64_t(f) << 20);
    x = ((x / f) << BXR_PROB_BITS) + (x % f) + cum;
  }
};

struct ItemCode {
  std::vector<uint16_t> words[BXR_STREAMS];         // decode order, all chunks of the item
  std::vector<uint8_t> per_chunk[BXR_STREAMS];      // words consumed in each chunk
  uint32_t state[BXR_STREAMS];
  std::vector<std::vector<uint32_t>> exceptions;    // per chunk: {segment | column in segment << 9 | exponent << 14}
};

void encode_item(const Source& src, const bxr_item& it, const uint8_t* base, const uint32_t* freq, const uint32_t* cum,
                 ItemCode& code) {
  const uint32_t nch = it.chunk_end - it.chunk_begin;
  std::vector<uint16_t> rev;
  code.exceptions.assign(nch, {});
  for (uint32_t sid = 0; sid < BXR_STREAMS; ++sid) {
    const uint32_t piece = sid / BXR_ROWS, r = sid % BXR_ROWS;  // piece = 2q + d: 16 columns of the chunk
    const uint32_t row = it.row_block * BXR_ROWS + r;
    const uint32_t b = base[row];
    rev.clear();
    StreamCoder coder;
    coder.out = &rev;
    auto& counts = code.per_chunk[sid];
    counts.assign(nch, 0);
    for (uint32_t c = it.chunk_end; c-- > it.chunk_begin;) {
      const size_t before = rev.size();
      for (int t = BXR_STEPS - 1; t >= 0; --t) {
        const uint32_t col = c * BXR_COLS + piece * BXR_STREAM_COLS + 2 * uint32_t(t);
        const uint32_t e0 = exponent_of(src.padded(row, col, base)), e1 = exponent_of(src.padded(row, col + 1, base));
        const uint32_t n0 = nibble_of(e0, b), n1 = nibble_of(e1, b);
        // an exponent outside the row window is coded as nibble 15 and listed with the chunk
        const uint32_t seg = (piece / 2) * BXR_ROWS + r, in_seg = (piece & 1) * BXR_STREAM_COLS + 2 * uint32_t(t);
        if (n0 == BXR_ESCAPE) code.exceptions[c - it.chunk_begin].push_back(seg | in_seg << 9 | e0 << 14);
        if (n1 == BXR_ESCAPE) code.exceptions[c - it.chunk_begin].push_back(seg | (in_seg + 1) << 9 | e1 << 14);
        const uint32_t sym = n0 | n1 << 4;
        coder.put_symbol(freq[sym], cum[sym]);
      }
      const size_t used = rev.size() - before;
      counts[c - it.chunk_begin] = uint8_t(used);  // at most one word per step: 8 per chunk
    }
    code.state[sid] = coder.x;
    code.words[sid].assign(rev.rbegin(), rev.rend());
  }
}

uint64_t align16(uint64_t v) { return (v + 15) & ~uint64_t(15); }

// ---- window mode ------------------------------------------------------------------------------------------
// Row windows: the 8 consecutive exponents [base, base + 7] that cover most of the row.
std::vector<uint8_t> choose_window_bases(const Source& src, uint32_t rows_pad, uint32_t threads) {
  std::vector<uint8_t> base(rows_pad);
  parallel_for(rows_pad, threads, [&](uint32_t r) {
    uint32_t h[256 + 8] = {0};
    for (uint32_t c = 0; c < src.cols; ++c) ++h[exponent_of(src.at(r, c))];
    uint32_t run = 0, best = 0, best_base = 0;
    for (uint32_t e = 0; e < 8; ++e) run += h[e];
    for (uint32_t b = 0;; ++b) {
      if (run > best) { best = run; best_base = b; }
      if (b == BXW_BASE_MAX) break;
      run += h[b + 8];
      run -= h[b];
    }
    base[r] = uint8_t(best_base);
  });
  return base;
}

// Where the word of (row in warp, column in the lane's 32) sits in the warp's part of the operand tile.
inline uint32_t window_place(uint32_t q, uint32_t rl, uint32_t j) {
  return rl * 64 + ((((q & 1) * 4 + j / 8) ^ (rl & 7)) * 8) + (j & 7);
}

// One chunk blob in window mode; false when the entry lists do not fit the slot.
bool window_blob(const Source& src, uint32_t row_block, uint32_t chunk, const uint8_t* base, std::vector<uint8_t>& blob) {
  std::vector<uint16_t> entries[16];
  std::vector<uint32_t> far;
  std::vector<uint8_t> fixed(BXW_LIST_AT, 0);
  auto* codes = reinterpret_cast<uint32_t*>(fixed.data() + BXW_CODES_AT);
  for (uint32_t warp = 0; warp < 16; ++warp) {
    const uint32_t q = warp >> 2;
    for (uint32_t rl = 0; rl < 32; ++rl) {
      const uint32_t r = (warp & 3) * 32 + rl, row = row_block * BXR_ROWS + r, b = base[row];
      uint32_t code[32];
      for (uint32_t j = 0; j < 32; ++j) {
        const uint32_t col = chunk * BXR_COLS + q * 32 + j;
        // a padded column never reaches an output: it carries the window's first exponent and a zero raw byte
        const uint16_t w = col < src.cols ? src.at(row, col) : uint16_t(b << 7);
        const int delta = int(exponent_of(w)) - int(b);
        fixed[BXW_RAW_AT + (size_t(2 * q + j / 16) * BXR_ROWS + r) * 16 + j % 16] = raw_byte_of(w);
        if (delta >= 0 && delta <= 7) { code[j] = uint32_t(delta); continue; }
        code[j] = 0;
        const uint32_t place = window_place(q, rl, j);
        int field = delta;
        if (delta < -15 || delta > 15) {
          field = BXW_DELTA_FAR;
          far.push_back(warp << BXW_PLACE_BITS | place | exponent_of(w) << 16);
        }
        entries[warp].push_back(uint16_t(place | (uint32_t(field) & 31u) << BXW_PLACE_BITS));
      }
      uint32_t word[3] = {0, 0, 0};
      for (uint32_t p = 0; p < 15; ++p) word[p / 5] |= code[2 * p] << (1 + 3 * (p % 5)) | code[2 * p + 1] << (17 + 3 * (p % 5));
      for (uint32_t t = 0; t < 3; ++t) word[t] |= ((code[30] >> t) & 1u) | ((code[31] >> t) & 1u) << 16;
      for (uint32_t t = 0; t < 3; ++t) codes[t * BXR_SEGMENTS + q * BXR_ROWS + r] = word[t];
    }
  }
  size_t total = 0;
  auto* warp_end = reinterpret_cast<uint16_t*>(fixed.data() + BXW_WARP_END_AT);
  for (uint32_t w = 0; w < 16; ++w) { warp_end[w] = uint16_t(total); total += entries[w].size(); }
  if (total > BXW_ENTRY_MAX || far.size() > BXW_FAR_MAX) return false;
  warp_end[16] = uint16_t(total);
  const uint16_t n_far = uint16_t(far.size());
  std::memcpy(fixed.data() + BXW_FAR_COUNT_AT, &n_far, 2);
  const size_t far_at = (BXW_LIST_AT + 2 * total + 3) & ~size_t(3);
  blob.assign((far_at + 4 * far.size() + 15) & ~size_t(15), 0);
  std::memcpy(blob.data(), fixed.data(), BXW_LIST_AT);
  size_t at = BXW_LIST_AT;
  for (uint32_t w = 0; w < 16; ++w) {
    if (!entries[w].empty()) std::memcpy(blob.data() + at, entries[w].data(), 2 * entries[w].size());
    at += 2 * entries[w].size();
  }
  if (!far.empty()) std::memcpy(blob.data() + far_at, far.data(), 4 * far.size());
  return true;
}

// Inverse of window_blob, written the way a GPU warp works: fixed codes first, then the entry lists.
bool window_unblob(const uint8_t* blob, uint64_t blob_bytes, const uint8_t* base_rows, uint16_t* tile /* [128][128] */) {
  if (blob_bytes < BXW_LIST_AT) return false;
  uint16_t warp_end[17], n_far;
  std::memcpy(warp_end, blob + BXW_WARP_END_AT, sizeof warp_end);
  std::memcpy(&n_far, blob + BXW_FAR_COUNT_AT, 2);
  const size_t total = warp_end[16];
  const size_t far_at = (BXW_LIST_AT + 2 * total + 3) & ~size_t(3);
  if (total > BXW_ENTRY_MAX || n_far > BXW_FAR_MAX || far_at + 4ull * n_far > blob_bytes) return false;
  const auto* codes = reinterpret_cast<const uint32_t*>(blob + BXW_CODES_AT);
  for (uint32_t q = 0; q < BXR_PHASES; ++q)
    for (uint32_t r = 0; r < BXR_ROWS; ++r) {
      uint32_t word[3];
      for (uint32_t t = 0; t < 3; ++t) word[t] = codes[t * BXR_SEGMENTS + q * BXR_ROWS + r];
      const uint32_t b = base_rows[r];
      for (uint32_t j = 0; j < 32; ++j) {
        const uint32_t p = j / 2, odd = j & 1;
        uint32_t code;
        if (p < 15) code = (word[p / 5] >> (1 + 3 * (p % 5) + 16 * odd)) & 7u;
        else code = ((word[0] >> (16 * odd)) & 1u) | ((word[1] >> (16 * odd)) & 1u) << 1 | ((word[2] >> (16 * odd)) & 1u) << 2;
        const uint32_t e = (b + code) & 0xFFu, byte = blob[BXW_RAW_AT + (size_t(2 * q + j / 16) * BXR_ROWS + r) * 16 + j % 16];
        tile[r * BXR_COLS + q * 32 + j] = uint16_t((byte & 0x80) << 8 | e << 7 | (byte & 0x7F));
      }
    }
  for (uint32_t warp = 0; warp < 16; ++warp) {
    if (warp_end[warp] > warp_end[warp + 1]) return false;
    for (uint32_t i = warp_end[warp]; i < warp_end[warp + 1]; ++i) {
      uint16_t v;
      std::memcpy(&v, blob + BXW_LIST_AT + 2 * size_t(i), 2);
      const uint32_t place = v & ((1u << BXW_PLACE_BITS) - 1), q = warp >> 2, rl = place >> 6;
      const uint32_t unit = ((place >> 3) & 7u) ^ (rl & 7u), j = (unit & 3u) * 8 + (place & 7u);
      if ((unit >> 2) != (q & 1u)) return false;
      const int delta = int(int16_t(v)) >> BXW_PLACE_BITS;  // sign-extended 5-bit field
      uint16_t& w = tile[((warp & 3) * 32 + rl) * BXR_COLS + q * 32 + j];
      if (delta != BXW_DELTA_FAR) {
        w = uint16_t(int(w) + delta * 128);
        continue;
      }
      bool found = false;
      for (uint32_t f = 0; f < n_far && !found; ++f) {
        uint32_t x;
        std::memcpy(&x, blob + far_at + 4 * size_t(f), 4);
        if ((x & 0x7FFFu) == (warp << BXW_PLACE_BITS | place)) { w = uint16_t((w & 0x807Fu) | ((x >> 16) & 0xFFu) << 7); found = true; }
      }
      if (!found) return false;
    }
  }
  return true;
}

// ---- wide-window mode -------------------------------------------------------------------------------------
// Row windows: the 16 consecutive exponents [base, base + 15] that cover most of the row.
std::vector<uint8_t> choose_window4_bases(const Source& src, uint32_t rows_pad, uint32_t threads) {
  std::vector<uint8_t> base(rows_pad);
  parallel_for(rows_pad, threads, [&](uint32_t r) {
    uint32_t h[256 + 16] = {0};
    for (uint32_t c = 0; c < src.cols; ++c) ++h[exponent_of(src.at(r, c))];
    uint32_t run = 0, best = 0, best_base = 0;
    for (uint32_t e = 0; e < 16; ++e) run += h[e];
    for (uint32_t b = 0;; ++b) {
      if (run >= best) { best = run; best_base = b; }   // ties go to the higher window: the tail below is the long one
      if (b == BXQ_BASE_MAX) break;
      run += h[b + 16];
      run -= h[b];
    }
    base[r] = uint8_t(best_base);
  });
  return base;
}

bool window4_blob(const Source& src, uint32_t row_block, uint32_t chunk, const uint8_t* base, std::vector<uint8_t>& blob) {
  std::vector<uint32_t> entries[16];
  std::vector<uint8_t> fixed(BXQ_LIST_AT, 0);
  auto* codes = reinterpret_cast<uint32_t*>(fixed.data() + BXQ_CODES_AT);
  for (uint32_t warp = 0; warp < 16; ++warp) {
    const uint32_t q = warp >> 2;
    for (uint32_t rl = 0; rl < 32; ++rl) {
      const uint32_t r = (warp & 3) * 32 + rl, row = row_block * BXR_ROWS + r, b = base[row];
      uint32_t word[4] = {0, 0, 0, 0};
      for (uint32_t j = 0; j < 32; ++j) {
        const uint32_t col = chunk * BXR_COLS + q * 32 + j;
        // a padded column never reaches an output: it carries the window's first exponent and a zero raw byte
        const uint16_t w = col < src.cols ? src.at(row, col) : uint16_t(b << 7);
        const uint32_t e = exponent_of(w);
        fixed[BXQ_RAW_AT + (size_t(2 * q + j / 16) * BXR_ROWS + r) * 16 + j % 16] = raw_byte_of(w);
        uint32_t code = e - b;  // wraps below the window
        if (code > 15) {
          code = 0;
          entries[warp].push_back(j | rl << 5 | e << 16);
        }
        const uint32_t p = j / 2;
        word[p / 4] |= code << (4 * (p % 4) + 16 * (j & 1));
      }
      for (uint32_t t = 0; t < 4; ++t) codes[t * BXR_SEGMENTS + q * BXR_ROWS + r] = word[t];
    }
  }
  size_t total = 0;
  auto* warp_end = reinterpret_cast<uint16_t*>(fixed.data() + BXQ_WARP_END_AT);
  for (uint32_t w = 0; w < 16; ++w) { warp_end[w] = uint16_t(total); total += entries[w].size(); }
  if (total > BXQ_ENTRY_MAX) return false;
  warp_end[16] = uint16_t(total);
  blob.assign((BXQ_LIST_AT + 4 * total + 15) & ~size_t(15), 0);
  std::memcpy(blob.data(), fixed.data(), BXQ_LIST_AT);
  size_t at = BXQ_LIST_AT;
  for (uint32_t w = 0; w < 16; ++w) {
    if (!entries[w].empty()) std::memcpy(blob.data() + at, entries[w].data(), 4 * entries[w].size());
    at += 4 * entries[w].size();
  }
  return true;
}

bool window4_unblob(const uint8_t* blob, uint64_t blob_bytes, const uint8_t* base_rows, uint16_t* tile /* [128][128] */) {
  if (blob_bytes < BXQ_LIST_AT) return false;
  uint16_t warp_end[17];
  std::memcpy(warp_end, blob + BXQ_WARP_END_AT, sizeof warp_end);
  const size_t total = warp_end[16];
  if (total > BXQ_ENTRY_MAX || BXQ_LIST_AT + 4ull * total > blob_bytes) return false;
  const auto* codes = reinterpret_cast<const uint32_t*>(blob + BXQ_CODES_AT);
  for (uint32_t q = 0; q < BXR_PHASES; ++q)
    for (uint32_t r = 0; r < BXR_ROWS; ++r)
      for (uint32_t j = 0; j < 32; ++j) {
        const uint32_t p = j / 2, word = codes[(p / 4) * BXR_SEGMENTS + q * BXR_ROWS + r];
        const uint32_t code = (word >> (4 * (p % 4) + 16 * (j & 1))) & 15u;
        const uint32_t e = (base_rows[r] + code) & 0xFFu, byte = blob[BXQ_RAW_AT + (size_t(2 * q + j / 16) * BXR_ROWS + r) * 16 + j % 16];
        tile[r * BXR_COLS + q * 32 + j] = uint16_t((byte & 0x80) << 8 | e << 7 | (byte & 0x7F));
      }
  for (uint32_t warp = 0; warp < 16; ++warp) {
    if (warp_end[warp] > warp_end[warp + 1]) return false;
    for (uint32_t i = warp_end[warp]; i < warp_end[warp + 1]; ++i) {
      uint32_t v;
      std::memcpy(&v, blob + BXQ_LIST_AT + 4 * size_t(i), 4);
      if ((v & 0xFC00u) || (v >> 24)) return false;
      const uint32_t j = v & 31u, rl = (v >> 5) & 31u, e = (v >> 16) & 0xFFu;
      uint16_t& w = tile[((warp & 3) * 32 + rl) * BXR_COLS + (warp >> 2) * 32 + j];
      w = uint16_t((w & 0x807Fu) | e << 7);
    }
  }
  return true;
}

// Structural check of an image before any of its offsets is followed, on the host or on the GPU: header fields, every
// array inside the image, the work partition (it must be the one this library computes for the shape and worker
// count: the kernels derive part of it themselves), the blob index and the per-mode size limits of a blob.  Cheap:
// it reads the header, the item list and the blob index, never the blobs.
bool image_is_well_formed(const uint8_t* img, uint64_t bytes) {
  if (!img || bytes < sizeof(bxr_header)) return false;
  bxr_header h;
  std::memcpy(&h, img, sizeof h);
  if (h.magic != BXR_MAGIC || h.layout_version != BXR_LAYOUT_VERSION || h.mode > BXR_MODE_WINDOW4) return false;
  if (h.total_bytes != bytes || !h.rows || !h.cols || !h.workers || h.workers > 4096) return false;
  if (h.row_blocks != (h.rows + BXR_ROWS - 1) / BXR_ROWS || h.chunks != (h.cols + BXR_COLS - 1) / BXR_COLS) return false;
  const uint64_t nblobs = uint64_t(h.row_blocks) * h.chunks;
  if (nblobs > 0xFFFFFFFEull) return false;
  const bool coded = h.mode == BXR_MODE_CODED;
  auto inside = [&](uint64_t at, uint64_t size, uint64_t align) {
    return at >= sizeof(bxr_header) && (at % align) == 0 && size <= bytes && at <= bytes - size;
  };
  if (!inside(h.base_at, uint64_t(h.row_blocks) * BXR_ROWS, 1)) return false;
  if (coded && !inside(h.lut_at, 4ull * BXR_PROB_TOTAL, 16)) return false;
  if (!inside(h.items_at, sizeof(bxr_item) * uint64_t(h.items), 16)) return false;
  if (!inside(h.worker_items_at, 4ull * (h.workers + 1ull), 4)) return false;
  if (coded && !inside(h.states_at, 4ull * BXR_STREAMS * h.items, 16)) return false;
  if (!inside(h.blob_index_at, 4ull * (nblobs + 1), 4)) return false;
  if (!inside(h.blobs_at, 0, 16)) return false;
  // the arrays follow one another in the builder's order and none reaches into the next
  const uint64_t begin[7] = {h.lut_at, h.base_at, h.items_at, h.worker_items_at, h.states_at, h.blob_index_at, h.blobs_at};
  const uint64_t size[6] = {coded ? 4ull * BXR_PROB_TOTAL : 0, uint64_t(h.row_blocks) * BXR_ROWS, sizeof(bxr_item) * uint64_t(h.items),
                            4ull * (h.workers + 1ull), coded ? 4ull * BXR_STREAMS * h.items : 0, 4ull * (nblobs + 1)};
  for (int i = 0; i < 6; ++i)
    if (begin[i] > begin[i + 1] || size[i] > begin[i + 1] - begin[i]) return false;
  // the work partition
  const Plan plan = make_plan(h.rows, h.cols, h.workers);
  if (plan.items.size() != h.items || plan.partial_slots != h.partial_slots) return false;
  if (std::memcmp(img + h.items_at, plan.items.data(), sizeof(bxr_item) * plan.items.size()) != 0) return false;
  if (std::memcmp(img + h.worker_items_at, plan.worker_items.data(), 4ull * (h.workers + 1ull)) != 0) return false;
  // the blob index: ascending, inside the image, every blob within the limits of its mode
  const auto* index = reinterpret_cast<const uint32_t*>(img + h.blob_index_at);
  uint64_t lo = 0, hi = 0;
  switch (h.mode) {
    case BXR_MODE_RAW: lo = hi = BXR_RAW_TILE_BYTES; break;
    case BXR_MODE_WINDOW: lo = BXW_LIST_AT; hi = BXR_BLOB_MAX; break;
    case BXR_MODE_WINDOW4: lo = BXQ_LIST_AT; hi = BXQ_BLOB_MAX; break;
    default: lo = BXR_WORDS_AT + 4; hi = BXR_BLOB_MAX; break;
  }
  if (index[0] != 0) return false;
  for (uint64_t b = 0; b < nblobs; ++b) {
    if (index[b + 1] < index[b]) return false;
    const uint64_t size = uint64_t(index[b + 1] - index[b]) << 4;
    if (size < lo || size > hi) return false;
    if (h.blob_stride16 && index[b] != b * h.blob_stride16) return false;
  }
  if (h.blob_stride16 && (h.mode != BXR_MODE_WINDOW4 || index[nblobs] != nblobs * h.blob_stride16)) return false;
  if (h.blobs_at + (uint64_t(index[nblobs]) << 4) != bytes) return false;
  // row windows
  const uint32_t base_max = h.mode == BXR_MODE_WINDOW4 ? BXQ_BASE_MAX : h.mode == BXR_MODE_WINDOW ? BXW_BASE_MAX : 241u;
  const uint8_t* base = img + h.base_at;
  for (uint64_t r = 0; r < uint64_t(h.row_blocks) * BXR_ROWS; ++r)
    if (base[r] > base_max) return false;
  return true;
}

}  // namespace

extern "C" {

uint32_t bxr_layout_version(void) { return BXR_LAYOUT_VERSION; }

// 0 when the image is structurally sound (see image_is_well_formed), 1 otherwise.  Never throws, never reads outside
// [image, image + image_bytes).
int bxr_validate(const uint8_t* image, uint64_t image_bytes) {
  try {
    return image_is_well_formed(image, image_bytes) ? 0 : 1;
  } catch (...) {
    return 1;
  }
}


void bxr_free(void* p) { std::free(p); }

// Builds the image.  workers = CTAs the kernels will run (one per SM); threads = host threads.
// layout = BXR_MODE_CODED (rANS exponent streams), BXR_MODE_WINDOW (fixed 3-bit codes), BXR_MODE_WINDOW4 (fixed 4-bit
// codes) or BXR_MODE_RAW (no coding).  A chunk that does not fit its slot demotes the whole image: window4 or window
// -> coded -> raw.
// Returns 0, 1 bad arguments, 2 out of memory, 3 other failure.  The image is malloc'ed; free with bxr_free.
int bxr_build(const uint16_t* words, uint32_t rows, uint32_t cols, uint32_t workers, uint32_t threads,
              uint32_t layout, const uint8_t* source_sha256, uint8_t** image, uint64_t* image_bytes) {
  try {
    if (!words || !rows || !cols || !workers || workers > 4096 || !image || !image_bytes || layout > BXR_MODE_WINDOW4) return 1;
    if (!threads) threads = std::max(1u, std::thread::hardware_concurrency());
    const Source src{words, rows, cols};
    Plan plan = make_plan(rows, cols, workers);
    const uint32_t rows_pad = plan.row_blocks * BXR_ROWS, cols_pad = plan.chunks * BXR_COLS;
    const uint32_t nblobs = plan.row_blocks * plan.chunks;
    const uint32_t nitems = uint32_t(plan.items.size());

    std::vector<uint8_t> base(rows_pad, 0);
    std::vector<uint32_t> lut(BXR_PROB_TOTAL, 0);
    std::vector<std::vector<uint8_t>> blobs(nblobs);
    std::vector<uint32_t> states(size_t(nitems) * BXR_STREAMS, BXR_STATE_LOW);
    bool raw_mode = layout == BXR_MODE_RAW;
    bool window_mode = layout == BXR_MODE_WINDOW;
    bool window4_mode = layout == BXR_MODE_WINDOW4;

    if (window4_mode) {
      base = choose_window4_bases(src, rows_pad, threads);
      std::atomic<bool> overflow{false};
      parallel_for(nblobs, threads, [&](uint32_t bi) {
        if (overflow.load()) return;
        if (!window4_blob(src, bi / plan.chunks, bi % plan.chunks, base.data(), blobs[bi])) overflow.store(true);
      });
      if (overflow.load()) {
        window4_mode = false;
        for (auto& b : blobs) b.clear();
      }
    }

    if (window_mode) {
      base = choose_window_bases(src, rows_pad, threads);
      std::atomic<bool> overflow{false};
      parallel_for(nblobs, threads, [&](uint32_t bi) {
        if (overflow.load()) return;
        if (!window_blob(src, bi / plan.chunks, bi % plan.chunks, base.data(), blobs[bi])) overflow.store(true);
      });
      if (overflow.load()) {
        window_mode = false;
        for (auto& b : blobs) b.clear();
      }
    }

    if (!raw_mode && !window_mode && !window4_mode) {
      base = choose_bases(src, rows_pad, threads);
      // pair statistics
      std::vector<std::vector<uint64_t>> local(threads, std::vector<uint64_t>(256, 0));
      {
        std::atomic<uint32_t> next{0};
        std::vector<std::thread> pool;
        for (uint32_t t = 0; t < threads; ++t)
          pool.emplace_back([&, t] {
            auto& cnt = local[t];
            for (uint32_t r = next.fetch_add(1); r < rows_pad; r = next.fetch_add(1))
              for (uint32_t c = 0; c < cols_pad; c += 2)
                ++cnt[nibble_of(exponent_of(src.padded(r, c, base.data())), base[r]) |
                      nibble_of(exponent_of(src.padded(r, c + 1, base.data())), base[r]) << 4];
          });
        for (auto& th : pool) th.join();
      }
      std::vector<uint64_t> counts(256, 0);
      for (auto& l : local)
        for (int s = 0; s < 256; ++s) counts[s] += l[s];
      uint32_t freq[256], cum[256];
      quantise_pairs(counts, freq);
      // A record has 12 bits for the frequency: a symbol that owns every slot cedes one to an unused symbol.
      for (uint32_t s = 0; s < 256; ++s)
        if (freq[s] == BXR_PROB_TOTAL) { freq[s] -= 1; freq[s ? 0 : 1] += 1; }
      uint32_t run = 0;
      for (uint32_t s = 0; s < 256; ++s) { cum[s] = run; run += freq[s]; }
      for (uint32_t s = 0; s < 256; ++s) {
        const uint32_t n0 = (s & 15) == BXR_ESCAPE ? 0 : (s & 15), n1 = (s >> 4) == BXR_ESCAPE ? 0 : (s >> 4);
        for (uint32_t slot = cum[s]; slot < cum[s] + freq[s]; ++slot) lut[slot] = n0 | (slot - cum[s]) << 4 | n1 << 16 | freq[s] << 20;
      }

      std::atomic<bool> overflow{false};
      parallel_for(nitems, threads, [&](uint32_t i) {
        if (overflow.load()) return;
        const bxr_item& it = plan.items[i];
        auto code = std::make_unique<ItemCode>();
        encode_item(src, it, base.data(), freq, cum, *code);
        std::copy(code->state, code->state + BXR_STREAMS, &states[size_t(i) * BXR_STREAMS]);
        std::vector<uint32_t> cursor(BXR_STREAMS, 0);
        for (uint32_t c = it.chunk_begin; c < it.chunk_end; ++c) {
          const uint32_t k = c - it.chunk_begin;
          uint32_t total = 0;
          for (uint32_t sid = 0; sid < BXR_STREAMS; ++sid) total += code->per_chunk[sid][k];
          std::vector<uint32_t>& exc = code->exceptions[k];
          std::sort(exc.begin(), exc.end(), [](uint32_t a, uint32_t b) { return (a & 0x3FFF) < (b & 0x3FFF); });
          const uint64_t exc_at = (BXR_WORDS_AT + 2ull * total + 3) & ~3ull;
          const uint64_t blob_bytes = align16(exc_at + 4 + 4ull * exc.size());
          if (total > BXR_WORDS_MAX || exc.size() > BXR_EXC_MAX || blob_bytes > BXR_BLOB_MAX) { overflow.store(true); return; }
          std::vector<uint8_t>& blob = blobs[size_t(it.row_block) * plan.chunks + c];
          blob.assign(size_t(blob_bytes), 0);
          const uint32_t n_exc = uint32_t(exc.size());
          std::memcpy(blob.data() + exc_at, &n_exc, 4);
          if (n_exc) std::memcpy(blob.data() + exc_at + 4, exc.data(), 4ull * n_exc);
          for (uint32_t v : exc) blob[BXR_EXC_BITS_AT + ((v & 511) >> 3)] |= uint8_t(1u << (v & 7));
          uint8_t* raw = blob.data() + BXR_RAW_AT;
          for (uint32_t piece = 0; piece < 2 * BXR_PHASES; ++piece)
            for (uint32_t r = 0; r < BXR_ROWS; ++r) {
              uint8_t* dst = raw + (size_t(piece) * BXR_ROWS + r) * 16;
              const uint32_t row = it.row_block * BXR_ROWS + r, col = c * BXR_COLS + piece * BXR_STREAM_COLS;
              for (uint32_t e = 0; e < 16; ++e) dst[e] = raw_byte_of(src.padded(row, col + e, base.data()));
            }
          uint16_t* w = reinterpret_cast<uint16_t*>(blob.data() + BXR_WORDS_AT);
          uint32_t at = 0;
          for (uint32_t g = 0; g < BXR_SEGMENTS; ++g) {
            const uint32_t q = g / BXR_ROWS, r = g % BXR_ROWS;
            const uint32_t fwd = (2 * q) * BXR_ROWS + r, bwd = (2 * q + 1) * BXR_ROWS + r;
            const uint32_t nf = code->per_chunk[fwd][k], nb = code->per_chunk[bwd][k];
            blob[g] = uint8_t(nf + nb);
            for (uint32_t e = 0; e < nf; ++e) w[at + e] = code->words[fwd][cursor[fwd] + e];
            for (uint32_t e = 0; e < nb; ++e) w[at + nf + nb - 1 - e] = code->words[bwd][cursor[bwd] + e];
            cursor[fwd] += nf;
            cursor[bwd] += nb;
            at += nf + nb;
          }
        }
      });
      if (overflow.load()) raw_mode = true;
    }

    if (raw_mode) {
      std::fill(base.begin(), base.end(), 0);
      std::fill(states.begin(), states.end(), BXR_STATE_LOW);
      parallel_for(nblobs, threads, [&](uint32_t bi) {
        const uint32_t rb = bi / plan.chunks, c = bi % plan.chunks;
        std::vector<uint8_t>& blob = blobs[bi];
        blob.assign(BXR_RAW_TILE_BYTES, 0);
        for (uint32_t a = 0; a < 2; ++a)
          for (uint32_t r = 0; r < BXR_ROWS; ++r)
            for (uint32_t j = 0; j < 8; ++j) {
              uint16_t* dst = reinterpret_cast<uint16_t*>(blob.data() + a * 16384 + r * 128 + ((j ^ (r & 7)) * 16));
              for (uint32_t e = 0; e < 8; ++e) dst[e] = src.padded(rb * BXR_ROWS + r, c * BXR_COLS + a * 64 + j * 8 + e, base.data());
            }
      });
    }

    bxr_header h{};
    h.magic = BXR_MAGIC;
    h.mode = raw_mode ? BXR_MODE_RAW : window4_mode ? BXR_MODE_WINDOW4 : window_mode ? BXR_MODE_WINDOW : BXR_MODE_CODED;
    const bool coded = !raw_mode && !window_mode && !window4_mode;
    h.rows = rows;
    h.cols = cols;
    h.row_blocks = plan.row_blocks;
    h.chunks = plan.chunks;
    h.workers = workers;
    h.items = nitems;
    h.partial_slots = plan.partial_slots;
    uint64_t at = align16(sizeof(bxr_header));
    at = (at + 255) & ~uint64_t(255);
    h.lut_at = at;            at += coded ? sizeof(uint32_t) * BXR_PROB_TOTAL : 0;
    h.base_at = at;           at = align16(at + rows_pad);
    h.items_at = at;          at = align16(at + sizeof(bxr_item) * nitems);
    h.worker_items_at = at;   at = align16(at + 4ull * (workers + 1));
    h.states_at = at;         at = align16(at + (coded ? 4ull * states.size() : 0));
    h.blob_index_at = at;     at = align16(at + 4ull * (nblobs + 1));
    at = (at + 255) & ~uint64_t(255);
    h.blobs_at = at;
    // Wide-window blobs differ only by their (rare) exception entries: pad them to one size, so that a kernel can
    // address blob b without looking its offset up (the index is written all the same).
    uint32_t blob_stride16 = 0;
    if (window4_mode) {
      size_t lo = SIZE_MAX, hi = 0;
      for (const auto& b : blobs) { lo = std::min(lo, b.size()); hi = std::max(hi, b.size()); }
      if (hi - lo <= 512) {
        for (auto& b : blobs) b.resize(hi, 0);
        blob_stride16 = uint32_t(hi >> 4);
      }
    }
    h.blob_stride16 = blob_stride16;
    h.layout_version = BXR_LAYOUT_VERSION;
    std::vector<uint32_t> index(nblobs + 1);
    uint64_t run = 0;
    for (uint32_t b = 0; b < nblobs; ++b) { index[b] = uint32_t(run >> 4); run += blobs[b].size(); }
    if ((run >> 4) > 0xFFFFFFFFull) return 3;
    index[nblobs] = uint32_t(run >> 4);
    h.total_bytes = at + run;
    h.coded_bytes = run + (coded ? 4ull * states.size() : 0) + 4ull * (nblobs + 1);
    if (source_sha256) std::memcpy(h.source_sha256, source_sha256, 32);

    auto* img = static_cast<uint8_t*>(std::calloc(size_t(h.total_bytes), 1));
    if (!img) return 2;
    std::memcpy(img, &h, sizeof h);
    if (coded) std::memcpy(img + h.lut_at, lut.data(), sizeof(uint32_t) * BXR_PROB_TOTAL);
    std::memcpy(img + h.base_at, base.data(), rows_pad);
    std::memcpy(img + h.items_at, plan.items.data(), sizeof(bxr_item) * nitems);
    std::memcpy(img + h.worker_items_at, plan.worker_items.data(), 4ull * (workers + 1));
    if (coded) std::memcpy(img + h.states_at, states.data(), 4ull * states.size());
    std::memcpy(img + h.blob_index_at, index.data(), 4ull * (nblobs + 1));
    parallel_for(nblobs, threads, [&](uint32_t b) {
      std::memcpy(img + h.blobs_at + (uint64_t(index[b]) << 4), blobs[b].data(), blobs[b].size());
    });
    *image = img;
    *image_bytes = h.total_bytes;
    return 0;
  } catch (const std::bad_alloc&) {
    return 2;
  } catch (...) {
    return 3;
  }
}

// Host twin of the GPU decoder.  Writes rows*cols words.  Returns 0, 1 bad arguments / malformed header,
// 2 a stream that reads outside its segment or does not end in the canonical state.
int bxr_decode_host(const uint8_t* img, uint64_t bytes, uint16_t* out) {
  try {
    if (!img || !out || bytes < sizeof(bxr_header)) return 1;
    bxr_header h;
    std::memcpy(&h, img, sizeof h);
    if (!image_is_well_formed(img, bytes)) return 1;   // every offset followed below has been checked
    const auto* items = reinterpret_cast<const bxr_item*>(img + h.items_at);
    const auto* index = reinterpret_cast<const uint32_t*>(img + h.blob_index_at);
    auto put = [&](uint32_t row, uint32_t col, uint16_t w) {
      if (row < h.rows && col < h.cols) out[size_t(row) * h.cols + col] = w;
    };
    if (h.mode == BXR_MODE_RAW) {
      for (uint32_t rb = 0; rb < h.row_blocks; ++rb)
        for (uint32_t c = 0; c < h.chunks; ++c) {
          const uint8_t* blob = img + h.blobs_at + (uint64_t(index[size_t(rb) * h.chunks + c]) << 4);
          for (uint32_t a = 0; a < 2; ++a)
            for (uint32_t r = 0; r < BXR_ROWS; ++r)
              for (uint32_t j = 0; j < 8; ++j) {
                const auto* srcp = reinterpret_cast<const uint16_t*>(blob + a * 16384 + r * 128 + ((j ^ (r & 7)) * 16));
                for (uint32_t e = 0; e < 8; ++e) put(rb * BXR_ROWS + r, c * BXR_COLS + a * 64 + j * 8 + e, srcp[e]);
              }
        }
      return 0;
    }
    const uint8_t* base = img + h.base_at;
    if (h.mode == BXR_MODE_WINDOW || h.mode == BXR_MODE_WINDOW4) {
      std::vector<uint16_t> tile(size_t(BXR_ROWS) * BXR_COLS);
      for (uint32_t rb = 0; rb < h.row_blocks; ++rb)
        for (uint32_t c = 0; c < h.chunks; ++c) {
          const size_t bi = size_t(rb) * h.chunks + c;
          const uint8_t* blob = img + h.blobs_at + (uint64_t(index[bi]) << 4);
          const uint64_t blob_bytes = uint64_t(index[bi + 1] - index[bi]) << 4;
          const bool ok = h.mode == BXR_MODE_WINDOW ? window_unblob(blob, blob_bytes, base + size_t(rb) * BXR_ROWS, tile.data())
                                                    : window4_unblob(blob, blob_bytes, base + size_t(rb) * BXR_ROWS, tile.data());
          if (!ok) return 2;
          for (uint32_t r = 0; r < BXR_ROWS; ++r)
            for (uint32_t j = 0; j < BXR_COLS; ++j) put(rb * BXR_ROWS + r, c * BXR_COLS + j, tile[r * BXR_COLS + j]);
        }
      return 0;
    }
    const auto* lut = reinterpret_cast<const uint32_t*>(img + h.lut_at);
    const auto* states = reinterpret_cast<const uint32_t*>(img + h.states_at);
    for (uint32_t i = 0; i < h.items; ++i) {
      const bxr_item& it = items[i];
      std::vector<uint32_t> x(states + size_t(i) * BXR_STREAMS, states + size_t(i + 1) * BXR_STREAMS);
      for (uint32_t c = it.chunk_begin; c < it.chunk_end; ++c) {
        const size_t bi = size_t(it.row_block) * h.chunks + c;
        const uint8_t* blob = img + h.blobs_at + (uint64_t(index[bi]) << 4);
        const uint64_t blob_bytes = uint64_t(index[bi + 1] - index[bi]) << 4;
        const auto* words = reinterpret_cast<const uint16_t*>(blob + BXR_WORDS_AT);
        const int64_t nwords = (int64_t(blob_bytes) - BXR_WORDS_AT) / 2;
        uint32_t start[BXR_SEGMENTS + 1];
        start[0] = 0;
        for (uint32_t g = 0; g < BXR_SEGMENTS; ++g) start[g + 1] = start[g] + blob[g];
        if (int64_t(start[BXR_SEGMENTS]) > nwords) return 2;
        for (uint32_t sid = 0; sid < BXR_STREAMS; ++sid) {
          const uint32_t piece = sid / BXR_ROWS, r = sid % BXR_ROWS, g = (piece / 2) * BXR_ROWS + r;
          const bool backward = piece & 1;
          int64_t cur = backward ? int64_t(start[g + 1]) - 1 : int64_t(start[g]);
          const int step = backward ? -1 : 1;
          uint32_t s = x[sid];
          const uint32_t row = it.row_block * BXR_ROWS + r, b = base[row];
          const uint8_t* bytes16 = blob + BXR_RAW_AT + (size_t(piece) * BXR_ROWS + r) * 16;
          for (uint32_t t = 0; t < BXR_STEPS; ++t) {
            const uint32_t rec = lut[s & (BXR_PROB_TOTAL - 1)];
            s = BXR_REC_FREQ(rec) * (s >> BXR_PROB_BITS) + BXR_REC_BIAS(rec);
            if (s < BXR_STATE_LOW) {
              if (cur < int64_t(start[g]) || cur >= int64_t(start[g + 1])) return 2;
              s = (s << 16) | words[cur];
              cur += step;
            }
            const uint32_t e0 = BXR_REC_N0(rec) + b, e1 = BXR_REC_N1(rec) + b;
            const uint32_t b0 = bytes16[2 * t], b1 = bytes16[2 * t + 1];
            const uint32_t col = c * BXR_COLS + piece * BXR_STREAM_COLS + 2 * t;
            put(row, col, uint16_t((b0 & 0x80) << 8 | (e0 & 0xFF) << 7 | (b0 & 0x7F)));
            put(row, col + 1, uint16_t((b1 & 0x80) << 8 | (e1 & 0xFF) << 7 | (b1 & 0x7F)));
          }
          x[sid] = s;
        }
        // exceptions: the true exponent replaces the placeholder the stream produced
        const uint64_t exc_at = (BXR_WORDS_AT + 2ull * start[BXR_SEGMENTS] + 3) & ~3ull;
        if (exc_at + 4 > blob_bytes) return 2;
        uint32_t n_exc;
        std::memcpy(&n_exc, blob + exc_at, 4);
        if (n_exc > BXR_EXC_MAX || exc_at + 4 + 4ull * n_exc > blob_bytes) return 2;
        for (uint32_t i = 0; i < n_exc; ++i) {
          uint32_t v;
          std::memcpy(&v, blob + exc_at + 4 + 4ull * i, 4);
          const uint32_t g = v & 511, in_seg = (v >> 9) & 31, e = (v >> 14) & 255;
          if (!((blob[BXR_EXC_BITS_AT + (g >> 3)] >> (g & 7)) & 1)) return 2;
          const uint32_t q = g / BXR_ROWS, r = g % BXR_ROWS;
          const uint32_t row = it.row_block * BXR_ROWS + r, col = c * BXR_COLS + q * 32 + in_seg;
          const uint32_t byte = blob[BXR_RAW_AT + (size_t(2 * q + in_seg / 16) * BXR_ROWS + r) * 16 + in_seg % 16];
          put(row, col, uint16_t((byte & 0x80) << 8 | e << 7 | (byte & 0x7F)));
        }
      }
      for (uint32_t sid = 0; sid < BXR_STREAMS; ++sid)
        if (x[sid] != BXR_STATE_LOW) return 2;
    }
    return 0;
  } catch (...) {
    return 3;
  }
}

}  // extern "C"
