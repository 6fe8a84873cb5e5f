/*
 * CPU oracle for the BCTX v1 context codec: a plain-C restatement of the reference
 * algorithm.  TEST INFRASTRUCTURE ONLY.  Nothing in the product package may call,
 * link or load this file; it exists so that tests, the smoke check and the bench's
 * cpu_baseline leg have an independent answer to compare the CUDA path against.
 *
 * Parity status: PINNED.  tests/test_oracle_golden.py checks this file against golden
 * vectors produced by the reference's own Python+C++ codec (tests/golden/make_golden.py)
 * and, where oracle/_ref/libbcx_ref.so was built from the reference sources, against that
 * library call by call.
 *
 * Each function names the reference lines it restates
 * (paths relative to the reference project root, cr/ = context-runtime/georefine_context_runtime/).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_SCALE 16u
#define ORC_TOTAL (1u << ORC_SCALE)
#define ORC_LOW   (1u << 23)

/* cr/bitexact_context_ans.cpp:9-12 -- 10-bit "main" symbol and 6-bit residual of a BF16 word */
static uint32_t orc_main(uint16_t w)  { return (uint32_t)((w >> 7) & 0xFFu) * 4u + ((w >> 5) & 3u); }
static uint32_t orc_resid(uint16_t w) { return (uint32_t)(w >> 15) * 32u + (w & 31u); }

/* cr/bitexact_context_codec.py:425-426 -- inverse of the split */
uint16_t orc_join(uint32_t main_sym, uint32_t resid) {
  return (uint16_t)(((main_sym >> 2) << 7) | ((main_sym & 3u) << 5) | (resid & 31u) | ((resid >> 5) << 15));
}

/* cr/bitexact_context_ans.cpp:13-16 */
static uint32_t orc_ctx(uint64_t i, uint32_t cols, const uint8_t *rc, const uint8_t *cc, uint32_t nc) {
  return (uint32_t)rc[i / cols] * nc + cc[i % cols];
}

typedef struct { uint32_t sym; uint64_t rem; } orc_rem_t;
static int orc_cmp_desc(const void *pa, const void *pb) {      /* larger remainder first, then smaller symbol */
  const orc_rem_t *a = (const orc_rem_t *)pa, *b = (const orc_rem_t *)pb;
  if (a->rem != b->rem) return a->rem > b->rem ? -1 : 1;
  return a->sym < b->sym ? -1 : (a->sym > b->sym);
}
static int orc_cmp_asc(const void *pa, const void *pb) {       /* smaller remainder first, then larger symbol */
  const orc_rem_t *a = (const orc_rem_t *)pa, *b = (const orc_rem_t *)pb;
  if (a->rem != b->rem) return a->rem < b->rem ? -1 : 1;
  return a->sym > b->sym ? -1 : (a->sym < b->sym);
}

/* cr/bitexact_context_ans.cpp:17-67 -- counts -> frequencies summing to 2^16, every seen symbol >= 1,
 * surplus/deficit spread by largest (smallest) remainder with symbol-order tie breaks. */
static int orc_normalize(const uint64_t *cnt, uint32_t vocab, uint32_t *out, orc_rem_t *scratch) {
  uint64_t total = 0;
  for (uint32_t s = 0; s < vocab; ++s) total += cnt[s];
  if (!total) return 0;
  uint32_t used = 0;
  int64_t sum = 0;
  for (uint32_t s = 0; s < vocab; ++s) {
    if (!cnt[s]) { out[s] = 0; continue; }
    uint64_t scaled = cnt[s] * (uint64_t)ORC_TOTAL;
    uint32_t f = (uint32_t)(scaled / total);
    if (f == 0) f = 1;
    out[s] = f;
    sum += f;
    scratch[used].sym = s;
    scratch[used].rem = scaled % total;
    ++used;
  }
  if (sum < (int64_t)ORC_TOTAL) {
    qsort(scratch, used, sizeof *scratch, orc_cmp_desc);
    uint32_t lack = ORC_TOTAL - (uint32_t)sum;
    for (uint32_t j = 0; j < lack; ++j) out[scratch[j % used].sym] += 1;
  } else if (sum > (int64_t)ORC_TOTAL) {
    qsort(scratch, used, sizeof *scratch, orc_cmp_asc);
    uint32_t extra = (uint32_t)sum - ORC_TOTAL;
    for (uint32_t j = 0; extra; j = (j + 1) % used) {
      uint32_t s = scratch[j].sym;
      if (out[s] > 1) { out[s] -= 1; --extra; }
    }
  }
  return 1;
}

static void orc_dims(uint32_t kind, uint32_t nr, uint32_t nc, uint32_t *vocab, uint32_t *nctx) {
  *vocab = kind ? 64u : 1024u;
  *nctx = kind ? 1024u : nr * nc;
}

/* cr/bitexact_context_ans.cpp:267-290 (and the counting half of :235-252) */
int orc_frequencies(const uint16_t *w, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t *rc,
                    const uint8_t *cc, uint32_t nr, uint32_t nc, uint32_t kind, uint32_t *freq) {
  uint32_t vocab, nctx;
  orc_dims(kind, nr, nc, &vocab, &nctx);
  if (!w || !rc || !cc || !freq || n != (uint64_t)rows * cols) return 1;
  uint64_t *counts = (uint64_t *)calloc((size_t)nctx * vocab, sizeof(uint64_t));
  orc_rem_t *scratch = (orc_rem_t *)malloc(sizeof(orc_rem_t) * vocab);
  if (!counts || !scratch) { free(counts); free(scratch); return 2; }
  for (uint64_t i = 0; i < n; ++i) {
    uint32_t s = kind ? orc_resid(w[i]) : orc_main(w[i]);
    uint32_t cx = kind ? orc_main(w[i]) : orc_ctx(i, cols, rc, cc, nc);
    counts[(size_t)cx * vocab + s] += 1;
  }
  for (uint32_t cx = 0; cx < nctx; ++cx)
    orc_normalize(counts + (size_t)cx * vocab, vocab, freq + (size_t)cx * vocab, scratch);
  free(counts);
  free(scratch);
  return 0;
}

/* cr/bitexact_context_ans.cpp:75-109,235-266 -- symbols are coded last to first; the bytes pushed
 * during renormalisation are emitted in reverse so the decoder reads forward.  Layout of the result:
 * 4 bytes little-endian final encoder state, then the renormalisation bytes in decode order. */
int orc_encode(const uint16_t *w, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t *rc,
               const uint8_t *cc, uint32_t nr, uint32_t nc, uint32_t kind, uint32_t *freq,
               uint8_t **stream, size_t *stream_n) {
  if (!stream || !stream_n) return 1;
  int st = orc_frequencies(w, n, rows, cols, rc, cc, nr, nc, kind, freq);
  if (st) return st;
  uint32_t vocab, nctx;
  orc_dims(kind, nr, nc, &vocab, &nctx);
  uint32_t *start = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)nctx * vocab);
  size_t cap = (size_t)(n / 2) + 64, used = 0;
  uint8_t *rev = (uint8_t *)malloc(cap);
  if (!start || !rev) { free(start); free(rev); return 2; }
  for (uint32_t cx = 0; cx < nctx; ++cx) {
    uint32_t run = 0;
    for (uint32_t s = 0; s < vocab; ++s) { start[(size_t)cx * vocab + s] = run; run += freq[(size_t)cx * vocab + s]; }
  }
  uint32_t x = ORC_LOW;
  for (uint64_t i = n; i-- > 0;) {
    uint32_t s = kind ? orc_resid(w[i]) : orc_main(w[i]);
    uint32_t cx = kind ? orc_main(w[i]) : orc_ctx(i, cols, rc, cc, nc);
    uint32_t f = freq[(size_t)cx * vocab + s], c = start[(size_t)cx * vocab + s];
    if (!f) { free(start); free(rev); return 3; }
    uint64_t limit = ((uint64_t)(ORC_LOW >> ORC_SCALE) << 8) * f;
    while (x >= limit) {
      if (used == cap) {
        cap *= 2;
        uint8_t *grown = (uint8_t *)realloc(rev, cap);
        if (!grown) { free(start); free(rev); return 2; }
        rev = grown;
      }
      rev[used++] = (uint8_t)(x & 255u);
      x >>= 8;
    }
    x = ((x / f) << ORC_SCALE) + (x % f) + c;
  }
  uint8_t *out = (uint8_t *)malloc(used + 4);
  if (!out) { free(start); free(rev); return 2; }
  out[0] = (uint8_t)x; out[1] = (uint8_t)(x >> 8); out[2] = (uint8_t)(x >> 16); out[3] = (uint8_t)(x >> 24);
  for (size_t k = 0; k < used; ++k) out[4 + k] = rev[used - 1 - k];
  free(start);
  free(rev);
  *stream = out;
  *stream_n = used + 4;
  return 0;
}

void orc_free(void *p) { free(p); }

/* Shared forward walk: cr/bitexact_context_ans.cpp:110-160 (decode) and
 * cr/bitexact_context_gpu_index.cpp:21-137 (decode + restart points).  The reference finds the symbol
 * with a 65536-entry inverse table; the answer is the unique s with start[s] <= slot < start[s]+freq[s],
 * found here by bisection over the prefix sums (zero-frequency symbols can never own a slot).
 * stride == 0 means "no restart points wanted".  Outputs are written only on success. */
static int orc_walk(const uint8_t *stream, size_t bytes, uint64_t n, uint32_t cols, const uint8_t *rc,
                    const uint8_t *cc, uint32_t nr, uint32_t nc, uint32_t kind, const uint16_t *resctx,
                    const uint32_t *freq, uint32_t stride, uint32_t *states, uint32_t *offsets, uint16_t *out) {
  uint32_t vocab, nctx;
  orc_dims(kind, nr, nc, &vocab, &nctx);
  if (bytes < 4) return 3;
  /* prefix sums with a sentinel column; a context must be empty or sum to exactly 2^16 */
  uint32_t *pre = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)nctx * (vocab + 1));
  uint8_t *live = (uint8_t *)malloc(nctx);
  uint16_t *sym = (uint16_t *)malloc(sizeof(uint16_t) * (size_t)(n ? n : 1));
  uint64_t marks = stride ? (n + stride - 1) / stride : 0;
  uint32_t *st = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)(marks ? marks : 1));
  uint32_t *of = (uint32_t *)malloc(sizeof(uint32_t) * (size_t)(marks ? marks : 1));
  int rcode = 0;
  if (!pre || !live || !sym || !st || !of) { rcode = 5; goto done; }
  for (uint32_t cx = 0; cx < nctx; ++cx) {
    uint64_t run = 0;
    uint32_t *p = pre + (size_t)cx * (vocab + 1);
    for (uint32_t s = 0; s < vocab; ++s) {
      uint32_t f = freq[(size_t)cx * vocab + s];
      p[s] = (uint32_t)run;
      if (f > ORC_TOTAL || run + f > ORC_TOTAL) { rcode = 2; goto done; }
      run += f;
    }
    p[vocab] = (uint32_t)run;
    if (run != 0 && run != ORC_TOTAL) { rcode = 2; goto done; }
    live[cx] = run == ORC_TOTAL;
  }
  {
    uint32_t x = (uint32_t)stream[0] | (uint32_t)stream[1] << 8 | (uint32_t)stream[2] << 16 | (uint32_t)stream[3] << 24;
    if (x < ORC_LOW) { rcode = 3; goto done; }
    size_t ip = 4;
    uint64_t mark = 0, next_mark = 0;
    for (uint64_t i = 0; i < n; ++i) {
      if (stride && i == next_mark) {
        if (ip > 0xFFFFFFFFull) { rcode = 4; goto done; }
        st[mark] = x; of[mark] = (uint32_t)ip; ++mark; next_mark += stride;
      }
      uint32_t cx = kind ? resctx[i] : orc_ctx(i, cols, rc, cc, nc);
      if (cx >= nctx || !live[cx]) { rcode = 2; goto done; }
      const uint32_t *p = pre + (size_t)cx * (vocab + 1);
      uint32_t slot = x & (ORC_TOTAL - 1);
      uint32_t lo = 0, hi = vocab;                 /* invariant: p[lo] <= slot < p[hi] */
      while (hi - lo > 1) { uint32_t mid = (lo + hi) >> 1; if (p[mid] <= slot) lo = mid; else hi = mid; }
      uint32_t f = p[lo + 1] - p[lo];
      if (!f || slot - p[lo] >= f) { rcode = 2; goto done; }
      sym[i] = (uint16_t)lo;
      uint64_t nx = (uint64_t)f * (x >> ORC_SCALE) + (slot - p[lo]);
      if (nx > 0xFFFFFFFFull) { rcode = 3; goto done; }
      x = (uint32_t)nx;
      while (x < ORC_LOW) {
        if (ip >= bytes) { rcode = 3; goto done; }
        x = (x << 8) | stream[ip++];
      }
    }
    if (ip != bytes || x != ORC_LOW) { rcode = 3; goto done; }   /* canonical end only */
  }
  if (out) memcpy(out, sym, sizeof(uint16_t) * (size_t)n);
  if (stride) { memcpy(states, st, sizeof(uint32_t) * (size_t)marks); memcpy(offsets, of, sizeof(uint32_t) * (size_t)marks); }
done:
  free(pre); free(live); free(sym); free(st); free(of);
  return rcode;
}

/* cr/bitexact_context_ans.cpp:291-308: 0 ok, 1 bad arguments, 2 malformed stream or tables */
int orc_decode(const uint8_t *stream, size_t bytes, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t *rc,
               const uint8_t *cc, uint32_t nr, uint32_t nc, uint32_t kind, const uint16_t *resctx,
               const uint32_t *freq, uint16_t *out) {
  if (!stream || !rc || !cc || !freq || !out || !cols || !rows || kind > 1 || !nr || !nc || nr > 64 || nc > 16 ||
      (kind && !resctx) || n != (uint64_t)rows * cols)
    return 1;
  return orc_walk(stream, bytes, n, cols, rc, cc, nr, nc, kind, resctx, freq, 0, NULL, NULL, out) ? 2 : 0;
}

/* cr/bitexact_context_gpu_index.cpp:21-137: 1 arguments/labels, 2 tables, 3 stream/state,
 * 4 offset overflow, 5 out of memory */
int orc_checkpoint(const uint8_t *stream, size_t bytes, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t *rc,
                   const uint8_t *cc, uint32_t nr, uint32_t nc, uint32_t kind, const uint16_t *resctx,
                   const uint32_t *freq, uint32_t stride, uint32_t *states, uint32_t *offsets, uint16_t *out) {
  if (!stream || !rc || !cc || !freq || !states || !offsets || !out || !rows || !cols || !nr || !nc || nr > 64 ||
      nc > 16 || !stride || kind > 1 || (kind == 1 && !resctx) || n != (uint64_t)rows * cols || !n || bytes < 4 ||
      bytes > 0xFFFFFFFFull)
    return 1;
  for (uint32_t r = 0; r < rows; ++r) if (rc[r] >= nr) return 1;
  for (uint32_t c = 0; c < cols; ++c) if (cc[c] >= nc) return 1;
  if (kind == 1) for (uint64_t i = 0; i < n; ++i) if (resctx[i] >= 1024u) return 1;
  return orc_walk(stream, bytes, n, cols, rc, cc, nr, nc, kind, resctx, freq, stride, states, offsets, out);
}

/* cr/bitexact_context_ans.cpp:328-344 -- residuals packed 6 bits each, most significant bit first */
int orc_pack6(const uint16_t *w, uint64_t n, uint8_t **out, size_t *bytes) {
  if (!w || !out || !bytes) return 1;
  size_t z = (size_t)((n * 6 + 7) / 8);
  uint8_t *p = (uint8_t *)calloc(z ? z : 1, 1);
  if (!p) return 2;
  for (uint64_t i = 0; i < n; ++i) {
    uint32_t v = orc_resid(w[i]);
    uint64_t bit = i * 6;
    uint32_t sh = 10u - (uint32_t)(bit & 7);          /* position inside a 16-bit big-endian window */
    uint32_t win = v << sh;
    p[bit >> 3] |= (uint8_t)(win >> 8);
    if (win & 0xFFu) p[(bit >> 3) + 1] |= (uint8_t)win;
  }
  *out = p;
  *bytes = z;
  return 0;
}

/* cr/bitexact_context_ans.cpp:345-359 -- exact length and zero padding bits required */
int orc_unpack6(const uint8_t *in, size_t bytes, uint64_t n, uint16_t *out) {
  if (!in || !out || bytes != (size_t)((n * 6 + 7) / 8)) return 1;
  uint32_t tail = (uint32_t)(n * 6 % 8);
  if (tail && (in[bytes - 1] & ((1u << (8 - tail)) - 1u))) return 2;
  for (uint64_t i = 0; i < n; ++i) {
    uint64_t bit = i * 6;
    size_t b = (size_t)(bit >> 3);
    uint32_t win = (uint32_t)in[b] << 8 | (b + 1 < bytes ? in[b + 1] : 0u);
    out[i] = (uint16_t)((win >> (10u - (uint32_t)(bit & 7))) & 63u);
  }
  return 0;
}
