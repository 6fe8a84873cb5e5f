// Fused kernels over window-mode images (bxr_format.h, BXR_MODE_WINDOW): the same persistent, warp-specialised
// pipeline and the same work partition as bxr_kernel, but the exponent of a weight is a fixed 3-bit code, so a
// decoder lane reconstructs two BF16 words with one shift, two masks, one byte permute and one three-input add;
// there is no slot table, no stream state and no dependency chain between weights.  With the decode this cheap
// what limits the kernel is the serial work of its single-thread roles, so those are kept short: the MMA warp
// waits on one barrier per chunk, issues the chunk's eight MMAs and commits once.
//   * kDense : decode twin (parity tests, ResidentWeight.decode),
//   * kUmma  : decoded words go into the 128-byte-swizzled K-major tile consumed by tcgen05.mma (any batch size;
//              the batch of one runs here too, padded to the narrowest tile).
// Weights outside a row's window (about 1.2 % on Gaussian rows) are patched after the fixed-code pass: the chunk
// carries one entry list per decoder warp, and the lanes of the warp take one entry each, whoever owns the row.
#pragma once
#include "bxr_kernels.cuh"

namespace grb {

constexpr int kWinWarpLoader = 16;    // bulk copies of chunk blobs
constexpr int kWinWarpMma = 17;       // TMEM owner; MMA issuer of the even chunks of every item
constexpr int kWinWarpXLoader = 18;   // TMA loads of activation tiles
constexpr int kWinWarpMmaOdd = 19;    // MMA issuer of the odd chunks (its own accumulator; the epilogue adds the two)
constexpr int kWinWarpEpilogue = 20;  // 4 warps; warp % 4 = the TMEM lane quarter a warp may read

// Shared-memory plan.  An operand stage holds the decoded weights of one chunk (two 128 x 64 atoms, 32 KB); the
// activations of a chunk (two NB x 64 atoms) have a ring of their own because they come from L2 with a latency of
// about a microsecond and are requested kXLag chunks ahead of the weights they will meet.
template <int MODE, int NB>
struct BxwSmem {
  // two operand stages: chunk v of the CTA uses stage v % 2, and the MMA issuer of that parity is the only one that
  // ever waits on the stage's barrier, so it sees every phase of it
  static constexpr int kOp = (MODE == kUmma) ? 2 : 0;
  static constexpr int kX = (MODE == kUmma) ? (NB <= 64 ? 4 : 2) : 0;
  static constexpr int kXLag = (kX >= 4) ? 2 : 1;
  static constexpr uint32_t kOpStage = 2 * kAtomBytes;
  static constexpr uint32_t kXStage = 2 * NB * 128;
  static constexpr uint32_t kReserve = 1024 /* alignment slack */ + 512 /* barriers, flags */;
  static constexpr int kInFit = int((232448u - kReserve - kOp * kOpStage - kX * kXStage) / BXR_BLOB_MAX);
  static constexpr int kIn = kInFit > 8 ? 8 : kInFit;
  static constexpr uint32_t op = 0;
  static constexpr uint32_t xs = op + kOp * kOpStage;
  static constexpr uint32_t in = xs + kX * kXStage;
  static constexpr uint32_t bars = in + kIn * BXR_BLOB_MAX;
  // barrier order: in_full, in_empty [kIn each]; op_full, op_empty [kOp each]; x_full [kX]; acc_full, acc_empty
  // [2 each]; final
  static constexpr uint32_t nbars = 2 * kIn + 2 * kOp + kX + 4 + 1;
  static constexpr uint32_t misc = (bars + 8 * nbars + 15) & ~15u;  // tmem base, abort flag, decision
  static constexpr uint32_t total = misc + 48;
  static constexpr uint32_t alloc = total + 1024;
  static_assert(MODE != kUmma || kIn >= 4, "ring too shallow");
  // what keeps the activation loader at most one barrier phase behind the MMA warp (see its role below)
  static_assert(MODE != kUmma || (kXLag < kX && kOp + kXLag + 1 > kX), "activation ring and lag do not fit the operand ring");
  static_assert(8 * nbars + 64 <= 512, "barrier area");
  static_assert(alloc <= 232448, "exceeds the 227 KB of shared memory a CTA may opt into");
};

// Exponent fields are taken with one mask and moved with one multiply-add whose addend is the row base (in both
// halves): the mask runs on the integer pipe, the multiply-add on the FMA pipe, which the decoder otherwise leaves
// idle.  (The multipliers are kernel parameters so that the compiler does not turn them back into shifts.)
// Word layout: pair k has its fields at bits 1+3k and 17+3k; `hi` is the same word shifted right by 6, which
// brings pairs 3 and 4 to where pairs 1 and 2 are.
struct BxwWord {
  uint32_t lo, hi;
  __device__ __forceinline__ explicit BxwWord(uint32_t w) : lo(w), hi(w >> 6) {}
};
template <int K>
__device__ __forceinline__ uint32_t bxw_exponents(const BxwWord& w, const BxwPowers& p, uint32_t base2) {
  if constexpr (K == 0) return (w.lo & (BXW_PAIR_MASK >> 6)) * p.p6 + base2;
  else if constexpr (K == 1) return (w.lo & (BXW_PAIR_MASK >> 3)) * p.p3 + base2;
  else if constexpr (K == 2) return (w.lo & BXW_PAIR_MASK) * p.p0 + base2;
  else if constexpr (K == 3) return (w.hi & (BXW_PAIR_MASK >> 3)) * p.p3 + base2;
  else return (w.hi & BXW_PAIR_MASK) * p.p0 + base2;
}
// The pair spread over the spare bits 0 and 16 of the three code words.
__device__ __forceinline__ uint32_t bxw_spare_exponents(uint32_t a, uint32_t b, uint32_t c, const BxwPowers& p, uint32_t base2) {
  return (a & 0x00010001u) * p.p7 + ((b & 0x00010001u) * p.p8 + ((c & 0x00010001u) * p.p9 + base2));
}
// raw bytes (sign << 7 | mantissa) of two columns merged with their exponents
__device__ __forceinline__ uint32_t bxw_join(uint32_t raw4, uint32_t selector, uint32_t exponents) {
  return (__byte_perm(raw4, 0, selector) & 0x807F807Fu) | exponents;
}

// The 32 weights of a lane: code words a, b, c and the raw bytes of its two 16-column pieces.
__device__ __forceinline__ void bxw_decode32(uint32_t wa, uint32_t wb, uint32_t wc, const uint4& rf, const uint4& rb,
                                             const BxwPowers& p, uint32_t base2, uint4 (&out)[4]) {
  const BxwWord a(wa), b(wb), c(wc);
  out[0].x = bxw_join(rf.x, 0x1100, bxw_exponents<0>(a, p, base2));
  out[0].y = bxw_join(rf.x, 0x3322, bxw_exponents<1>(a, p, base2));
  out[0].z = bxw_join(rf.y, 0x1100, bxw_exponents<2>(a, p, base2));
  out[0].w = bxw_join(rf.y, 0x3322, bxw_exponents<3>(a, p, base2));
  out[1].x = bxw_join(rf.z, 0x1100, bxw_exponents<4>(a, p, base2));
  out[1].y = bxw_join(rf.z, 0x3322, bxw_exponents<0>(b, p, base2));
  out[1].z = bxw_join(rf.w, 0x1100, bxw_exponents<1>(b, p, base2));
  out[1].w = bxw_join(rf.w, 0x3322, bxw_exponents<2>(b, p, base2));
  out[2].x = bxw_join(rb.x, 0x1100, bxw_exponents<3>(b, p, base2));
  out[2].y = bxw_join(rb.x, 0x3322, bxw_exponents<4>(b, p, base2));
  out[2].z = bxw_join(rb.y, 0x1100, bxw_exponents<0>(c, p, base2));
  out[2].w = bxw_join(rb.y, 0x3322, bxw_exponents<1>(c, p, base2));
  out[3].x = bxw_join(rb.z, 0x1100, bxw_exponents<2>(c, p, base2));
  out[3].y = bxw_join(rb.z, 0x3322, bxw_exponents<3>(c, p, base2));
  out[3].z = bxw_join(rb.w, 0x1100, bxw_exponents<4>(c, p, base2));
  out[3].w = bxw_join(rb.w, 0x3322, bxw_spare_exponents(wa, wb, wc, p, base2));
}

template <int MODE, int NB>
__global__ void __launch_bounds__(MODE == kUmma ? kThreadsUmma : kThreadsSimt, 1)
bxw_kernel(const BxrArgs args, const __grid_constant__ CUtensorMap tmap_x) {
  using L = BxwSmem<MODE, NB>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t worker = blockIdx.x;

  RoleCtx ctx;
  ctx.smem = smem;
  ctx.bars = smem + L::bars;
  ctx.abort_addr = smem + L::misc + 4;
  ctx.status = args.status;
  ctx.suspend = false;  // this pipeline is latency-bound: plain probes wake up sooner
  const uint32_t bar_in_full = ctx.bars, bar_in_empty = bar_in_full + 8 * L::kIn;
  const uint32_t bar_op_full = bar_in_empty + 8 * L::kIn, bar_op_empty = bar_op_full + 8 * L::kOp;
  const uint32_t bar_x_full = bar_op_empty + 8 * L::kOp;
  const uint32_t bar_acc_full = bar_x_full + 8 * L::kX, bar_acc_empty = bar_acc_full + 16, bar_final = bar_acc_empty + 16;
  constexpr uint32_t kTmemCols = 4 * NB;  // {even, odd chunk accumulator} x two items in flight
  constexpr uint32_t kOpN = L::kOp ? L::kOp : 1;
  constexpr uint32_t kXN = L::kX ? L::kX : 1;

  // Work of this CTA, known from the arguments alone; the blob loader asks for its first offsets before anything
  // else so that the first copy can leave as soon as the barriers exist.
  const uint64_t units = uint64_t(args.row_blocks) * args.chunks;
  const uint32_t unit_begin = uint32_t(units * worker / args.workers);
  const uint32_t unit_count = uint32_t(units * (worker + 1) / args.workers) - unit_begin;
  uint32_t first_i0 = 0, first_i1 = 0;
  if (warp == kWinWarpLoader && unit_count) {
    const uint32_t mine = unit_begin + min(uint32_t(lane), unit_count - 1);
    first_i0 = __ldg(args.blob_index + mine);
    first_i1 = __ldg(args.blob_index + mine + 1);
  }
  if (warp == 0) {  // one barrier per lane
    static_assert(L::nbars <= 32, "one lane per barrier");
    const uint32_t i = lane;
    uint32_t count = 1;                                                          // in_full, op_empty, x_full
    if (i >= uint32_t(L::kIn) && i < 2u * L::kIn) count = kDecoderWarps;          // in_empty
    else if (i >= 2u * L::kIn && i < 2u * L::kIn + L::kOp) count = kDecoderWarps + 1;  // op_full: + the loader's go-ahead
    else if (i >= 2u * L::kIn + 2 * L::kOp + L::kX) {
      const uint32_t j = i - (2u * L::kIn + 2 * L::kOp + L::kX);                  // acc_full x2, acc_empty x2, final
      count = j < 2 ? 2u : 4u;                                                   // both MMA issuers / the epilogue warps
    }
    if (i < L::nbars) mbar_init(ctx.bars + 8 * i, count);
    // flags: abort at misc + 4, epilogue decision at misc + 8, final decision at misc + 16 (misc + 0 receives the TMEM
    // base address from the allocating warp and is left alone here)
    if (i == 0) asm volatile("st.shared.v2.u32 [%0], {%1, %1};" ::"r"(smem + L::misc + 8), "r"(0u) : "memory");
    if (i == 1) asm volatile("st.shared.u32 [%0], %1;" ::"r"(smem + L::misc + 4), "r"(0u) : "memory");
    if (i == 2 || i == 3) asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(smem + L::misc + 16 * (i - 1)), "r"(0u) : "memory");
    mbar_fence_init();
  }
  if (MODE == kUmma && warp == kWinWarpMma) {
    tmem_alloc(smem + L::misc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // The image is never written by a kernel: everything up to the first access to x, bias, y or the workspace may
  // overlap the tail of the previous kernel in the stream.
  grid_dependents_may_launch();
  if (MODE == kDense) grid_dependency_wait();
  uint32_t tmem_base = 0;
  if (MODE == kUmma) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(smem + L::misc));

  const uint32_t item_begin = args.worker_items[worker], item_end = args.worker_items[worker + 1];

  if (warp < kDecoderWarps) {
    // ------------------------------------------------------------------ decoders: 32 weights per lane and chunk
    const uint32_t q = warp >> 2, r = (warp & 3) * 32 + lane;
    const uint32_t seg = q * BXR_ROWS + r;
    uint32_t s = 0, ph = 0;    // input ring slot of the current chunk and its phase parity
    uint32_t so = 0, pho = 0;  // operand stage of the current chunk
    const uint32_t raw_at = BXW_RAW_AT + ((2 * q) * BXR_ROWS + r) * 16;
    const uint32_t code_at = BXW_CODES_AT + 4 * seg;
    const uint32_t atom_at = (q >> 1) * kAtomBytes;
    uint32_t st_at[4];         // swizzled 16-byte positions of this lane's four stores inside its atom
#pragma unroll
    for (int i = 0; i < 4; ++i) st_at[i] = r * 128 + ((((q & 1) * 4 + i) ^ (r & 7)) << 4);
    bool live = true;
    for (uint32_t it = item_begin; it < item_end && live; ++it) {
      const bxr_item item = args.items[it];
      const uint32_t row = item.row_block * BXR_ROWS + r;
      const uint32_t base2 = uint32_t(args.base[row]) * 0x00800080u;
      for (uint32_t c = item.chunk_begin; c < item.chunk_end; ++c) {
        if (!ctx.wait(bar_in_full + 8 * s, ph)) { live = false; break; }
        const uint32_t blob = smem + L::in + s * BXR_BLOB_MAX;
        const uint32_t wa = lds32(blob + code_at), wb = lds32(blob + code_at + 4 * BXR_SEGMENTS),
                       wc = lds32(blob + code_at + 8 * BXR_SEGMENTS);
        const uint4 raw_f = lds128(blob + raw_at);
        const uint4 raw_b = lds128(blob + raw_at + BXR_ROWS * 16);
        // Entries of this warp: weights outside their row window.  An entry names the word (by its place in the
        // warp's part of the operand tile) and the exponent correction.  Lane i takes the warp's i-th entry, whoever
        // owns the row, and builds the complete BF16 word now, so that after the fixed-code pass only a 2-byte
        // store is left and the blob's slot can be handed back before the operand stage is even free.  Corrupt
        // bounds are clamped so that every read stays inside the slot.
        const uint32_t e_lo = lds_u16(blob + BXW_WARP_END_AT + 2 * warp);
        const uint32_t e_hi = min(lds_u16(blob + BXW_WARP_END_AT + 2 * warp + 2), uint32_t(BXW_ENTRY_MAX));
        const bool mine = e_lo + lane < e_hi;
        const uint32_t entry = mine ? lds_u16(blob + BXW_LIST_AT + 2 * (e_lo + lane)) : 0u;
        const uint32_t place = entry & ((1u << BXW_PLACE_BITS) - 1);
        const int delta = int(entry << 16) >> (16 + BXW_PLACE_BITS);
        const uint32_t p_rl = place >> 6, p_unit = ((place >> 3) & 7u) ^ (p_rl & 7u), p_j = (p_unit & 3u) * 8 + (place & 7u);
        const uint32_t p_byte = lds_u8(blob + BXW_RAW_AT + ((2 * q + (p_j >> 4)) * BXR_ROWS + (warp & 3) * 32 + p_rl) * 16 + (p_j & 15u));
        const uint32_t p_exp = (__shfl_sync(0xFFFFFFFFu, base2, p_rl) >> 7) + uint32_t(delta);
        const uint32_t p_word = (p_byte & 0x80u) << 8 | (p_exp & 0xFFu) << 7 | (p_byte & 0x7Fu);
        // rare: more than 32 entries in this warp's part of the chunk, or an exponent too far off for the 5-bit field
        const bool slow = __any_sync(0xFFFFFFFFu, (mine && delta == BXW_DELTA_FAR) || e_hi > e_lo + 32);
        uint4 out[4];
        bxw_decode32(wa, wb, wc, raw_f, raw_b, args.kw, base2, out);
        if (!slow) {  // everything this warp needs from the blob is in registers
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_in_empty + 8 * s);
        }
        uint32_t a_tile = 0;
        if (MODE == kUmma) {
          if (!ctx.wait(bar_op_empty + 8 * so, pho ^ 1)) { live = false; break; }
          a_tile = smem + L::op + so * L::kOpStage + atom_at;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (MODE == kUmma) {
            sts128(a_tile + st_at[i], out[i]);
          } else if (row < args.rows) {
            const uint32_t col = c * BXR_COLS + q * 32 + i * 8;
            uint16_t* dst = args.dense + size_t(row) * args.cols + col;
            if (col + 8 <= args.cols && (args.cols & 7) == 0) {
              *reinterpret_cast<uint4*>(dst) = out[i];
            } else {
              const uint32_t ww[4] = {out[i].x, out[i].y, out[i].z, out[i].w};
              for (int e = 0; e < 8; ++e)
                if (col + e < args.cols) dst[e] = uint16_t(ww[e >> 1] >> (16 * (e & 1)));
            }
          }
        }
        __syncwarp();  // the fixed-code pass of every lane is in place before another lane patches it
        if (mine && delta != BXW_DELTA_FAR) {
          if (MODE == kUmma) {
            sts_u16(a_tile + (warp & 3) * 4096 + 2 * place, p_word);
          } else {
            const uint32_t prow = item.row_block * BXR_ROWS + (warp & 3) * 32 + p_rl, pcol = c * BXR_COLS + q * 32 + p_j;
            if (prow < args.rows && pcol < args.cols) args.dense[size_t(prow) * args.cols + pcol] = uint16_t(p_word);
          }
        }
        if (slow) {
          // far entries among the first 32, and every entry beyond them: read the word back and correct it
          for (uint32_t i = e_lo + lane; i < e_hi; i += 32) {
            const uint32_t v = lds_u16(blob + BXW_LIST_AT + 2 * i);
            const uint32_t pl = v & ((1u << BXW_PLACE_BITS) - 1);
            const int dl = int(v << 16) >> (16 + BXW_PLACE_BITS);
            if (i < e_lo + 32 && dl != BXW_DELTA_FAR) continue;  // already done above
            uint32_t far_e = 0;
            if (dl == BXW_DELTA_FAR) {
              const uint32_t total = min(lds_u16(blob + BXW_WARP_END_AT + 32), uint32_t(BXW_ENTRY_MAX));
              const uint32_t n_far = min(lds_u16(blob + BXW_FAR_COUNT_AT), uint32_t(BXW_FAR_MAX));
              const uint32_t far_at = blob + ((BXW_LIST_AT + 2 * total + 3) & ~3u);
              const uint32_t key = uint32_t(warp) << BXW_PLACE_BITS | pl;
              for (uint32_t f = 0; f < n_far; ++f) {
                const uint32_t x = lds32(far_at + 4 * f);
                if ((x & 0x7FFFu) == key) far_e = (x >> 16) & 0xFFu;
              }
            }
            if (MODE == kUmma) {
              const uint32_t at = a_tile + (warp & 3) * 4096 + 2 * pl;
              const uint32_t old = lds_u16(at);
              sts_u16(at, dl == BXW_DELTA_FAR ? ((old & 0x807Fu) | far_e << 7) : old + uint32_t(dl) * args.kw.p7);
            } else {
              const uint32_t rl = pl >> 6, unit = ((pl >> 3) & 7u) ^ (rl & 7u), j = (unit & 3u) * 8 + (pl & 7u);
              const uint32_t prow = item.row_block * BXR_ROWS + (warp & 3) * 32 + rl, pcol = c * BXR_COLS + q * 32 + j;
              if (prow < args.rows && pcol < args.cols) {
                volatile uint16_t* w = args.dense + size_t(prow) * args.cols + pcol;
                const uint32_t old = *w;
                *w = uint16_t(dl == BXW_DELTA_FAR ? ((old & 0x807Fu) | far_e << 7) : old + uint32_t(dl) * 128u);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_in_empty + 8 * s);
        }
        if (MODE == kUmma) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_op_full + 8 * so);
          if (++so == kOpN) { so = 0; pho ^= 1; }
        } else {
          __syncwarp();
        }
        if (++s == L::kIn) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == kWinWarpLoader) {
    // ------------------------------------------------------------------ chunk blobs, one bulk copy each
    uint32_t issued = 0;
    for (uint32_t u0 = 0; u0 < unit_count; u0 += 32) {
      uint32_t i0 = first_i0, i1 = first_i1;
      if (u0) {
        const uint32_t mine = unit_begin + min(u0 + lane, unit_count - 1);
        i0 = __ldg(args.blob_index + mine);
        i1 = __ldg(args.blob_index + mine + 1);
      }
      const uint32_t n = min(32u, unit_count - u0);
      bool live = true;
      for (uint32_t i = 0; i < n && live; ++i) {
        const uint32_t u = u0 + i, s = u % L::kIn, ph = (u / L::kIn) & 1;
        const uint32_t b0 = __shfl_sync(0xFFFFFFFFu, i0, i), b1 = __shfl_sync(0xFFFFFFFFu, i1, i);
        const uint32_t bytes = (b1 - b0) << 4;
        if (ctx.aborted() || !ctx.wait(bar_in_empty + 8 * s, ph ^ 1)) { live = false; break; }
        if (b1 < b0 || bytes > BXR_BLOB_MAX || bytes < BXW_LIST_AT) {
          ctx.abort(kStatusBadArgument);
          live = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(bar_in_full + 8 * s, bytes);
          bulk_g2s(smem + L::in + s * BXR_BLOB_MAX, args.blobs + (size_t(b0) << 4), bytes, bar_in_full + 8 * s);
        }
        issued = u + 1;
      }
      if (!live) break;
    }
    // after an abort: give copies still in flight a bounded time to land before the CTA exits
    if (ctx.aborted() && lane == 0)
      for (uint32_t u = (issued > uint32_t(L::kIn) ? issued - L::kIn : 0); u < issued; ++u) mbar_wait(bar_in_full + 8 * (u % L::kIn), (u / L::kIn) & 1);
  } else if (MODE == kUmma && warp == kWinWarpXLoader) {
    // ------------------------------------------------------------------ activation tiles by TMA, and the go-ahead
    // One thread.  Chunk v of this CTA (in the order the items list them) uses activation stage v % kX and operand
    // stage v % kOp.  The tiles of chunk v are requested once chunk v - kX has been multiplied (its stage is free);
    // kXLag chunks later the thread waits for them and gives the MMA warp the go-ahead by arriving on the operand
    // stage's `full` barrier, which the decoder warps complete.  "Chunk c has been multiplied" is the phase of
    // op_empty[c % kOp] that the MMA warp's commit completes; this thread is never more than one phase behind it,
    // because the multiply of chunk c + kOp needs its own go-ahead.
    if (lane == 0) {
      grid_dependency_wait();
      bool live = true;
      uint32_t it_v = item_begin, c_v = 0;  // cursor of the chunk to request: item and chunk inside it
      bxr_item item_v = args.items[item_begin < item_end ? item_begin : 0];
      c_v = item_v.chunk_begin;
      auto multiplied = [&](uint32_t c) { return ctx.wait(bar_op_empty + 8 * (c % kOpN), (c / kOpN) & 1); };
      for (uint32_t v = 0; v < unit_count + L::kXLag && live; ++v) {
        if (ctx.aborted()) break;
        if (v < unit_count) {
          if (v >= kXN && !multiplied(v - kXN)) { live = false; break; }
          const uint32_t sx = v % kXN, stage = smem + L::xs + sx * L::kXStage;
          mbar_arrive_expect_tx(bar_x_full + 8 * sx, L::kXStage);
          tma_load_2d(stage, &tmap_x, int(c_v * BXR_COLS), 0, bar_x_full + 8 * sx);
          tma_load_2d(stage + NB * 128, &tmap_x, int(c_v * BXR_COLS + 64), 0, bar_x_full + 8 * sx);
          if (++c_v == item_v.chunk_end && it_v + 1 < item_end) {
            item_v = args.items[++it_v];
            c_v = item_v.chunk_begin;
          }
        }
        if (v >= uint32_t(L::kXLag)) {
          const uint32_t w = v - L::kXLag;
          if (!ctx.wait(bar_x_full + 8 * (w % kXN), (w / kXN) & 1)) { live = false; break; }
          if (w >= kOpN && !multiplied(w - kOpN)) { live = false; break; }
          mbar_arrive(bar_op_full + 8 * (w % kOpN));
        }
      }
    }
  } else if (MODE == kUmma && (warp == kWinWarpMma || warp == kWinWarpMmaOdd)) {
    // ------------------------------------------------------------------ MMA issue: one wait, eight MMAs, one commit
    // Two issuers take the chunks of the CTA in turn (even / odd position in the CTA's chunk sequence) and accumulate
    // into accumulators of their own, so that one of them can wait for its next chunk while the other keeps the
    // tensor pipe fed.  Which chunk goes where depends on the image's work partition only, never on the batch size.
    static_assert(MODE != kUmma || kOpN == 2, "an issuer owns the operand stage of its parity");
    constexpr uint32_t idesc = umma_idesc_bf16(NB);
    const uint32_t parity = warp == kWinWarpMmaOdd ? 1u : 0u;
    uint32_t n_item = 0, so = 0, pho = 0, sx = 0;
    bool live = true;
    for (uint32_t it = item_begin; it < item_end && live; ++it, ++n_item) {
      const bxr_item item = args.items[it];
      const uint32_t buf = n_item & 1;
      if (ctx.aborted() || !ctx.wait(bar_acc_empty + 8 * buf, ((n_item >> 1) & 1) ^ 1)) { live = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (2 * buf + parity) * NB;
      uint32_t accumulate = 0;
      for (uint32_t c = item.chunk_begin; c < item.chunk_end; ++c) {
        if (so == parity) {
          if (!ctx.wait(bar_op_full + 8 * so, pho)) { live = false; break; }
          tc_fence_after();
          if (lane == 0) {
            const uint64_t adesc = umma_desc_sw128(smem + L::op + so * L::kOpStage), bdesc = umma_desc_sw128(smem + L::xs + sx * L::kXStage);
#pragma unroll
            for (uint32_t a = 0; a < 2; ++a)
#pragma unroll
              for (uint32_t k = 0; k < 4; ++k) {
                umma_bf16(d_tmem, adesc + a * (kAtomBytes >> 4) + 2 * k, bdesc + a * (NB * 128 >> 4) + 2 * k, idesc, accumulate);
                accumulate = 1;
              }
            umma_commit(bar_op_empty + 8 * so);
          }
          __syncwarp();
        }
        if (++so == kOpN) { so = 0; pho ^= 1; }
        if (++sx == kXN) sx = 0;
      }
      // the accumulator of this issuer is complete when its MMAs are; an issuer without a chunk in the item (a
      // single-chunk item of the other parity) only reports in
      if (live && lane == 0) {
        if (accumulate) umma_commit(bar_acc_full + 8 * buf);
        else mbar_arrive(bar_acc_full + 8 * buf);
      }
      __syncwarp();
    }
  } else if (MODE == kUmma && warp >= kWinWarpEpilogue) {
    // ------------------------------------------------------------------ TMEM -> y, or -> FP32 partial tile
    const uint32_t e = warp - kWinWarpEpilogue;  // == warp % 4: the TMEM lane quarter this warp may read
    const uint32_t r = e * 32 + lane;
    const uint32_t mcols = (args.m + 7) & ~7u;
    uint32_t n_item = 0, u_seen = 0;  // u_seen: chunks of this CTA before the current item
    bool live = true;
    grid_dependency_wait();  // bias, y, partial tiles and counters may belong to the previous kernel
    for (uint32_t it = item_begin; it < item_end && live; ++it, ++n_item) {
      const bxr_item item = args.items[it];
      const uint32_t buf = n_item & 1;
      if (ctx.aborted() || !ctx.wait(bar_acc_full + 8 * buf, (n_item >> 1) & 1)) { live = false; break; }
      tc_fence_after();
      const uint32_t row = item.row_block * BXR_ROWS + r;
      const uint32_t taddr = tmem_base + ((e * 32) << 16) + 2 * buf * NB;
      const uint32_t n_chunks = item.chunk_end - item.chunk_begin;
      const bool two = n_chunks > 1;                               // both issuers had a chunk of this item
      const uint32_t only = two ? 0u : (u_seen & 1u) * NB;          // else: the accumulator of the chunk's parity
      u_seen += n_chunks;
      const float b = (args.bias && row < args.rows) ? __bfloat162float(args.bias[row]) : 0.f;
      for (uint32_t m0 = 0; m0 < mcols; m0 += 8) {
        uint32_t v[8];
        tmem_ld8(taddr + only + m0, v);
        if (two) {  // even chunks + odd chunks, one FP32 addition per output
          uint32_t o[8];
          tmem_ld8(taddr + NB + m0, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] = __float_as_uint(__fadd_rn(__uint_as_float(v[i]), __uint_as_float(o[i])));
        } else {
          tmem_ld_wait();
        }
        if (item.parts == 1) {
          if (row < args.rows)
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (m0 + i < args.m) {
                const float f = __uint_as_float(v[i]);
                args.y[size_t(m0 + i) * args.ldy + row] = __float2bfloat16_rn(args.bias ? __fadd_rn(f, b) : f);
              }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) args.partials[(size_t(item.slot) * NB + m0 + i) * BXR_ROWS + r] = __uint_as_float(v[i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
      if (item.parts > 1) {
        __threadfence();
        named_barrier(1, 128);
        if (e == 0 && lane == 0) {
          const uint32_t prev = atomicAdd(args.counters + item.row_block, 1u);
          asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(smem + L::misc + 8), "r"(prev) : "memory");
        }
        named_barrier(1, 128);
        uint32_t prev;
        asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(prev) : "r"(smem + L::misc + 8));
        if (prev == item.parts - 1) {  // every partial tile of this row block is in memory: add them in K order
          __threadfence();
          const uint32_t first = item.slot - item.part;
          if (it + 1 == item_end) {
            // the CTA's last item: the decoder warps have nothing left to do and share the reduction (below)
            if (e == 0 && lane == 0)
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(smem + L::misc + 16), "r"(1u), "r"(item.row_block),
                           "r"(first), "r"(item.parts) : "memory");
          } else {
            reduce_row_block<NB>(args, item.row_block, first, item.parts, e, 4, lane);
          }
          if (e == 0 && lane == 0) args.counters[item.row_block] = 0;
        }
        named_barrier(1, 128);  // the decision word may be rewritten
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_final);
  }

  // A row block whose last partial tile came from this CTA's final item is reduced by the 16 decoder warps and
  // the 4 epilogue warps together.
  if (MODE == kUmma && (warp < kDecoderWarps || warp >= kWinWarpEpilogue)) {
    if (ctx.wait(bar_final, 0)) {
      const uint4 decision = lds128(smem + L::misc + 16);  // {reduce?, row block, first slot, parts}
      if (decision.x)
        reduce_row_block<NB>(args, decision.y, decision.z, decision.w, warp < kDecoderWarps ? warp : warp - 4, kDecoderWarps + 4, lane);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (MODE == kUmma && warp == kWinWarpMma) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace grb
