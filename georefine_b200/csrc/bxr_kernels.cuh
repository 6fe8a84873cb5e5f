// Fused kernels over the BXR1 resident layout (bxr_format.h): one persistent CTA per worker walks its
// share of (row block, chunk) units.  A chunk blob arrives in shared memory by one bulk copy; 16 warps
// decode it (one rANS stream per lane, two weights per step) and the reconstructed BF16 words go
//   * kDense : to global memory (the decode twin used by decode() and by the parity tests),
//   * kGemv  : into FP32 FMA chains against up to 8 activation rows (CUDA cores), or
//   * kUmma  : into a 128-byte-swizzled K-major operand tile consumed by tcgen05.mma with the FP32
//              accumulator in TMEM (weights are the M=128 operand, the batch is N).
// They stand where the reference runs decode_words + F.linear
// (context-runtime/georefine_context_runtime/bitexact_context_gpu.py:130-157,
// bitexact_context_serving.py:365-376) and its fused MIV / BI linears (glc_serve/miv_gemv.py:125-191,
// glc_serve/bi_csrc/bi_gemm.cuh:797-916).  The reduction order of every output element depends only on
// the image (shape, worker count), never on the batch size.
#pragma once
#include <cuda.h>

#include "bxr_format.h"
#include "device_utils.cuh"

namespace grb {

enum BxrMode { kDense = 0, kGemv = 1, kUmma = 2 };

constexpr int kDecoderWarps = 16;
constexpr int kWarpLoader = 16;    // bulk copies of chunk blobs
constexpr int kWarpScanner = 17;   // segment offsets (and FP32 activations for the GEMV)
constexpr int kWarpMma = 18;       // TMEM owner and MMA issuer
constexpr int kWarpXLoader = 19;   // TMA loads of activation tiles
constexpr int kWarpEpilogue = 20;  // 4 warps, TMEM lane quarter = warp % 4
constexpr int kThreadsUmma = 24 * 32;
constexpr int kThreadsSimt = 18 * 32;

constexpr uint32_t kLutBytes = 4 * BXR_PROB_TOTAL;
constexpr uint32_t kSegOffBytes = 1040;  // u16[513] rounded up
constexpr uint32_t kAtomBytes = 16384;  // 128 rows x 64 BF16
constexpr uint32_t kInGuard = 128;      // a corrupt stream may read up to 50 bytes past its slot
constexpr int kGemvMaxM = 8;

// Powers of two passed as kernel parameters so that the compiler keeps `x * 2^k + y` a multiply-add on the FMA
// pipe instead of a shift and an add on the busier integer pipe.
struct BxrPowers {
  uint32_t p7, p16;  // 128, 65536
};

// The same device for the window-mode decoder: 1, 8, 64, 128, 256, 512.
struct BxwPowers {
  uint32_t p0, p3, p6, p7, p8, p9;
};

struct BxrArgs {
  // image
  const uint32_t* lut;
  BxrPowers k;
  BxwPowers kw;
  const uint8_t* base;
  const bxr_item* items;
  const uint32_t* worker_items;
  const uint32_t* states;
  const uint32_t* blob_index;
  const uint8_t* blobs;
  uint32_t blob_stride16;      // nonzero: blobs of one size (16-byte units), blob b at b * size; else see blob_index
  uint32_t rows, cols, row_blocks, chunks, workers;
  uint32_t raw;                // image holds plain pre-swizzled tiles (BXR_MODE_RAW): kUmma only, no decoders
  uint32_t window;             // image holds fixed 3-bit exponent codes (BXR_MODE_WINDOW): served by bxw_kernel
  uint32_t window4;            // image holds fixed 4-bit exponent codes (BXR_MODE_WINDOW4): served by bxq_kernel
  // call
  uint32_t m;                  // activation rows in this launch (<= NB, <= 8 for the GEMV)
  const __nv_bfloat16* x;      // GEMV only (the UMMA path reads x through the tensor map)
  long long ldx;
  __nv_bfloat16* y;
  long long ldy;
  const __nv_bfloat16* bias;   // optional, one per weight row
  float* partials;             // FP32 [partial_slots][NB][128]
  uint32_t* counters;          // [row_blocks], zero between calls
  uint16_t* dense;             // kDense: rows x cols words
  uint32_t* status;
  uint32_t cluster;            // bxq_kernel: > 1 = launched as clusters of this many CTAs, one cluster per row block
  // bxq_kernel, optional: the image the NEXT launch in the stream will read (blobs of one size).  A CTA whose own
  // loads have all been issued asks the L2 for the first blobs of the next launch's CTAs, so that HBM keeps working
  // through this launch's tail and the next launch's prologue.
  const uint8_t* next_blobs;
  uint32_t next_blob_bytes, next_units, next_workers;
};

template <int MODE, int NB>
struct BxrSmem {
  static constexpr int kIn = (MODE == kUmma && NB <= 32) ? 5 : 4;
  static constexpr int kOp = (MODE == kUmma) ? ((NB >= 128) ? 3 : 4) : 0;
  static constexpr uint32_t kOpStage = kAtomBytes + NB * 128;
  static constexpr uint32_t kXStage = (MODE == kGemv) ? kGemvMaxM * BXR_COLS * 4 : 0;  // FP32 activations per chunk
  static constexpr uint32_t lut = 0;
  static constexpr uint32_t op = lut + kLutBytes;
  static constexpr uint32_t in = op + kOp * kOpStage;
  static constexpr uint32_t segoff = in + kIn * BXR_BLOB_MAX + kInGuard;
  static constexpr uint32_t xf32 = segoff + kIn * kSegOffBytes;
  static constexpr uint32_t bars = (xf32 + kIn * kXStage + 15) & ~15u;
  // barrier order: in_full, in_ready, in_empty [kIn each]; op_full, op_empty [kOp each]; acc_full, acc_empty [2 each]
  static constexpr uint32_t nbars = 3 * kIn + 2 * kOp + 4 + 2;  // + the table's arrival barrier, + the final decision
  static constexpr uint32_t misc = (bars + 8 * nbars + 15) & ~15u;  // tmem base, abort flag, reduce flag, spare
  static constexpr uint32_t red = misc + 48;          // GEMV: FP32 [4 phases][128 rows][8]
  static constexpr uint32_t total = red + (MODE == kGemv ? 4 * 128 * kGemvMaxM * 4 : 0);
  static constexpr uint32_t alloc = total + 1024;     // slack to align the base to 1024
  static_assert(alloc <= 232448, "exceeds the 227 KB of shared memory a CTA may opt into");
};

struct RoleCtx {
  uint32_t smem;       // aligned base (shared address)
  uint32_t bars;
  uint32_t abort_addr; // shared address of the abort flag
  uint32_t* status;
  bool suspend = true;  // barrier probes may park the thread (see mbar_try_wait)
  __device__ __forceinline__ bool aborted() const {
    uint32_t v;
    asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(abort_addr));
    return v != 0;
  }
  __device__ __forceinline__ void abort(uint32_t bits) const {
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort_addr), "r"(1u) : "memory");
    atomicOr(status, bits);
  }
  // Bounded wait; on expiry marks the CTA aborted.  The first wait of the launch to give up also records where:
  // bits 8..15 of the status word receive 1 + the barrier's index in the kernel's barrier area, bits 16..23 the CTA
  // (diagnostic only).
  __device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity) const {
    if (mbar_wait(bar, parity, suspend)) return true;
    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(abort_addr), "r"(1u) : "memory");
    if ((atomicOr(status, kStatusTimeout) & kStatusTimeout) == 0)
      atomicOr(status, ((((bar - bars) >> 3) + 1u) & 0xFFu) << 8 | (blockIdx.x & 0xFFu) << 16);
    return false;
  }
};

// The two rANS streams of a lane (the forward and the backward reader of one segment), advanced together
// so that their dependency chains overlap.  A step of a stream yields the exponent bits of two weights in
// packed-BF16 position (bits 7..14 and 23..30).
struct LaneDecoder {
  uint32_t xf, xb;   // rANS states
  uint32_t wf, wb;   // shared addresses of the next 16-bit word of each stream
  uint32_t lut;      // shared address of the slot records
  uint32_t base2;    // row base replicated into both exponent fields
  BxrPowers k;

  __device__ __forceinline__ void start_chunk(uint32_t first_f, uint32_t first_b) {
    wf = first_f;
    wb = first_b;
  }
  // (x << 16) | word, written as one multiply-add
  __device__ __forceinline__ void refill_f() {
    if (xf < BXR_STATE_LOW) { xf = xf * k.p16 + lds_u16(wf); wf += 2; }
  }
  __device__ __forceinline__ void refill_b() {
    if (xb < BXR_STATE_LOW) { xb = xb * k.p16 + lds_u16(wb); wb -= 2; }
  }
  // One step of both streams.  The record layout keeps the integer-pipe work low: the frequency is the top
  // field (one shift), the nibble pair becomes the exponent pair with one mask and one multiply-add.
  __device__ __forceinline__ void step(uint32_t& ef, uint32_t& eb) {
    const uint32_t af = lut + ((xf & (BXR_PROB_TOTAL - 1)) << 2), ab = lut + ((xb & (BXR_PROB_TOTAL - 1)) << 2);
    const uint32_t rf = lds32(af), rb = lds32(ab);
    xf = BXR_REC_FREQ(rf) * (xf >> BXR_PROB_BITS) + BXR_REC_BIAS(rf);
    xb = BXR_REC_FREQ(rb) * (xb >> BXR_PROB_BITS) + BXR_REC_BIAS(rb);
    refill_f();
    refill_b();
    ef = (rf & BXR_LUT_NIBBLES) * k.p7 + base2;
    eb = (rb & BXR_LUT_NIBBLES) * k.p7 + base2;
  }
};

// Two raw bytes (sign << 7 | mantissa) and two exponents -> two BF16 words in one register.
__device__ __forceinline__ uint32_t join_pair(uint32_t raw4, uint32_t selector, uint32_t expo) {
  return (__byte_perm(raw4, 0, selector) & 0x807F807Fu) | expo;
}

// Decodes 8 consecutive weights of each of the lane's two streams from 8 raw bytes per stream.
__device__ __forceinline__ void decode8x2(LaneDecoder& d, uint32_t f_lo, uint32_t f_hi, uint32_t b_lo, uint32_t b_hi,
                                          uint4& wf, uint4& wb) {
  uint32_t ef, eb;
  d.step(ef, eb);
  wf.x = join_pair(f_lo, 0x1100, ef);
  wb.x = join_pair(b_lo, 0x1100, eb);
  d.step(ef, eb);
  wf.y = join_pair(f_lo, 0x3322, ef);
  wb.y = join_pair(b_lo, 0x3322, eb);
  d.step(ef, eb);
  wf.z = join_pair(f_hi, 0x1100, ef);
  wb.z = join_pair(b_hi, 0x1100, eb);
  d.step(ef, eb);
  wf.w = join_pair(f_hi, 0x3322, ef);
  wb.w = join_pair(b_hi, 0x3322, eb);
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

// Ordered reduction of the FP32 partial tiles of one row block: y[m, row] = bf16(sum over parts in K order
// (+ bias)).  Called by the CTA that delivered the last tile.  `group` warps share the work: warp g takes the
// batch rows g, g + group, ...; a lane takes 4 consecutive weight rows (one float4 per tile).  The tiles come from
// other SMs through the L2, a round trip of half a microsecond: a thread asks for MS batch rows x PS tiles at once
// and adds them, in tile order, when they are there.  Tile `own` (an index among the parts; none if >= parts) is
// read from shared memory at `own_tile` instead, in the same [batch row][128 weight rows] order.
template <int NB, int MS, int PS>
__device__ __forceinline__ void reduce_row_block_by(const BxrArgs& args, uint32_t row_block, uint32_t first, uint32_t parts,
                                                    uint32_t g, uint32_t group, uint32_t lane, uint32_t own, uint32_t own_tile) {
  const uint32_t r4 = lane * 4, row4 = row_block * BXR_ROWS + r4;
  if (row4 >= args.rows) return;
  float bias4[4] = {0.f, 0.f, 0.f, 0.f};
  if (args.bias)
    for (int i = 0; i < 4; ++i)
      if (row4 + i < args.rows) bias4[i] = __bfloat162float(args.bias[row4 + i]);
  const bool whole = row4 + 3 < args.rows;
  for (uint32_t m0 = g; m0 < args.m; m0 += MS * group) {
    float4 t[MS];
    for (uint32_t p0 = 0; p0 < parts; p0 += PS) {
      float4 v[MS][PS];
#pragma unroll
      for (int j = 0; j < MS; ++j)
#pragma unroll
        for (int q = 0; q < PS; ++q) {
          const uint32_t m = m0 + group * j, p = p0 + q;
          if (m < args.m && p < parts) {
            if (p == own) {
              const uint4 u = lds128(own_tile + (m * BXR_ROWS + r4) * 4);
              v[j][q] = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
            } else {
              v[j][q] = __ldcg(reinterpret_cast<const float4*>(args.partials + (size_t(first + p) * NB + m) * BXR_ROWS + r4));
            }
          } else {
            v[j][q] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
        }
#pragma unroll
      for (int q = 0; q < PS; ++q) {
        if (p0 + q >= parts) break;
#pragma unroll
        for (int j = 0; j < MS; ++j) {
          if (p0 + q == 0) {
            t[j] = v[j][q];  // the first tile is taken as it is (adding it to zero would lose the sign of a -0)
          } else {
            t[j].x = __fadd_rn(t[j].x, v[j][q].x);
            t[j].y = __fadd_rn(t[j].y, v[j][q].y);
            t[j].z = __fadd_rn(t[j].z, v[j][q].z);
            t[j].w = __fadd_rn(t[j].w, v[j][q].w);
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < MS; ++j) {
      const uint32_t m = m0 + group * j;
      if (m >= args.m) continue;
      const float f[4] = {t[j].x, t[j].y, t[j].z, t[j].w};
      __nv_bfloat16* dst = args.y + size_t(m) * args.ldy + row4;
      if (whole && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
        __nv_bfloat162 lo, hi;
        lo.x = __float2bfloat16_rn(args.bias ? __fadd_rn(f[0], bias4[0]) : f[0]);
        lo.y = __float2bfloat16_rn(args.bias ? __fadd_rn(f[1], bias4[1]) : f[1]);
        hi.x = __float2bfloat16_rn(args.bias ? __fadd_rn(f[2], bias4[2]) : f[2]);
        hi.y = __float2bfloat16_rn(args.bias ? __fadd_rn(f[3], bias4[3]) : f[3]);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&lo);
        packed.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(dst) = packed;
      } else {
        for (int i = 0; i < 4; ++i)
          if (row4 + i < args.rows) dst[i] = __float2bfloat16_rn(args.bias ? __fadd_rn(f[i], bias4[i]) : f[i]);
      }
    }
  }
}
template <int NB>
__device__ __forceinline__ void reduce_row_block(const BxrArgs& args, uint32_t row_block, uint32_t first, uint32_t parts,
                                                 uint32_t g, uint32_t group, uint32_t lane, uint32_t own = 0xFFFFFFFFu,
                                                 uint32_t own_tile = 0) {
  // eight loads in flight per thread either way
  if (parts <= 2) reduce_row_block_by<NB, 4, 2>(args, row_block, first, parts, g, group, lane, own, own_tile);
  else reduce_row_block_by<NB, 2, 4>(args, row_block, first, parts, g, group, lane, own, own_tile);
}

template <int MODE, int NB>
__global__ void __launch_bounds__(MODE == kUmma ? kThreadsUmma : kThreadsSimt, 1)
bxr_kernel(const BxrArgs args, const __grid_constant__ CUtensorMap tmap_x) {
  using L = BxrSmem<MODE, NB>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t worker = blockIdx.x;

  RoleCtx ctx;
  ctx.smem = smem;
  ctx.bars = smem + L::bars;
  ctx.abort_addr = smem + L::misc + 4;
  ctx.status = args.status;
  const uint32_t bar_in_full = ctx.bars, bar_in_ready = bar_in_full + 8 * L::kIn, bar_in_empty = bar_in_ready + 8 * L::kIn;
  const uint32_t bar_op_full = bar_in_empty + 8 * L::kIn, bar_op_empty = bar_op_full + 8 * L::kOp;
  const uint32_t bar_acc_full = bar_op_empty + 8 * L::kOp, bar_acc_empty = bar_acc_full + 16, bar_lut = bar_acc_empty + 16, bar_final = bar_lut + 8;
  constexpr uint32_t kTmemCols = (2 * NB < 32) ? 32 : 2 * NB;
  constexpr uint32_t kOpN = L::kOp ? L::kOp : 1;  // ring length of the operand stages (unused outside kUmma)

  if (threadIdx.x == 0) {
    for (int i = 0; i < L::kIn; ++i) {
      mbar_init(bar_in_full + 8 * i, 1);
      mbar_init(bar_in_ready + 8 * i, 1);
      mbar_init(bar_in_empty + 8 * i, kDecoderWarps);
    }
    for (int i = 0; i < L::kOp; ++i) {
      // coded image: 8 decoder warps + the activation TMA; raw image: the tile copy + the activation TMA
      mbar_init(bar_op_full + 8 * i, args.raw ? 2 : kDecoderWarps / 2 + 1);
      mbar_init(bar_op_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      // GEMV: pair 0 guards the cross-phase reduction buffer (filled by 16 warps, drained by 4)
      mbar_init(bar_acc_full + 8 * i, MODE == kGemv ? kDecoderWarps : 1);
      mbar_init(bar_acc_empty + 8 * i, 4);
    }
    mbar_init(bar_lut, 1);
    mbar_init(bar_final, 4);  // one arrival per epilogue warp once its items are done
    // flags: abort at misc + 4, decisions at misc + 8 and misc + 16 (misc + 0 receives the TMEM base address from the
    // allocating warp and is left alone here)
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(smem + L::misc + 4), "r"(0u) : "memory");
    asm volatile("st.shared.v2.u32 [%0], {%1, %1};" ::"r"(smem + L::misc + 8), "r"(0u) : "memory");
    for (int i = 1; i < 3; ++i) asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(smem + L::misc + 16 * i), "r"(0u) : "memory");
    mbar_fence_init();
  }
  if (MODE == kUmma && warp == kWarpMma) {
    tmem_alloc(smem + L::misc, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // The image (table, blobs, states) is never written by a kernel, so everything up to the first access to x,
  // bias, y or the workspace may overlap the tail of the previous kernel in the stream; the roles that touch
  // those call grid_dependency_wait() first.
  grid_dependents_may_launch();
  if (MODE == kDense) grid_dependency_wait();
  uint32_t tmem_base = 0;
  if (MODE == kUmma) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(smem + L::misc));

  const uint32_t item_begin = args.worker_items[worker], item_end = args.worker_items[worker + 1];
  const uint64_t units = uint64_t(args.row_blocks) * args.chunks;
  const uint32_t unit_begin = uint32_t(units * worker / args.workers);
  const uint32_t unit_count = uint32_t(units * (worker + 1) / args.workers) - unit_begin;

  if (warp < kDecoderWarps) {
    // ------------------------------------------------------------------ decoders: one segment (2 streams) per lane
    if (MODE == kUmma && args.raw) goto roles_done;  // nothing to decode
    const uint32_t q = warp >> 2, r = (warp & 3) * 32 + lane;
    const uint32_t seg = q * BXR_ROWS + r, atom = q >> 1;
    LaneDecoder d;
    d.lut = smem + L::lut;
    d.k = args.k;
    uint32_t u = 0;
    // ring positions advance by increments (no division in the chunk loop); per-lane offsets are fixed
    uint32_t s = 0, ph = 0;                          // input ring slot of chunk u and its phase parity
    uint32_t so = atom % kOpN, pho = 0;              // operand ring stage of half-stage 2u + atom
    const uint32_t raw_at = BXR_RAW_AT + ((2 * q) * BXR_ROWS + r) * 16;
    const uint32_t exc_bit_at = BXR_EXC_BITS_AT + (seg >> 3), exc_bit = 1u << (seg & 7);
    const uint32_t seg_at = smem + L::segoff + 2 * seg;
    uint32_t st_at[4];                               // swizzled 16-byte positions of this lane's four stores
#pragma unroll
    for (int i = 0; i < 4; ++i) st_at[i] = r * 128 + ((((q & 1) * 4 + i) ^ (r & 7)) << 4);
    bool live = ctx.wait(bar_lut, 0);  // the slot records arrive by a bulk copy the loader issued first
    for (uint32_t it = item_begin; it < item_end && live; ++it) {
      const bxr_item item = args.items[it];
      const uint32_t row = item.row_block * BXR_ROWS + r;
      d.xf = args.states[size_t(it) * BXR_STREAMS + (2 * q) * BXR_ROWS + r];
      d.xb = args.states[size_t(it) * BXR_STREAMS + (2 * q + 1) * BXR_ROWS + r];
      d.base2 = uint32_t(args.base[row]) * 0x00800080u;
      float acc[MODE == kGemv ? kGemvMaxM : 1];
#pragma unroll
      for (int m = 0; m < (MODE == kGemv ? kGemvMaxM : 1); ++m) acc[m] = 0.f;
      for (uint32_t c = item.chunk_begin; c < item.chunk_end; ++c, ++u) {
        // in_ready is posted by the scanner after it has itself observed the blob's arrival (in_full)
        if (!ctx.wait(bar_in_ready + 8 * s, ph)) { live = false; break; }
        const uint32_t blob = smem + L::in + s * BXR_BLOB_MAX;
        const uint32_t bounds = lds32_unaligned_pair(seg_at + s * kSegOffBytes);
        d.start_chunk(blob + BXR_WORDS_AT + 2 * (bounds & 0xFFFFu), blob + BXR_WORDS_AT + 2 * (bounds >> 16) - 2);
        uint32_t a_tile = 0;
        if (MODE == kUmma) {
          if (!ctx.wait(bar_op_empty + 8 * so, pho ^ 1)) { live = false; break; }
          a_tile = smem + L::op + so * L::kOpStage;
        }
        const uint4 raw_f = lds128(blob + raw_at);
        const uint4 raw_b = lds128(blob + raw_at + BXR_ROWS * 16);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          uint4 w2[2];
          decode8x2(d, k ? raw_f.z : raw_f.x, k ? raw_f.w : raw_f.y, k ? raw_b.z : raw_b.x, k ? raw_b.w : raw_b.y, w2[0], w2[1]);
#pragma unroll
          for (int dir = 0; dir < 2; ++dir) {
            const uint4 w = w2[dir];
            const uint32_t cin = (2 * q + dir) * BXR_STREAM_COLS + k * 8;  // column inside the chunk
            const uint32_t col = c * BXR_COLS + cin;
            if (MODE == kUmma) {
              sts128(a_tile + st_at[dir * 2 + k], w);
            } else if (MODE == kDense) {
              if (row < args.rows) {
                uint16_t* dst = args.dense + size_t(row) * args.cols + col;
                if (col + 8 <= args.cols && (args.cols & 7) == 0) {
                  *reinterpret_cast<uint4*>(dst) = w;
                } else {
                  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
                  for (int e = 0; e < 8; ++e)
                    if (col + e < args.cols) dst[e] = uint16_t(ww[e >> 1] >> (16 * (e & 1)));
                }
              }
            } else {
              const float wf[8] = {bf16_lo(w.x), bf16_hi(w.x), bf16_lo(w.y), bf16_hi(w.y),
                                   bf16_lo(w.z), bf16_hi(w.z), bf16_lo(w.w), bf16_hi(w.w)};
              const uint32_t xs = smem + L::xf32 + s * L::kXStage + cin * 4;
#pragma unroll
              for (int m = 0; m < kGemvMaxM; ++m) {
                if (m < NB) {  // NB carries the batch size for the GEMV instantiations
                  const uint4 x0 = lds128(xs + m * BXR_COLS * 4), x1 = lds128(xs + m * BXR_COLS * 4 + 16);
                  float a = acc[m];
                  a = __fmaf_rn(__uint_as_float(x0.x), wf[0], a);
                  a = __fmaf_rn(__uint_as_float(x0.y), wf[1], a);
                  a = __fmaf_rn(__uint_as_float(x0.z), wf[2], a);
                  a = __fmaf_rn(__uint_as_float(x0.w), wf[3], a);
                  a = __fmaf_rn(__uint_as_float(x1.x), wf[4], a);
                  a = __fmaf_rn(__uint_as_float(x1.y), wf[5], a);
                  a = __fmaf_rn(__uint_as_float(x1.z), wf[6], a);
                  a = __fmaf_rn(__uint_as_float(x1.w), wf[7], a);
                  acc[m] = a;
                }
              }
            }
          }
        }
        // Exceptions (exponents outside the row window, ~1.5e-4 of the weights): the stream produced the
        // placeholder exponent base[row]; the lane that owns the segment patches its own output from the list.
        if (lds_u8(blob + exc_bit_at) & exc_bit) {
          const uint32_t total = lds_u16(seg_at - 2 * seg + s * kSegOffBytes + 2 * BXR_SEGMENTS);
          const uint32_t exc_at = blob + ((BXR_WORDS_AT + 2 * total + 3) & ~3u);
          const uint32_t n_exc = min(lds32(exc_at), uint32_t(BXR_EXC_MAX));
          for (uint32_t i = 0; i < n_exc; ++i) {
            const uint32_t v = lds32(exc_at + 4 + 4 * i);
            if ((v & 511u) != seg) continue;
            const uint32_t in_seg = (v >> 9) & 31u, e = (v >> 14) & 255u;
            const uint32_t byte = lds_u8(blob + raw_at + (in_seg >> 4) * BXR_ROWS * 16 + (in_seg & 15u));
            const uint32_t word = (byte & 0x80u) << 8 | e << 7 | (byte & 0x7Fu);
            if (MODE == kUmma) {
              sts_u16(a_tile + r * 128 + ((((q & 1) * 4 + (in_seg >> 3)) ^ (r & 7)) << 4) + 2 * (in_seg & 7u), word);
            } else if (MODE == kDense) {
              const uint32_t col = c * BXR_COLS + q * 32 + in_seg;
              if (row < args.rows && col < args.cols) args.dense[size_t(row) * args.cols + col] = uint16_t(word);
            } else {
              // the chain already holds x * placeholder: take it out and put the true product in
              const float good = __uint_as_float(word << 16);
              const float wrong = __uint_as_float(((byte & 0x80u) << 8 | (d.base2 & 0x7F80u) | (byte & 0x7Fu)) << 16);
              const uint32_t xs = smem + L::xf32 + s * L::kXStage + (q * 32 + in_seg) * 4;
#pragma unroll
              for (int m = 0; m < kGemvMaxM; ++m)
                if (m < NB) {
                  float xv;
                  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(xv) : "r"(xs + m * BXR_COLS * 4));
                  acc[m] = __fmaf_rn(xv, good, __fmaf_rn(-xv, wrong, acc[m]));
                }
            }
          }
        }
        if (MODE == kUmma) {
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_op_full + 8 * so);
          so += 2;
          if (so >= kOpN) { so -= kOpN; pho ^= 1; }
        } else {
          __syncwarp();
        }
        if (lane == 0) mbar_arrive(bar_in_empty + 8 * s);
        if (++s == L::kIn) { s = 0; ph ^= 1; }
      }
      if (!live) break;
      if (d.xf != BXR_STATE_LOW || d.xb != BXR_STATE_LOW) atomicOr(args.status, kStatusCheckpoint);
      if (MODE == kGemv) {
        if (it == item_begin) grid_dependency_wait();  // y, partial sums and counters
        // phases of a row are added in phase order, parts of a row block in part order
        const uint32_t red = smem + L::red;
        const uint32_t n_item = it - item_begin;
        if (!ctx.wait(bar_acc_empty, (n_item & 1) ^ 1)) break;  // previous item's sums have been read
#pragma unroll
        for (int m = 0; m < kGemvMaxM; ++m)
          if (m < NB) asm volatile("st.shared.f32 [%0], %1;" ::"r"(red + ((q * BXR_ROWS + r) * kGemvMaxM + m) * 4), "f"(acc[m]) : "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_full);
        bool last_part = item.parts == 1;
        if (q == 0) {
          if (!ctx.wait(bar_acc_full, n_item & 1)) break;
          float tot[kGemvMaxM];
#pragma unroll
          for (int m = 0; m < kGemvMaxM; ++m) {
            tot[m] = 0.f;
            if (m < NB) {
              float t;
              asm volatile("ld.shared.f32 %0, [%1];" : "=f"(t) : "r"(red + ((0 * BXR_ROWS + r) * kGemvMaxM + m) * 4));
#pragma unroll
              for (int p = 1; p < BXR_PHASES; ++p) {
                float v;
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(red + ((p * BXR_ROWS + r) * kGemvMaxM + m) * 4));
                t = __fadd_rn(t, v);
              }
              tot[m] = t;
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acc_empty);
          if (item.parts > 1) {
#pragma unroll
            for (int m = 0; m < kGemvMaxM; ++m)
              if (m < NB) args.partials[(size_t(item.slot) * kGemvMaxM + m) * BXR_ROWS + r] = tot[m];
            __threadfence();
          }
          named_barrier(3, 128);
          if (item.parts > 1) {
            uint32_t prev = 0;
            if (warp == 0 && lane == 0) prev = atomicAdd(args.counters + item.row_block, 1u);
            prev = __shfl_sync(0xFFFFFFFFu, prev, 0);
            // warps 1..3 learn the decision through shared memory
            if (warp == 0 && lane == 0) asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(smem + L::misc + 8), "r"(prev) : "memory");
            named_barrier(3, 128);
            asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(prev) : "r"(smem + L::misc + 8));
            last_part = prev == item.parts - 1;
            if (last_part) {
              __threadfence();
              const uint32_t first = item.slot - item.part;
#pragma unroll
              for (int m = 0; m < kGemvMaxM; ++m)
                if (m < NB) {
                  float t = __ldcg(args.partials + (size_t(first) * kGemvMaxM + m) * BXR_ROWS + r);
                  for (uint32_t p = 1; p < item.parts; ++p)
                    t = __fadd_rn(t, __ldcg(args.partials + (size_t(first + p) * kGemvMaxM + m) * BXR_ROWS + r));
                  tot[m] = t;
                }
              if (warp == 0 && lane == 0) args.counters[item.row_block] = 0;
            }
          }
          if (last_part && row < args.rows) {
            const float b = args.bias ? __bfloat162float(args.bias[row]) : 0.f;
#pragma unroll
            for (int m = 0; m < kGemvMaxM; ++m)
              if (m < NB && m < int(args.m))
                args.y[size_t(m) * args.ldy + row] = __float2bfloat16_rn(args.bias ? __fadd_rn(tot[m], b) : tot[m]);
          }
        }
      }
    }
  } else if (warp == kWarpLoader) {
    // ------------------------------------------------------------------ chunk blobs, one bulk copy each
    if (MODE == kUmma && args.raw) {
      // raw image: every chunk blob is the 128x128 BF16 tile already in operand order (two 16 KB atoms);
      // copy each atom straight into its operand stage
      if (lane == 0) {
        bool live = true;
        for (uint32_t u = 0; u < unit_count && live; ++u)
          for (uint32_t a = 0; a < 2; ++a) {
            const uint32_t hs = 2 * u + a, so = hs % kOpN, pho = (hs / kOpN) & 1;
            if (ctx.aborted() || !ctx.wait(bar_op_empty + 8 * so, pho ^ 1)) { live = false; break; }
            mbar_arrive_expect_tx(bar_op_full + 8 * so, kAtomBytes);
            bulk_g2s(smem + L::op + so * L::kOpStage, args.blobs + (size_t(unit_begin + u) * 2 + a) * kAtomBytes, kAtomBytes,
                     bar_op_full + 8 * so);
          }
      }
      goto roles_done;
    }
    if (lane == 0) {  // the 16 KB slot-record table (L2 hits after the first CTA)
      mbar_arrive_expect_tx(bar_lut, kLutBytes);
      bulk_g2s(smem + L::lut, args.lut, kLutBytes, bar_lut);
    }
    uint32_t issued = 0;
    for (uint32_t u0 = 0; u0 < unit_count; u0 += 32) {
      const uint32_t mine = unit_begin + min(u0 + lane, unit_count - 1);
      const uint32_t i0 = __ldg(args.blob_index + mine), i1 = __ldg(args.blob_index + mine + 1);
      const uint32_t n = min(32u, unit_count - u0);
      bool live = true;
      for (uint32_t i = 0; i < n && live; ++i) {
        const uint32_t u = u0 + i, s = u % L::kIn, ph = (u / L::kIn) & 1;
        const uint32_t b0 = __shfl_sync(0xFFFFFFFFu, i0, i), b1 = __shfl_sync(0xFFFFFFFFu, i1, i);
        uint32_t bytes = (b1 - b0) << 4;
        if (ctx.aborted() || !ctx.wait(bar_in_empty + 8 * s, ph ^ 1)) { live = false; break; }
        if (b1 < b0 || bytes > BXR_BLOB_MAX || bytes < BXR_WORDS_AT) {
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
    if (ctx.aborted() && lane == 0) {
      mbar_wait(bar_lut, 0);
      for (uint32_t u = (issued > uint32_t(L::kIn) ? issued - L::kIn : 0); u < issued; ++u) mbar_wait(bar_in_full + 8 * (u % L::kIn), (u / L::kIn) & 1);
    }
  } else if (warp == kWarpScanner) {
    // ------------------------------------------------------------------ segment offsets per chunk
    if (MODE == kUmma && args.raw) goto roles_done;
    uint32_t u = 0;
    bool live = true;
    for (uint32_t it = item_begin; it < item_end && live; ++it) {
      const bxr_item item = args.items[it];
      for (uint32_t c = item.chunk_begin; c < item.chunk_end; ++c, ++u) {
        const uint32_t s = u % L::kIn, ph = (u / L::kIn) & 1;
        if (ctx.aborted() || !ctx.wait(bar_in_full + 8 * s, ph)) { live = false; break; }
        const uint32_t blob = smem + L::in + s * BXR_BLOB_MAX;
        const uint4 cnt = lds128(blob + 16 * lane);  // this lane's 16 segment counts
        const uint32_t cw[4] = {cnt.x, cnt.y, cnt.z, cnt.w};
        uint32_t pre[16];
        uint32_t run = 0;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          pre[e] = run;
          run += (cw[e >> 2] >> (8 * (e & 3))) & 0xFFu;
        }
        uint32_t incl = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const uint32_t v = __shfl_up_sync(0xFFFFFFFFu, incl, o);
          if (lane >= o) incl += v;
        }
        const uint32_t excl = incl - run;
        const uint32_t total = __shfl_sync(0xFFFFFFFFu, incl, 31);
        if (total > BXR_WORDS_MAX) {  // cannot come from the builder; refuse rather than read elsewhere
          ctx.abort(kStatusBadArgument);
          live = false;
          break;
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint4 o4;
          o4.x = (excl + pre[8 * h + 0]) | (excl + pre[8 * h + 1]) << 16;
          o4.y = (excl + pre[8 * h + 2]) | (excl + pre[8 * h + 3]) << 16;
          o4.z = (excl + pre[8 * h + 4]) | (excl + pre[8 * h + 5]) << 16;
          o4.w = (excl + pre[8 * h + 6]) | (excl + pre[8 * h + 7]) << 16;
          sts128(smem + L::segoff + s * kSegOffBytes + 32 * lane + 16 * h, o4);
        }
        if (lane == 31) asm volatile("st.shared.u16 [%0], %1;" ::"r"(smem + L::segoff + s * kSegOffBytes + 1024), "h"(uint16_t(total)) : "memory");
        if (MODE == kGemv) {
          if (u == 0) grid_dependency_wait();  // x may be the previous kernel's output
          // activations of this chunk as FP32: [m][128]
          const uint32_t xs = smem + L::xf32 + s * L::kXStage;
          for (int m = 0; m < kGemvMaxM; ++m)
            if (m < NB) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const uint32_t col = c * BXR_COLS + e * 32 + lane;
                float v = 0.f;
                if (m < int(args.m) && col < args.cols) v = __bfloat162float(args.x[size_t(m) * args.ldx + col]);
                asm volatile("st.shared.f32 [%0], %1;" ::"r"(xs + (m * BXR_COLS + e * 32 + lane) * 4), "f"(v) : "memory");
              }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_in_ready + 8 * s);
      }
    }
  } else if (MODE == kUmma && warp == kWarpXLoader) {
    // ------------------------------------------------------------------ activation half-tiles by TMA
    if (lane == 0) {
      grid_dependency_wait();
      uint32_t u = 0;
      bool live = true;
      for (uint32_t it = item_begin; it < item_end && live; ++it) {
        const bxr_item item = args.items[it];
        for (uint32_t c = item.chunk_begin; c < item.chunk_end && live; ++c, ++u)
          for (uint32_t a = 0; a < 2; ++a) {
            const uint32_t hs = 2 * u + a, so = hs % kOpN, pho = (hs / kOpN) & 1;
            if (ctx.aborted() || !ctx.wait(bar_op_empty + 8 * so, pho ^ 1)) { live = false; break; }
            mbar_arrive_expect_tx(bar_op_full + 8 * so, NB * 128);
            tma_load_2d(smem + L::op + so * L::kOpStage + kAtomBytes, &tmap_x, int(c * BXR_COLS + a * 64), 0, bar_op_full + 8 * so);
          }
      }
    }
  } else if (MODE == kUmma && warp == kWarpMma) {
    // ------------------------------------------------------------------ MMA issue
    constexpr uint32_t idesc = umma_idesc_bf16(NB);
    uint32_t u = 0, n_item = 0;
    bool live = true;
    for (uint32_t it = item_begin; it < item_end && live; ++it, ++n_item) {
      const bxr_item item = args.items[it];
      const uint32_t buf = n_item & 1;
      if (ctx.aborted() || !ctx.wait(bar_acc_empty + 8 * buf, ((n_item >> 1) & 1) ^ 1)) { live = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * NB;
      uint32_t first = 1;
      for (uint32_t c = item.chunk_begin; c < item.chunk_end && live; ++c, ++u)
        for (uint32_t a = 0; a < 2; ++a) {
          const uint32_t hs = 2 * u + a, so = hs % kOpN, pho = (hs / kOpN) & 1;
          if (ctx.aborted() || !ctx.wait(bar_op_full + 8 * so, pho)) { live = false; break; }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t stage = smem + L::op + so * L::kOpStage;
            const uint64_t adesc = umma_desc_sw128(stage), bdesc = umma_desc_sw128(stage + kAtomBytes);
#pragma unroll
            for (uint32_t k = 0; k < 4; ++k) {
              umma_bf16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, first ? 0u : 1u);
              first = 0;
            }
            umma_commit(bar_op_empty + 8 * so);
          }
          __syncwarp();
        }
      if (live && lane == 0) umma_commit(bar_acc_full + 8 * buf);
      __syncwarp();
    }
  } else if (MODE == kUmma && warp >= kWarpEpilogue) {
    // ------------------------------------------------------------------ TMEM -> y, or -> FP32 partial tile
    const uint32_t e = warp - kWarpEpilogue;  // == warp % 4: the TMEM lane quarter this warp may read
    const uint32_t r = e * 32 + lane;
    const uint32_t mcols = (args.m + 7) & ~7u;
    uint32_t n_item = 0;
    bool live = true;
    grid_dependency_wait();  // bias, y, partial tiles and counters may belong to the previous kernel
    for (uint32_t it = item_begin; it < item_end && live; ++it, ++n_item) {
      const bxr_item item = args.items[it];
      const uint32_t buf = n_item & 1;
      if (ctx.aborted() || !ctx.wait(bar_acc_full + 8 * buf, (n_item >> 1) & 1)) { live = false; break; }
      tc_fence_after();
      const uint32_t row = item.row_block * BXR_ROWS + r;
      const uint32_t taddr = tmem_base + ((e * 32) << 16) + buf * NB;
      const float b = (args.bias && row < args.rows) ? __bfloat162float(args.bias[row]) : 0.f;
      for (uint32_t m0 = 0; m0 < mcols; m0 += 8) {
        uint32_t v[8];
        tmem_ld8(taddr + m0, v);
        tmem_ld_wait();
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
          if (it + 1 == item_end && !args.raw) {
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
  // the 4 epilogue warps together (20 warps instead of 4 on the critical tail of the kernel).
  if (MODE == kUmma && !args.raw && (warp < kDecoderWarps || warp >= kWarpEpilogue)) {
    if (ctx.wait(bar_final, 0)) {
      const uint4 decision = lds128(smem + L::misc + 16);  // {reduce?, row block, first slot, parts}
      if (decision.x)
        reduce_row_block<NB>(args, decision.y, decision.z, decision.w, warp < kDecoderWarps ? warp : warp - 4, kDecoderWarps + 4, lane);
    }
  }

roles_done:
  tc_fence_before();
  __syncthreads();
  if (MODE == kUmma && warp == kWarpMma) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace grb
