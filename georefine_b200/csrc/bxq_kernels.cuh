// Fused kernels over wide-window images (bxr_format.h, BXR_MODE_WINDOW4): 4-bit exponent codes inside a 16-binade
// row window, so that a weight outside its window is a rarity (fewer than one in ten thousand on Gaussian rows) and
// the decoded words never have to touch shared memory:
//   * kUmma  : a lane holds the 32 weights of its row and phase in 16 registers and writes them with one tcgen05.st
//              into tensor memory, where tcgen05.mma takes them as its A operand (M = 128 weight rows; the batch is
//              N, read from shared memory).  Shared memory carries only what comes from outside the SM: chunk blobs
//              and activation tiles.  Two threads issue the MMAs, chunk about, each into an accumulator of its own.  (In the 3-bit window kernel the operand tile lives in shared memory, and its
//              stores plus the tensor core's reads of it are more than 40 % of all shared-memory traffic, which sets
//              that kernel's pace; its per-chunk exception patching is what keeps it from using tensor memory: done
//              in registers it costs more instructions than the decode itself.)
//   * kDense : decode twin (parity tests, ResidentWeight.decode).
// Same persistent, warp-specialised pipeline and work partition as the other fused kernels; any batch size, the
// batch of one padded to the narrowest tile.
#pragma once
#include "bxr_kernels.cuh"

namespace grb {

constexpr int kWideWarpLoader = 16;    // bulk copies of chunk blobs
constexpr int kWideWarpMma = 17;       // TMEM owner and MMA issuer of the even chunks of an item
constexpr int kWideWarpMma2 = 19;      // MMA issuer of the odd chunks
constexpr int kWideWarpXLoader = 18;   // TMA loads of activation tiles
constexpr int kWideWarpEpilogue = 20;  // 4 warps: warp % 4 = the tensor-memory lane quarter a warp may read

// Tensor memory: columns [0, 256) accumulators, FP32: an item has two, one per MMA issuer (even chunks, odd chunks;
// the epilogue adds them), NB columns each.  Up to NB = 64 two items fit (one being multiplied, one being drained);
// at NB = 128 there is room for one, and the issuers wait for the drain at an item boundary while the decoders fill
// the operand stages.  Columns [256, 512): the decoded weights of four chunks, 64 columns each (two 128 x 64 atoms, two
// BF16 per column).  (The narrow tiles would leave room for six or seven stages and a deeper activation ring; measured at
// NB = 16 with 7 stages, 8 activation stages and 6 requests in flight, every M = 1 launch got slower, gate|up by 4.6 us.)
constexpr int kWideNextBlobs = 8;      // blobs per CTA of the next launch that a finishing CTA asks the L2 for
constexpr uint32_t kWideTmemCols = 512;
template <int NB>
constexpr int kWideStages = 4;
template <int NB>
constexpr uint32_t kWideOperandCol = kWideTmemCols - 64u * kWideStages<NB>;

// Shared-memory plan: a ring of chunk blobs and a ring of activation tiles (two NB x 64 atoms per chunk), the
// latter requested kXLag chunks ahead of the weights they will meet (they come from L2 with a latency of about a
// microsecond).
template <int MODE, int NB>
struct BxqSmem {
  static constexpr int kOp = (MODE == kUmma) ? kWideStages<NB> : 0;
  static constexpr int kX = (MODE == kUmma) ? (NB <= 64 ? 4 : 3) : 0;
  static constexpr int kXLag = 2;
  static constexpr uint32_t kXStage = 2 * NB * 128;
  static constexpr uint32_t kReserve = 1024 /* alignment slack */ + 512 /* barriers, flags */;
  // the epilogue warps turn their accumulator columns around in shared memory (a lane holds one weight row, memory
  // wants consecutive rows together): 16 columns x 32 rows x 4 bytes per warp
  static constexpr uint32_t kTurn = (MODE == kUmma) ? 2048u : 0u;
  static constexpr int kInFit = int((232448u - kReserve - kX * kXStage - 4 * kTurn) / BXQ_BLOB_MAX);
  static constexpr int kIn = kInFit > 7 ? 7 : kInFit;   // (more barriers would not fit the one-per-lane set-up)
  static constexpr uint32_t xs = 0;
  static constexpr uint32_t turn = xs + kX * kXStage;
  static constexpr uint32_t in = turn + 4 * kTurn;
  static constexpr uint32_t bars = in + kIn * BXQ_BLOB_MAX;
  // barrier order: in_full, in_empty [kIn each]; op_full, op_empty [kOp each]; x_full [kX]; acc_full, acc_empty
  // [2 each]; final; tile_full, tile_used [kRing each] (the closing reduction)
  static constexpr uint32_t kRing = (NB <= 64) ? 4 : 2;  // tiles in flight in the closing reduction (kWideTileRing)
  static constexpr uint32_t nbars = 2 * kIn + 2 * kOp + kX + 4 + 1 + 2 * kRing;
  static constexpr uint32_t misc = (bars + 8 * nbars + 15) & ~15u;  // tmem base, abort flag, decision
  static constexpr uint32_t total = misc + 48;
  static constexpr uint32_t alloc = total + 1024;
  static_assert(MODE != kUmma || kIn >= 4, "ring too shallow");
  // what keeps the activation loader at most one barrier phase behind the MMA issuer (see its role below)
  static_assert(MODE != kUmma || (kXLag < kX && kOp + kXLag + 1 > kX), "activation ring and lag do not fit the operand ring");
  static_assert(MODE != kUmma || 2 * NB * (NB <= 64 ? 2 : 1) <= int(kWideOperandCol<NB>), "accumulators overlap the operand columns");
  static_assert(8 * nbars + 64 <= 512, "barrier area");
  static_assert(MODE != kUmma || (1 + kRing) * NB * 512u <= bars, "the closing reduction's tiles would overwrite the barriers");
  static_assert(alloc <= 232448, "exceeds the 227 KB of shared memory a CTA may opt into");
};

// A code word holds four column pairs: pair k has the code of its even column in bits [4k, 4k+4) and that of its odd
// column 16 bits higher.  One mask and one multiply-add (whose addend is the row base in both halves) put a pair into
// packed-BF16 exponent position; `hi` is the word shifted right by 8, which brings pairs 2 and 3 to where pairs 0
// and 1 are.  The mask runs on the integer pipe, the multiply-add on the FMA pipe (the multipliers are kernel
// parameters so that the compiler does not turn them back into shifts).
template <int K>
__device__ __forceinline__ uint32_t bxq_exponents(uint32_t lo, uint32_t hi, const BxwPowers& p, uint32_t base2) {
  if constexpr (K == 0) return (lo & BXQ_PAIR_MASK) * p.p7 + base2;
  else if constexpr (K == 1) return (lo & (BXQ_PAIR_MASK << 4)) * p.p3 + base2;
  else if constexpr (K == 2) return (hi & BXQ_PAIR_MASK) * p.p7 + base2;
  else return (hi & (BXQ_PAIR_MASK << 4)) * p.p3 + base2;
}
// raw bytes (sign << 7 | mantissa) of two columns merged with their exponents
__device__ __forceinline__ uint32_t bxq_join(uint32_t raw4, uint32_t selector, uint32_t exponents) {
  return (__byte_perm(raw4, 0, selector) & 0x807F807Fu) | exponents;
}
// The 32 weights of a lane, two per register in column order: four code words and the raw bytes of its two
// 16-column pieces.
__device__ __forceinline__ void bxq_decode32(const uint32_t (&w)[4], const uint4& rf, const uint4& rb, const BxwPowers& p,
                                             uint32_t base2, uint32_t (&out)[16]) {
  const uint32_t raw[8] = {rf.x, rf.y, rf.z, rf.w, rb.x, rb.y, rb.z, rb.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t lo = w[j], hi = w[j] >> 8;
    out[4 * j + 0] = bxq_join(raw[2 * j], 0x1100, bxq_exponents<0>(lo, hi, p, base2));
    out[4 * j + 1] = bxq_join(raw[2 * j], 0x3322, bxq_exponents<1>(lo, hi, p, base2));
    out[4 * j + 2] = bxq_join(raw[2 * j + 1], 0x1100, bxq_exponents<2>(lo, hi, p, base2));
    out[4 * j + 3] = bxq_join(raw[2 * j + 1], 0x3322, bxq_exponents<3>(lo, hi, p, base2));
  }
}
// An exception entry applied to the registers of the lane that owns it: the exponent field of one half of one
// register is replaced.  The register index is data, so the choice is sixteen predicated operations; this runs only
// for the rare warp that has entries at all.
__device__ __forceinline__ void bxq_patch(uint32_t (&out)[16], uint32_t column, uint32_t exponent) {
  const uint32_t reg = column >> 1, sh = (column & 1u) ? 16u : 0u;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    if (reg == uint32_t(i)) out[i] = (out[i] & ~(0x7F80u << sh)) | (exponent & 0xFFu) << (7 + sh);
}

// The work of a CTA is a contiguous range of the (row block, chunk) sequence; an item is the part of it that lies in
// one row block.  Everything but the epilogue needs only the geometry of an item, which follows from the range by
// arithmetic: no load stands between the start of a CTA and its first blob, window base and multiply.  (The item
// list in the image holds the same geometry plus the partial-tile bookkeeping - part, parts, slot - which the
// epilogue reads with plenty of time to spare; bxr_validate checks that the two agree.)
struct WideSpan {
  uint32_t row_block, chunk_begin, chunk_end;
};
__device__ __forceinline__ WideSpan wide_span(uint32_t unit, uint32_t unit_end, uint32_t chunks) {
  const uint32_t rb = unit / chunks, c0 = unit - rb * chunks;
  return {rb, c0, min(chunks, c0 + (unit_end - unit))};
}

// The closing reduction of a split row block, by the (kDecoderWarps + 4) x 32 threads that have nothing else left
// to do: y[m, row] = bf16(sum of the row block's FP32 tiles in K order (+ bias)).  A reducing SM has to pull
// (parts - 1) x NB x 512 bytes through its one L2 port, so the tiles come by bulk copy, kWideTileRing<NB> in flight,
// into the shared memory the pipeline no longer needs (from byte T on, T = NB x 512; the CTA's own last tile, if it
// takes part, lies at [0, T) and was never in memory).  A thread owns the same few float4 positions of every tile and
// keeps their running sums in registers.  `fetched` counts the tiles brought in so far by this CTA (barrier phases).
template <int NB>
constexpr uint32_t kWideTileRing = NB <= 64 ? 4 : 2;  // (1 + ring) x NB x 512 bytes of shared memory

template <int NB>
__device__ __forceinline__ void bxq_reduce_row_block(const BxrArgs& args, const RoleCtx& ctx, uint32_t row_block, uint32_t first,
                                                     uint32_t parts, uint32_t own, uint32_t smem, uint32_t bar_full, uint32_t bar_used,
                                                     uint32_t t, uint32_t& fetched) {
  constexpr uint32_t kThreads = (kDecoderWarps + 4) * 32;
  constexpr int kMine = (NB * 32 + kThreads - 1) / kThreads;  // float4 positions per thread
  constexpr uint32_t kTile = NB * BXR_ROWS * 4;
  const uint32_t mcols = (args.m + 7) & ~7u, total = mcols * 32, bytes = mcols * BXR_ROWS * 4;
  const uint32_t remote = parts - (own < parts ? 1u : 0u);
  const uint32_t lane = t & 31;
  uint32_t asked = 0;  // remote tiles requested in this call
  bool live = true;
  constexpr uint32_t kRing = kWideTileRing<NB>;
  auto ask = [&](uint32_t j) {  // thread 0: the j-th remote tile into buffer (fetched + j) % kRing, once its last readers are done
    const uint32_t n = fetched + j, b = n % kRing, p = j + ((own < parts && own <= j) ? 1u : 0u);
    if (!ctx.wait(bar_used + 8 * b, ((n / kRing) & 1) ^ 1)) { live = false; return; }
    mbar_arrive_expect_tx(bar_full + 8 * b, bytes);
    bulk_g2s(smem + kTile * (1 + b), args.partials + size_t(first + p) * NB * BXR_ROWS, bytes, bar_full + 8 * b, l2_policy_evict_first());
    asked = j + 1;
  };
  if (t == 0)
    for (uint32_t j = 0; j < kRing && j < remote && live; ++j) ask(j);
  float4 sum[kMine];
  uint32_t j = 0;  // remote tiles consumed
  for (uint32_t p = 0; p < parts && live; ++p) {
    uint32_t src = smem, b = 0;
    if (p != own) {
      const uint32_t n = fetched + j;
      b = n % kRing;
      if (!ctx.wait(bar_full + 8 * b, (n / kRing) & 1)) { live = false; break; }
      src = smem + kTile * (1 + b);
    }
#pragma unroll
    for (int k = 0; k < kMine; ++k) {
      const uint32_t at = t + k * kThreads;
      if (at < total) {
        const uint4 u = lds128(src + at * 16);
        if (p == 0) {  // taken as it is: adding it to zero would lose the sign of a -0
          sum[k] = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
        } else {
          sum[k].x = __fadd_rn(sum[k].x, __uint_as_float(u.x));
          sum[k].y = __fadd_rn(sum[k].y, __uint_as_float(u.y));
          sum[k].z = __fadd_rn(sum[k].z, __uint_as_float(u.z));
          sum[k].w = __fadd_rn(sum[k].w, __uint_as_float(u.w));
        }
      }
    }
    if (p != own) {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_used + 8 * b);
      if (t == 0 && j + kRing < remote) ask(j + kRing);
      ++j;
    }
  }
  if (t == 0 && !live)  // unwinding: copies still in flight must land before the CTA may exit
    for (uint32_t k = j; k < asked; ++k) mbar_wait(bar_full + 8 * ((fetched + k) % kRing), ((fetched + k) / kRing) & 1);
  fetched += remote;
  if (!live) return;
#pragma unroll
  for (int k = 0; k < kMine; ++k) {
    const uint32_t at = t + k * kThreads, m = at >> 5, row4 = row_block * BXR_ROWS + (at & 31) * 4;
    if (at >= total || m >= args.m || row4 >= args.rows) continue;
    float f[4] = {sum[k].x, sum[k].y, sum[k].z, sum[k].w};
    if (args.bias)
      for (int i = 0; i < 4; ++i)
        if (row4 + i < args.rows) f[i] = __fadd_rn(f[i], __bfloat162float(args.bias[row4 + i]));
    __nv_bfloat16* dst = args.y + size_t(m) * args.ldy + row4;
    if (row4 + 3 < args.rows && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
      __nv_bfloat162 lo, hi;
      lo.x = __float2bfloat16_rn(f[0]);
      lo.y = __float2bfloat16_rn(f[1]);
      hi.x = __float2bfloat16_rn(f[2]);
      hi.y = __float2bfloat16_rn(f[3]);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst) = packed;
    } else {
      for (int i = 0; i < 4; ++i)
        if (row4 + i < args.rows) dst[i] = __float2bfloat16_rn(f[i]);
    }
  }
}

// The closing reduction of a row block whose parts belong to the CTAs of one thread-block cluster (the partition is
// "aligned": workers = row blocks x P, CTA rank r of cluster b owns part r of row block b, in K order).  Every CTA has
// left its FP32 tile at the start of its shared memory; after the cluster barrier each CTA adds the P tiles of ITS share
// of the batch columns (m = rank, rank + P, ...) in rank order - its own from local shared memory, the others over
// distributed shared memory - and writes y.  No partial tile goes to global memory, no counter, no fence, and the work
// of the reduction is spread over the P SMs.  t = index of the calling thread among the (kDecoderWarps + 4) x 32.
template <int NB>
__device__ __forceinline__ void bxq_reduce_in_cluster(const BxrArgs& args, uint32_t row_block, uint32_t smem, uint32_t t) {
  constexpr uint32_t kThreads = (kDecoderWarps + 4) * 32;
  const uint32_t parts = args.cluster, rank = cluster_rank();
  const uint32_t mcols = (args.m + 7) & ~7u;
  const uint32_t mine = rank < mcols ? (mcols - rank + parts - 1) / parts : 0;  // batch columns rank, rank + P, ... below mcols
  for (uint32_t i = t; i < mine * 32; i += kThreads) {
    const uint32_t m = rank + (i >> 5) * parts, at = (m << 5) | (i & 31);
    const uint32_t row4 = row_block * BXR_ROWS + (i & 31) * 4;
    if (m >= args.m || row4 >= args.rows) continue;
    uint4 u[8];  // every part's piece first (independent loads in flight), then the sum in K order
#pragma unroll
    for (uint32_t p = 0; p < 8; ++p)
      if (p < parts) u[p] = p == rank ? lds128(smem + at * 16) : lds128_cluster(cluster_map(smem + at * 16, p));
    // part 0 is taken as it is: adding it to zero would lose the sign of a -0
    float f[4] = {__uint_as_float(u[0].x), __uint_as_float(u[0].y), __uint_as_float(u[0].z), __uint_as_float(u[0].w)};
#pragma unroll
    for (uint32_t p = 1; p < 8; ++p)
      if (p < parts) {
        f[0] = __fadd_rn(f[0], __uint_as_float(u[p].x));
        f[1] = __fadd_rn(f[1], __uint_as_float(u[p].y));
        f[2] = __fadd_rn(f[2], __uint_as_float(u[p].z));
        f[3] = __fadd_rn(f[3], __uint_as_float(u[p].w));
      }
    if (args.bias)
      for (int k = 0; k < 4; ++k)
        if (row4 + k < args.rows) f[k] = __fadd_rn(f[k], __bfloat162float(args.bias[row4 + k]));
    __nv_bfloat16* dst = args.y + size_t(m) * args.ldy + row4;
    if (row4 + 3 < args.rows && (reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
      __nv_bfloat162 lo, hi;
      lo.x = __float2bfloat16_rn(f[0]);
      lo.y = __float2bfloat16_rn(f[1]);
      hi.x = __float2bfloat16_rn(f[2]);
      hi.y = __float2bfloat16_rn(f[3]);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst) = packed;
    } else {
      for (int k = 0; k < 4; ++k)
        if (row4 + k < args.rows) dst[k] = __float2bfloat16_rn(f[k]);
    }
  }
}

template <int MODE, int NB>
__global__ void __launch_bounds__(MODE == kUmma ? kThreadsUmma : kThreadsSimt, 1)
bxq_kernel(const BxrArgs args, const __grid_constant__ CUtensorMap tmap_x) {
  using L = BxqSmem<MODE, NB>;
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
  const uint32_t bar_tile_full = bar_final + 8, bar_tile_used = bar_tile_full + 8 * L::kRing;
  constexpr uint32_t kTmemCols = kWideTmemCols;
  constexpr uint32_t kOpN = L::kOp ? L::kOp : 1;
  constexpr uint32_t kXN = L::kX ? L::kX : 1;
  constexpr uint32_t kAccBufs = NB <= 64 ? 2 : 1;  // items whose accumulators fit tensor memory at once

  // The blob loader's own barriers first of all (blobs of one size: it needs nothing else to start its copies): their
  // fences complete while the CTA's share of the work is being computed.
  if (warp == kWideWarpLoader && args.blob_stride16 && lane == 0) {
    for (uint32_t n = 0; n < uint32_t(L::kIn); ++n) mbar_init(bar_in_full + 8 * n, 1);
    mbar_fence_init();
    fence_proxy_async_smem();
  }
  // Work of this CTA, known from the arguments alone; the blob loader asks for its first offsets before anything
  // else so that the first copy can leave as soon as the barriers exist.
  const uint64_t units = uint64_t(args.row_blocks) * args.chunks;
  const uint32_t unit_begin = uint32_t(units * worker / args.workers);
  const uint32_t unit_count = uint32_t(units * (worker + 1) / args.workers) - unit_begin;
  uint32_t first_i0 = 0, first_i1 = 0;
  if (warp == kWideWarpLoader && unit_count && !args.blob_stride16) {
    const uint32_t mine = unit_begin + min(uint32_t(lane), unit_count - 1);
    first_i0 = __ldg(args.blob_index + mine);
    first_i1 = __ldg(args.blob_index + mine + 1);
  }
  const uint32_t unit_end = unit_begin + unit_count;
  // Decoders: the window base of this thread's row in the CTA's first item, asked for before anything else.
  uint32_t first_base = 0;
  if (warp < kDecoderWarps && unit_count) first_base = args.base[(unit_begin / args.chunks) * BXR_ROWS + (warp & 3) * 32 + lane];
  // Epilogue: where the CTA's items are in the image's list (their partial-tile bookkeeping); needed much later.
  uint32_t item_begin = 0, item_end = 0;
  if (MODE == kUmma && warp >= kWideWarpEpilogue) {
    item_begin = __ldg(args.worker_items + worker);
    item_end = __ldg(args.worker_items + worker + 1);
  }
  // An SM runs the launches of a stream back to back, so whatever a CTA does before its first multiply is not hidden
  // behind the previous launch on the SM that finished last.  The longest wait in it is the first blob's trip from
  // HBM: with blobs of one size the loader needs nothing but its own barriers to start it, and sets those up itself.
  uint32_t early = 0;
  if (warp == kWideWarpLoader && args.blob_stride16) {
    const uint32_t bytes = args.blob_stride16 << 4;
    if (bytes <= BXQ_BLOB_MAX && bytes >= BXQ_LIST_AT) early = min(unit_count, uint32_t(L::kIn));
    if (lane == 0) {
      const uint64_t once = l2_policy_evict_first();
      for (uint32_t u = 0; u < early; ++u) {
        mbar_arrive_expect_tx(bar_in_full + 8 * u, bytes);
        bulk_g2s(smem + L::in + u * BXQ_BLOB_MAX, args.blobs + size_t(unit_begin + u) * bytes, bytes, bar_in_full + 8 * u, once);
      }
    }
    __syncwarp();
  }
  if (warp == 0) {  // one or two barriers per lane
    static_assert(L::nbars <= 64, "two barriers per lane at most");
    const uint32_t i = lane;
#pragma unroll
    for (uint32_t n = i; n < L::nbars; n += 32) {
      if (n < uint32_t(L::kIn) && args.blob_stride16) continue;                    // in_full: the loader's own (above)
      uint32_t count = 1;                                                          // in_full, op_empty, x_full
      if (n >= uint32_t(L::kIn) && n < 2u * L::kIn) count = kDecoderWarps;          // in_empty
      else if (n >= 2u * L::kIn && n < 2u * L::kIn + L::kOp) count = kDecoderWarps + 1;  // op_full: + the loader's go-ahead
      else if (n >= 2u * L::kIn + 2 * L::kOp + L::kX) {
        const uint32_t j = n - (2u * L::kIn + 2 * L::kOp + L::kX);  // acc_full x2, acc_empty x2, final, tile_full x2, tile_used x2
        count = j < 2 ? 2u : j < 5 ? 4u : j < 5 + L::kRing ? 1u : uint32_t(kDecoderWarps + 4);  // acc_full: both MMA issuers commit
      }
      mbar_init(ctx.bars + 8 * n, count);
    }
    // flags: abort at misc + 4, epilogue decision at misc + 8, final decision at misc + 16 (misc + 0 receives the TMEM
    // base address from the allocating warp and is left alone here)
    if (i == 0) asm volatile("st.shared.v2.u32 [%0], {%1, %1};" ::"r"(smem + L::misc + 8), "r"(0u) : "memory");
    if (i == 1) asm volatile("st.shared.u32 [%0], %1;" ::"r"(smem + L::misc + 4), "r"(0u) : "memory");
    if (i == 2 || i == 3) asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(smem + L::misc + 16 * (i - 1)), "r"(0u) : "memory");
    mbar_fence_init();
  }
  if (MODE == kUmma && warp == kWideWarpMma) {
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


  if (warp < kDecoderWarps) {
    // ------------------------------------------------------------------ decoders: 32 weights per lane and chunk
    const uint32_t q = warp >> 2, rg = warp & 3, r = rg * 32 + lane;
    uint32_t s = 0, ph = 0;    // input ring slot of the current chunk and its phase parity
    uint32_t so = 0, pho = 0;  // operand stage (tensor memory) of the current chunk
    const uint32_t raw_at = BXQ_RAW_AT + ((2 * q) * BXR_ROWS + r) * 16;
    const uint32_t code_at = BXQ_CODES_AT + 4 * (q * BXR_ROWS + r);
    // this lane's 16 operand columns: lane = row, columns = its 32 weights inside the chunk's atom
    const uint32_t operand_at = ((rg * 32u) << 16) + kWideOperandCol<NB> + (q >> 1) * 32 + (q & 1) * 16;
    bool live = true;
    uint32_t next_base = first_base;
    for (uint32_t u = unit_begin; u < unit_end && live;) {
      const WideSpan item = wide_span(u, unit_end, args.chunks);
      u += item.chunk_end - item.chunk_begin;
      const uint32_t row = item.row_block * BXR_ROWS + r;
      const uint32_t base2 = next_base * 0x00800080u;
      if (u < unit_end) next_base = args.base[row + BXR_ROWS];  // the next item's base: on its way while this item is decoded
      for (uint32_t c = item.chunk_begin; c < item.chunk_end; ++c) {
        if (!ctx.wait(bar_in_full + 8 * s, ph)) { live = false; break; }
        const uint32_t blob = smem + L::in + s * BXQ_BLOB_MAX;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = lds32(blob + code_at + 4 * BXR_SEGMENTS * j);
        const uint4 raw_f = lds128(blob + raw_at);
        const uint4 raw_b = lds128(blob + raw_at + BXR_ROWS * 16);
        const uint32_t e_lo = lds_u16(blob + BXQ_WARP_END_AT + 2 * warp);
        const uint32_t e_hi = min(lds_u16(blob + BXQ_WARP_END_AT + 2 * warp + 2), uint32_t(BXQ_ENTRY_MAX));
        uint32_t out[16];
        bxq_decode32(w, raw_f, raw_b, args.kw, base2, out);
        // Exceptions (weights outside their row window): rare.  Every lane reads the same entry; its owner acts.
        // Corrupt bounds are clamped so that every read stays inside the slot.
        for (uint32_t i = e_lo; i < e_hi; ++i) {
          const uint32_t v = lds32(blob + BXQ_LIST_AT + 4 * i);
          if (((v >> 5) & 31u) == uint32_t(lane)) bxq_patch(out, v & 31u, v >> 16);
        }
        __syncwarp();   // every lane has what it needs from the blob: hand the slot back
        if (lane == 0) mbar_arrive(bar_in_empty + 8 * s);
        if (MODE == kUmma) {
          if (!ctx.wait(bar_op_empty + 8 * so, pho ^ 1)) { live = false; break; }
          tc_fence_after();
          tmem_st16(tmem_base + operand_at + so * 64, out);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_op_full + 8 * so);
          if (++so == kOpN) { so = 0; pho ^= 1; }
        } else if (row < args.rows) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t col = c * BXR_COLS + q * 32 + i * 8;
            uint16_t* dst = args.dense + size_t(row) * args.cols + col;
            if (col + 8 <= args.cols && (args.cols & 7) == 0) {
              *reinterpret_cast<uint4*>(dst) = make_uint4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
            } else {
              for (int e = 0; e < 8; ++e)
                if (col + e < args.cols) dst[e] = uint16_t(out[4 * i + (e >> 1)] >> (16 * (e & 1)));
            }
          }
        }
        if (++s == L::kIn) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == kWideWarpLoader) {
    // ------------------------------------------------------------------ chunk blobs, one bulk copy each
    uint32_t issued = 0;
    const uint64_t once = l2_policy_evict_first();  // a blob is read once per launch
    for (uint32_t u0 = 0; u0 < unit_count; u0 += 32) {
      uint32_t i0 = first_i0, i1 = first_i1;
      if (args.blob_stride16) {  // blobs of one size: no offsets to look up
        i0 = (unit_begin + min(u0 + lane, unit_count - 1)) * args.blob_stride16;
        i1 = i0 + args.blob_stride16;
      } else if (u0) {
        const uint32_t mine = unit_begin + min(u0 + lane, unit_count - 1);
        i0 = __ldg(args.blob_index + mine);
        i1 = __ldg(args.blob_index + mine + 1);
      }
      const uint32_t n = min(32u, unit_count - u0);
      bool live = true;
      for (uint32_t i = 0; i < n && live; ++i) {
        const uint32_t u = u0 + i, s = u % L::kIn, ph = (u / L::kIn) & 1;
        const uint32_t b0 = __shfl_sync(0xFFFFFFFFu, i0, i), b1 = __shfl_sync(0xFFFFFFFFu, i1, i);
        if (u < early) {  // requested before the set-up
          issued = u + 1;
          continue;
        }
        const uint32_t bytes = (b1 - b0) << 4;
        if (ctx.aborted() || !ctx.wait(bar_in_empty + 8 * s, ph ^ 1)) { live = false; break; }
        if (b1 < b0 || bytes > BXQ_BLOB_MAX || bytes < BXQ_LIST_AT) {
          ctx.abort(kStatusBadArgument);
          live = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(bar_in_full + 8 * s, bytes);
          bulk_g2s(smem + L::in + s * BXQ_BLOB_MAX, args.blobs + (size_t(b0) << 4), bytes, bar_in_full + 8 * s, once);
        }
        issued = u + 1;
      }
      if (!live) break;
    }
    // Every load of this CTA is on its way: from here on it asks HBM for nothing.  Ask the L2 for what the next launch
    // of the stream will want first - the leading blobs of its CTAs w, w + workers, ... (consecutive in memory) - so
    // that they arrive during this launch's tail and the next launch's set-up.
    if (MODE == kUmma && args.next_blobs && lane == 0 && !ctx.aborted()) {
      for (uint32_t w2 = worker; w2 < args.next_workers; w2 += args.workers) {
        const uint32_t b0 = uint32_t(uint64_t(args.next_units) * w2 / args.next_workers);
        const uint32_t b1 = uint32_t(uint64_t(args.next_units) * (w2 + 1) / args.next_workers);
        const uint32_t n = min(b1 - b0, uint32_t(kWideNextBlobs));
        for (uint32_t b = 0; b < n; ++b) bulk_prefetch_l2(args.next_blobs + size_t(b0 + b) * args.next_blob_bytes, args.next_blob_bytes);
      }
    }
    // after an abort: give copies still in flight a bounded time to land before the CTA exits
    if (ctx.aborted() && lane == 0)
      for (uint32_t u = (issued > uint32_t(L::kIn) ? issued - L::kIn : 0); u < issued; ++u) mbar_wait(bar_in_full + 8 * (u % L::kIn), (u / L::kIn) & 1);
  } else if (MODE == kUmma && warp == kWideWarpXLoader) {
    // ------------------------------------------------------------------ activation tiles by TMA, and the go-ahead
    // One thread.  Chunk v of this CTA (in the order the items list them) uses activation stage v % kX and operand
    // stage v % kOp (tensor memory).  The tiles of chunk v are requested once chunk v - kX has been multiplied (its stage is free);
    // kXLag chunks later the thread waits for them and gives the MMA warp the go-ahead by arriving on the operand
    // stage's `full` barrier, which the decoder warps complete.  "Chunk c has been multiplied" is the phase of
    // op_empty[c % kOp] that the MMA warp's commit completes; this thread is never more than one phase behind it,
    // because the multiply of chunk c + kOp needs its own go-ahead.
    if (lane == 0) {
      grid_dependency_wait();
      const uint64_t stay = l2_policy_evict_last();  // every CTA reads the same activation tiles
      bool live = true;
      uint32_t c_v = unit_begin % args.chunks;  // the chunk (column block) to request next: wraps at the end of a row block
      auto multiplied = [&](uint32_t c) { return ctx.wait(bar_op_empty + 8 * (c % kOpN), (c / kOpN) & 1); };
      for (uint32_t v = 0; v < unit_count + L::kXLag && live; ++v) {
        if (ctx.aborted()) break;
        // the go-ahead first: the request below waits for a multiply that may need it
        if (v >= uint32_t(L::kXLag)) {
          const uint32_t w = v - L::kXLag;
          if (!ctx.wait(bar_x_full + 8 * (w % kXN), (w / kXN) & 1)) { live = false; break; }
          if (w >= kOpN && !multiplied(w - kOpN)) { live = false; break; }
          mbar_arrive(bar_op_full + 8 * (w % kOpN));
        }
        if (v < unit_count) {
          if (v >= kXN && !multiplied(v - kXN)) { live = false; break; }
          const uint32_t sx = v % kXN, stage = smem + L::xs + sx * L::kXStage;
          mbar_arrive_expect_tx(bar_x_full + 8 * sx, L::kXStage);
          tma_load_2d(stage, &tmap_x, int(c_v * BXR_COLS), 0, bar_x_full + 8 * sx, stay);
          tma_load_2d(stage + NB * 128, &tmap_x, int(c_v * BXR_COLS + 64), 0, bar_x_full + 8 * sx, stay);
          if (++c_v == args.chunks) c_v = 0;
        }
      }
    }
  } else if (MODE == kUmma && (warp == kWideWarpMma || warp == kWideWarpMma2)) {
    // ------------------------------------------------------------------ MMA issue: one wait, eight MMAs, one commit
    // Issuing takes a thread about a hundred cycles per MMA, more than the tensor core needs for it: two threads
    // take turns chunk by chunk.  The order of additions has to be a fixed one, so each has an accumulator of its own:
    // chunk i of an item (counted from the item's first) goes to accumulator i mod 2, whatever the batch size.
    constexpr uint32_t idesc = umma_idesc_bf16(NB);
    const uint32_t which = warp == kWideWarpMma2 ? 1u : 0u;
    uint32_t n_item = 0, so = 0, pho = 0, sx = 0;
    bool live = true;
    for (uint32_t u = unit_begin; u < unit_end && live; ++n_item) {
      const WideSpan item = wide_span(u, unit_end, args.chunks);
      u += item.chunk_end - item.chunk_begin;
      const uint32_t buf = n_item % kAccBufs, use = n_item / kAccBufs;
      if (ctx.aborted() || !ctx.wait(bar_acc_empty + 8 * buf, (use & 1) ^ 1)) { live = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + (buf * 2 + which) * NB;
      for (uint32_t c = item.chunk_begin; c < item.chunk_end; ++c) {
        const uint32_t i = c - item.chunk_begin;
        if ((i & 1) == which) {
          if (!ctx.wait(bar_op_full + 8 * so, pho)) { live = false; break; }
          tc_fence_after();
          if (lane == 0) {
            const uint32_t a_tmem = tmem_base + kWideOperandCol<NB> + so * 64;
            const uint64_t bdesc = umma_desc_sw128(smem + L::xs + sx * L::kXStage);
            uint32_t accumulate = i >= 2 ? 1u : 0u;
#pragma unroll
            for (uint32_t a = 0; a < 2; ++a)
#pragma unroll
              for (uint32_t k = 0; k < 4; ++k) {
                umma_bf16_ts(d_tmem, a_tmem + a * 32 + k * 8, bdesc + a * (NB * 128 >> 4) + 2 * k, idesc, accumulate);
                accumulate = 1;
              }
            umma_commit(bar_op_empty + 8 * so);
          }
          __syncwarp();
        }
        if (++so == kOpN) { so = 0; pho ^= 1; }
        if (++sx == kXN) sx = 0;
      }
      if (live && lane == 0) umma_commit(bar_acc_full + 8 * buf);
      __syncwarp();
    }
  } else if (MODE == kUmma && warp >= kWideWarpEpilogue) {
    // ------------------------------------------------------------------ TMEM -> y, or -> FP32 partial tile
    const uint32_t e = warp - kWideWarpEpilogue;  // == warp % 4: the TMEM lane quarter this warp may read
    const uint32_t r = e * 32 + lane;
    const uint32_t mcols = (args.m + 7) & ~7u;
    uint32_t n_item = 0;
    bool live = true, early_taken = false;
    const uint64_t stay = l2_policy_evict_last();  // partial tiles are read back within the launch
    grid_dependency_wait();  // bias, y, partial tiles and counters may belong to the previous kernel
    bxr_item item = {};
    if (item_begin < item_end) item = args.items[item_begin];
    for (uint32_t it = item_begin; it < item_end && live; ++it, ++n_item) {
      if (it != item_begin) item = args.items[it];
      const uint32_t buf = n_item % kAccBufs, use = n_item / kAccBufs;
      if (ctx.aborted() || !ctx.wait(bar_acc_full + 8 * buf, use & 1)) { live = false; break; }
      tc_fence_after();
      const uint32_t row = item.row_block * BXR_ROWS + r;
      const uint32_t taddr = tmem_base + ((e * 32) << 16) + buf * 2 * NB;   // even-chunk accumulator; the odd one NB columns on
      const bool two = item.chunk_end - item.chunk_begin > 1;                // a one-chunk item has no odd chunk
      const float b = (args.bias && row < args.rows) ? __bfloat162float(args.bias[row]) : 0.f;
      constexpr int kStep = 16;  // accumulator columns per tensor-memory load
      // The CTA's last item, if it is part of a split row block, keeps its tile in shared memory (all of it is free
      // by now: every blob and every activation tile has been multiplied).  If the other tiles of the row block are already in memory -
      // the usual case, they were finished long ago as some CTA's first item - this tile never goes to memory at
      // all: no store, no fence, no counter update on the tail of the kernel.
      const bool final_item = it + 1 == item_end;
      const bool in_cluster = args.cluster > 1;  // the CTA's one item is a part of its cluster's row block
      const bool keep = item.parts > 1 && (final_item || in_cluster);
      const uint32_t tile = smem;           // [batch row][128 weight rows] FP32, like a partial tile in memory
      uint32_t arrived = 0;
      if (keep && !in_cluster && e == 0 && lane == 0) arrived = ld_relaxed_gpu(args.counters + item.row_block);  // answer used after the drain; fenced there
      // A lane holds one weight row and kStep batch columns; y and the partial tiles keep the rows of one batch
      // column together.  Stored from the registers that is one narrow store instruction per column, and the
      // store queue, not the memory, sets the pace (a 128-column drain took 4 400 to 10 000 cycles).  So the
      // columns are turned around in shared memory and leave as 16-byte stores: 8 (y) or 4 (tiles) columns each.
      const uint32_t turn = smem + L::turn + e * L::kTurn;
      const bool y_wide = (reinterpret_cast<uintptr_t>(args.y) & 15u) == 0 && (args.ldy & 7u) == 0 &&
                          item.row_block * BXR_ROWS + e * 32 + 32 <= args.rows;
      for (uint32_t m0 = 0; m0 < mcols; m0 += kStep) {
        uint32_t v[kStep];
        tmem_ld16(taddr + m0, v);
        if (two) {
          uint32_t odd[kStep];
          tmem_ld16(taddr + NB + m0, odd);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < kStep; ++i) v[i] = __float_as_uint(__fadd_rn(__uint_as_float(v[i]), __uint_as_float(odd[i])));
        } else {
          tmem_ld_wait();
        }
        if (keep) {
#pragma unroll
          for (int i = 0; i < kStep; ++i)
            if (m0 + i < mcols) sts32(tile + ((m0 + i) * BXR_ROWS + r) * 4, v[i]);
        } else if (item.parts == 1) {
          if (y_wide) {
#pragma unroll
            for (int i = 0; i < kStep; ++i) {
              const float f = __uint_as_float(v[i]);
              const __nv_bfloat16 h = __float2bfloat16_rn(args.bias ? __fadd_rn(f, b) : f);
              sts_u16(turn + (i * 32 + lane) * 2, uint32_t(*reinterpret_cast<const uint16_t*>(&h)));
            }
            __syncwarp();
#pragma unroll
            for (int j = 0; j < kStep / 8; ++j) {  // a store: 8 columns x 64 bytes (32 rows)
              const uint32_t ml = j * 8 + (lane >> 2), m = m0 + ml;
              const uint4 piece = lds128(turn + ml * 64 + (lane & 3) * 16);
              if (m < args.m)
                *reinterpret_cast<uint4*>(args.y + size_t(m) * args.ldy + item.row_block * BXR_ROWS + e * 32 + (lane & 3) * 8) = piece;
            }
            __syncwarp();
          } else if (row < args.rows) {
#pragma unroll
            for (int i = 0; i < kStep; ++i)
              if (m0 + i < args.m) {
                const float f = __uint_as_float(v[i]);
                args.y[size_t(m0 + i) * args.ldy + row] = __float2bfloat16_rn(args.bias ? __fadd_rn(f, b) : f);
              }
          }
        } else {
#pragma unroll
          for (int i = 0; i < kStep; ++i) sts32(turn + (i * 32 + lane) * 4, v[i]);
          __syncwarp();
#pragma unroll
          for (int j = 0; j < kStep / 4; ++j) {  // a store: 4 columns x 128 bytes (32 rows)
            const uint32_t ml = j * 4 + (lane >> 3), m = m0 + ml;
            const uint4 piece = lds128(turn + ml * 128 + (lane & 7) * 16);
            if (m < mcols) stg128(args.partials + (size_t(item.slot) * NB + m) * BXR_ROWS + e * 32 + (lane & 7) * 4, piece, stay);
          }
          __syncwarp();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
      if (item.parts > 1 && !in_cluster) {
        // `prev` = how many tiles of the row block were in memory before this one; the CTA that completes the set
        // reduces it.  Flag words: misc + 8 and misc + 12.
        uint32_t prev;
        if (keep) {
          fence_proxy_async_smem();  // the tile may leave through a bulk copy
          if (e == 0 && lane == 0) asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(smem + L::misc + 8), "r"(arrived) : "memory");
          named_barrier(1, 128);
          asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(prev) : "r"(smem + L::misc + 8));
          if (prev != item.parts - 1) {  // someone else is still missing: publish the tile like any other
            if (e == 0 && lane == 0) {
              bulk_s2g(args.partials + size_t(item.slot) * NB * BXR_ROWS, tile, mcols * BXR_ROWS * 4);
              bulk_commit_and_wait();
              fence_proxy_async_all();
              __threadfence();
              const uint32_t before = atomicAdd(args.counters + item.row_block, 1u);
              asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(smem + L::misc + 12), "r"(before) : "memory");
            }
            named_barrier(1, 128);
            asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(prev) : "r"(smem + L::misc + 12));
          }
        } else {
          __threadfence();
          named_barrier(1, 128);
          if (e == 0 && lane == 0) {
            const uint32_t before = atomicAdd(args.counters + item.row_block, 1u);
            asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(smem + L::misc + 8), "r"(before) : "memory");
          }
          named_barrier(1, 128);
          asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(prev) : "r"(smem + L::misc + 8));
        }
        if (prev == item.parts - 1) {  // every other tile of this row block is in memory: add them in K order
          __threadfence();
          const uint32_t first = item.slot - item.part;
          // Reduced at the end of the CTA by the decoder and epilogue warps together (below).  Only the first and the
          // last item of a CTA can be part of a split row block, hence two decision slots; anything else is reduced here.
          if (final_item || !early_taken) {
            if (e == 0 && lane == 0)  // {1 | (index + 1 of the tile kept in shared memory) << 8, row block, first slot, parts}
              asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(smem + L::misc + (final_item ? 16 : 32)),
                           "r"(1u | (keep ? (item.part + 1u) << 8 : 0u)), "r"(item.row_block), "r"(first), "r"(item.parts) : "memory");
            early_taken = early_taken || !final_item;
          } else {
            reduce_row_block<NB>(args, item.row_block, first, item.parts, e, 4, lane);
          }
          if (e == 0 && lane == 0) args.counters[item.row_block] = 0;
        }
        named_barrier(1, 128);  // the flag words may be rewritten
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(bar_final);
  }

  if (MODE == kUmma && args.cluster > 1) {
    // One cluster per row block: every CTA's tile is in its shared memory once its epilogue is through; the cluster
    // barrier makes the tiles visible to the peers, the second one keeps every CTA's shared memory alive until the
    // peers have read it.  Every thread of every CTA gets here on every path (all other waits are bounded).
    const bool worker_thread = warp < kDecoderWarps || warp >= kWideWarpEpilogue;
    const bool drained = worker_thread ? ctx.wait(bar_final, 0) : true;
    __syncwarp();
    cluster_sync();
    if (worker_thread && drained && unit_count)
      bxq_reduce_in_cluster<NB>(args, unit_begin / args.chunks, smem, (warp < kDecoderWarps ? warp : warp - 4) * 32 + lane);
    __syncwarp();
    cluster_sync();
  }

  // Row blocks whose last partial tile came from this CTA are reduced by the 16 decoder warps and the 4 epilogue
  // warps together, once the epilogue has drained the CTA's last item.
  if (MODE == kUmma && args.cluster <= 1 && (warp < kDecoderWarps || warp >= kWideWarpEpilogue)) {
    if (ctx.wait(bar_final, 0)) {
      uint32_t fetched = 0;  // tiles brought in so far: position in the two-buffer ring
#pragma unroll 1
      for (uint32_t at = 32; at >= 16; at -= 16) {
        const uint4 decision = lds128(smem + L::misc + at);  // {reduce? | own tile << 8, row block, first slot, parts}
        if (decision.x)
          bxq_reduce_row_block<NB>(args, ctx, decision.y, decision.z, decision.w, (decision.x >> 8) - 1u, smem, bar_tile_full, bar_tile_used,
                                   (warp < kDecoderWarps ? warp : warp - 4) * 32 + lane, fetched);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (MODE == kUmma && warp == kWideWarpMma) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace grb
