// Sum of the BF16 partial outputs of a row-parallel linear across the GPUs of one node, over peer memory.
//
// Every rank owns a control block (flags) and a receive area that the other ranks have mapped (CUDA IPC over NVLink).
// One launch per rank, the same launch on every rank:
//   1. push: every CTA copies its share of the rank's partial output (written by the kernel before this one in the
//      stream) into slot [call parity][rank] of every peer's receive area - posted stores, no round trip;
//   2. announce: the last CTA to finish pushing stores the call's number into slot [rank] of every peer's flags;
//   3. every CTA waits until the flags of this rank show the call's number for every peer (a poll of local memory),
//      then adds its share of all partials - the own one from where it is, the others from the local receive area -
//      in FP32 in rank order (so every rank gets the same bits) and writes BF16 to the local output.
// One barrier per call is enough because the receive slots alternate with the call's parity: a rank can be writing
// call k + 2 into a peer's slot only after that peer has announced call k + 1, i.e. after it finished reading call k.
// The call's number lives in device memory and is advanced by the kernel itself, so a launch can be replayed from a
// CUDA graph.  Waits are polls with a time limit (a launch argument); on expiry the status word gets kStatusTimeout
// and the kernel finishes without waiting further: nothing is added, the output is left as it was, the tickets are
// cleared and the call number still advances, so the context stays usable.  After a timeout the ranks no longer agree
// on the call number: the caller zeroes every rank's control block before the group is used again.
// No multicast, no TMA.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "device_utils.cuh"

namespace grb {

constexpr int kPeerMaxRanks = 8;
constexpr int kPeerThreads = 256;
constexpr int kPeerMaxCtas = 128;         // all resident at once: CTAs of a launch wait for one another's pushes
constexpr uint32_t kPeerFlagStride = 32;  // u32 slots between the flags of two ranks (128 bytes: one line each)

// Layout of a rank's control block (u32 slots): ready[r] at r * stride, the call number at 8 * stride, the two CTA
// tickets (pushed, finished) at 9 and 10 * stride.
constexpr uint32_t kPeerReadyAt = 0, kPeerCallAt = 8 * kPeerFlagStride, kPeerPushedAt = 9 * kPeerFlagStride,
                   kPeerFinishedAt = 10 * kPeerFlagStride, kPeerControlWords = 11 * kPeerFlagStride;

struct PeerArgs {
  const __nv_bfloat16* partial;        // local: this rank's partial output
  uint8_t* receive[kPeerMaxRanks];     // every rank's receive area for this reduction as mapped here: [2][world] blocks
  uint32_t* control[kPeerMaxRanks];    // every rank's control block as mapped here
  __nv_bfloat16* out;                  // local
  uint64_t block_bytes;                // size of one [parity][source rank] block of a receive area (>= 2 * elems)
  uint32_t elems;                      // multiple of 8
  uint32_t rank, world;
  uint32_t* status;
  unsigned long long wait_limit_ns;    // how long a rank waits for its peers' flags before it gives up
};

__device__ __forceinline__ uint32_t peer_poll(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void peer_post(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Waits until the flag has reached `call`; false after the time limit.
__device__ __forceinline__ bool peer_wait(const uint32_t* flag, uint32_t call, unsigned long long limit_ns) {
  if (int32_t(peer_poll(flag) - call) >= 0) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 32; ++i)
      if (int32_t(peer_poll(flag) - call) >= 0) return true;
    if (global_ns() - t0 > limit_ns) return false;
  }
}

__global__ void __launch_bounds__(kPeerThreads) peer_allreduce_kernel(const PeerArgs a) {
  __shared__ uint32_t ok_all, last;
  uint32_t* mine = a.control[a.rank];
  if (threadIdx.x == 0) ok_all = 1;
  // Launched with programmatic stream serialisation: up to here the launch may overlap the tail of the kernel before
  // it, which writes the partial (or, if that is another reduction, the call number); the kernel after may start its
  // own prologue now and waits for this one where it must.
  grid_dependency_wait();
  grid_dependents_may_launch();
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(mine + kPeerCallAt) + 1;  // rewritten only by the last CTA, at its end
  const uint32_t parity = call & 1;
  const uint32_t vectors = a.elems >> 3, stride = gridDim.x * kPeerThreads;
  const uint4* own = reinterpret_cast<const uint4*>(a.partial);
  // 1. push
  for (uint32_t v = blockIdx.x * kPeerThreads + threadIdx.x; v < vectors; v += stride) {
    const uint4 x = own[v];
#pragma unroll
    for (uint32_t r = 0; r < kPeerMaxRanks; ++r)
      if (r < a.world && r != a.rank) reinterpret_cast<uint4*>(a.receive[r] + (parity * a.world + a.rank) * a.block_bytes)[v] = x;
  }
  __syncthreads();
  // 2. announce, by the CTA that completes the rank's push.  Release side: one system-scope fence per CTA after the
  //    CTA's barrier (it covers every thread's stores), then the ticket.  Acquire side: the CTA that draws the last
  //    ticket fences again before its threads post the flags, so that every other CTA's pushes are ordered before them.
  if (threadIdx.x == 0) {
    __threadfence_system();
    const bool completes = atomicAdd(mine + kPeerPushedAt, 1u) == gridDim.x - 1;
    if (completes) __threadfence_system();
    last = completes ? 1u : 0u;
  }
  __syncthreads();
  if (last && threadIdx.x < a.world && threadIdx.x != a.rank) peer_post(a.control[threadIdx.x] + kPeerReadyAt + a.rank * kPeerFlagStride, call);
  // 3. wait for everybody's data, add
  if (threadIdx.x < a.world && threadIdx.x != a.rank && !peer_wait(mine + kPeerReadyAt + threadIdx.x * kPeerFlagStride, call, a.wait_limit_ns)) {
    ok_all = 0;
    atomicOr(a.status, kStatusTimeout);
  }
  __syncthreads();
  if (ok_all) {
    const uint8_t* got = a.receive[a.rank] + uint64_t(parity) * a.world * a.block_bytes;
    for (uint32_t v = blockIdx.x * kPeerThreads + threadIdx.x; v < vectors; v += stride) {
      uint4 part[kPeerMaxRanks];
#pragma unroll
      for (uint32_t r = 0; r < kPeerMaxRanks; ++r)
        if (r < a.world) part[r] = r == a.rank ? own[v] : __ldcg(reinterpret_cast<const uint4*>(got + r * a.block_bytes) + v);
      float sum[8];
#pragma unroll
      for (uint32_t r = 0; r < kPeerMaxRanks; ++r)
        if (r < a.world) {
          const uint32_t w[4] = {part[r].x, part[r].y, part[r].z, part[r].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = __uint_as_float(w[i] << 16), hi = __uint_as_float(w[i] & 0xFFFF0000u);
            sum[2 * i] = r ? __fadd_rn(sum[2 * i], lo) : lo;
            sum[2 * i + 1] = r ? __fadd_rn(sum[2 * i + 1], hi) : hi;
          }
        }
      uint4 o;
      uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 h = __floats2bfloat162_rn(sum[2 * i], sum[2 * i + 1]);
        ow[i] = *reinterpret_cast<const uint32_t*>(&h);
      }
      reinterpret_cast<uint4*>(a.out)[v] = o;
    }
  }
  // the last CTA to finish advances the call number and clears the tickets for the next launch
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(mine + kPeerFinishedAt, 1u) == gridDim.x - 1) {
    mine[kPeerPushedAt] = 0;
    mine[kPeerFinishedAt] = 0;
    __threadfence();
    *reinterpret_cast<volatile uint32_t*>(mine + kPeerCallAt) = call;
  }
}

}  // namespace grb
