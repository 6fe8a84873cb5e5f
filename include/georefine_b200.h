/*
 * georefine_b200 -- C ABI of the B200-native BCTX path: plain pointers and sizes, no torch types.
 *
 * One shared library (libgeorefine_b200.so) exports three groups of entry points:
 *
 *   1. bcx_*   host coder and restart index.  Same names, argument lists, status codes and ownership
 *              rules as the reference's ctypes ABI, so existing bindings load this library unchanged.
 *   2. grb_bctx_*  CUDA decode of unchanged BCTX streams from their restart index (replaces the launch of
 *              the reference's Triton kernels).
 *   3. bxr_* / grb_bxr_*  the resident layout and the fused decode-GEMV / decode-GEMM kernels over it
 *              (replace the reference's decode + F.linear and its fused native linears).
 *
 * Reference paths below are relative to the reference project root;
 * cr/ = context-runtime/georefine_context_runtime/, gs/ = context-runtime/glc_serve/.
 *
 * Device entry points take raw device pointers and a CUDA stream handle (cudaStream_t passed as void*),
 * never allocate, never synchronise with the host, and return an int: 0 on success, GRB_ERR_* otherwise.
 * Faults found while a kernel runs (corrupt stream, expired wait) are reported through a caller-owned
 * 32-bit device status word (GRB_STATUS_* bits, OR-ed in); a nonzero word means the output must be discarded.
 */
#ifndef GEOREFINE_B200_H
#define GEOREFINE_B200_H

#include <stddef.h>
#include <stdint.h>

#include "../georefine_b200/csrc/bxr_format.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------------------------------------------
 * 1. Host coder (CPU).  Status: 0 ok, 1 bad arguments, 2 malformed stream or tables / out of memory,
 *    3 internal failure.  Outputs are untouched unless the call returns 0.  No global state; safe to call
 *    from several threads.
 * ------------------------------------------------------------------------------------------------- */

/* Replaces bcx_encode, cr/bitexact_context_ans.cpp:235-266.  kind 0 codes the 10-bit main symbol under
 * nr*nc (row class x column class) models, kind 1 the 6-bit residual under 1024 models selected by the main
 * symbol.  freq receives nctx*vocab frequencies (each context sums to 65536).  *stream is malloc'ed: release
 * it with bcx_free. */
int bcx_encode(const uint16_t* words, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* row_class,
               const uint8_t* col_class, uint32_t nr, uint32_t nc, uint32_t kind, uint32_t* freq, uint8_t** stream,
               size_t* stream_bytes);

/* Replaces bcx_frequencies, cr/bitexact_context_ans.cpp:267-290 (tables only, no stream). */
int bcx_frequencies(const uint16_t* words, uint64_t n, uint32_t rows, uint32_t cols, const uint8_t* row_class,
                    const uint8_t* col_class, uint32_t nr, uint32_t nc, uint32_t kind, uint32_t* freq);

/* Replace bcx_decode / bcx_decode_compact, cr/bitexact_context_ans.cpp:291-326.  resctx (kind 1 only) holds
 * the main symbol of every element.  Rejects anything but the canonical end of stream. */
int bcx_decode(const uint8_t* stream, size_t stream_bytes, uint64_t n, uint32_t rows, uint32_t cols,
               const uint8_t* row_class, const uint8_t* col_class, uint32_t nr, uint32_t nc, uint32_t kind,
               const uint16_t* resctx, const uint32_t* freq, uint16_t* symbols);
int bcx_decode_compact(const uint8_t* stream, size_t stream_bytes, uint64_t n, uint32_t rows, uint32_t cols,
                       const uint8_t* row_class, const uint8_t* col_class, uint32_t nr, uint32_t nc, uint32_t kind,
                       const uint16_t* resctx, const uint32_t* freq, uint16_t* symbols);

/* Replaces bcx_free, cr/bitexact_context_ans.cpp:327. */
void bcx_free(void* p);

/* Replace bcx_pack6 / bcx_unpack6, cr/bitexact_context_ans.cpp:328-359: residuals, 6 bits each, most
 * significant bit first; unpack6 wants exactly ceil(6n/8) bytes with zero padding bits (2 otherwise). */
int bcx_pack6(const uint16_t* words, uint64_t n, uint8_t** out, size_t* bytes);
int bcx_unpack6(const uint8_t* in, size_t bytes, uint64_t n, uint16_t* residuals);

/* Replaces bcx_checkpoint, cr/bitexact_context_gpu_index.cpp:21-137.  Walks the stream once and records the
 * decoder state and byte offset in front of every stride-th symbol (offsets count from the start of the
 * stream, so the first pair is (initial state, 4)).  Status: 0 ok, 1 arguments or labels, 2 tables,
 * 3 stream/state, 4 offset beyond 32 bits, 5 out of memory, 6 other. */
int bcx_checkpoint(const uint8_t* stream, size_t stream_bytes, uint64_t n, uint32_t rows, uint32_t cols,
                   const uint8_t* row_class, const uint8_t* col_class, uint32_t nr, uint32_t nc, uint32_t kind,
                   const uint16_t* resctx, const uint32_t* freq, uint32_t stride, uint32_t* states,
                   uint32_t* offsets, uint16_t* symbols);

/* Tables for grb_bctx_decode_words: cum = u32[nctx][vocab+1] prefix sums, bucket = u16[nctx][4096] symbol
 * owning the first slot of each 16-slot bucket.  Takes the place of the cumulative tables the reference
 * builds in CudaContextTensor.__init__, cr/bitexact_context_gpu.py:120-125.  0 ok, 1 arguments, 2 tables. */
int grb_bctx_build_lookup(const uint32_t* freq, uint32_t nctx, uint32_t vocab, uint32_t* cum, uint16_t* bucket);

/* ---------------------------------------------------------------------------------------------------
 * 2. CUDA decode of unchanged BCTX streams.
 * ------------------------------------------------------------------------------------------------- */

#define GRB_OK 0
#define GRB_ERR_ARGUMENT 1      /* null pointer, bad size, misaligned buffer */
#define GRB_ERR_UNSUPPORTED 2   /* e.g. batch larger than the entry point handles */
#define GRB_ERR_WORKSPACE 3     /* workspace too small */
#define GRB_ERR_STATIC_LIMIT 4  /* the image needs more scratch than the built-in array of grb_bxr_gemv_static */
#define GRB_ERR_CUDA 100        /* + cudaError_t of the failing runtime call */

#define GRB_STATUS_BAD_SYMBOL 1u
#define GRB_STATUS_OVERRUN 2u
#define GRB_STATUS_LOW_STATE 4u
#define GRB_STATUS_CHECKPOINT 8u
#define GRB_STATUS_TIMEOUT 16u      /* a bounded wait ran out; the fused kernels also record where: bits 8..15 =
                                      1 + index of the first barrier that gave up, bits 16..23 = its CTA (diagnostic) */
#define GRB_STATUS_BAD_ARGUMENT 32u

/* Device pointers of one indexed frame: the arrays CudaContextTensor keeps in .buffers
 * (cr/bitexact_context_gpu.py:109-128) plus the lookup tables above. */
typedef struct grb_bctx_tensor {
  uint64_t n;                 /* rows * cols */
  uint32_t rows, cols;
  uint32_t nr, nc;
  uint32_t mode;              /* 0 raw6 residual, 128 conditional residual stream */
  uint32_t stride;            /* words per restart block */
  const uint8_t* row_class;   /* u8[rows] */
  const uint8_t* col_class;   /* u8[cols] */
  const uint8_t* main_stream; uint64_t main_bytes;
  const uint32_t* main_states; const uint32_t* main_offsets;   /* u32[ceil(n/stride)] */
  const uint32_t* main_cum;   const uint16_t* main_bucket;
  const uint8_t* residual_stream; uint64_t residual_bytes;     /* raw6 bytes or the conditional stream */
  const uint32_t* residual_states; const uint32_t* residual_offsets;  /* mode 128 only */
  const uint32_t* residual_cum;    const uint16_t* residual_bucket;   /* mode 128 only */
  /* log2 of the slots per bucket of the two inverse indexes; 0 = 4, the tables grb_bctx_build_lookup writes.  A caller
   * may thin them out (every 2^(shift-4)-th entry, [nctx][65536 >> shift]) so that all contexts' tables stay in L1:
   * the walk is one serial chain per lane, and a first-level miss costs it an L2 round trip per symbol. */
  uint32_t main_bucket_shift, residual_bucket_shift;
} grb_bctx_tensor;

/* Replaces the launch of decode_words, cr/bitexact_context_gpu.py:130-152 / bitexact_context_gpu_kernels.py:
 * 114-169.  block_ids == NULL decodes blocks 0..count-1, otherwise the listed blocks (gather).  out receives
 * count*stride words, block-major.  *status is OR-ed with GRB_STATUS_* bits; the caller zeroes it. */
int grb_bctx_decode_words(const grb_bctx_tensor* tensor, const int64_t* block_ids, uint64_t count, uint16_t* out,
                          uint32_t* status, void* cuda_stream);

/* ---------------------------------------------------------------------------------------------------
 * 3. Resident layout (bxr_format.h) and the fused kernels.
 * ------------------------------------------------------------------------------------------------- */

/* Host: re-codes decoded BF16 words into a resident image for `workers` persistent CTAs (the SM count of the
 * target GPU).  Stands where the reference transcodes a frame into its runtime formats at load
 * (gs/bctx_v21_transcode.py:59-560; gs/tbe_desc.py:42-51).  layout: 3 = fixed 4-bit exponent codes in a 16-binade
 * row window with a (nearly empty) exception list and chunk blobs of one size (the role of the reference's TBE
 * container, gl/tbe_container.py:259-404; 1.506 bytes per weight, the fastest kernel), 2 = 3-bit codes in an 8-binade
 * window (1.406 bytes per weight), 0 = entropy-coded exponent streams (rANS; 1.365-1.39 bytes per weight, the slowest
 * kernel), 1 = plain tiles.  An image whose chunks do not fit is demoted 3 or 2 -> 0 -> 1; the header's `mode` says
 * what was built.
 * source_sha256 (optional, 32 bytes) is copied into the header.  *image is malloc'ed: release with bxr_free.
 * 0 ok, 1 arguments, 2 out of memory, 3 other. */
int bxr_build(const uint16_t* words, uint32_t rows, uint32_t cols, uint32_t workers, uint32_t host_threads,
              uint32_t layout, const uint8_t* source_sha256, uint8_t** image, uint64_t* image_bytes);
void bxr_free(void* p);

/* Structural check of an image before any offset inside it is followed, by the host twin or by a kernel: layout
 * version (bxr_layout_version(), bumped on every format change), header fields, every array inside
 * [image, image + image_bytes), the work partition (it must be the one this library computes for the shape and worker
 * count), an ascending blob index and the per-mode size limits of every blob.  Reads the header, the item list and the
 * blob index only.  0 sound, 1 malformed.  Loaders call it on every image that did not come straight out of bxr_build
 * (a disk cache, a file): the reference's transcode cache makes the same kind of check on its entries
 * (gs/transcode_cache.py) before trusting them. */
int bxr_validate(const uint8_t* image, uint64_t image_bytes);
uint32_t bxr_layout_version(void);

/* Host twin of the GPU decoder, used to bind an image to its source digest before upload (the check the
 * reference makes at cr/bitexact_context_gpu.py:104-105).  Runs bxr_validate first.  0 ok, 1 malformed image,
 * 2 corrupt stream. */
int bxr_decode_host(const uint8_t* image, uint64_t image_bytes, uint16_t* words);

/* Bytes of caller-owned device scratch the fused entry points need for this image and batch tile:
 * FP32 partial tiles of row blocks shared by several CTAs, preceded by one counter per row block.
 * The scratch must be zero-filled once after allocation; the kernels leave the counters at zero. */
uint64_t grb_bxr_workspace_bytes(const bxr_header* header, uint32_t max_m);

/* Decode twin: writes rows*cols BF16 words.  Replaces CudaContextTensor.decode() for a resident image,
 * cr/bitexact_context_gpu.py:154-157. */
int grb_bxr_decode(const void* device_image, const bxr_header* header, uint16_t* out, uint32_t* status,
                   void* cuda_stream);

/* y[m, n] = bf16( sum_k x[m, k] * W[n, k] (+ bias[n]) ), FP32 accumulation, W decoded on the fly.
 *   x: BF16 [m, cols], row stride ldx elements, 16-byte aligned, ldx % 8 == 0;  y: BF16 [m, rows], stride ldy.
 *
 * grb_bxr_gemm (any m; tcgen05/TMEM) replaces bi_gemm_dense, gs/bi_csrc/bi_api.h:55-57 and the simple path
 * BctxLinear.forward, cr/bitexact_context_serving.py:365-376.  Rows of y do not depend on m.
 * grb_bxr_gemv (m <= 8; CUDA cores) replaces miv_tbe_gemv, gs/miv_tbe_csrc/miv_tbe.h:57-65, and
 * miv_gemv_out, gs/miv_gemv.py:125-191, with the same M-invariance among m = 1..8.
 * The two entry points use different reduction orders; a caller that needs bitwise equal rows across batch
 * sizes must stay with one of them. */
int grb_bxr_gemm(const void* device_image, const bxr_header* header, const void* x, int64_t ldx, uint32_t m, void* y,
                 int64_t ldy, const void* bias, void* workspace, uint64_t workspace_bytes, uint32_t* status,
                 void* cuda_stream);
int grb_bxr_gemv(const void* device_image, const bxr_header* header, const void* x, int64_t ldx, uint32_t m, void* y,
                 int64_t ldy, const void* bias, void* workspace, uint64_t workspace_bytes, uint32_t* status,
                 void* cuda_stream);

/* grb_bxr_gemm with a hint: next_image / next_header name the resident image the NEXT fused launch of the same stream
 * will read (the order of the linears of a decoder layer is fixed, so an engine knows it; the reference's engine fixes
 * the same order when it captures a whole decode step, gs/fastdec.py:706-956).  CTAs that have issued their last load
 * ask the L2 for the first blobs of the next launch, so that HBM keeps working through this launch's tail and the next
 * launch's set-up.  Only a hint: results do not depend on it; NULL (or an image in another layout) means no hint. */
int grb_bxr_gemm_next(const void* device_image, const bxr_header* header, const void* x, int64_t ldx, uint32_t m, void* y,
                      int64_t ldy, const void* bias, void* workspace, uint64_t workspace_bytes, uint32_t* status,
                      void* cuda_stream, const void* next_device_image, const bxr_header* next_header);

/* y[m, n] = bf16( sum_k x[m, k] * W[n, k] (+ bias[n]) ) for a DENSE BF16 weight W [rows, cols] (row stride ldw), m <= 8.
 * Replaces miv_gemv_out / linear, gs/miv_gemv.py:125-191,916-959, with its numerical contract: lanes walk 16-byte
 * vectors in increasing k, eight FMAs per vector in element order, xor butterfly, K slices added in slice order, bias
 * in FP32, one rounding; rows of y are bitwise independent of m (1..8).  The number of K slices depends on the shape
 * and the SM count only.  It is the dense yardstick the fused kernels are compared with, and the linear for weights
 * that are kept uncompressed.  cols % 8 == 0, ldw % 8 == 0, ldx % 8 == 0, W and x 16-byte aligned.  No allocation, no
 * host synchronisation. */
int grb_dense_gemv_bf16(const void* w, int64_t ldw, uint32_t rows, uint32_t cols, const void* x, int64_t ldx, uint32_t m,
                        void* y, int64_t ldy, const void* bias, void* cuda_stream);

/* grb_bxr_gemv without caller-provided scratch.  This entry point has no counterpart in the reference.
 *
 * It is for callers that are not in a position to allocate device memory at all: a plugin loaded into a
 * serving process whose host has already handed every free byte of HBM to its own pool (KV cache, activations)
 * and offers the plugin no allocator, or code that runs where a call into the driver's allocator is forbidden
 * or may block (inside a latency-critical decode loop, while another thread holds the device for a capture).
 * Such a caller passes only inputs and outputs; the FP32 partial sums and the per-row-block counters of the
 * GEMV live in a fixed array that is part of the library image itself (grb_static_scratch_bytes() = 4 MiB per
 * GPU that loads the library, held until the process exits).  The call makes no cudaMalloc, cudaFree or other
 * allocating call.
 *
 *  - Limit: images whose GEMV scratch (one counter per 128-row block plus 4 KiB per shared partial tile, 8 KiB for
 *    the window layouts) exceeds the array are refused with GRB_ERR_STATIC_LIMIT.  A 34816 x 5120 weight built for
 *    148 workers needs about 1.7 MiB.  Every refusal (this one, a batch above 8, a null or misaligned pointer, a bad
 *    stride) comes before anything is put on the stream: the output and the array are left as they were.
 *  - First use: the first call on each device looks up the array's device address (with that device current)
 *    and keeps it; make that first call outside any stream capture.
 *  - Sharing: every call on a device uses the same array.  The counters are cleared on the given stream at
 *    the start of each call, so a call does not depend on what the previous one left behind, but two calls
 *    that can overlap on the GPU (different streams, no dependency) race on it and must not be issued.
 *  - Results are bitwise those of grb_bxr_gemv (same kernel, same reduction order); m <= 8. */
uint64_t grb_static_scratch_bytes(void);
int grb_bxr_gemv_static(const void* device_image, const bxr_header* header, const void* x, int64_t ldx, uint32_t m,
                        void* y, int64_t ldy, const void* bias, uint32_t* status, void* cuda_stream);

/* Registers, spills and shared memory of the compiled kernels, for tuning records (the reference reads the
 * same from its card in bi_kernel_attrs, gs/bi_csrc/bi_gemm.cuh:1104-1121).  which: 0 BCTX decode; entropy-coded
 * images: 1 decode twin, 2 GEMV (m=1), 3 GEMM (batch tile 16), 4 GEMM (batch tile 128); 3-bit window images: 5 decode
 * twin, 6 GEMM (tile 16), 7 GEMM (tile 128); 4-bit window images: 8 decode twin, 9 GEMM (tile 16), 10 GEMM (tile 128).
 * out = {registers, local bytes, static smem, max dynamic smem, max threads}. */
int grb_kernel_attributes(int which, int out[5]);

/* ---------------------------------------------------------------------------------------------------
 * 4. Row-parallel linears across the GPUs of one node: the sum of the per-GPU partial outputs.
 * ------------------------------------------------------------------------------------------------- */

/* The reference runs a linear on one device (its multi-device code places whole layers,
 * glc_loader/tbe_device_map.py:46-56); a tensor-parallel deployment of the fused linears needs the partial outputs
 * of the column-split weights (O and down projections) added across GPUs.  grb_peer_allreduce_bf16 does that over
 * peer memory, one launch per rank, the same call on every rank in the same order:
 *   partial      this rank's partial output (elems BF16, 16-byte aligned), written by the preceding kernel of `stream`;
 *   receives[r]  rank r's receive area for this reduction as mapped into this process (CUDA IPC or any other peer
 *                mapping; receives[rank] is the local one): 2 * world blocks of block_bytes (>= 2 * elems, a multiple
 *                of 16), indexed [call parity][source rank]; never touched by the host;
 *   controls[r]  rank r's control block (grb_peer_control_bytes() bytes, 128-byte aligned, zeroed once before the
 *                first call, never touched by the host afterwards), mapped likewise; one block per rank serves all
 *                reductions of that rank, which must then be issued one after another on one stream;
 *   out          local result: BF16(sum over r in rank order of rank r's partial), FP32 accumulation, the same bits on
 *                every rank; may not alias the partial.
 * Every rank copies its partial into the peers' receive areas (posted stores over NVLink), announces it with a flag,
 * waits for the peers' flags and adds.  The partial may be overwritten as soon as the launch has completed locally.
 * The call allocates nothing and does not synchronise with the host; it can be captured in a CUDA graph (the call
 * counter lives in the control block).  A peer that never makes the matching call shows as GRB_STATUS_TIMEOUT in
 * *status after wait_limit_ns nanoseconds (0 = the default, two seconds): nothing spins without a limit, the kernel
 * returns by itself, `out` is left as it was and the context stays usable.  The ranks then disagree on the call
 * number: zero every rank's control block before the group reduces again.  world <= 8, elems % 8 == 0.
 * grb_peer_enable(device) enables access from the current device to a peer's memory (GRB_ERR_UNSUPPORTED if the
 * two are not connected). */
uint64_t grb_peer_control_bytes(void);
int grb_peer_enable(int peer_device);
/* Buffers the ranks of a node can map from one another (CUDA IPC).  grb_peer_alloc: a zeroed device allocation of
 * its own on the current device and the 64-byte handle that names it; grb_peer_open: maps the allocation behind a
 * handle received from another process for the current device; grb_peer_close / grb_peer_free undo them.  Set-up
 * calls: they allocate and synchronise. */
int grb_peer_alloc(uint64_t bytes, void** ptr, uint8_t handle[64]);
int grb_peer_free(void* ptr);
int grb_peer_open(const uint8_t handle[64], void** ptr);
int grb_peer_close(void* ptr);
int grb_peer_allreduce_bf16(const void* partial, void* const* receives, void* const* controls, uint64_t block_bytes, uint32_t rank,
                            uint32_t world, void* out, uint64_t elems, uint64_t wait_limit_ns, uint32_t* status, void* cuda_stream);

/* ---------------------------------------------------------------------------------------------------
 * 5. The other kernels of a batched decode step (everything between the fused linears).  BF16 in and out, FP32
 *    arithmetic, every row computed by CTAs of its own in a fixed order, so a row does not depend on the batch it is in.
 *    No allocation, no host synchronisation.
 * ------------------------------------------------------------------------------------------------- */

/* Replaces rmsnorm_kernel, gs/fastdec_kernels.cu:83-110.  If delta: h = bf16(h + delta), written back (the residual
 * add).  out = bf16(h * rsqrt(mean(h^2) + eps) * (unit_offset ? 1 + weight : weight)).  hidden % 8 == 0, <= 16384. */
int grb_rmsnorm_bf16(void* h, int64_t ldh, const void* delta, int64_t ldd, const void* weight, void* out, int64_t ldo,
                     uint32_t rows, uint32_t hidden, float eps, int unit_offset, void* cuda_stream);

/* Replaces silu_mul_kernel, gs/fastdec_kernels.cu:451-459: out[r, i] = bf16(bf16(silu(gate_up[r, i])) * gate_up[r, f + i]). */
int grb_silu_mul_bf16(const void* gate_up, int64_t ldg, void* out, int64_t ldo, uint32_t rows, uint32_t f, void* cuda_stream);

/* Replaces argmax_kernel, gs/fastdec_kernels.cu:462-488: index of the first maximum of every row. */
int grb_argmax_bf16(const void* logits, int64_t ld, uint32_t rows, uint32_t vocab, int32_t* out, void* cuda_stream);

/* One attention step over a paged KV cache: rotary embedding of the query and key heads and the append of keys and
 * values at each row's position, then decode attention in splits of 256 positions merged in split order.  Replaces
 * attn_prep / attn_split / attn_combine, gs/fastdec_kernels.cu:324-448, and their batched twins with a page table
 * (gs/bidec.py:71-81).  Plain grouped-query attention with head dimension 128: no per-head norm, no output gate.
 * Row r is position row_pos[r] of the sequence in slot row_seq[r]; several rows of one sequence at consecutive
 * positions (a prompt chunk, a speculative verify) are handled in one call: all appends happen before any read.
 * A page holds 256 positions of one sequence as [kv head][256][128]; page_table[slot * max_pages + p / 256] names it. */
typedef struct grb_attn_step {
  const void* qkv;            /* BF16 [rows][ldq]: nq query heads | nkv key heads | nkv value heads */
  int64_t ldq;
  const void* cos_table;      /* BF16 [positions][128] (second half repeats the first, the rotate-half convention) */
  const void* sin_table;
  const int32_t* row_seq;     /* [rows] */
  const int32_t* row_pos;     /* [rows] */
  const int32_t* page_table;  /* [slots][max_pages] */
  uint32_t max_pages;
  void* k_pages;              /* BF16 [pages][nkv][256][128] */
  void* v_pages;
  void* q;                    /* scratch: BF16 [rows][nq][128] */
  float* part_acc;            /* scratch: [rows][nq][max_splits][128]; a split is 128 positions, half a page */
  float* part_ml;             /* scratch: [rows][nq][max_splits][2]; max_splits <= 2 * max_pages */
  void* out;                  /* BF16 [rows][nq * 128] */
  uint32_t rows, nq, nkv, head_dim, max_splits;   /* head_dim must be 128; nq / nkv in {1, 2, 4, 5, 8} */
  float scaling;              /* 1 / sqrt(head_dim) */
} grb_attn_step;
int grb_attn_decode_bf16(const grb_attn_step* step, void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif
