// BXR1: the resident layout the fused decode-GEMV/GEMM kernels stream from HBM.
//
// A BCTX frame is one serial rANS stream per tensor; it restarts only at indexed checkpoints and its
// bytes are scattered relative to the columns they code.  At load time the decoded words are re-coded
// into this layout, which keeps the frame's information (bit-exact BF16 words) but is organised for a
// B200 SM: everything one CTA needs for 128 rows x 128 columns is one contiguous, 16-byte aligned blob
// that a single bulk copy brings into shared memory.
//
//   word     = sign(1) exponent(8) mantissa(7)
//   raw byte = sign << 7 | mantissa                       stored verbatim, 1 byte per weight
//   exponent -> nibble n = exponent - base[row] when 0 <= n <= 14, else n = 15 ("escape", the 8-bit
//               exponent follows in the same stream at probability 1/256)
//   symbol   = n(col 2t) | n(col 2t+1) << 4                one rANS step decodes two weights
//   rANS     : 32-bit state, lower bound 2^16, 16-bit words, 12-bit probabilities, one static table
//              per tensor stored as 4096 slot records {freq | esc flags | bias, exponent bits}
//
// Geometry.  Rows are grouped in row blocks of 128 (one UMMA M tile), columns in chunks of 128.  Inside a
// chunk every row has 4 independent streams ("phases"), phase q coding columns [32q, 32q+32) of the chunk
// in 16 steps.  A stream runs through consecutive chunks of one work item without being flushed; a lane
// owns one stream, so 16 warps decode a chunk of a row block in lock step without ever communicating.
// The words consumed by a stream while it decodes one chunk are stored with that chunk: streams 2h and
// 2h+1 of a row share one segment, the even one reading forward from the segment's first word, the odd
// one backward from its last, so one byte (the segment's word count) locates both.
//
// Chunk blob (size = multiple of 16 bytes, at most kBlobMax):
//   [0,256)          u8  count[256]         words in segment g = h*128 + r           (h = phase / 2)
//   [256,16640)      u8  raw[4][2][128][16] piece (q, j, r) = raw bytes of row r, chunk columns 32q+16j..+15
//   [16640, ...)     u16 words              segments in order g, then zero padding
//
// Work items.  The K range of every row block is cut so that `workers` CTAs get equal numbers of chunks
// (a contiguous range of the (row block, chunk) sequence each).  An item is the part of one row block
// that one worker owns; streams restart (4-byte state per stream) at the start of every item.  A row
// block covered by several items is reduced from FP32 partial tiles in item order, which depends only on
// the shape and `workers`, never on the batch size.
#pragma once
#include <stdint.h>

#define BXR_MAGIC 0x31525842u /* "BXR1" */
#define BXR_ROWS 128
#define BXR_COLS 128
#define BXR_PHASES 4
#define BXR_PHASE_COLS 32
#define BXR_STEPS 16
#define BXR_STREAMS 512  /* per row block: phase * 128 + row */
#define BXR_SEGMENTS 256 /* per chunk: (phase / 2) * 128 + row */
#define BXR_COUNT_BYTES 256
#define BXR_RAW_BYTES 16384
#define BXR_WORDS_AT (BXR_COUNT_BYTES + BXR_RAW_BYTES)
#define BXR_BLOB_MAX 24576 /* shared-memory slot per chunk blob */
#define BXR_WORDS_MAX ((BXR_BLOB_MAX - BXR_WORDS_AT) / 2)
#define BXR_PROB_BITS 12
#define BXR_PROB_TOTAL 4096
#define BXR_STATE_LOW 65536u
#define BXR_ESCAPE 15
#define BXR_MODE_CODED 0
#define BXR_MODE_RAW 1 /* chunk blob = the 128x128 BF16 tile itself, already in UMMA operand order */
#define BXR_RAW_TILE_BYTES 32768

/* Slot record of the pair table: lo = freq[0,13) | esc0 << 13 | esc1 << 14 | bias << 16,
 * hi = n0 << 7 | n1 << 23 (escaped nibbles contribute 0). */
#define BXR_LUT_ESC0 0x2000u
#define BXR_LUT_ESC1 0x4000u
#define BXR_LUT_FREQ_MASK 0x1FFFu

typedef struct bxr_item {
  uint32_t row_block;  /* which 128-row block */
  uint32_t chunk_begin, chunk_end;
  uint32_t part;       /* index of this item among the items of its row block, in K order */
  uint32_t parts;      /* how many items share the row block */
  uint32_t slot;       /* partial-tile slot in the workspace when parts > 1 */
  uint32_t reserved[2];
} bxr_item;

/* Host-side description of one resident tensor; every offset is in bytes from the start of the image. */
typedef struct bxr_header {
  uint32_t magic, mode;
  uint32_t rows, cols;            /* logical shape */
  uint32_t row_blocks, chunks;    /* padded shape / 128 */
  uint32_t workers, items;
  uint32_t partial_slots;         /* FP32 partial tiles the workspace must hold */
  uint32_t reserved0;
  uint64_t lut_at;                /* u64[4096] slot records (absent in raw mode) */
  uint64_t base_at;               /* u8[row_blocks*128] exponent base per row */
  uint64_t items_at;              /* bxr_item[items] */
  uint64_t worker_items_at;       /* u32[workers+1]: items of worker w are [v[w], v[w+1]) */
  uint64_t states_at;             /* u32[items][512] start state of every stream */
  uint64_t blob_index_at;         /* u32[row_blocks*chunks+1] blob offsets in 16-byte units from blobs_at */
  uint64_t blobs_at;
  uint64_t total_bytes;
  uint64_t coded_bytes;           /* blobs + states + index: what one pass of the kernel streams */
  uint8_t source_sha256[32];      /* digest of the little-endian source words, as in the BCTX header */
} bxr_header;
