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
//   exponent -> nibble n = exponent - base[row] when 0 <= n <= 14, else n = 15 ("exception": the decoder
//               emits exponent base[row] for it and the true 8-bit exponent is patched in afterwards from
//               the chunk's exception list; about 1.5e-4 of the weights on Gaussian rows)
//   symbol   = n(col 2t) | n(col 2t+1) << 4                one rANS step decodes two weights
//   rANS     : 32-bit state, lower bound 2^16, 16-bit words, 12-bit probabilities, one static table
//              per tensor stored as 4096 32-bit slot records {n0, bias, n1, freq}; the decode loop has no
//              data-dependent branch
//
// Geometry.  Rows are grouped in row blocks of 128 (one UMMA M tile), columns in chunks of 128.  Inside a
// chunk every row has 8 independent streams of 16 columns (8 steps) each.  A stream runs through the
// consecutive chunks of one work item without being flushed.  Streams 2q and 2q+1 of a row (columns
// [32q, 32q+16) and [32q+16, 32q+32) of the chunk) belong to one lane, which decodes them interleaved: two
// independent dependency chains per lane.  The words the two streams consume while they decode one chunk
// are stored with that chunk in one segment: the even stream reads forward from the segment's first word,
// the odd one backward from its last, so one byte (the segment's word count) locates both.  16 warps
// decode a chunk of a row block in lock step without ever communicating.
//
// Chunk blob (size = multiple of 16 bytes, at most BXR_BLOB_MAX):
//   [0,512)          u8  count[512]         words in segment g = q*128 + r
//   [512,576)        u8  exc_bits[64]       bit g set: segment g has at least one exception in this chunk
//   [576,16960)      u8  raw[8][128][16]    piece (s, r) = raw bytes of row r, chunk columns 16s..16s+15
//   [16960, ...)     u16 words              segments in order g
//   then, 4-byte aligned: u32 exception count, u32 entries {segment[0,9) | column in segment[9,14) |
//   exponent[14,22)} sorted by segment, then zero padding
//
// Work items.  The K range of every row block is cut so that `workers` CTAs get equal numbers of chunks
// (a contiguous range of the (row block, chunk) sequence each).  An item is the part of one row block
// that one worker owns; streams restart (4-byte state per stream) at the start of every item.  A row
// block covered by several items is reduced from FP32 partial tiles in item order, which depends only on
// the shape and `workers`, never on the batch size.
#pragma once
#include <stdint.h>

#define BXR_MAGIC 0x31525842u /* "BXR1" */
/* Bumped whenever a blob layout, the work partition or the header changes: an image of another version is refused by
 * bxr_validate (and by the disk cache, whose key includes it) instead of being streamed by kernels that no longer
 * understand it. */
#define BXR_LAYOUT_VERSION 2u
#define BXR_ROWS 128
#define BXR_COLS 128
#define BXR_PHASES 4       /* lanes per row: phase q owns chunk columns [32q, 32q+32) */
#define BXR_STREAM_COLS 16
#define BXR_STEPS 8        /* two weights per step */
#define BXR_STREAMS 1024   /* per row block: (2q + d) * 128 + row, d = 0 forward / 1 backward reader */
#define BXR_SEGMENTS 512   /* per chunk: q * 128 + row */
#define BXR_COUNT_BYTES 512
#define BXR_EXC_BITS_AT 512
#define BXR_RAW_AT 576
#define BXR_RAW_BYTES 16384
#define BXR_WORDS_AT (BXR_RAW_AT + BXR_RAW_BYTES)
#define BXR_EXC_MAX 1024 /* exception entries a decoder will look at in one chunk */
#define BXR_BLOB_MAX 24576 /* shared-memory slot per chunk blob */
#define BXR_WORDS_MAX ((BXR_BLOB_MAX - BXR_WORDS_AT - 16) / 2)
#define BXR_PROB_BITS 12
#define BXR_PROB_TOTAL 4096
#define BXR_STATE_LOW 65536u
#define BXR_ESCAPE 15
#define BXR_MODE_CODED 0
#define BXR_MODE_RAW 1 /* chunk blob = the 128x128 BF16 tile itself, already in UMMA operand order */
#define BXR_RAW_TILE_BYTES 32768
#define BXR_MODE_WINDOW 2 /* fixed 3-bit exponent codes inside an 8-binade row window; see below */

/* Window mode.  Same geometry, work items, blob index and raw-byte order as the coded mode, but the exponent of
 * a weight is a fixed 3-bit code: exponent = base[row] + code, base[row] in [0, 248].  A weight whose exponent
 * lies outside its row window carries code 0 and an entry in the chunk's list that says by how much the word the
 * decoder produced is off.  No entropy coder: no slot table, no stream states, no word segments; a decoder lane
 * needs only masks, multiply-adds and byte permutes, and any lane of a warp can patch any of the warp's weights.
 *
 * A lane (phase q, row r) owns the 32 chunk columns [32q, 32q+32) of its row = 16 column pairs.  Its codes are
 * three 32-bit words A, B, C (codes[j][q*128 + r], j = 0..2).  Word j holds pairs 5j..5j+4: pair 5j+k has the code
 * of its even column in bits [1+3k, 4+3k) and the code of its odd column 16 bits higher, so that one mask and one
 * multiply put both into packed-BF16 exponent position (bits 7..9 and 23..25).  Pair 15 is spread over the spare
 * bits: bit 0 of A, B, C = bits 0, 1, 2 of the even column's code, bit 16 of A, B, C likewise for the odd column.
 *
 * Chunk blob in window mode (multiple of 16 bytes, at most BXR_BLOB_MAX):
 *   [0,34)        u16 warp_end[17]     entries of decoder warp w = [warp_end[w], warp_end[w+1]); warp w covers
 *                                      phase w/4, rows 32*(w%4) .. +31
 *   [34,36)       u16 n_far
 *   [64,16448)    u8  raw[8][128][16]  as in the coded mode
 *   [16448,22592) u32 codes[3][512]
 *   [22592, ...)  u16 entries          place[0,11) | delta[11,16).  place = where the weight's BF16 word sits in
 *                                      the warp's 32 rows x 128 bytes of the operand tile, in 2-byte units:
 *                                      row in warp * 64 + (16-byte unit ^ (row & 7)) * 8 + column & 7, with
 *                                      unit = (q & 1) * 4 + (column in the lane's 32) / 8.  delta = true exponent
 *                                      - base[row] as a 5-bit two's complement number (-15..-1 or 8..15); the
 *                                      patch adds delta << 7 to the word.  delta = -16: see the far list
 *   then, 4-byte aligned: u32 far[n_far] = warp << 11 | place, exponent << 16
 */
#define BXW_WARP_END_AT 0
#define BXW_FAR_COUNT_AT 34
#define BXW_RAW_AT 64
#define BXW_CODES_AT (BXW_RAW_AT + BXR_RAW_BYTES)
#define BXW_LIST_AT (BXW_CODES_AT + 3 * 4 * BXR_SEGMENTS)
#define BXW_FAR_MAX 64
#define BXW_ENTRY_MAX ((BXR_BLOB_MAX - BXW_LIST_AT - 4 * BXW_FAR_MAX - 16) / 2)
#define BXW_PAIR_MASK 0x03800380u
#define BXW_PLACE_BITS 11
#define BXW_DELTA_FAR (-16)
#define BXW_BASE_MAX 248

/* Wide-window mode.  As the window mode, with 4-bit codes: exponent = base[row] + code over a 16-binade window
 * (base in [0, 240]).  On Gaussian rows fewer than one weight in ten thousand falls outside, so exceptions are a rare
 * slow path, the decoder has no per-chunk patching to do, and the decoded words can stay in registers until they are
 * written to tensor memory.  12 bits per weight.
 *
 * A lane (phase q, row r) owns the 32 chunk columns [32q, 32q+32) of its row = 16 column pairs; its codes are four
 * 32-bit words (codes[j][q*128 + r], j = 0..3).  Word j holds pairs 4j..4j+3: pair 4j+k has the code of its even
 * column in bits [4k, 4k+4) and the code of its odd column 16 bits higher.
 *
 * Chunk blob in wide-window mode (multiple of 16 bytes, at most BXQ_BLOB_MAX):
 *   [0,34)        u16 warp_end[17]     entries of decoder warp w = [warp_end[w], warp_end[w+1]); warp w covers phase
 *                                      w/4, rows 32*(w%4) .. +31, one lane per row
 *   [64,16448)    u8  raw[8][128][16]  as in the coded mode
 *   [16448,24640) u32 codes[4][512]
 *   [24640, ...)  u32 entries          column in the lane's 32 [0,5) | lane [5,10) | true exponent [16,24); the
 *                                      weight carries code 0
 */
#define BXR_MODE_WINDOW4 3
#define BXQ_WARP_END_AT 0
#define BXQ_RAW_AT 64
#define BXQ_CODES_AT (BXQ_RAW_AT + BXR_RAW_BYTES)
#define BXQ_LIST_AT (BXQ_CODES_AT + 4 * 4 * BXR_SEGMENTS)
#define BXQ_BLOB_MAX 25600 /* shared-memory slot per chunk blob in this mode */
#define BXQ_ENTRY_MAX ((BXQ_BLOB_MAX - BXQ_LIST_AT - 16) / 4)
#define BXQ_PAIR_MASK 0x000F000Fu
#define BXQ_BASE_MAX 240

/* Slot record of the pair table, 32 bits: n0[0,4) | bias[4,16) | n1[16,20) | freq[20,32).  freq <= 4095.
 * (record & 0x000F000F) * 128 is the pair of relative exponents in packed-BF16 position (an exception nibble is
 * stored as 0), freq is the top field, bias = (record >> 4) & 0xFFF. */
#define BXR_LUT_NIBBLES 0x000F000Fu
#define BXR_REC_FREQ(rec) ((rec) >> 20)
#define BXR_REC_BIAS(rec) (((rec) >> 4) & 0xFFFu)
#define BXR_REC_N0(rec) ((rec) & 15u)
#define BXR_REC_N1(rec) (((rec) >> 16) & 15u)

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
  uint32_t blob_stride16;         /* nonzero: every blob has this size (16-byte units) and blob b starts at b * size */
  uint32_t layout_version;        /* BXR_LAYOUT_VERSION of the builder */
  uint32_t reserved0;
  uint64_t lut_at;                /* u32[4096] slot records (absent in raw mode) */
  uint64_t base_at;               /* u8[row_blocks*128] exponent base per row */
  uint64_t items_at;              /* bxr_item[items] */
  uint64_t worker_items_at;       /* u32[workers+1]: items of worker w are [v[w], v[w+1]) */
  uint64_t states_at;             /* u32[items][1024] start state of every stream */
  uint64_t blob_index_at;         /* u32[row_blocks*chunks+1] blob offsets in 16-byte units from blobs_at */
  uint64_t blobs_at;
  uint64_t total_bytes;
  uint64_t coded_bytes;           /* blobs + states + index: what one pass of the kernel streams */
  uint8_t source_sha256[32];      /* digest of the little-endian source words, as in the BCTX header */
} bxr_header;
