/*
 * jointqk_b200 -- C ABI of the compress-then-attend key path for NVIDIA B200 (sm_100a).
 *
 * The reference (Amir-zsh/JointQK) is pure Python/PyTorch and has no FFI; each entry point
 * below names the reference function whose work it takes over, by path inside that project.
 *
 * Conventions
 *   - every function returns 0 on success, a negative JQK_E_* code for a rejected argument
 *     and a positive cudaError_t value when a CUDA call failed; jqk_last_error() returns a
 *     thread-local human-readable message for the last non-zero return on this thread;
 *   - every pointer except `tables` (a host struct of device pointers), and where marked
 *     "host", is a device pointer on the current device; buffers are borrowed for the
 *     duration of the call (asynchronous on `stream`), nothing is allocated or freed;
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream;
 *   - the library keeps no mutable global state except what is documented per function.
 *
 * Paged storage (new in this build; the reference stores dequantised floats)
 *   - a page holds JQK_PAGE_TOKENS consecutive keys of one sequence for all kv heads;
 *   - K pool:  uint32 [n_pages][n_kv_heads][words_per_record][16]; word w of key t of head h
 *     in page p is k_pool[((p*H + h)*words_per_record + w)*16 + t];
 *   - V pool:  bf16   [n_pages][n_kv_heads][d][16], dims-major inside a (page, head) block: the value
 *     of key slot t, dim i sits at element i*16 + (((t>>3) ^ ((i>>2)&1)) << 3) + (t&7) of the block
 *     (a 16-dim x 16-key tile is one ldmatrix of the decode kernel; the two 8-key halves of a row
 *     are swapped on dims 4..7 mod 8 to spread shared-memory banks);
 *   - page_table: int32 [n_seqs][page_table_stride], logical page -> physical page.
 */
#ifndef JOINTQK_B200_H_
#define JOINTQK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JQK_PAGE_TOKENS 16
#define JQK_MAX_DIM 128        /* head_dim: multiple of 16, at most 128 */
#define JQK_MAX_COLS 128       /* coordinates that carry >0 bits, padded to 16 */
#define JQK_MAX_WORDS 16       /* uint32 words per record */
#define JQK_MAX_WIDE 32        /* columns of 5..8 bits per head */
#define JQK_MAX_VALUE_WIDE_LEVELS 6144 /* sum of 2^width over a head's wide columns that packed-VALUE decode holds */
#define JQK_MAX_TABLES 208     /* lookups per record (see jqk_head_tables.table_fields) */
#define JQK_DESC_INTS 32       /* int32 per head in jqk_head_tables.desc */
#define JQK_MAX_GROUP 4        /* q heads scored together by one thread block */

#define JQK_DTYPE_F32 0
#define JQK_DTYPE_BF16 1
#define JQK_DTYPE_F16 2

#define JQK_E_ARG (-1)         /* null pointer, bad size or stride */
#define JQK_E_LAYOUT (-2)      /* head tables inconsistent with the call */
#define JQK_E_UNSUPPORTED (-3) /* shape outside what the kernels implement */
#define JQK_E_WORKSPACE (-4)   /* workspace too small */

/* Bits of the device status word (int32, OR-ed by kernels, never cleared by them). */
#define JQK_STATUS_BAD_PAGE 1      /* page index outside [0, n_pages) - access skipped */
#define JQK_STATUS_WAIT_EXPIRED 2  /* a bounded wait on an mbarrier gave up */
#define JQK_STATUS_BAD_LENGTH 4    /* a length reaches past what the call was sized for (a context longer
                                      than max_seq_len, a token range past the page-table row): the
                                      excess is ignored */

/*
 * Per-head device tables built on the host from a fitted compressor
 * (reference object: PerCoordCompressor, experiments/stage1/toolkit/per_coord_quantization.py:43-121;
 * fields derive from its bits_int, forward_map, inverse_map and codebooks_padded).
 * "Column" c is the c-th coordinate with >0 bits in ascending record bit position.
 *
 *   desc          int32 [H][JQK_DESC_INTS]: d, n_cols, n_active, n_words, n_a_words, n_c_words,
 *                 n_tables, payload_bits, then word_col_begin[0..n_words] at offset 8
 *   col_meta      int32 [H][128]: width | bitpos << 4 | coord << 16 for column c (width 0 and
 *                 coord 255 = padding column)
 *   table_fields  int32 [H][JQK_MAX_TABLES][4]: col | width << 8 | shift << 12, or -1
 *   fwd_cols      float [H][d][128]: forward_map[i][coord(c)]
 *   thresholds    float [H][128][16]: code = #{l < 15 : x >= thresholds[c][l]} (+inf padded)
 *   cb_cols       float [H][128][16]: codebooks_padded[coord(c)][l], 0 beyond the last level
 *   qproj_cols    float [H][d][128]: inverse_map[coord(c)][i] (query projection)
 *   inv_rows      float [H][128][d]: inverse_map[coord(c)][i] (reconstruction)
 *   fwd_limbs     bf16  [H][3][128][d]: three-way bf16 split of fwd_cols with column c scaled by
 *                 1 / sigma of its coordinate, column-major (limb l, column c, dim i), for the
 *                 tensor-core transform, whose values are then quantised against the unit Lloyd-Max
 *                 levels of the column's width; may be NULL (the CUDA-core kernel runs)
 *   center        float [H][d] or NULL: a mean that is subtracted from every input row before the
 *                 transform and added back after reconstruction (the reference's CenteredCompressor,
 *                 experiments/stage1/toolkit/v_compressor_adapter.py:46-72, used on the value side);
 *   center_cols   float [H][128] or NULL: center @ (the scaled basis that fwd_limbs holds), column c;
 *                 with it the tensor-core compress kernel serves centred tables as well (it
 *                 transforms the raw rows and subtracts this constant from every column)
 *   wide_thr / wide_cb  float [H][JQK_MAX_WIDE][256] or NULL: decision thresholds (+inf padded) and levels
 *                 of the columns that carry 5..8 bits (what the reference's cap of 8 gives outlier
 *                 channels, per_coord_quantization.py:365-379); such a column takes one byte of the
 *                 record, its rows here are indexed by column - desc[30] (desc[31] = how many).  They
 *                 are written, read back and reconstructed by jqk_compress_paged / jqk_decompress_paged
 *                 / jqk_unpack_codes on the CUDA cores.  The score and decode entry points give a wide
 *                 column of w bits a lookup table of 2^w entries (2^(w-4) of the JQK_MAX_TABLES slots of
 *                 16 entries, behind the 16-entry tables; desc n_tables counts them all); tables whose
 *                 lookups do not fit the slots have decodable = 0 and get JQK_E_UNSUPPORTED there.  As
 *                 packed-VALUE tables (jqk_decode_attend_packed_values) the levels of a head's wide
 *                 columns are held as they are, JQK_MAX_VALUE_WIDE_LEVELS entries at most
 *                 (value_decodable)
 *   unit_wide_thr float [4][256] or NULL: unit decision thresholds of the widths 5..8 (+inf padded); with it
 *                 (and fwd_limbs) the tensor-core compress kernel serves tables with wide columns: a wide
 *                 column's code is found by binary search over the row of its width
 *   unit_pre      uint8 [4][128], unit_thr float [4][16] (HOST values, +inf padded), unit_aff float [2]
 *                 (HOST): the shared coarse-to-exact quantiser of the tensor-core kernel for widths
 *                 1..4: cell = low 7 bits of clamp(x * aff[0] + aff[1]) (aff[1] includes 2^23),
 *                 j = unit_pre[w-1][cell], code = (j & 15) + (x >= unit_thr flattened [j])
 */
typedef struct jqk_head_tables {
  int32_t n_heads;
  int32_t d;
  int32_t words_per_record; /* K pool stride in words: max n_words over the heads */
  int32_t n_wide;           /* largest number of 5..8-bit columns of a head (0: every code has at most 4 bits) */
  const int32_t* desc;
  const int32_t* col_meta;
  const int32_t* table_fields;
  const float* fwd_cols;
  const float* thresholds;
  const float* cb_cols;
  const float* qproj_cols;
  const float* inv_rows;
  const uint16_t* fwd_limbs;
  const uint8_t* unit_pre;
  const float* center;
  const float* center_cols;
  float unit_thr[64];
  float unit_aff[2];
  const float* wide_thr;
  const float* wide_cb;
  const float* unit_wide_thr;
  int32_t decodable;        /* every head's lookup tables fit the decode kernels' table memory (JQK_MAX_TABLES slots) */
  int32_t value_decodable;  /* as VALUE tables: the levels of every head's wide columns fit (JQK_MAX_VALUE_WIDE_LEVELS) */
} jqk_head_tables;

/* Library version: major << 16 | minor.  The minor number changes whenever struct jqk_head_tables or
 * an entry point's arguments change; a binding compares it, and the struct's size, with its own. */
#define JQK_VERSION ((0 << 16) | 2)
int32_t jqk_version(void);
/* sizeof(struct jqk_head_tables) as the library was built. */
size_t jqk_head_tables_bytes(void);

/* Message for the last non-zero return on the calling thread ("" if none). */
const char* jqk_last_error(void);

/*
 * Prefill compression: basis transform, per-coordinate nearest-centroid quantisation and
 * bit-packing into pages.  Replaces the forward half of PerCoordCompressor.roundtrip
 * (per_coord_quantization.py:132-157) for all heads of a layer, i.e. the per-head loop of
 * JointQKPress._quantize_layer (experiments/stage1/toolkit/jointqk_press.py:253-256).
 *
 *   keys        [n_seqs][H][*][d] of key_dtype with element strides (seq, head, token); d contiguous
 *   n_tokens    int32 [n_seqs] keys to compress per sequence in this call
 *   seq_starts  int32 [n_seqs] position in the sequence of keys[...][0] (NULL = 0); the
 *               destination of key t is slot (seq_starts+t) % 16 of logical page (seq_starts+t)/16
 *   max_tokens  largest n_tokens[] value (host), sizes the grid
 *   status      int32 device word, see JQK_STATUS_*
 * The tensor-core kernel (bf16 keys, head_dim 128) is launched as a programmatic dependent: its
 * set-up reads the tables' arrays while the previous kernel on the stream may still run, so that
 * kernel must not be the one that writes them (tables are written once, by copies from the host).
 */
int32_t jqk_compress_paged(const jqk_head_tables* tables, const void* keys, int32_t key_dtype,
                           int64_t seq_stride, int64_t head_stride, int64_t token_stride,
                           int32_t n_seqs, const int32_t* n_tokens, const int32_t* seq_starts,
                           int32_t max_tokens, const int32_t* page_table,
                           int32_t page_table_stride, int32_t n_pages, uint32_t* k_pool,
                           int32_t* status, void* stream);

/*
 * Values into pages: transposes rows [token][dim] into the V pool's (page, head) blocks (layout at the
 * top of this file), converting to bf16.  The reference leaves values in the HF cache and appends the
 * newest token each step (experiments/stage1/toolkit/jointqk_press.py:298-307); this is that append
 * for the paged pool, used by prefill and by every decode step.
 *   values      [n_seqs][n_kv_heads][*][d] of dtype with element strides (seq, head, token); d contiguous
 *   n_tokens, seq_starts, max_tokens, page_table: as in jqk_compress_paged; slots outside
 *               [seq_starts, seq_starts + n_tokens) of a page keep their contents
 *   v_pool      bf16 [n_pages][n_kv_heads][d][16]
 */
int32_t jqk_store_values_paged(const void* values, int32_t dtype, int64_t seq_stride, int64_t head_stride,
                               int64_t token_stride, int32_t n_seqs, int32_t n_kv_heads, int32_t d,
                               const int32_t* n_tokens, const int32_t* seq_starts, int32_t max_tokens,
                               const int32_t* page_table, int32_t page_table_stride, int32_t n_pages,
                               void* v_pool, int32_t* status, void* stream);

/*
 * Reconstruction from pages: unpack, centroid lookup, inverse map.  Replaces the second half
 * of PerCoordCompressor.roundtrip (per_coord_quantization.py:158-164).
 *   seq_starts  int32 [n_seqs] position in the sequence of the first key to reconstruct (NULL = 0);
 *               row t of the output is key seq_starts + t
 *   out  float [n_seqs][H][max_tokens][d] (contiguous); rows beyond n_tokens[s] are not written
 */
int32_t jqk_decompress_paged(const jqk_head_tables* tables, int32_t n_seqs,
                             const int32_t* n_tokens, const int32_t* seq_starts, int32_t max_tokens,
                             const int32_t* page_table, int32_t page_table_stride,
                             int32_t n_pages, const uint32_t* k_pool, float* out,
                             int32_t* status, void* stream);

/*
 * Integer codes in coordinate order (0 for coordinates with 0 bits).  The reference never
 * returns its argmin indices (per_coord_quantization.py:156-160); this exposes them for
 * bit-exact parity checks.
 *   codes  uint8 [n_seqs][H][max_tokens][d]
 */
int32_t jqk_unpack_codes(const jqk_head_tables* tables, int32_t n_seqs, const int32_t* n_tokens,
                         int32_t max_tokens, const int32_t* page_table,
                         int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                         uint8_t* codes, int32_t* status, void* stream);

/*
 * Round trip without a packed record, for allocations the record does not hold (more than
 * JQK_MAX_WIDE coordinates above 4 bits, or more than 32 * JQK_MAX_WORDS bits per key: what the
 * reference's default cap of 8 gives from budgets of about 3.5 bits per coordinate on).  Replaces
 * PerCoordCompressor.roundtrip (experiments/stage1/toolkit/per_coord_quantization.py:123-165) and,
 * with `center`, CenteredCompressor.roundtrip (v_compressor_adapter.py:64-72) for such objects:
 * x = (row - center) @ forward_map, code_j = #{l : x_j >= thresholds[j][l]}, x_hat_j =
 * levels[j][code_j], out = x_hat @ inverse_map + center.
 *   forward_maps / inverse_maps  float [H][d][d] row-major
 *   thresholds  float [H][d][255] exact fp32 decision thresholds of coordinate j, +inf padded
 *   levels      float [H][d][256] its levels (codebooks_padded row), 0 beyond the last
 *   widths      int32 [H][d]      bits of coordinate j, 0..8
 *   rows        [H][n_tokens][d] of `dtype` with the given strides in elements
 *   out         float [H][n_tokens][d] or NULL;  codes  uint8 [H][n_tokens][d] or NULL
 */
int32_t jqk_roundtrip_dense(const float* forward_maps, const float* inverse_maps, const float* thresholds,
                            const float* levels, const int32_t* widths, const float* center,
                            int32_t n_heads, int32_t d, const void* rows, int32_t dtype,
                            int64_t head_stride, int64_t token_stride, int64_t n_tokens, float* out,
                            uint8_t* codes, void* stream);

/*
 * Attention logits of queries against packed keys, q . k_hat / sqrt(d).  Replaces compute_attention_metrics' candidate logits
 * (experiments/stage1/toolkit/eval.py:21) with GQA grouping as in repeat_kv_states
 * (experiments/stage1/toolkit/metric_transform.py:21-27).
 *   table_mode 0: fp32 sum over coordinates of q'_c * codebook[c][code] (evaluation, top-1 metrics);
 *              1: the decode kernel's 16-bit fixed-point lookup tables (what decode attention scores with)
 *   q       [n_seqs][n_q_heads][n_queries][d] of q_dtype, contiguous
 *   scores  float [n_seqs][n_q_heads][n_queries][max_tokens]; entries beyond seq_lens[s] untouched
 */
int32_t jqk_score_paged(const jqk_head_tables* tables, int32_t table_mode, const void* q, int32_t q_dtype,
                        int32_t n_seqs, int32_t n_q_heads, int32_t n_queries,
                        const int32_t* seq_lens, int32_t max_tokens, const int32_t* page_table,
                        int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                        float* scores, int32_t* status, void* stream);

/*
 * Bytes of zero-initialised workspace jqk_decode_attend needs.  The caller zeroes it once;
 * the kernel leaves its counters at zero when it finishes, so the same buffer can be passed
 * to the next call on the same stream without clearing.
 */
size_t jqk_decode_workspace_bytes(int32_t n_seqs, int32_t n_q_heads, int32_t n_kv_heads,
                                  int32_t max_splits);

/*
 * One decode step of attention over packed keys and bf16 values for one layer:
 * out = softmax(q . k_hat / sqrt(d)) @ V.  In the reference this is stock attention over the
 * reconstructed cache (jointqk_press.py:306-307 swaps it in); the scores follow eval.py:20-21.
 *   q                bf16 [n_seqs][n_q_heads][d]
 *   seq_lens         int32 [n_seqs] context length per sequence (0 allowed: output zeros)
 *   max_seq_len      largest seq_lens[] value (host)
 *   tokens_per_split keys handled by one thread block (multiple of 32; 0 = choose)
 *   out              [n_seqs][n_q_heads][d] of out_dtype (JQK_DTYPE_F32 or JQK_DTYPE_BF16)
 *   workspace        from jqk_decode_workspace_bytes with max_splits >= ceil(max_seq_len/tokens_per_split)
 */
int32_t jqk_decode_attend(const jqk_head_tables* tables, const void* q, int32_t n_seqs,
                          int32_t n_q_heads, const int32_t* seq_lens, int32_t max_seq_len,
                          int32_t tokens_per_split, const int32_t* page_table,
                          int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                          const void* v_pool, void* out, int32_t out_dtype, void* workspace,
                          size_t workspace_bytes, int32_t* status, void* stream);

/*
 * One step of a generate loop in one launch: append the newest token of every sequence, attend,
 * advance the lengths.  Replaces the reference's Mode-B step, which compresses the new key into the
 * cache entry (experiments/stage1/toolkit/jointqk_press.py:298-304) and then runs stock attention,
 * and does the work of jqk_compress_paged + jqk_store_values_paged + jqk_decode_attend for that
 * token in a single kernel:
 *   - new_k / new_v: one row of d elements per (sequence, kv head), element (s, h, i) at
 *     s * seq_stride + h * head_stride + i (strides in elements), dtypes k_dtype / v_dtype
 *     (JQK_DTYPE_*);
 *   - the row of sequence s goes to position seq_lens[s]; its page must already be in page_table;
 *     the key's codes are bit-identical to those jqk_compress_paged writes for the same row;
 *   - the step attends over seq_lens[s] + 1 keys; max_seq_len (grid and workspace sizing) must
 *     cover that;
 *   - when the launch is done seq_lens[s] has been advanced by one for every sequence, so the call
 *     can be replayed from a CUDA graph without host work in between.
 *   - flags: JQK_APPEND_OWN_KEY_EXACT scores the appended key from its exact values in this step
 *     and from its codes in every later one, which is what the reference's Mode B does (its hook
 *     compresses a decode key after the attention of the step that produced it); without the flag
 *     the new key is scored from its codes like every other key.
 * bf16 value pool only (no packed values); tables without a centre.  Everything else as in
 * jqk_decode_attend.
 */
#define JQK_APPEND_OWN_KEY_EXACT 1
int32_t jqk_decode_append_attend(const jqk_head_tables* tables, const void* q, const void* new_k,
                                 const void* new_v, int32_t k_dtype, int32_t v_dtype, int64_t k_seq_stride,
                                 int64_t k_head_stride, int64_t v_seq_stride, int64_t v_head_stride,
                                 int32_t n_seqs, int32_t n_q_heads, int32_t* seq_lens, int32_t max_seq_len,
                                 int32_t tokens_per_split, const int32_t* page_table,
                                 int32_t page_table_stride, int32_t n_pages, uint32_t* k_pool, void* v_pool,
                                 void* out, int32_t out_dtype, int32_t flags, void* workspace,
                                 size_t workspace_bytes, int32_t* status, void* stream);

/*
 * jqk_decode_append_attend with the values stored as packed codes (see
 * jqk_decode_attend_packed_values): the new value row has its mean subtracted in fp32 and is
 * compressed through `v_tables` exactly as jqk_compress_paged would, into `v_code_pool`.  The flag
 * JQK_APPEND_OWN_KEY_EXACT applies to the key only; the new value is read from its codes.
 */
int32_t jqk_decode_append_attend_packed_values(
    const jqk_head_tables* tables, const jqk_head_tables* v_tables, const void* q, const void* new_k, const void* new_v,
    int32_t k_dtype, int32_t v_dtype, int64_t k_seq_stride, int64_t k_head_stride, int64_t v_seq_stride,
    int64_t v_head_stride, int32_t n_seqs, int32_t n_q_heads, int32_t* seq_lens, int32_t max_seq_len,
    int32_t tokens_per_split, const int32_t* page_table, int32_t page_table_stride, int32_t n_pages, uint32_t* k_pool,
    uint32_t* v_code_pool, void* out, int32_t out_dtype, int32_t flags, void* workspace, size_t workspace_bytes,
    int32_t* status, void* stream);

/*
 * jqk_decode_attend over packed values: the value pool holds codes of a second per-coordinate
 * compressor (`v_tables`, optionally centred) in the same paged record format as the keys, written
 * by jqk_compress_paged with those tables.  The kernel dequantises a tile of values into shared
 * memory (bf16 centroids), accumulates softmax-weighted sums in the value basis and applies the
 * value side's inverse map and mean once per query head at the end:
 * out = (sum_t p_t x_hat_t) @ inverse_map_v + mu_v.  In the reference the same result comes from stock
 * attention over values reconstructed by the V-side compressor
 * (experiments/stage1/toolkit/v_compressor_adapter.py:46-72,165-226; jointqk_press.py:262-266).
 *   v_code_pool  uint32 [n_pages][n_kv_heads][v_tables->words_per_record][16]
 * Everything else as in jqk_decode_attend (same workspace size).
 */
int32_t jqk_decode_attend_packed_values(const jqk_head_tables* tables, const jqk_head_tables* v_tables,
                                        const void* q, int32_t n_seqs, int32_t n_q_heads,
                                        const int32_t* seq_lens, int32_t max_seq_len, int32_t tokens_per_split,
                                        const int32_t* page_table, int32_t page_table_stride, int32_t n_pages,
                                        const uint32_t* k_pool, const uint32_t* v_code_pool, void* out,
                                        int32_t out_dtype, void* workspace, size_t workspace_bytes,
                                        int32_t* status, void* stream);

/*
 * jqk_decode_attend from host memory, one call per decode step (no counterpart in the reference,
 * whose attention inputs are device tensors of the model): copies the query from `q_host` to the
 * device, runs the step, copies the result to `out_host` and waits for it, all on `stream`.
 *   q_host     bf16 [n_seqs][n_q_heads][d] anywhere in host memory
 *   q_pinned   page-locked host staging of the same size (the query is copied there first, so the
 *              transfer is asynchronous); may equal q_host if that is page-locked already
 *   q_dev      device staging for the query, same size
 *   out_dev    device staging for the result, [n_seqs][n_q_heads][d] of out_dtype
 *              either may be NULL (page-locked host memory is device-addressable): without q_dev the
 *              blocks read the query from q_pinned themselves, without out_dev the block that finishes a
 *              head writes its result into out_host itself, and the matching copy command is not issued
 *   out_host   page-locked host memory of the same size; valid when the call returns
 * Everything else as in jqk_decode_attend.  h2d / d2h bytes per call: the sizes of q and out.
 */
int32_t jqk_decode_attend_host(const jqk_head_tables* tables, const void* q_host, void* q_pinned, void* q_dev,
                               int32_t n_seqs, int32_t n_q_heads, const int32_t* seq_lens, int32_t max_seq_len,
                               int32_t tokens_per_split, const int32_t* page_table, int32_t page_table_stride,
                               int32_t n_pages, const uint32_t* k_pool, const void* v_pool, void* out_dev,
                               void* out_host, int32_t out_dtype, void* workspace, size_t workspace_bytes,
                               int32_t* status, void* stream);

/*
 * jqk_decode_attend for callers that must not allocate (no counterpart in the reference, which
 * leaves all memory to torch).  Some hosts of this library cannot call cudaMalloc on the decode
 * path at all: a serving engine that has handed every byte of device memory to its own pool at
 * start-up, a plugin that runs inside another process's memory budget, code that runs while an
 * allocator lock is held.  For them the split-key scratch is a fixed array inside the library,
 * JQK_DECODE_STATIC_SCRATCH_BYTES per device, held from the moment the library is loaded on a
 * device until the process exits.  Inputs and outputs are still the caller's.
 *
 *   - a call whose splits need more than the array (see jqk_decode_workspace_bytes) is rejected
 *     with JQK_E_WORKSPACE and a message that says how much was needed;
 *   - no cudaMalloc / cudaFree / allocating library routine is called, ever;
 *   - the first call on a device looks up the array's device address and zeroes its ticket area
 *     on `stream`; make that first call outside any stream capture;
 *   - all calls on a device share the one array: two calls that overlap on the GPU (different
 *     streams, or graphs replayed concurrently) race on it and produce garbage.  Calls that are
 *     ordered on one stream are safe; each launch leaves the tickets at zero for the next.
 * Arguments are those of jqk_decode_attend without workspace / workspace_bytes.
 */
#define JQK_DECODE_STATIC_SCRATCH_BYTES (8 * 1024 * 1024)
int32_t jqk_decode_attend_static(const jqk_head_tables* tables, const void* q, int32_t n_seqs,
                                 int32_t n_q_heads, const int32_t* seq_lens, int32_t max_seq_len,
                                 int32_t tokens_per_split, const int32_t* page_table,
                                 int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                                 const void* v_pool, void* out, int32_t out_dtype, int32_t* status,
                                 void* stream);

/*
 * Self-test of the library's bounded device-side wait (no counterpart in the reference): one warp
 * waits, with the same routine every kernel here uses, on an mbarrier that nothing completes.
 * After `limit_us` microseconds the wait gives up, the kernel ORs JQK_STATUS_WAIT_EXPIRED into
 * `status` (device int32) and returns normally; the context stays usable.  limit_us in 1..100000.
 */
int32_t jqk_selftest_bounded_wait(int32_t limit_us, int32_t* status, void* stream);

/* tokens_per_split that jqk_decode_attend would choose for this shape (host helper): every
 * sequence is taken to be max_seq_len long. */
int32_t jqk_decode_default_split(int32_t n_seqs, int32_t n_q_heads, int32_t n_kv_heads,
                                 int32_t max_seq_len);

/* The same choice for a batch whose context lengths the host knows (host_seq_lens is HOST memory,
 * int32 [n_seqs]): the block count is fitted to whole waves of one block per SM.  Pass the result
 * as tokens_per_split. */
int32_t jqk_decode_split_for_lengths(const int32_t* host_seq_lens, int32_t n_seqs, int32_t n_q_heads,
                                     int32_t n_kv_heads);

/*
 * Calibration moments: accumulates (+=) the per-kv-head sums over tokens
 *   sq_sum  += sum_g sum_t q_g q_g^T      (pooled over the q heads of the group)
 *   sk_sum  += sum_t k k^T
 *   cqk_sum += sum_t mean_g(q_g) k^T
 * for one layer.  Replaces the einsums of compute_moments_from_tensors
 * (experiments/stage1/calibration/compute_stats.py:118-123) and of the streaming
 * accumulators (experiments/stage1/toolkit/moments.py:68,110).
 *   q  [n_q_heads][n_tokens][d], k [n_kv_heads][n_tokens][d] of dtype (bf16, f16 or f32); tokens are
 *      d elements apart, heads q_head_stride / k_head_stride elements apart
 *   sq_sum, sk_sum, cqk_sum  float [n_kv_heads][d][d]; any of them may be NULL to skip it
 *   q_sum, k_sum  float [n_kv_heads][d]: first moments from the same pass, += sum_g sum_t q_g and
 *      += sum_t k (compute_stats.py:125-126; the value moments sv_sum / sum_v of :124,127 come from a
 *      call with the values as `k`); NULL to skip
 *   max_chain_tokens  bound on the length of one fp32 running sum inside the tensor core (0 = the
 *      default, 2048 tokens).  The tensor core truncates when it accumulates, so the relative error of
 *      a sum grows with the chain (about 2e-5 at 2048 tokens, 4e-6 at 512); shorter chains are more
 *      accurate and somewhat slower (more, smaller blocks)
 *   workspace / workspace_bytes: scratch from jqk_moments_workspace_bytes; its first int32 is a
 *      device status word (JQK_STATUS_*), OR-ed by the kernel, zeroed by the caller; may be NULL
 */
int32_t jqk_moments_accumulate(const void* q, const void* k, int32_t dtype, int64_t n_tokens,
                               int64_t q_head_stride, int64_t k_head_stride, int32_t n_q_heads, int32_t n_kv_heads, int32_t d, float* sq_sum,
                               float* sk_sum, float* cqk_sum, float* q_sum, float* k_sum,
                               int32_t max_chain_tokens, void* workspace,
                               size_t workspace_bytes, void* stream);

size_t jqk_moments_workspace_bytes(int64_t n_tokens, int32_t n_q_heads, int32_t n_kv_heads,
                                   int32_t d);

#ifdef __cplusplus
}
#endif
#endif /* JOINTQK_B200_H_ */
