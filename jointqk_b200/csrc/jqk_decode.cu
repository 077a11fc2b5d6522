// Scoring of packed keys through shared-memory lookup tables, and paged decode attention.
//
// Reference semantics: logits = q . k_hat / sqrt(d) (experiments/stage1/toolkit/eval.py:20-21)
// with the GQA grouping of metric_transform.py:21-27, then softmax and a product with V.  The
// reference runs stock attention over a reconstructed fp16/bf16 cache
// (experiments/stage1/toolkit/jointqk_press.py:306-307); here no key is ever dequantised.
//
// Decode kernel, one thread block per (key split, kv head x q-head block, sequence), one block per SM:
//   * prologue: project the <=4 queries of the group and build the lookup tables (jqk_tables.cuh),
//     or copy the tables a table kernel built once per group when the grid is larger than one
//     wave.  The global reads of the build are the first thing a block issues; the pages of its
//     first tiles are in flight while the tables are built;
//   * each warp owns a contiguous run of 32-key tiles and stages their pages itself: lane 0 issues
//     cp.async.bulk copies (K: two tiles deep, V: one) that complete on the warp's own mbarriers.
//     A lane scores one key: per record word one shared-memory read of the word, then one 8-byte
//     table read per lookup (16-entry tables of 128 bytes: no bank conflicts), accumulated as
//     packed 16-bit integer sums;
//   * online softmax per warp, branch-free (integer tile maximum by one warp reduction per head;
//     the sum of the weights stays per lane until the end); P is split into two bf16 terms
//     (hi + lo) so that the weights keep fp32-level accuracy;
//   * P.V on the tensor cores as out^T[dims x heads] += V^T[dims x keys] . P^T[keys x heads] with
//     mma.sync m16n8k16 (four query heads do not fill a tcgen05 tile): columns 0..3 carry the hi
//     terms of the four heads and 4..7 the lo terms.  V pages are stored dims-major and swizzled
//     in HBM (see the V layout in include/jointqk_b200.h), so one ldmatrix.x4 yields the A
//     fragment of 16 dims x 16 keys;
//   * the partial results of the splits are merged by the last block of the group to finish
//     (atomic ticket), with one memory round trip, no second launch.
// Every wait on a copy is bounded; an expired wait sets JQK_STATUS_WAIT_EXPIRED and skips the tile.
#include <limits.h>
#include <string.h>

#include <atomic>
#include <type_traits>
#include <mutex>

#include "jqk_sm100.cuh"
#include "jqk_tables.cuh"

namespace jqk {

constexpr int SCORE_THREADS = TBL_THREADS;
constexpr int TBL_BUILD_THREADS = 512;
constexpr int DEC_THREADS = 384;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int TILE_TOK = 32;        // keys per warp step (two pages)
constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------------------------------
// Score kernel (evaluation / parity): one block per (key chunk, kv head x q block, seq x query)
// ---------------------------------------------------------------------------------------
constexpr int SCORE_CHUNK = 2048;

__global__ void __launch_bounds__(SCORE_THREADS)
score_kernel(jqk_head_tables tb, int table_mode, const void* __restrict__ q, int q_dtype, int n_q_heads, int n_queries,
             const int32_t* __restrict__ seq_lens, int max_tokens, const int32_t* __restrict__ page_table,
             int pt_stride, int n_pages, const uint32_t* __restrict__ k_pool, float* __restrict__ scores,
             int32_t* status) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TableSmem& sm = *reinterpret_cast<TableSmem*>(smem_raw);
  const int group = n_q_heads / tb.n_heads;
  const int q_blocks = (group + JQK_MAX_GROUP - 1) / JQK_MAX_GROUP;
  const int head = blockIdx.y / q_blocks, qb = blockIdx.y % q_blocks;
  const int seq = blockIdx.z / n_queries, qi = blockIdx.z % n_queries;
  const int len = min(seq_lens[seq], max_tokens);
  const int t_begin = blockIdx.x * SCORE_CHUNK;
  if (t_begin >= len) return;
  const int t_end = min(len, t_begin + SCORE_CHUNK);
  const HeadDesc hd = load_desc(tb.desc, head);
  const int d = hd.d;
  const int g0 = qb * JQK_MAX_GROUP, n_group = min(JQK_MAX_GROUP, group - g0);
  const int qh0 = head * group + g0;
  const size_t q_elem0 = (((size_t)seq * n_q_heads + qh0) * n_queries + qi) * d;
  const char* q_ptr = (const char*)q + q_elem0 * (q_dtype == JQK_DTYPE_F32 ? 4 : 2);
  {
    if (tb.n_wide) {  // (the struct's count: the same in every block)
      const TableLoads ld = issue_table_loads<true>(tb, head, d, q_ptr, q_dtype, (size_t)n_queries * d, n_group);
      build_tables<true>(sm, hd, ld, tb.wide_cb + (size_t)head * JQK_MAX_WIDE * 256);
    } else {
      const TableLoads ld = issue_table_loads(tb, head, d, q_ptr, q_dtype, (size_t)n_queries * d, n_group);
      build_tables(sm, hd, ld);
    }
  }
  const float* wide_cb = hd.n_wide ? tb.wide_cb + (size_t)head * JQK_MAX_WIDE * 256 : nullptr;
  const float inv_sqrt_d = 1.0f / sqrtf((float)d);
  for (int tok = t_begin + threadIdx.x; tok < t_end; tok += blockDim.x) {
    const int page = lookup_page(page_table, pt_stride, seq, tok / JQK_PAGE_TOKENS, n_pages, status);
    if (page < 0) continue;
    const uint32_t* kp = k_pool + ((size_t)page * tb.n_heads + head) * tb.words_per_record * JQK_PAGE_TOKENS +
                         (tok % JQK_PAGE_TOKENS);
    float sv[JQK_MAX_GROUP];
    if (table_mode) {  // the decode kernel's fixed-point tables
      int acc[JQK_MAX_GROUP];
      auto word = [kp](int w) { return __ldg(kp + w * JQK_PAGE_TOKENS); };
      if (hd.n_wide)
        score_record<true>(word, TableView{sm.lut, sm.dshift, sm.bias, sm.woff}, hd.n_a_words, hd.n_c_words, hd.n_words, acc, hd.n_wide);
      else
        score_record<false>(word, TableView{sm.lut, sm.dshift, sm.bias}, hd.n_a_words, hd.n_c_words, hd.n_words, acc);
#pragma unroll
      for (int h = 0; h < JQK_MAX_GROUP; ++h) sv[h] = (float)acc[h] * sm.scale[h];
    } else {           // plain fp32: sum_c q'_c * cb[c][code_c], column after column
#pragma unroll
      for (int h = 0; h < JQK_MAX_GROUP; ++h) sv[h] = 0.f;
      const int32_t* meta = tb.col_meta + (size_t)head * 128;
      for (int c = 0; c < hd.n_active; ++c) {
        const int m = __ldg(meta + c);
        const int bp = (m >> 4) & 1023;
        const uint32_t word = __ldg(kp + (bp >> 5) * JQK_PAGE_TOKENS);
        const uint32_t code = (word >> (bp & 31)) & ((1u << (m & 15)) - 1u);
        const float x = (m & 15) > 4 ? __ldg(wide_cb + (size_t)(c - hd.wide_first) * 256 + code) : sm.cb[c * 16 + code];
        const float4 qp = *reinterpret_cast<const float4*>(sm.qproj[c]);
        sv[0] = fmaf(qp.x, x, sv[0]); sv[1] = fmaf(qp.y, x, sv[1]);
        sv[2] = fmaf(qp.z, x, sv[2]); sv[3] = fmaf(qp.w, x, sv[3]);
      }
    }
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) {
      if (h < n_group)
        scores[(((size_t)seq * n_q_heads + qh0 + h) * n_queries + qi) * max_tokens + tok] = sv[h] * inv_sqrt_d;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Decode attention
// ---------------------------------------------------------------------------------------
struct DecodeWs {
  TableRecord* tables;     // [n_seqs][n_kv_heads * q_blocks]
  float* part_m;           // [n_seqs][n_q_heads][max_splits]
  float* part_l;           // [n_seqs][n_q_heads][max_splits]
  float* part_acc;         // [n_seqs][n_q_heads][max_splits][128]
  unsigned int* counters;  // [n_seqs][n_kv_heads * q_blocks]
  int max_splits;
  unsigned int* grid_ticket;  // one counter for the whole launch (append variant: who advances the lengths)
  int late_wait;              // the kernel right before this one on the stream is this call's table kernel
};

// Per-warp staging of one tile: the two V pages (dims-major, see the V page layout in the file
// header) and the two K pages, filled by bulk asynchronous copies that the warp issues itself.
// With packed values (VQ) the copies bring the two pages of V codes into `vq` and the warp
// dequantises them into `v`, in the same dims-major layout (rows are then columns of the value
// basis), so the tensor-core product reads either kind the same way.
constexpr int K_STAGE_STRIDE = JQK_MAX_WORDS * JQK_PAGE_TOKENS * 4 + 64;  // +64 B: the two pages hit different banks
constexpr int V_PAGE_SMEM = JQK_PAGE_TOKENS * JQK_MAX_DIM * 2;            // 4096
template <bool VQ> struct TileStageT;
template <> struct alignas(128) TileStageT<false> {
  uint8_t v[2][V_PAGE_SMEM];         // the two V pages of the current tile, 2 x 4096 B
  uint8_t k[2][2][K_STAGE_STRIDE];   // the K pages of two tiles (double buffer), 4 x 1088 B
};
template <> struct alignas(128) TileStageT<true> {
  uint8_t v[2][V_PAGE_SMEM + 64];    // dequantised values of the current tile (+64 B: a lane-per-key store
                                     // of one column touches both pages, which must not share banks)
  uint8_t k[2][2][K_STAGE_STRIDE];
  uint8_t vq[2][K_STAGE_STRIDE];     // the two pages of V codes of the current tile
};

constexpr int VQ_WIDE_ENTRIES = JQK_MAX_VALUE_WIDE_LEVELS;
static_assert(VQ_WIDE_ENTRIES >= JQK_MAX_COLS * 16, "the lane-interleaved level words of the narrow form use the wide levels' room");   // levels of all byte-wide value columns of a head that the block can hold
template <bool VQ> struct DecodeSmemT;
template <> struct DecodeSmemT<false> {
  union {            // the tables this block scores with:
    TableRecord rec;   //   a copy of the table kernel's record, or
    TableSmem build;   //   tables built by the block itself (few blocks: latency matters more than repeated work)
  } t;
  TileStageT<false> stage[DEC_WARPS];
  uint64_t tfull;
  uint64_t kfull[DEC_WARPS][2];
  uint64_t vfull[DEC_WARPS];
  alignas(16) __nv_bfloat16 pbuf[DEC_WARPS][2][JQK_MAX_GROUP][TILE_TOK];  // P hi / lo per warp
  float wm[DEC_WARPS][JQK_MAX_GROUP];
  float wl[DEC_WARPS][JQK_MAX_GROUP];
  int is_last;
  // the key and value row appended by this launch (blocks of the last split only)
  float ap_k[JQK_MAX_DIM];
  uint32_t ap_words[JQK_MAX_WORDS];
  __nv_bfloat16 ap_v[JQK_MAX_DIM];
  float ap_dot[JQK_MAX_GROUP];   // q_h . k_new, exact
  int ap_page, ap_last;
};
template <> struct DecodeSmemT<true> {
  struct { TableRecord rec; } t;     // the key tables always come from the table kernel
  TileStageT<true> stage[DEC_WARPS];
  uint64_t tfull;
  uint64_t kfull[DEC_WARPS][2];
  uint64_t vfull[DEC_WARPS];
  alignas(16) __nv_bfloat16 pbuf[DEC_WARPS][2][JQK_MAX_GROUP][TILE_TOK];
  float wm[DEC_WARPS][JQK_MAX_GROUP];
  float wl[DEC_WARPS][JQK_MAX_GROUP];
  int is_last;
  // the row appended by this launch (blocks of the last split only): the key's and the value's codes
  float ap_k[JQK_MAX_DIM];       // the key row, then the centred value row
  uint32_t ap_words[JQK_MAX_WORDS];
  uint32_t apv_words[JQK_MAX_WORDS];
  float ap_dot[JQK_MAX_GROUP];
  int ap_page, ap_last;
  alignas(16) int32_t vmeta[JQK_MAX_COLS];        // value columns: width | bit position << 4 | first entry of its levels in vcb << 14
  // value codebooks, bf16 (what the tensor-core product multiplies): 16 entries per column, then
  // the 2^width levels of each column of 5..8 bits, one column after the other
  __nv_bfloat16 vcb[JQK_MAX_COLS * 16 + VQ_WIDE_ENTRIES];
};
// A warp's stage doubles as its output staging [JQK_MAX_GROUP][128] floats after the last tile.
static_assert(sizeof(TileStageT<false>) >= sizeof(float) * JQK_MAX_GROUP * JQK_MAX_DIM, "stage too small for the partial output");
static_assert(sizeof(DecodeSmemT<true>) <= 232448 && sizeof(DecodeSmemT<false>) <= 232448, "decode shared memory");
static_assert(offsetof(DecodeSmemT<true>, pbuf) % 16 == 0, "the packed-value epilogue writes float4 into pbuf");

__device__ __forceinline__ void store_out(void* out, int out_dtype, size_t idx, float v) {
  if (out_dtype == JQK_DTYPE_F32) ((float*)out)[idx] = v;
  else ((__nv_bfloat16*)out)[idx] = __float2bfloat16(v);
}

// 2^x for x <= 0 (or -inf): one MUFU instruction, results below the normal range flush to zero.
// Two ulps of error are far inside what the softmax weights need (they are rounded to two bf16
// terms afterwards).
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Bulk asynchronous copy global -> shared (16-byte aligned, size a multiple of 16), completing on `bar`.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)) : "memory");
}
// The same for data that is read once per launch (K and V pages): marked evict-first in L2, so the
// stream does not push out what every launch reuses (the per-head tables and projection matrices).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void bulk_load_stream(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_addr(dst)), "l"(src), "r"(bytes), "r"(smem_addr(bar)), "l"(policy) : "memory");
}
__device__ __forceinline__ void bar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// Bounded wait (two seconds of %globaltimer by default): a copy that never completes ends in a
// status bit and a skipped tile, not in a hung device.
constexpr unsigned long long DEC_WAIT_NS = 2000000000ull;
__device__ __forceinline__ bool bar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit_ns = DEC_WAIT_NS) {
  return sm100::mbar_wait_timed<0>(bar, parity, limit_ns);
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// 32 page ids of a warp's window, validated; -1 beyond the sequence or outside the pool.
__device__ __forceinline__ int load_page_window(const int32_t* __restrict__ page_table, int pt_stride, int seq,
                                                int first_lp, int n_seq_pages, int n_pages, int32_t* status) {
  const int lp = first_lp + (threadIdx.x & 31);
  if (lp >= n_seq_pages || lp >= pt_stride) return -1;
  return lookup_page(page_table, pt_stride, seq, lp, n_pages, status);
}


// Builds the lookup tables of every (sequence, kv head, q-head block) once per decode step; the
// decode blocks of all key splits of that group then only copy them.  One block per group.
__global__ void __launch_bounds__(TBL_BUILD_THREADS)
decode_tables_kernel(jqk_head_tables tb, const __nv_bfloat16* __restrict__ q, int n_q_heads, TableRecord* __restrict__ recs) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  TableSmem& sm = *reinterpret_cast<TableSmem*>(smem_raw);
  const int group = n_q_heads / tb.n_heads;
  const int q_blocks = (group + JQK_MAX_GROUP - 1) / JQK_MAX_GROUP;
  const int head = blockIdx.x / q_blocks, qb = blockIdx.x % q_blocks, seq = blockIdx.y;
  const int g0 = qb * JQK_MAX_GROUP, n_group = min(JQK_MAX_GROUP, group - g0);
  // the decode launch that follows may start (its blocks wait for these records where they need them)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const HeadDesc hd = load_desc(tb.desc, head);
  {
    const __nv_bfloat16* qg = q + ((size_t)seq * n_q_heads + head * group + g0) * hd.d;
    if (tb.n_wide) {
      const TableLoads ld = issue_table_loads<true>(tb, head, hd.d, qg, JQK_DTYPE_BF16, (size_t)hd.d, n_group);
      build_tables<true>(sm, hd, ld, tb.wide_cb + (size_t)head * JQK_MAX_WIDE * 256);
    } else {
      const TableLoads ld = issue_table_loads(tb, head, hd.d, qg, JQK_DTYPE_BF16, (size_t)hd.d, n_group);
      build_tables(sm, hd, ld);
    }
  }
  TableRecord* rec = recs + (size_t)seq * gridDim.x + blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(sm.lut);
  uint4* dst = reinterpret_cast<uint4*>(rec->lut);
  for (int e = threadIdx.x; e < hd.n_tables * 8; e += blockDim.x) dst[e] = src[e];
  if (threadIdx.x < TBL_WORDS) rec->dshift[threadIdx.x] = sm.dshift[threadIdx.x];
  if (threadIdx.x < JQK_MAX_GROUP) rec->scale[threadIdx.x] = sm.scale[threadIdx.x];
  if (threadIdx.x == 0) rec->bias = sm.bias;
  if (threadIdx.x < JQK_MAX_WIDE) rec->woff[threadIdx.x] = sm.woff[threadIdx.x];
}

// What the kernel needs of the value-side tables when values are stored as packed codes.
struct ValueSide {
  const int32_t* desc;      // [H][JQK_DESC_INTS]
  const int32_t* col_meta;  // [H][128]
  const float* cb_cols;     // [H][128][16]
  const float* inv_rows;    // [H][128][d]
  const float* center;      // [H][d] or null
  int n_heads, wpr;
  const float* fwd_cols;    // [H][d][128]  (append variant: the new value row is compressed in the kernel)
  const float* thresholds;  // [H][128][16]
  const float* wide_cb;     // [H][JQK_MAX_WIDE][256] levels of the columns of 5..8 bits, or null
  const float* wide_thr;    // [H][JQK_MAX_WIDE][256] their thresholds (append variant), or null
};

// The newest token of every sequence, appended by the decode launch itself (k == nullptr: none).
// Position seq_lens[s] takes the row; the launch attends over seq_lens[s] + 1 keys and its last
// block to finish advances every length by one.
struct AppendSide {
  const void* k;            // [n_seqs][n_kv_heads][d] through the strides below (elements)
  const void* v;
  int k_dtype, v_dtype;     // JQK_DTYPE_* of k and of v
  long long k_seq_stride, k_head_stride, v_seq_stride, v_head_stride;
  uint32_t* k_pool;         // the pools again, writable
  __nv_bfloat16* v_pool;
  int32_t* seq_lens;        // the lengths again, writable
  int n_seqs;
  int own_key_exact;        // score the appended key from its exact values in this step (its codes serve later steps)
};

__device__ __forceinline__ float load_elem_f32(const void* p, int dtype, size_t i) {
  if (dtype == JQK_DTYPE_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == JQK_DTYPE_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// (sum_t p_t x_hat_t) / L in the value basis -> attention output: one 128 x d product per query head
// with the value side's inverse map, plus the mean the values were centred with.  `yb`: shared,
// [JQK_MAX_GROUP][128] normalised sums, then JQK_MAX_GROUP flags (some key was attended).
template <int D>
__device__ __forceinline__ void values_to_output(const float* yb, int n_group, const ValueSide& vs, int head, int n_cols,
                                                 void* out, int out_dtype, size_t qrow0) {
  const float* inv = vs.inv_rows + (size_t)head * 128 * D;
  for (int e = threadIdx.x; e < n_group * D; e += DEC_THREADS) {
    const int h = e / D, i = e % D;
    float a = 0.f;
#pragma unroll 8
    for (int cc = 0; cc < n_cols; ++cc) a = fmaf(yb[h * 128 + cc], __ldg(inv + (size_t)cc * D + i), a);
    const bool some = yb[JQK_MAX_GROUP * 128 + h] != 0.f;
    if (vs.center && some) a += vs.center[(size_t)head * D + i];
    store_out(out, out_dtype, (qrow0 + h) * D + i, some ? a : 0.f);
  }
}

// Code of column `col` of one row (`row`: D values in shared memory), with the arithmetic of
// compress_token_kernel: the dims in ascending order with fused multiply-adds.  The column's
// descriptor and threshold row are fetched ahead of the dot product, whose 128 reads of the basis go
// out 64 at a time: the latency of a block that appends is a few memory round trips, not a dozen.
template <int D>
__device__ __forceinline__ uint32_t column_code(const float* row, const float* __restrict__ fwd_cols,
                                                const int32_t* __restrict__ col_meta, const float* __restrict__ thresholds,
                                                const float* __restrict__ wide_thr, int wide_first, int head, int col, int& m_out) {
  const int m = __ldg(col_meta + (size_t)head * 128 + col);
  const float4* th4 = reinterpret_cast<const float4*>(thresholds + ((size_t)head * 128 + col) * 16);
  const float4 t0 = __ldg(th4), t1 = __ldg(th4 + 1), t2 = __ldg(th4 + 2), t3 = __ldg(th4 + 3);
  const float* w = fwd_cols + (size_t)head * D * 128 + col;
  float x = 0.f;
#pragma unroll 64
  for (int i = 0; i < D; ++i) x = fmaf(row[i], __ldg(w + (size_t)i * 128), x);
  m_out = m;
  const int width = m & 15;
  if (width > 4) return threshold_code(x, width, nullptr, wide_thr + ((size_t)head * JQK_MAX_WIDE + (col - wide_first)) * 256);
  // (+inf beyond the column's 2^width - 1 thresholds: counting all fifteen gives the same code)
  const float th[15] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y, t1.z, t1.w, t2.x, t2.y, t2.z, t2.w, t3.x, t3.y, t3.z};
  uint32_t code = 0;
#pragma unroll
  for (int l = 0; l < 15; ++l) code += (x >= th[l]) ? 1u : 0u;
  return code;
}

// The appended key of (seq, head): transformed and quantised exactly as compress_token_kernel does
// (thread = column, the dims in ascending order with fused multiply-adds: the same bits), the value
// row converted to bf16.  Both stay in shared memory for the warp whose tile holds the position;
// with `write` they also go to their slot of the tail page.  Called by all threads of the block.
template <int D>
__device__ __noinline__ void append_row(DecodeSmemT<false>& sm, const float* __restrict__ fwd_cols,
                                        const int32_t* __restrict__ col_meta, const float* __restrict__ thresholds,
                                        int n_heads, int wpr, int n_active, int n_words, const void* k_row,
                                        const void* v_row, int k_dtype, int v_dtype, uint32_t* k_pool, __nv_bfloat16* v_pool,
                                        int head, int seq, bool write, int pos,
                                        const int32_t* __restrict__ page_table, int pt_stride, int n_pages,
                                        int32_t* status, const __nv_bfloat16* __restrict__ q_rows, int n_group,
                                        const float* __restrict__ wide_thr, int wide_first) {
  const int tid = threadIdx.x;
  int m_col = 0;
  if (tid < D) {
    sm.ap_k[tid] = load_elem_f32(k_row, k_dtype, tid);
  } else if (tid >= 128 && tid < 128 + D) {
    sm.ap_v[tid - 128] = __float2bfloat16(load_elem_f32(v_row, v_dtype, tid - 128));
  } else if (tid >= 256 && tid < 256 + JQK_MAX_WORDS) {
    sm.ap_words[tid - 256] = 0u;
  } else if (tid == DEC_THREADS - 1) {
    sm.ap_page = lookup_page(page_table, pt_stride, seq, pos / JQK_PAGE_TOKENS, n_pages, status);
  }
  __syncthreads();
  if (tid < n_active) {
    const uint32_t code = column_code<D>(sm.ap_k, fwd_cols, col_meta, thresholds, wide_thr, wide_first, head, tid, m_col);
    const int bp = (m_col >> 4) & 1023;
    atomicOr(&sm.ap_words[bp >> 5], code << (bp & 31));
  } else if (q_rows && tid >= 256) {   // the exact scores of the new key: one warp per query head of the group
    const int h = (tid - 256) >> 5, lane = tid & 31;
    if (h < n_group) {
      float dot = 0.f;
      for (int i = lane; i < D; i += 32) dot = fmaf(__bfloat162float(q_rows[(size_t)h * D + i]), sm.ap_k[i], dot);
      dot = warp_sum(dot);
      if (lane == 0) sm.ap_dot[h] = dot;
    }
  }
  __syncthreads();
  const int page = sm.ap_page;
  if (write && page >= 0) {
    const int slot = pos % JQK_PAGE_TOKENS;
    if (tid < n_words) {
      k_pool[(((size_t)page * n_heads + head) * wpr + tid) * JQK_PAGE_TOKENS + slot] = sm.ap_words[tid];
    } else if (tid >= 128 && tid < 128 + D) {
      const int i = tid - 128;
      v_pool[((size_t)page * n_heads + head) * (size_t)(JQK_PAGE_TOKENS * D) + i * JQK_PAGE_TOKENS +
                (((slot >> 3) ^ ((i >> 2) & 1)) * 8) + (slot & 7)] = sm.ap_v[i];
    }
  }
}

// One row of D values in shared memory (`row`) -> its record words in `words` (zeroed by the caller),
// with the arithmetic of compress_token_kernel: thread = column, dims in ascending order.
template <int D>
__device__ __forceinline__ void quantise_row(const float* row, uint32_t* words, const float* __restrict__ fwd_cols,
                                             const int32_t* __restrict__ col_meta, const float* __restrict__ thresholds,
                                             int head, int n_active, const float* __restrict__ wide_thr, int wide_first) {
  const int tid = threadIdx.x;
  if (tid < n_active) {
    int m;
    const uint32_t code = column_code<D>(row, fwd_cols, col_meta, thresholds, wide_thr, wide_first, head, tid, m);
    const int bp = (m >> 4) & 1023;
    atomicOr(&words[bp >> 5], code << (bp & 31));
  }
}

// The append with packed values: the key as in append_row, then the value row (mean subtracted in
// fp32, as the reference's wrapper does before its transform) through the value side's tables; both
// records stay in shared memory and, with `write`, go to the tail pages of the two code pools.
template <int D>
__device__ __noinline__ void append_row_packed(DecodeSmemT<true>& sm, const float* __restrict__ k_fwd,
                                               const int32_t* __restrict__ k_meta, const float* __restrict__ k_thr,
                                               int n_heads, int k_wpr, int k_active, int k_words,
                                               const float* __restrict__ v_fwd, const int32_t* __restrict__ v_meta,
                                               const float* __restrict__ v_thr, const float* __restrict__ v_center,
                                               int v_wpr, int v_active, int v_words, const void* k_row, const void* v_row,
                                               int k_dtype, int v_dtype, uint32_t* k_pool, uint32_t* v_pool, int head, int seq,
                                               bool write, int pos, const int32_t* __restrict__ page_table, int pt_stride,
                                               int n_pages, int32_t* status, const __nv_bfloat16* __restrict__ q_rows, int n_group,
                                               const float* __restrict__ k_wide_thr, int k_wide_first,
                                               const float* __restrict__ v_wide_thr, int v_wide_first) {
  const int tid = threadIdx.x;
  if (tid < D) {
    sm.ap_k[tid] = load_elem_f32(k_row, k_dtype, tid);
  } else if (tid >= 256 && tid < 256 + JQK_MAX_WORDS) {
    sm.ap_words[tid - 256] = 0u;
    sm.apv_words[tid - 256] = 0u;
  } else if (tid == DEC_THREADS - 1) {
    sm.ap_page = lookup_page(page_table, pt_stride, seq, pos / JQK_PAGE_TOKENS, n_pages, status);
  }
  __syncthreads();
  quantise_row<D>(sm.ap_k, sm.ap_words, k_fwd, k_meta, k_thr, head, k_active, k_wide_thr, k_wide_first);
  if (q_rows && tid >= 256) {
    const int h = (tid - 256) >> 5, lane = tid & 31;
    if (h < n_group) {
      float dot = 0.f;
      for (int i = lane; i < D; i += 32) dot = fmaf(__bfloat162float(q_rows[(size_t)h * D + i]), sm.ap_k[i], dot);
      dot = warp_sum(dot);
      if (lane == 0) sm.ap_dot[h] = dot;
    }
  }
  __syncthreads();
  if (tid < D) {
    float v = load_elem_f32(v_row, v_dtype, tid);
    if (v_center) v -= v_center[(size_t)head * D + tid];
    sm.ap_k[tid] = v;
  }
  __syncthreads();
  quantise_row<D>(sm.ap_k, sm.apv_words, v_fwd, v_meta, v_thr, head, v_active, v_wide_thr, v_wide_first);
  __syncthreads();
  const int page = sm.ap_page;
  if (write && page >= 0) {
    const int slot = pos % JQK_PAGE_TOKENS;
    if (tid < k_words)
      k_pool[(((size_t)page * n_heads + head) * k_wpr + tid) * JQK_PAGE_TOKENS + slot] = sm.ap_words[tid];
    else if (tid >= 128 && tid < 128 + v_words)
      v_pool[(((size_t)page * n_heads + head) * v_wpr + (tid - 128)) * JQK_PAGE_TOKENS + slot] = sm.apv_words[tid - 128];
  }
}

// D = head_dim (64 or 128).  VQ: values are packed codes of a second compressor (v_pool is then the
// uint32 code pool, `vs` its tables); the keys' tables then always come from the table kernel.
template <int D, bool BUILD_IN_BLOCK, bool VQ, bool APPEND, bool WIDE = false>
__global__ void __launch_bounds__(DEC_THREADS, 1)
decode_kernel(jqk_head_tables tb, const __nv_bfloat16* __restrict__ q, int n_q_heads,
              const int32_t* __restrict__ seq_lens, int tokens_per_split,
              const int32_t* __restrict__ page_table, int pt_stride, int n_pages,
              const uint32_t* __restrict__ k_pool, const void* __restrict__ v_pool_raw,
              void* __restrict__ out, int out_dtype, DecodeWs ws, int32_t* status, ValueSide vs, AppendSide ap) {
  static_assert(!(VQ && BUILD_IN_BLOCK), "packed values need the table kernel");
  constexpr int DT = D / 16;                       // 16-dim MMA tiles
  constexpr uint32_t V_PAGE_BYTES = JQK_PAGE_TOKENS * D * 2;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  DecodeSmemT<VQ>& sm = *reinterpret_cast<DecodeSmemT<VQ>*>(smem_raw);
  const __nv_bfloat16* v_pool = reinterpret_cast<const __nv_bfloat16*>(v_pool_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, c = lane & 3;
  const int group = n_q_heads / tb.n_heads;
  const int q_blocks = (group + JQK_MAX_GROUP - 1) / JQK_MAX_GROUP;
  const int head = blockIdx.y / q_blocks, qb = blockIdx.y % q_blocks;
  const int seq = blockIdx.z, split = blockIdx.x;
  // Launched as a programmatic dependent: everything up to here overlaps the tail of the previous
  // kernel on the stream; nothing in memory is read or written before that kernel has completed.
  // One exception: when the previous kernel is this call's own table kernel (ws.late_wait), it
  // writes nothing but the table records, and everything older on the stream was complete before it
  // started; the block then waits only where it needs the records, and its lengths, page ids and
  // first page copies run beside the table build.
  bool waited = true;
  if constexpr (!BUILD_IN_BLOCK) waited = !ws.late_wait;
  if (waited) asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // A context longer than the call was sized for (max_seq_len on the host side fixed the grid and
  // the workspace) is cut to what the grid covers and flagged; otherwise the ticket below would
  // never see its last block.
  int len = seq_lens[seq];
  // The table build's reads go out at once, in the same round trip as the length: nothing a block
  // does later is queued ahead of them (a block that turns out to have no keys has read in vain).
  const int g0 = qb * JQK_MAX_GROUP, n_group = min(JQK_MAX_GROUP, group - g0);
  const int qh0 = head * group + g0;
  TableLoads tloads;
  if constexpr (BUILD_IN_BLOCK)
    tloads = issue_table_loads<WIDE>(tb, head, D, q + ((size_t)seq * n_q_heads + qh0) * D, JQK_DTYPE_BF16, (size_t)D, n_group);
  if constexpr (APPEND) len += 1;  // this launch attends over the key it appends
  // Append variant: every block of the launch passes here exactly once on its way out, all of its
  // threads together.  Each has read its length by then, so the block that takes the last ticket
  // may advance the lengths for the next launch.
  // (The ticket is taken in two halves so that the merging block can put the atomic in flight before
  // its merge and read the answer after it: its round trip is then off the step's critical path.)
  [[maybe_unused]] unsigned int ticket_prev = 0u;
  auto take_ticket = [&]() {   // after a barrier that all threads of the block have passed since reading their length
    if constexpr (APPEND)
      if (tid == 0)
        asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(ticket_prev) : "l"(ws.grid_ticket) : "memory");
  };
  auto finish_ticket = [&]() {
    if constexpr (APPEND) {
      if (tid == 0) {
        const bool last = ticket_prev == gridDim.x * gridDim.y * gridDim.z - 1u;
        if (last) *ws.grid_ticket = 0u;
        sm.ap_last = last ? 1 : 0;
      }
      __syncthreads();
      if (sm.ap_last)
        for (int s2 = tid; s2 < ap.n_seqs; s2 += DEC_THREADS) ap.seq_lens[s2] += 1;
    }
  };
  auto leave = [&]() {
    if constexpr (APPEND) {
      __syncthreads();
      take_ticket();
      finish_ticket();
    }
  };
  {
    const long long cap = (long long)gridDim.x * tokens_per_split;
    if (len > cap) {
      len = (int)cap;
      if (threadIdx.x == 0 && split == 0 && status) atomicOr(status, JQK_STATUS_BAD_LENGTH);
    }
  }
  const int n_splits = (len + tokens_per_split - 1) / tokens_per_split;
  if (len <= 0) {  // empty context: defined output (zeros), written by split 0
    if (split == 0)
      for (int e = tid; e < n_group * D; e += DEC_THREADS)
        store_out(out, out_dtype, ((size_t)seq * n_q_heads + qh0 + e / D) * D + e % D, 0.f);
    leave();
    return;
  }
  if (split >= n_splits) { leave(); return; }
  const HeadDesc hd = load_desc(tb.desc, head);
  const int t_begin = split * tokens_per_split;
  const int t_end = min(len, t_begin + tokens_per_split);
  const int n_seq_pages = (len + JQK_PAGE_TOKENS - 1) / JQK_PAGE_TOKENS;
  const int wpr = tb.words_per_record;
  const size_t k_page_words = (size_t)tb.n_heads * wpr * JQK_PAGE_TOKENS;
  const size_t v_page_elems = (size_t)tb.n_heads * JQK_PAGE_TOKENS * D;
  const uint32_t* k_head = k_pool + (size_t)head * wpr * JQK_PAGE_TOKENS;
  const __nv_bfloat16* v_head = v_pool + (size_t)head * JQK_PAGE_TOKENS * D;
  const uint32_t k_page_bytes = (uint32_t)hd.n_words * JQK_PAGE_TOKENS * 4;
  // packed values: pages of the value code pool, one head's block inside a page
  const uint32_t* vq_head = nullptr;
  size_t vq_page_words = 0;
  uint32_t vq_page_bytes = 0;
  int v_n_active = 0, v_wide_first = 0, v_n_wide = 0;
  if constexpr (VQ) {
    const HeadDesc vhd = load_desc(vs.desc, head);
    vq_head = reinterpret_cast<const uint32_t*>(v_pool_raw) + (size_t)head * vs.wpr * JQK_PAGE_TOKENS;
    vq_page_words = (size_t)vs.n_heads * vs.wpr * JQK_PAGE_TOKENS;
    vq_page_bytes = (uint32_t)vhd.n_words * JQK_PAGE_TOKENS * 4;
    v_n_active = vhd.n_active;
    v_wide_first = vhd.wide_first;
    v_n_wide = vhd.n_wide;
  }

  // ---- this warp's run of tiles and its page ids ----
  const int tiles_total = (t_end - t_begin + TILE_TOK - 1) / TILE_TOK;
  const int tiles_per_warp = (tiles_total + DEC_WARPS - 1) / DEC_WARPS;
  const int tile_lo = min(tiles_total, warp * tiles_per_warp);
  const int n_my = min(tiles_total, tile_lo + tiles_per_warp) - tile_lo;
  const int lp0 = t_begin / JQK_PAGE_TOKENS + 2 * tile_lo;  // first logical page of this warp
  int pg_cur = load_page_window(page_table, pt_stride, seq, lp0, n_seq_pages, n_pages, status);
  int pg_next = load_page_window(page_table, pt_stride, seq, lp0 + 32, n_seq_pages, n_pages, status);

  if (lane == 0) { bar_init(&sm.kfull[warp][0], 1); bar_init(&sm.kfull[warp][1], 1); bar_init(&sm.vfull[warp], 1); }
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  __syncwarp();

  // Lane 0 starts the copies of a tile (pages pg_lo / pg_hi, -1 = absent).  K pages of tile r go to
  // K buffer r & 1, V pages to the single V buffer.  Buffers are refilled by the warp that read
  // them, in program order after its last read, so no "empty" barriers are needed.
  TileStageT<VQ>& st = sm.stage[warp];
  const uint64_t stream_policy = l2_evict_first_policy();
  auto issue_keys = [&](int r, int pg_lo, int pg_hi) {
    if (lane == 0) {
      uint64_t* bar = &sm.kfull[warp][r & 1];
      const int t0 = t_begin + (tile_lo + r) * TILE_TOK;
      const bool ok0 = pg_lo >= 0, ok1 = pg_hi >= 0 && t0 + JQK_PAGE_TOKENS < t_end;
      bar_expect_tx(bar, ((ok0 ? 1u : 0u) + (ok1 ? 1u : 0u)) * k_page_bytes);
      if (ok0) bulk_load_stream(st.k[r & 1][0], k_head + (size_t)pg_lo * k_page_words, k_page_bytes, bar, stream_policy);
      if (ok1) bulk_load_stream(st.k[r & 1][1], k_head + (size_t)pg_hi * k_page_words, k_page_bytes, bar, stream_policy);
    }
  };
  auto issue_values = [&](int r, int pg_lo, int pg_hi) {
    if (lane == 0) {
      uint64_t* bar = &sm.vfull[warp];
      const int t0 = t_begin + (tile_lo + r) * TILE_TOK;
      const bool ok0 = pg_lo >= 0, ok1 = pg_hi >= 0 && t0 + JQK_PAGE_TOKENS < t_end;
      if constexpr (VQ) {
        bar_expect_tx(bar, ((ok0 ? 1u : 0u) + (ok1 ? 1u : 0u)) * vq_page_bytes);
        if (ok0) bulk_load_stream(st.vq[0], vq_head + (size_t)pg_lo * vq_page_words, vq_page_bytes, bar, stream_policy);
        if (ok1) bulk_load_stream(st.vq[1], vq_head + (size_t)pg_hi * vq_page_words, vq_page_bytes, bar, stream_policy);
      } else {
        bar_expect_tx(bar, ((ok0 ? 1u : 0u) + (ok1 ? 1u : 0u)) * V_PAGE_BYTES);
        if (ok0) bulk_load_stream(st.v[0], v_head + (size_t)pg_lo * v_page_elems, V_PAGE_BYTES, bar, stream_policy);
        if (ok1) bulk_load_stream(st.v[1], v_head + (size_t)pg_hi * v_page_elems, V_PAGE_BYTES, bar, stream_policy);
      }
    }
  };
  // the first copies go in flight before the tables exist, so HBM works during the prologue
  {
    const int p0 = __shfl_sync(0xffffffffu, pg_cur, 0), p1 = __shfl_sync(0xffffffffu, pg_cur, 1);
    const int p2 = __shfl_sync(0xffffffffu, pg_cur, 2), p3 = __shfl_sync(0xffffffffu, pg_cur, 3);
    if (n_my > 0) { issue_keys(0, p0, p1); issue_values(0, p0, p1); }
    if (n_my > 1) issue_keys(1, p2, p3);
  }

  // the block whose split ends the context takes the appended row (every query block keeps its own
  // copy in shared memory; the first one also writes it to the tail page)
  int ap_pos = -1;
  if constexpr (APPEND && VQ) {
    if (split == n_splits - 1) {
      ap_pos = len - 1;
      const HeadDesc vhd2 = load_desc(vs.desc, head);
      const size_t k_esz = ap.k_dtype == JQK_DTYPE_F32 ? 4 : 2, v_esz = ap.v_dtype == JQK_DTYPE_F32 ? 4 : 2;
      append_row_packed<D>(sm, tb.fwd_cols, tb.col_meta, tb.thresholds, tb.n_heads, tb.words_per_record, hd.n_active, hd.n_words,
                           vs.fwd_cols, vs.col_meta, vs.thresholds, vs.center, vs.wpr, vhd2.n_active, vhd2.n_words,
                           (const char*)ap.k + ((size_t)seq * ap.k_seq_stride + (size_t)head * ap.k_head_stride) * k_esz,
                           (const char*)ap.v + ((size_t)seq * ap.v_seq_stride + (size_t)head * ap.v_head_stride) * v_esz,
                           ap.k_dtype, ap.v_dtype, ap.k_pool, reinterpret_cast<uint32_t*>(ap.v_pool), head, seq, qb == 0, ap_pos,
                           page_table, pt_stride, n_pages, status,
                           ap.own_key_exact ? q + ((size_t)seq * n_q_heads + qh0) * D : nullptr, n_group,
                           tb.wide_thr, hd.wide_first, vs.wide_thr, vhd2.wide_first);
    }
  }
  if constexpr (APPEND && !VQ) {
    if (split == n_splits - 1) {
      ap_pos = len - 1;
      const size_t k_esz = ap.k_dtype == JQK_DTYPE_F32 ? 4 : 2, v_esz = ap.v_dtype == JQK_DTYPE_F32 ? 4 : 2;
      append_row<D>(sm, tb.fwd_cols, tb.col_meta, tb.thresholds, tb.n_heads, tb.words_per_record, hd.n_active, hd.n_words,
                    (const char*)ap.k + ((size_t)seq * ap.k_seq_stride + (size_t)head * ap.k_head_stride) * k_esz,
                    (const char*)ap.v + ((size_t)seq * ap.v_seq_stride + (size_t)head * ap.v_head_stride) * v_esz,
                    ap.k_dtype, ap.v_dtype, ap.k_pool, ap.v_pool, head, seq, qb == 0, ap_pos, page_table, pt_stride, n_pages, status,
                    ap.own_key_exact ? q + ((size_t)seq * n_q_heads + qh0) * D : nullptr, n_group, tb.wide_thr, hd.wide_first);
    }
  }

  float sc[JQK_MAX_GROUP];
  TableView tview;
  if constexpr (BUILD_IN_BLOCK) {
    build_tables<WIDE>(sm.t.build, hd, tloads, WIDE ? tb.wide_cb + (size_t)head * JQK_MAX_WIDE * 256 : nullptr);
    tview = TableView{sm.t.build.lut, sm.t.build.dshift, sm.t.build.bias, sm.t.build.woff};
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) sc[h] = sm.t.build.scale[h];
  } else {
    if constexpr (VQ) {
      // value-side tables of this head (static per head: no query enters them), and a clean tile:
      // rows of columns that carry no bits are never written by the dequantiser and must read as 0
      const int32_t* vcm = vs.col_meta + (size_t)head * 128;
      for (int e = tid; e < JQK_MAX_COLS; e += DEC_THREADS) {
        // (a descriptor past the last column reads code 0 of its own, all-zero, row)
        int m = (e < v_n_active) ? (__ldg(vcm + e) & 0x3FFF) : 0, base = e * 16;
        if ((m & 15) > 4) {  // a byte-wide column: its levels follow those of the wide columns before it
          base = JQK_MAX_COLS * 16;
          for (int j = v_wide_first; j < e; ++j) base += 1 << (__ldg(vcm + j) & 15);
        }
        sm.vmeta[e] = v_n_wide ? (m | (base << 14)) : m;
      }
      for (int i = warp; i < v_n_wide; i += DEC_WARPS) {  // a warp per byte-wide column: its 2^width levels
        const int m = __ldg(vcm + v_wide_first + i) & 15;
        int base = JQK_MAX_COLS * 16;
        for (int j = 0; j < i; ++j) base += 1 << (__ldg(vcm + v_wide_first + j) & 15);
        const float* row = vs.wide_cb + ((size_t)head * JQK_MAX_WIDE + i) * 256;
        for (int l = lane; l < (1 << m); l += 32) sm.vcb[base + l] = __float2bfloat16(__ldg(row + l));
      }
      for (int e = tid; e < JQK_MAX_COLS * 16; e += DEC_THREADS) {
        const int c = e >> 4, l = e & 15;
        const __nv_bfloat16 lvl = __float2bfloat16(__ldg(vs.cb_cols + (size_t)head * 128 * 16 + e));
        if (v_n_wide) sm.vcb[e] = lvl;
        else reinterpret_cast<uint32_t*>(sm.vcb)[((c >> 5) * 16 + l) * 32 + (c & 31)] = (uint32_t)__bfloat16_as_ushort(lvl);
      }
      uint4* z = reinterpret_cast<uint4*>(&st.v[0][0]);
      for (int e = lane; e < (int)(sizeof(st.v) / 16); e += 32) z[e] = make_uint4(0u, 0u, 0u, 0u);
    }
    // the finished tables of this (sequence, head group) come from the table kernel
    if (!waited) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0) {
      const TableRecord* rec = ws.tables + (size_t)seq * gridDim.y + blockIdx.y;
      const uint32_t lut_bytes = (uint32_t)hd.n_tables * 128u;
      bar_init(&sm.tfull, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      bar_expect_tx(&sm.tfull, lut_bytes + TABLE_RECORD_META_BYTES);
      if (lut_bytes) bulk_load(sm.t.rec.lut, rec->lut, lut_bytes, &sm.tfull);
      bulk_load(sm.t.rec.dshift, rec->dshift, TABLE_RECORD_META_BYTES, &sm.tfull);
    }
    __syncthreads();
    if (!bar_wait(&sm.tfull, 0) && tid == 0 && status) atomicOr(status, JQK_STATUS_WAIT_EXPIRED);
    tview = TableView{sm.t.rec.lut, sm.t.rec.dshift, sm.t.rec.bias, sm.t.rec.woff};
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) sc[h] = sm.t.rec.scale[h];
  }
  {
    const float f = kLog2e / sqrtf((float)D);
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) sc[h] *= f;
  }
  const int n_a_words = hd.n_a_words, n_c_words = hd.n_c_words, n_words = hd.n_words;

  float m_run[JQK_MAX_GROUP], l_run[JQK_MAX_GROUP];
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) { m_run[h] = -CUDART_INF_F; l_run[h] = 0.f; }
  float acc[DT][4];  // MMA tile j: rows = dims 16j + g (+8), cols = heads 2c, 2c+1
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[j][k] = 0.f;
  // ldmatrix row address of this lane inside a 16-dim x 16-key block of a V page (32-byte rows; the
  // two 16-byte halves of a row are swapped on rows 4..7 mod 8 so that eight rows hit eight bank groups)
  const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8;
  const uint32_t lm_off = (uint32_t)(lrow * 32 + (((lane >> 4) ^ ((lrow >> 2) & 1)) * 16));

  for (int r = 0; r < n_my; ++r) {
    if (r > 0 && (r & 15) == 0) {
      pg_cur = pg_next;
      pg_next = load_page_window(page_table, pt_stride, seq, lp0 + 2 * r + 32, n_seq_pages, n_pages, status);
    }
    const int t0 = t_begin + (tile_lo + r) * TILE_TOK;
    const int page_lo = __shfl_sync(0xffffffffu, pg_cur, (r & 15) << 1);
    const int page_hi = __shfl_sync(0xffffffffu, pg_cur, ((r & 15) << 1) | 1);
    bool landed = bar_wait(&sm.kfull[warp][r & 1], (r >> 1) & 1);

    if constexpr (APPEND) {
      if (ap_pos >= t0 && ap_pos < t0 + TILE_TOK) {  // the page copy may predate the append: take the record from the block's own copy
        const int slot = ap_pos - t0;
        uint32_t* kd = reinterpret_cast<uint32_t*>(st.k[r & 1][slot >> 4]) + (slot & 15);
        if (lane < n_words) kd[lane * JQK_PAGE_TOKENS] = sm.ap_words[lane];
        __syncwarp();
      }
    }

    // ---- score this lane's key from the staged record words ----
    const int tok = t0 + lane;
    const bool lane_ok = landed && tok < t_end && ((lane < 16) ? page_lo : page_hi) >= 0;
    int ia[JQK_MAX_GROUP];
    {
      const uint32_t* kw = reinterpret_cast<const uint32_t*>(st.k[r & 1][lane >> 4]) + (lane & 15);
      score_record<WIDE>([kw](int w) { return kw[w * JQK_PAGE_TOKENS]; }, tview, n_a_words, n_c_words, n_words, ia, WIDE ? hd.n_wide : 0);
    }
    if (!lane_ok) {
#pragma unroll
      for (int h = 0; h < JQK_MAX_GROUP; ++h) ia[h] = INT_MIN;
    }
    if constexpr (APPEND) {
      // the appended key attends with its exact values in the step that appends it (the reference
      // compresses a decode key after the step that produced it, jointqk_press.py:298-304)
      if (ap.own_key_exact && tok == ap_pos && lane_ok) {
        const float f = kLog2e / sqrtf((float)D);
#pragma unroll
        for (int h = 0; h < JQK_MAX_GROUP; ++h)
          if (sc[h] > 0.f) ia[h] = __float2int_rn(fminf(fmaxf(sm.ap_dot[h] * f / sc[h], -2147483520.f), 2147483520.f));
      }
    }

    // ---- online softmax: the tile maximum is an integer reduction (scores are scale * integer);
    //      the sum of the weights stays per lane and is reduced once after the last tile ----
    // Written without branches so that the four heads' dependent chains (reduction, conversion,
    // two exponentials, bf16 split) interleave instead of running one after the other.
    float alpha[JQK_MAX_GROUP];
    int imax[JQK_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) imax[h] = __reduce_max_sync(0xffffffffu, ia[h]);
    bool any = false, grew = false;
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) {
      const bool some = imax[h] != INT_MIN;
      const float m_tile = some ? (float)imax[h] * sc[h] : -CUDART_INF_F;
      const float m_new = fmaxf(m_run[h], m_tile);
      const bool up = m_new > m_run[h];
      alpha[h] = up ? exp2_fast(m_run[h] - m_new) : 1.f;  // first valid tile: exp2(-inf) = 0
      const float p = lane_ok ? exp2_fast((float)ia[h] * sc[h] - m_new) : 0.f;
      any |= some;
      grew |= up;
      m_run[h] = m_new;
      const __nv_bfloat16 p_hi = __float2bfloat16(p);
      const __nv_bfloat16 p_lo = __float2bfloat16(p - __bfloat162float(p_hi));
      sm.pbuf[warp][0][h][lane] = p_hi;
      sm.pbuf[warp][1][h][lane] = p_lo;
      l_run[h] = l_run[h] * alpha[h] + (__bfloat162float(p_hi) + __bfloat162float(p_lo));
    }
    landed = bar_wait(&sm.vfull[warp], r & 1) && landed;
    if (!landed && lane == 0 && status) atomicOr(status, JQK_STATUS_WAIT_EXPIRED);
    if constexpr (APPEND && !VQ) {
      if (ap_pos >= t0 && ap_pos < t0 + TILE_TOK) {
        const int ts = (ap_pos - t0) & 15;
        unsigned char* vt = reinterpret_cast<unsigned char*>(st.v[(ap_pos - t0) >> 4]);
        for (int d = lane; d < D; d += 32)
          *reinterpret_cast<__nv_bfloat16*>(vt + d * 32 + (((ts >> 3) ^ ((d >> 2) & 1)) * 16) + (ts & 7) * 2) = sm.ap_v[d];
      }
    }
    // keys past the end of the split inside a page that is present: their V columns may hold
    // anything (stale or never written), and 0 x NaN must not reach the accumulators
    if constexpr (VQ && APPEND) {
      if (ap_pos >= t0 && ap_pos < t0 + TILE_TOK) {   // the appended value's codes from the block's own copy
        const int slot = ap_pos - t0;
        uint32_t* vd = reinterpret_cast<uint32_t*>(st.vq[slot >> 4]) + (slot & 15);
        if (lane < (int)(vq_page_bytes / (JQK_PAGE_TOKENS * 4))) vd[lane * JQK_PAGE_TOKENS] = sm.apv_words[lane];
        __syncwarp();
      }
    }
    if constexpr (VQ) {
      // dequantise the tile: a lane owns columns (lane, lane + 32, ...) and walks the 16 keys of each
      // page for them, so a column's word index, shift and mask are loop constants, its 16 record words
      // arrive as four 16-byte reads (lanes whose columns share a word read the same bytes), sixteen
      // independent code -> bf16 level reads follow, and the 16 levels leave as two 16-byte stores: one
      // half-row each of the dims-major tile the tensor-core product reads (the halves of a row are
      // swapped on every other group of four columns, which also spreads a warp's stores over all
      // banks).  Keys past the end or on absent pages produce finite garbage that meets a zero weight.
      if (any && landed) {
        // (two forms: with byte-wide columns a descriptor also carries where the column's levels
        // start; without, the rows are 16 entries apart and the descriptor has 14 bits)
        auto dequantise = [&](auto with_wide) {
          constexpr bool VW = decltype(with_wide)::value;
          const unsigned short* vcb16 = reinterpret_cast<const unsigned short*>(sm.vcb);
#pragma unroll 1
          for (int c = lane; c < v_n_active; c += 32) {
            const int m = sm.vmeta[c];
            const int wi = VW ? ((m >> 9) & 31) : (m >> 9);       // bit position >> 5 = record word
            const uint32_t sh = (m >> 4) & 31, mask = (1u << (m & 15)) - 1u;
            // (without byte-wide columns the levels are stored lane-interleaved, a 32-bit word each:
            // level l of column lane + 32 k at word (16 k + l) * 32 + lane, so a warp's reads of random
            // levels fall into the lanes' own banks; the words take the room of the wide levels)
            const unsigned short* row = vcb16 + (m >> 14);
            const uint32_t* row32 = reinterpret_cast<const uint32_t*>(sm.vcb) + (c >> 5) * 512 + (c & 31);
            const uint32_t swap = (c >> 2) & 1;
#pragma unroll
            for (int pg = 0; pg < 2; ++pg) {
              const uint4* src = reinterpret_cast<const uint4*>(st.vq[pg] + wi * (JQK_PAGE_TOKENS * 4));
              const uint4 w0 = src[0], w1 = src[1], w2 = src[2], w3 = src[3];
              const uint32_t w[16] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w,
                                      w2.x, w2.y, w2.z, w2.w, w3.x, w3.y, w3.z, w3.w};
              uint32_t lv[16];
#pragma unroll
              for (int t = 0; t < 16; ++t) {
                const uint32_t code = (w[t] >> sh) & mask;
                lv[t] = VW ? (uint32_t)row[code] : row32[code * 32];
              }
              uint8_t* dst = st.v[pg] + c * 32;
              *reinterpret_cast<uint4*>(dst + (swap ? 16 : 0)) =
                  make_uint4(lv[0] | (lv[1] << 16), lv[2] | (lv[3] << 16), lv[4] | (lv[5] << 16), lv[6] | (lv[7] << 16));
              *reinterpret_cast<uint4*>(dst + (swap ? 0 : 16)) =
                  make_uint4(lv[8] | (lv[9] << 16), lv[10] | (lv[11] << 16), lv[12] | (lv[13] << 16), lv[14] | (lv[15] << 16));
            }
          }
        };
        if (v_n_wide) dequantise(std::true_type{});
        else dequantise(std::false_type{});
      }
    } else if (any && t0 + TILE_TOK > t_end) {
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        const int n_valid = min(JQK_PAGE_TOKENS, max(0, t_end - (t0 + JQK_PAGE_TOKENS * kb)));
        if (n_valid > 0 && n_valid < JQK_PAGE_TOKENS) {
          for (int d = lane; d < D; d += 32)
            for (int t = n_valid; t < JQK_PAGE_TOKENS; ++t)
              *reinterpret_cast<uint16_t*>(st.v[kb] + d * 32 + (((t >> 3) ^ ((d >> 2) & 1)) * 16) + (t & 7) * 2) = 0;
        }
      }
    }
    __syncwarp();
    if (any && landed) {
      if (grew) {
        const float a_even = (c & 1) ? alpha[2] : alpha[0];  // head 2c   (c >= 2: heads that do not exist)
        const float a_odd = (c & 1) ? alpha[3] : alpha[1];   // head 2c+1
#pragma unroll
        for (int j = 0; j < DT; ++j) { acc[j][0] *= a_even; acc[j][1] *= a_odd; acc[j][2] *= a_even; acc[j][3] *= a_odd; }
      }
#pragma unroll
      for (int kb = 0; kb < 2; ++kb) {
        const int pg = kb ? page_hi : page_lo;
        if (pg < 0 || t0 + JQK_PAGE_TOKENS * kb >= t_end) continue;  // warp-uniform
        // P^T fragment, column n = g: columns 0..3 carry the high bf16 terms of the four heads and
        // columns 4..7 (padding otherwise) the low terms, so one MMA per 16 dims covers both
        const uint32_t* prow = reinterpret_cast<const uint32_t*>(&sm.pbuf[warp][g >> 2][g & 3][JQK_PAGE_TOKENS * kb]);
        const uint32_t b0 = prow[c], b1 = prow[c + 4];
        const uint32_t vbase = smem_addr(st.v[kb]) + lm_off;
#pragma unroll
        for (int j = 0; j < DT; ++j) {
          uint32_t a0, a1, a2, a3;
          ldmatrix_x4(vbase + j * 512, a0, a1, a2, a3);
          mma_bf16_16816(acc[j], a0, a1, a2, a3, b0, b1);
        }
      }
    }
    __syncwarp();  // every lane is done with this stage and with pbuf
    {  // V of the next tile and K of the tile after it take the buffers this tile has just released
      const int r1 = r + 1, r2 = r + 2;
      const int s1 = ((r1 >> 4) == (r >> 4)) ? pg_cur : pg_next, s2 = ((r2 >> 4) == (r >> 4)) ? pg_cur : pg_next;
      const int v_lo = __shfl_sync(0xffffffffu, s1, (r1 & 15) << 1), v_hi = __shfl_sync(0xffffffffu, s1, ((r1 & 15) << 1) | 1);
      const int k_lo = __shfl_sync(0xffffffffu, s2, (r2 & 15) << 1), k_hi = __shfl_sync(0xffffffffu, s2, ((r2 & 15) << 1) | 1);
      if (r1 < n_my) issue_values(r1, v_lo, v_hi);
      if (r2 < n_my) issue_keys(r2, k_lo, k_hi);
    }
  }

  // ---- combine the warps of this block (each warp reuses its own first stage) ---------------
  float* wacc = reinterpret_cast<float*>(&sm.stage[0]);  // warp w at w * WACC_STRIDE floats
  constexpr int WACC_STRIDE = (int)(sizeof(TileStageT<VQ>) / sizeof(float));
  float* yb = reinterpret_cast<float*>(&sm.pbuf[0][0][0][0]);  // packed values: normalised sums in the value basis
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) l_run[h] = warp_sum(l_run[h]);
  if (lane == 0) {
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) { sm.wm[warp][h] = m_run[h]; sm.wl[warp][h] = l_run[h]; }
  }
  // lanes c and c + 2 hold the high-term and low-term sums of the same heads
#pragma unroll
  for (int j = 0; j < DT; ++j)
#pragma unroll
    for (int k = 0; k < 4; ++k) acc[j][k] += __shfl_down_sync(0xffffffffu, acc[j][k], 2);
  if (c < 2) {
#pragma unroll
    for (int j = 0; j < DT; ++j) {
      float* w0 = wacc + (size_t)warp * WACC_STRIDE + (2 * c) * JQK_MAX_DIM + 16 * j + g;
      float* w1 = w0 + JQK_MAX_DIM;
      w0[0] = acc[j][0]; w1[0] = acc[j][1];
      w0[8] = acc[j][2]; w1[8] = acc[j][3];
    }
  }
  __syncthreads();
  const bool single = (n_splits == 1);
  for (int e = tid; e < n_group * D; e += DEC_THREADS) {
    const int h = e / D, i = e % D;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm.wm[w][h]);
    float L = 0.f, A = 0.f;
    if (M > -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float f = exp2f(sm.wm[w][h] - M);
        L += sm.wl[w][h] * f;
        A += wacc[(size_t)w * WACC_STRIDE + h * JQK_MAX_DIM + i] * f;
      }
    }
    const size_t qrow = (size_t)seq * n_q_heads + qh0 + h;
    if (single) {
      if constexpr (VQ) {
        yb[h * 128 + i] = L > 0.f ? A / L : 0.f;
        if (i == 0) yb[JQK_MAX_GROUP * 128 + h] = L > 0.f ? 1.f : 0.f;
      } else {
        store_out(out, out_dtype, qrow * D + i, L > 0.f ? A / L : 0.f);
      }
    } else {
      const size_t pidx = qrow * ws.max_splits + split;
      ws.part_acc[pidx * JQK_MAX_DIM + i] = A;
      if (i == 0) { ws.part_m[pidx] = M; ws.part_l[pidx] = L; }
    }
  }
  if constexpr (VQ) {
    if (single) {
      __syncthreads();
      values_to_output<D>(yb, n_group, vs, head, v_n_active, out, out_dtype, (size_t)seq * n_q_heads + qh0);
    }
  }
  if (single) { leave(); return; }

  // ---- the last block of this (sequence, head group) to finish merges the splits ------------
  // Ticket with release/acquire at gpu scope: the barrier orders this block's partial results
  // before thread 0's atomic, whose release makes them visible to whoever takes a later ticket, and
  // whose acquire (for the last block) makes the other blocks' results visible to the loads below.
  __syncthreads();
  unsigned int* counter = ws.counters + (size_t)seq * gridDim.y + blockIdx.y;
  if (tid == 0) {
    unsigned int prev;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], 1;" : "=r"(prev) : "l"(counter) : "memory");
    sm.is_last = (prev == (unsigned int)(n_splits - 1));
  }
  __syncthreads();
  if (!sm.is_last) { leave(); return; }
  take_ticket();
  // A thread owns four output dims of one head and every third split: it first puts its partial
  // rows in flight (MERGE_BATCH independent 16-byte loads), then one warp per head turns the
  // splits' (max, sum) pairs into one weight per split, so a single memory round trip covers both.
  // (The stages are free: every warp is past the block-level combine.)
  constexpr int MERGE_GROUPS = DEC_THREADS / 128, MERGE_BATCH = 6;
  constexpr int F4 = D / 4;
  float* fac = reinterpret_cast<float*>(&sm.stage[0]);  // [n_splits][JQK_MAX_GROUP]
  float4* red = reinterpret_cast<float4*>(fac + (size_t)n_splits * JQK_MAX_GROUP);  // [MERGE_GROUPS][128]
  const int sg = tid >> 7, col = tid & 127;
  const int mh = col / F4, mi = col % F4;
  const bool m_active = mh < n_group;
  const float4* pa = reinterpret_cast<const float4*>(
      ws.part_acc + ((size_t)seq * n_q_heads + qh0 + (m_active ? mh : 0)) * ws.max_splits * JQK_MAX_DIM) + mi;
  float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int base = 0; base < n_splits; base += MERGE_GROUPS * MERGE_BATCH) {
    float4 raw[MERGE_BATCH];
#pragma unroll
    for (int j = 0; j < MERGE_BATCH; ++j) {
      const int s2 = base + sg + MERGE_GROUPS * j;
      raw[j] = (m_active && s2 < n_splits) ? __ldcg(pa + (size_t)s2 * (JQK_MAX_DIM / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (base == 0) {
      if (warp < n_group) {
        const size_t p0 = ((size_t)seq * n_q_heads + qh0 + warp) * ws.max_splits;
        const float m0 = (lane < n_splits) ? __ldcg(ws.part_m + p0 + lane) : -CUDART_INF_F;
        const float l0 = (lane < n_splits) ? __ldcg(ws.part_l + p0 + lane) : 0.f;
        float M = m0;
        for (int s2 = lane + 32; s2 < n_splits; s2 += 32) M = fmaxf(M, __ldcg(ws.part_m + p0 + s2));
        M = warp_max(M);
        const bool any = M > -CUDART_INF_F;
        float L = 0.f;
        if (lane < n_splits) {
          const float f = any ? exp2f(m0 - M) : 0.f;
          fac[lane * JQK_MAX_GROUP + warp] = f;
          L = l0 * f;
        }
        for (int s2 = lane + 32; s2 < n_splits; s2 += 32) {
          const float f = any ? exp2f(__ldcg(ws.part_m + p0 + s2) - M) : 0.f;
          fac[s2 * JQK_MAX_GROUP + warp] = f;
          L += __ldcg(ws.part_l + p0 + s2) * f;
        }
        L = warp_sum(L);
        if (lane == 0) sm.wl[0][warp] = L;
      }
      __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < MERGE_BATCH; ++j) {
      const int s2 = base + sg + MERGE_GROUPS * j;
      if (m_active && s2 < n_splits) {
        const float f = fac[s2 * JQK_MAX_GROUP + mh];
        sum.x = fmaf(raw[j].x, f, sum.x); sum.y = fmaf(raw[j].y, f, sum.y);
        sum.z = fmaf(raw[j].z, f, sum.z); sum.w = fmaf(raw[j].w, f, sum.w);
      }
    }
  }
  red[sg * 128 + col] = sum;
  __syncthreads();
  if (sg == 0 && m_active) {
    float4 a4 = red[col];
#pragma unroll
    for (int k = 1; k < MERGE_GROUPS; ++k) {
      const float4 o = red[k * 128 + col];
      a4.x += o.x; a4.y += o.y; a4.z += o.z; a4.w += o.w;
    }
    const float L = sm.wl[0][mh];
    if constexpr (VQ) {
      const float r = L > 0.f ? 1.f / L : 0.f;
      *reinterpret_cast<float4*>(yb + mh * 128 + 4 * mi) = make_float4(a4.x * r, a4.y * r, a4.z * r, a4.w * r);
      if (mi == 0) yb[JQK_MAX_GROUP * 128 + mh] = L > 0.f ? 1.f : 0.f;
    } else {
      const size_t o0 = ((size_t)seq * n_q_heads + qh0 + mh) * D + 4 * mi;
      store_out(out, out_dtype, o0 + 0, L > 0.f ? a4.x / L : 0.f);
      store_out(out, out_dtype, o0 + 1, L > 0.f ? a4.y / L : 0.f);
      store_out(out, out_dtype, o0 + 2, L > 0.f ? a4.z / L : 0.f);
      store_out(out, out_dtype, o0 + 3, L > 0.f ? a4.w / L : 0.f);
    }
  }
  if constexpr (VQ) {
    __syncthreads();
    values_to_output<D>(yb, n_group, vs, head, v_n_active, out, out_dtype, (size_t)seq * n_q_heads + qh0);
  }
  if (tid == 0) *counter = 0u;  // ready for the next launch that shares this workspace
  finish_ticket();
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }


static int q_blocks_for(int n_q_heads, int n_kv_heads) {
  const int group = n_q_heads / n_kv_heads;
  return (group + JQK_MAX_GROUP - 1) / JQK_MAX_GROUP;
}

}  // namespace jqk

using namespace jqk;

extern "C" size_t jqk_decode_workspace_bytes(int32_t n_seqs, int32_t n_q_heads, int32_t n_kv_heads,
                                             int32_t max_splits) {
  if (n_seqs <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_splits <= 0) return 0;
  const size_t rows = (size_t)n_seqs * n_q_heads * max_splits;
  const size_t groups = (size_t)n_seqs * n_kv_heads * q_blocks_for(n_q_heads, n_kv_heads);
  size_t b = 256;  // the launch-wide ticket of the append variant
  b += align_up(groups * sizeof(unsigned int), 256);
  b += align_up(rows * sizeof(float), 256) * 2;
  b += align_up(rows * JQK_MAX_DIM * sizeof(float), 256);
  b += align_up(groups * sizeof(TableRecord), 256);
  return b;
}

constexpr int MAX_SPLITS = 4096;  // the merge keeps one weight per split and head in shared memory

// Split size for a batch whose context lengths the host knows (host_lens == nullptr: all sequences
// at max_seq_len).  Blocks of `tps` keys run in waves of 148 (one block per SM); a block costs its
// keys plus a fixed share (table build or copy, block combine, merge) of about 1200 keys' worth of
// main-loop time.  The split that minimises waves x (tps + fixed) wins: for one short batch that is
// the smallest split that still fits one wave, for large batches a few thousand keys per block
// with the block count just under a multiple of 148.
static int32_t choose_split(const int32_t* host_lens, int n_seqs, int n_q_heads, int n_kv_heads, int max_seq_len) {
  const int unit = TILE_TOK * DEC_WARPS;  // one tile per warp: keeps the warps of a block level (384 keys)
  if (n_seqs <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_seq_len <= 0) return unit;
  const long long groups = (long long)n_kv_heads * q_blocks_for(n_q_heads, n_kv_heads);
  const long long fixed = 1200, slots = 148;
  long long best_cost = -1;
  int best = unit;
  const int max_units = (max_seq_len + unit - 1) / unit;
  for (int u = 1; u <= max_units; ++u) {
    const long long tps = (long long)u * unit;
    if ((max_seq_len + tps - 1) / tps > MAX_SPLITS) continue;
    long long blocks = 0;
    if (host_lens) {
      for (int s2 = 0; s2 < n_seqs; ++s2) blocks += (host_lens[s2] > 0) ? (host_lens[s2] + tps - 1) / tps : 0;
    } else {
      blocks = (long long)n_seqs * ((max_seq_len + tps - 1) / tps);
    }
    blocks *= groups;
    if (blocks <= 0) continue;
    const long long waves = (blocks + slots - 1) / slots;
    const long long cost = waves * (tps + fixed);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = (int)tps; }
  }
  return best;
}

extern "C" int32_t jqk_decode_default_split(int32_t n_seqs, int32_t n_q_heads, int32_t n_kv_heads,
                                            int32_t max_seq_len) {
  return choose_split(nullptr, n_seqs, n_q_heads, n_kv_heads, max_seq_len);
}

extern "C" int32_t jqk_decode_split_for_lengths(const int32_t* host_seq_lens, int32_t n_seqs, int32_t n_q_heads,
                                                int32_t n_kv_heads) {
  if (!host_seq_lens || n_seqs <= 0) return TILE_TOK * DEC_WARPS;
  int max_len = 0;
  for (int s2 = 0; s2 < n_seqs; ++s2) max_len = host_seq_lens[s2] > max_len ? host_seq_lens[s2] : max_len;
  return choose_split(host_seq_lens, n_seqs, n_q_heads, n_kv_heads, max_len);
}

extern "C" int32_t jqk_score_paged(const jqk_head_tables* tables, int32_t table_mode, const void* q, int32_t q_dtype,
                                   int32_t n_seqs, int32_t n_q_heads, int32_t n_queries,
                                   const int32_t* seq_lens, int32_t max_tokens, const int32_t* page_table,
                                   int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                                   float* scores, int32_t* status, void* stream) {
  int32_t rc = check_tables(tables);
  if (rc) return rc;
  if ((rc = check_decodable(tables, "jqk_score_paged"))) return rc;
  if (n_seqs < 0 || n_queries < 0 || max_tokens < 0) return fail(JQK_E_ARG, "negative size");
  if (n_seqs == 0 || n_queries == 0 || max_tokens == 0) return 0;
  if (!q || !seq_lens || !page_table || !k_pool || !scores) return fail(JQK_E_ARG, "null pointer argument");
  if (n_q_heads <= 0 || n_q_heads % tables->n_heads) return fail(JQK_E_ARG, "n_q_heads %d is not a multiple of the %d kv heads", n_q_heads, tables->n_heads);
  if (q_dtype != JQK_DTYPE_F32 && q_dtype != JQK_DTYPE_BF16 && q_dtype != JQK_DTYPE_F16) return fail(JQK_E_ARG, "unknown q dtype %d", q_dtype);
  if (table_mode != 0 && table_mode != 1) return fail(JQK_E_ARG, "table_mode must be 0 (fp32) or 1 (decode tables)");
  if ((long long)n_seqs * n_queries > 65535) return fail(JQK_E_UNSUPPORTED, "n_seqs * n_queries exceeds 65535");
  if (page_table_stride <= 0 || n_pages <= 0) return fail(JQK_E_ARG, "page_table_stride and n_pages must be positive");
  dim3 grid((max_tokens + SCORE_CHUNK - 1) / SCORE_CHUNK, tables->n_heads * q_blocks_for(n_q_heads, tables->n_heads),
            n_seqs * n_queries);
  JQK_SMEM_ONCE(score_kernel, sizeof(TableSmem), "score smem attribute");
  score_kernel<<<grid, SCORE_THREADS, sizeof(TableSmem), (cudaStream_t)stream>>>(
      *tables, table_mode, q, q_dtype, n_q_heads, n_queries, seq_lens, max_tokens, page_table, page_table_stride,
      n_pages, k_pool, scores, status);
  JQK_CUDA_OK(cudaGetLastError(), "score launch");
  return 0;
}

// One decode step; `v_tables` non-null: `v_pool` holds packed value codes of that compressor.
static int32_t decode_launch(const jqk_head_tables* tables, const jqk_head_tables* v_tables, const void* q, int32_t n_seqs,
                             int32_t n_q_heads, const int32_t* seq_lens, int32_t max_seq_len,
                             int32_t tokens_per_split, const int32_t* page_table,
                             int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                             const void* v_pool, void* out, int32_t out_dtype, void* workspace,
                             size_t workspace_bytes, int32_t* status, void* stream, const AppendSide* append = nullptr) {
  int32_t rc = check_tables(tables);
  if (rc) return rc;
  if ((rc = check_decodable(tables, "decode attention"))) return rc;
  if (v_tables) {
    rc = check_tables(v_tables);
    if (rc) return rc;
    if (v_tables->n_wide > 0 && !v_tables->value_decodable)
      return fail(JQK_E_UNSUPPORTED, "decode attention over packed values: the levels of a head's columns above 4 bits "
                                     "exceed the %d entries the kernel holds", VQ_WIDE_ENTRIES);
    if (v_tables->n_heads != tables->n_heads || v_tables->d != tables->d)
      return fail(JQK_E_LAYOUT, "key and value tables disagree on heads or head_dim");
  }
  if (n_seqs < 0 || max_seq_len < 0) return fail(JQK_E_ARG, "negative size");
  if (n_seqs == 0) return 0;
  if (!q || !seq_lens || !out) return fail(JQK_E_ARG, "null q, seq_lens or out");
  if (n_q_heads <= 0 || n_q_heads % tables->n_heads) return fail(JQK_E_ARG, "n_q_heads %d is not a multiple of the %d kv heads", n_q_heads, tables->n_heads);
  if (out_dtype != JQK_DTYPE_F32 && out_dtype != JQK_DTYPE_BF16) return fail(JQK_E_ARG, "out dtype must be f32 or bf16");
  if (n_seqs > 65535) return fail(JQK_E_UNSUPPORTED, "n_seqs %d exceeds 65535", n_seqs);
  if (tables->d != 128 && tables->d != 64) return fail(JQK_E_UNSUPPORTED, "decode attention is built for head_dim 64 and 128, got %d", tables->d);
  if (max_seq_len > 0 && (!page_table || !k_pool || !v_pool)) return fail(JQK_E_ARG, "null page_table, k_pool or v_pool");
  if (max_seq_len > 0 && (page_table_stride <= 0 || n_pages <= 0)) return fail(JQK_E_ARG, "page_table_stride and n_pages must be positive");
  if (max_seq_len > 0 && ((uintptr_t)v_pool % 16 || (uintptr_t)k_pool % 16)) return fail(JQK_E_ARG, "k_pool and v_pool must be 16-byte aligned");
  if (tokens_per_split == 0) tokens_per_split = jqk_decode_default_split(n_seqs, n_q_heads, tables->n_heads, max_seq_len);
  if (tokens_per_split < 0 || tokens_per_split % TILE_TOK) return fail(JQK_E_ARG, "tokens_per_split %d must be a positive multiple of %d", tokens_per_split, TILE_TOK);
  const int max_splits = max_seq_len > 0 ? (max_seq_len + tokens_per_split - 1) / tokens_per_split : 1;
  if (max_splits > MAX_SPLITS) return fail(JQK_E_UNSUPPORTED, "%d key splits exceed %d: use a larger tokens_per_split", max_splits, MAX_SPLITS);
  const int qbl = q_blocks_for(n_q_heads, tables->n_heads);
  DecodeWs ws{nullptr, nullptr, nullptr, nullptr, nullptr, max_splits, nullptr, 0};
  {
    const size_t need = jqk_decode_workspace_bytes(n_seqs, n_q_heads, tables->n_heads, max_splits);
    if (!workspace || workspace_bytes < need) return fail(JQK_E_WORKSPACE, "decode workspace needs %zu bytes, got %zu", need, workspace_bytes);
    if ((uintptr_t)workspace % 16) return fail(JQK_E_ARG, "workspace must be 16-byte aligned");
    const size_t rows = (size_t)n_seqs * n_q_heads * max_splits;
    char* p = (char*)workspace;
    ws.grid_ticket = (unsigned int*)p; p += 256;
    ws.counters = (unsigned int*)p; p += align_up((size_t)n_seqs * tables->n_heads * qbl * sizeof(unsigned int), 256);
    ws.part_m = (float*)p; p += align_up(rows * sizeof(float), 256);
    ws.part_l = (float*)p; p += align_up(rows * sizeof(float), 256);
    ws.part_acc = (float*)p; p += align_up(rows * JQK_MAX_DIM * sizeof(float), 256);
    ws.tables = (TableRecord*)p;
  }
  dim3 grid(max_splits, tables->n_heads * qbl, n_seqs);
  cudaStream_t st = (cudaStream_t)stream;
  // One wave of blocks or less: every block builds its own tables (no second launch on the
  // critical path).  More: a table kernel builds them once per group and the blocks copy them.
  const bool in_block = !v_tables && (long long)max_splits * tables->n_heads * qbl * n_seqs <= 148;
  if (max_seq_len > 0 && !in_block) {
    JQK_SMEM_ONCE(decode_tables_kernel, sizeof(TableSmem), "decode tables smem attribute");
    decode_tables_kernel<<<dim3(tables->n_heads * qbl, n_seqs), TBL_BUILD_THREADS, sizeof(TableSmem), st>>>(
        *tables, (const __nv_bfloat16*)q, n_q_heads, ws.tables);
    JQK_CUDA_OK(cudaGetLastError(), "decode tables launch");
    ws.late_wait = 1;
  }
  // Programmatic dependent launch: the blocks may become resident while the previous kernel on the
  // stream drains; they wait for it to complete (griddepcontrol.wait) before they touch memory.
  cudaLaunchAttribute pdl_attr[1];
  pdl_attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl_attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(DEC_THREADS);
  cfg.stream = st;
  cfg.attrs = pdl_attr;
  cfg.numAttrs = 1;
  ValueSide vs{nullptr, nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr, nullptr, nullptr, nullptr};
  AppendSide ap{};
  if (append) ap = *append;
  if (v_tables)
    vs = ValueSide{v_tables->desc, v_tables->col_meta, v_tables->cb_cols, v_tables->inv_rows, v_tables->center,
                   v_tables->n_heads, v_tables->words_per_record, v_tables->fwd_cols, v_tables->thresholds,
                   v_tables->wide_cb, v_tables->wide_thr};
#define JQK_LAUNCH_DECODE(DIM, INB, VQQ, APP, WID)                                                                    \
  do {                                                                                                                \
    cfg.dynamicSmemBytes = sizeof(DecodeSmemT<VQQ>);                                                                  \
    JQK_SMEM_ONCE((decode_kernel<DIM, INB, VQQ, APP, WID>), sizeof(DecodeSmemT<VQQ>), "decode smem attribute");       \
    JQK_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_kernel<DIM, INB, VQQ, APP, WID>, *tables, (const __nv_bfloat16*)q,    \
                                   n_q_heads, seq_lens, tokens_per_split, page_table, page_table_stride, n_pages,     \
                                   k_pool, v_pool, out, out_dtype, ws, status, vs, ap),                               \
                "decode launch");                                                                                     \
  } while (0)
  const bool wide = tables->n_wide > 0;   // byte-wide codes: head_dim 128 only
  if (wide && tables->d != 128) return fail(JQK_E_UNSUPPORTED, "codes above 4 bits are decoded for head_dim 128 only");
  if (v_tables && v_tables->n_wide > 0 && tables->d != 128)
    return fail(JQK_E_UNSUPPORTED, "value codes above 4 bits are decoded for head_dim 128 only");
  if (v_tables && append) {
    if (wide) JQK_LAUNCH_DECODE(128, false, true, true, true);
    else if (tables->d == 128) JQK_LAUNCH_DECODE(128, false, true, true, false);
    else JQK_LAUNCH_DECODE(64, false, true, true, false);
  } else if (v_tables) {
    if (wide) JQK_LAUNCH_DECODE(128, false, true, false, true);
    else if (tables->d == 128) JQK_LAUNCH_DECODE(128, false, true, false, false);
    else JQK_LAUNCH_DECODE(64, false, true, false, false);
  } else if (wide) {
    if (append) {
      if (in_block) JQK_LAUNCH_DECODE(128, true, false, true, true); else JQK_LAUNCH_DECODE(128, false, false, true, true);
    } else {
      if (in_block) JQK_LAUNCH_DECODE(128, true, false, false, true); else JQK_LAUNCH_DECODE(128, false, false, false, true);
    }
  } else if (append) {
    if (tables->d == 128) {
      if (in_block) JQK_LAUNCH_DECODE(128, true, false, true, false); else JQK_LAUNCH_DECODE(128, false, false, true, false);
    } else {
      if (in_block) JQK_LAUNCH_DECODE(64, true, false, true, false); else JQK_LAUNCH_DECODE(64, false, false, true, false);
    }
  } else if (tables->d == 128) {
    if (in_block) JQK_LAUNCH_DECODE(128, true, false, false, false); else JQK_LAUNCH_DECODE(128, false, false, false, false);
  } else {
    if (in_block) JQK_LAUNCH_DECODE(64, true, false, false, false); else JQK_LAUNCH_DECODE(64, false, false, false, false);
  }
#undef JQK_LAUNCH_DECODE
  JQK_CUDA_OK(cudaGetLastError(), "decode launch");
  return 0;
}

extern "C" int32_t jqk_decode_attend(const jqk_head_tables* tables, const void* q, int32_t n_seqs,
                                     int32_t n_q_heads, const int32_t* seq_lens, int32_t max_seq_len,
                                     int32_t tokens_per_split, const int32_t* page_table,
                                     int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                                     const void* v_pool, void* out, int32_t out_dtype, void* workspace,
                                     size_t workspace_bytes, int32_t* status, void* stream) {
  return decode_launch(tables, nullptr, q, n_seqs, n_q_heads, seq_lens, max_seq_len, tokens_per_split, page_table,
                       page_table_stride, n_pages, k_pool, v_pool, out, out_dtype, workspace, workspace_bytes, status, stream);
}

extern "C" int32_t jqk_decode_attend_packed_values(const jqk_head_tables* tables, const jqk_head_tables* v_tables,
                                                   const void* q, int32_t n_seqs, int32_t n_q_heads,
                                                   const int32_t* seq_lens, int32_t max_seq_len, int32_t tokens_per_split,
                                                   const int32_t* page_table, int32_t page_table_stride, int32_t n_pages,
                                                   const uint32_t* k_pool, const uint32_t* v_code_pool, void* out,
                                                   int32_t out_dtype, void* workspace, size_t workspace_bytes,
                                                   int32_t* status, void* stream) {
  if (!v_tables) return fail(JQK_E_ARG, "null value tables");
  return decode_launch(tables, v_tables, q, n_seqs, n_q_heads, seq_lens, max_seq_len, tokens_per_split, page_table,
                       page_table_stride, n_pages, k_pool, v_code_pool, out, out_dtype, workspace, workspace_bytes, status, stream);
}

// One step of a generate loop in one launch: the newest key and value row of every sequence go to
// position seq_lens[s] of its cache (compressed exactly as jqk_compress_paged would), the step
// attends over seq_lens[s] + 1 keys, and seq_lens is advanced by one when the launch is done.
static int32_t append_attend(const jqk_head_tables* tables, const jqk_head_tables* v_tables, const void* q,
                             const void* new_k, const void* new_v, int32_t k_dtype, int32_t v_dtype, int64_t k_seq_stride,
                             int64_t k_head_stride, int64_t v_seq_stride, int64_t v_head_stride, int32_t n_seqs,
                             int32_t n_q_heads, int32_t* seq_lens, int32_t max_seq_len, int32_t tokens_per_split,
                             const int32_t* page_table, int32_t page_table_stride, int32_t n_pages, uint32_t* k_pool,
                             void* v_pool, void* out, int32_t out_dtype, int32_t flags, void* workspace,
                             size_t workspace_bytes, int32_t* status, void* stream) {
  int32_t rc = check_tables(tables);
  if (rc) return rc;
  if (!new_k || !new_v) return fail(JQK_E_ARG, "null new_k or new_v");
  if (flags & ~JQK_APPEND_OWN_KEY_EXACT) return fail(JQK_E_ARG, "unknown flags 0x%x", flags);
  for (int32_t dt : {k_dtype, v_dtype})
    if (dt != JQK_DTYPE_F32 && dt != JQK_DTYPE_BF16 && dt != JQK_DTYPE_F16) return fail(JQK_E_ARG, "unknown dtype %d", dt);
  if (tables->center) return fail(JQK_E_UNSUPPORTED, "centred tables are for values; keys are appended uncentred");
  if (max_seq_len <= 0) return fail(JQK_E_ARG, "max_seq_len must cover the context after the append");
  AppendSide ap{new_k, new_v, k_dtype, v_dtype, (long long)k_seq_stride, (long long)k_head_stride, (long long)v_seq_stride,
                (long long)v_head_stride, k_pool, (__nv_bfloat16*)v_pool, seq_lens, n_seqs,
                (flags & JQK_APPEND_OWN_KEY_EXACT) ? 1 : 0};
  return decode_launch(tables, v_tables, q, n_seqs, n_q_heads, seq_lens, max_seq_len, tokens_per_split, page_table,
                       page_table_stride, n_pages, k_pool, v_pool, out, out_dtype, workspace, workspace_bytes, status,
                       stream, &ap);
}

extern "C" int32_t jqk_decode_append_attend(const jqk_head_tables* tables, const void* q, const void* new_k,
                                            const void* new_v, int32_t k_dtype, int32_t v_dtype, int64_t k_seq_stride,
                                            int64_t k_head_stride, int64_t v_seq_stride, int64_t v_head_stride,
                                            int32_t n_seqs, int32_t n_q_heads, int32_t* seq_lens, int32_t max_seq_len,
                                            int32_t tokens_per_split, const int32_t* page_table,
                                            int32_t page_table_stride, int32_t n_pages, uint32_t* k_pool, void* v_pool,
                                            void* out, int32_t out_dtype, int32_t flags, void* workspace,
                                            size_t workspace_bytes, int32_t* status, void* stream) {
  return append_attend(tables, nullptr, q, new_k, new_v, k_dtype, v_dtype, k_seq_stride, k_head_stride, v_seq_stride,
                       v_head_stride, n_seqs, n_q_heads, seq_lens, max_seq_len, tokens_per_split, page_table,
                       page_table_stride, n_pages, k_pool, v_pool, out, out_dtype, flags, workspace, workspace_bytes, status,
                       stream);
}

extern "C" int32_t jqk_decode_append_attend_packed_values(
    const jqk_head_tables* tables, const jqk_head_tables* v_tables, const void* q, const void* new_k, const void* new_v,
    int32_t k_dtype, int32_t v_dtype, int64_t k_seq_stride, int64_t k_head_stride, int64_t v_seq_stride,
    int64_t v_head_stride, int32_t n_seqs, int32_t n_q_heads, int32_t* seq_lens, int32_t max_seq_len,
    int32_t tokens_per_split, const int32_t* page_table, int32_t page_table_stride, int32_t n_pages, uint32_t* k_pool,
    uint32_t* v_code_pool, void* out, int32_t out_dtype, int32_t flags, void* workspace, size_t workspace_bytes,
    int32_t* status, void* stream) {
  if (!v_tables) return fail(JQK_E_ARG, "null value tables");
  return append_attend(tables, v_tables, q, new_k, new_v, k_dtype, v_dtype, k_seq_stride, k_head_stride, v_seq_stride,
                       v_head_stride, n_seqs, n_q_heads, seq_lens, max_seq_len, tokens_per_split, page_table,
                       page_table_stride, n_pages, k_pool, v_code_pool, out, out_dtype, flags, workspace, workspace_bytes,
                       status, stream);
}

extern "C" int32_t jqk_decode_attend_host(const jqk_head_tables* tables, const void* q_host, void* q_pinned,
                                          void* q_dev, int32_t n_seqs, int32_t n_q_heads, const int32_t* seq_lens,
                                          int32_t max_seq_len, int32_t tokens_per_split, const int32_t* page_table,
                                          int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                                          const void* v_pool, void* out_dev, void* out_host, int32_t out_dtype,
                                          void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  int32_t rc = check_tables(tables);
  if (rc) return rc;
  if (n_seqs <= 0 || n_q_heads <= 0) return fail(JQK_E_ARG, "n_seqs and n_q_heads must be positive");
  if (!q_host || !q_pinned || !out_host) return fail(JQK_E_ARG, "null host buffer");
  if (out_dtype != JQK_DTYPE_F32 && out_dtype != JQK_DTYPE_BF16) return fail(JQK_E_ARG, "out dtype must be f32 or bf16");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n = (size_t)n_seqs * n_q_heads * tables->d;
  const size_t q_bytes = n * 2, out_bytes = n * (out_dtype == JQK_DTYPE_F32 ? 4 : 2);
  if (q_pinned != q_host) memcpy(q_pinned, q_host, q_bytes);
  // Page-locked host memory is device-addressable.  Without q_dev the blocks read the query from
  // q_pinned themselves; without out_dev the block that finishes a head writes its result into
  // out_host itself (posted writes across the bus, no copy command after the kernel).
  if (q_dev) JQK_CUDA_OK(cudaMemcpyAsync(q_dev, q_pinned, q_bytes, cudaMemcpyHostToDevice, st), "query copy to the device");
  rc = jqk_decode_attend(tables, q_dev ? q_dev : q_pinned, n_seqs, n_q_heads, seq_lens, max_seq_len, tokens_per_split,
                         page_table, page_table_stride, n_pages, k_pool, v_pool, out_dev ? out_dev : out_host, out_dtype,
                         workspace, workspace_bytes, status, stream);
  if (rc) return rc;
  if (out_dev) JQK_CUDA_OK(cudaMemcpyAsync(out_host, out_dev, out_bytes, cudaMemcpyDeviceToHost, st), "result copy to the host");
  JQK_CUDA_OK(cudaStreamSynchronize(st), "waiting for the decode step");
  return 0;
}

// ---------------------------------------------------------------------------------------
// Decode attention for callers that cannot hand over a workspace
// ---------------------------------------------------------------------------------------
// The split-key partial results and the per-group tickets live in this fixed array, which every
// device that loads the library keeps until the process exits.
static __device__ __align__(256) unsigned char g_decode_scratch[JQK_DECODE_STATIC_SCRATCH_BYTES];

// Device address of g_decode_scratch on the current device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, so the address is asked for
// once per device, with that device current, and remembered.  At that moment the ticket area at the
// front of the array is also zeroed on `st`.  That is belt and braces: the array is zero when the
// module loads, and every launch that runs to its end leaves the tickets at zero (a context longer
// than the grid covers is clamped in the kernel, so the last block always turns up).  Only a
// launch that the driver aborts half-way can leave a ticket behind, and after that the context
// is unusable anyway.
// Host threads: the look-up is serialised by a mutex, so two threads that make the first call on a
// device at the same time get the same address and one clear; what they then launch on different
// streams still shares the one array and races on the GPU like any other overlapping pair of calls.
static int32_t decode_static_scratch(void** out, cudaStream_t st) {
  static std::atomic<void*> addr[64];
  static std::mutex first_call;
  int dev = 0;
  JQK_CUDA_OK(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= 64) return fail(JQK_E_UNSUPPORTED, "device ordinal %d outside 0..63", dev);
  void* p = addr[dev].load(std::memory_order_acquire);
  if (!p) {
    std::lock_guard<std::mutex> guard(first_call);
    p = addr[dev].load(std::memory_order_acquire);
    if (!p) {
      JQK_CUDA_OK(cudaGetSymbolAddress(&p, g_decode_scratch), "cudaGetSymbolAddress(decode scratch)");
      JQK_CUDA_OK(cudaMemsetAsync(p, 0, 65536, st), "clearing the decode tickets");
      addr[dev].store(p, std::memory_order_release);
    }
  }
  *out = p;
  return 0;
}

extern "C" int32_t jqk_decode_attend_static(const jqk_head_tables* tables, const void* q, int32_t n_seqs,
                                            int32_t n_q_heads, const int32_t* seq_lens, int32_t max_seq_len,
                                            int32_t tokens_per_split, const int32_t* page_table,
                                            int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                                            const void* v_pool, void* out, int32_t out_dtype, int32_t* status,
                                            void* stream) {
  int32_t rc = check_tables(tables);
  if (rc) return rc;
  if (n_seqs <= 0 || n_q_heads <= 0 || max_seq_len < 0)
    return jqk_decode_attend(tables, q, n_seqs, n_q_heads, seq_lens, max_seq_len, tokens_per_split, page_table,
                             page_table_stride, n_pages, k_pool, v_pool, out, out_dtype, nullptr, 0, status, stream);
  if (tokens_per_split == 0) tokens_per_split = jqk_decode_default_split(n_seqs, n_q_heads, tables->n_heads, max_seq_len);
  if (tokens_per_split < 0 || tokens_per_split % TILE_TOK) return fail(JQK_E_ARG, "tokens_per_split %d must be a positive multiple of %d", tokens_per_split, TILE_TOK);
  const int max_splits = max_seq_len > 0 ? (max_seq_len + tokens_per_split - 1) / tokens_per_split : 1;
  const size_t need = jqk_decode_workspace_bytes(n_seqs, n_q_heads, tables->n_heads, max_splits);
  if (need > (size_t)JQK_DECODE_STATIC_SCRATCH_BYTES)
    return fail(JQK_E_WORKSPACE,
                "this call needs %zu bytes of split scratch but the built-in array holds %d; use fewer splits "
                "(larger tokens_per_split), a smaller batch, or jqk_decode_attend with a caller workspace",
                need, (int)JQK_DECODE_STATIC_SCRATCH_BYTES);
  if (256 + (size_t)n_seqs * tables->n_heads * q_blocks_for(n_q_heads, tables->n_heads) * sizeof(unsigned int) > 65536)
    return fail(JQK_E_WORKSPACE, "too many (sequence, head group) pairs for the built-in ticket area");
  void* scratch = nullptr;
  rc = decode_static_scratch(&scratch, (cudaStream_t)stream);
  if (rc) return rc;
  return jqk_decode_attend(tables, q, n_seqs, n_q_heads, seq_lens, max_seq_len, tokens_per_split, page_table,
                           page_table_stride, n_pages, k_pool, v_pool, out, out_dtype, scratch,
                           (size_t)JQK_DECODE_STATIC_SCRATCH_BYTES, status, stream);
}

// ---------------------------------------------------------------------------------------
// Self-test of the bounded wait
// ---------------------------------------------------------------------------------------
namespace jqk {
// One warp waits on an mbarrier that nothing will ever complete, with the library's wait routine
// and a short limit.  The wait gives up, the status bit is set, the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(unsigned long long limit_ns, int32_t* status) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    bar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const bool done = bar_wait(&bar, 0, limit_ns);
  if (!done && threadIdx.x == 0 && status) atomicOr(status, JQK_STATUS_WAIT_EXPIRED);
}
}  // namespace jqk

extern "C" int32_t jqk_selftest_bounded_wait(int32_t limit_us, int32_t* status, void* stream) {
  if (!status) return fail(JQK_E_ARG, "null status word");
  if (limit_us <= 0 || limit_us > 100000) return fail(JQK_E_ARG, "limit_us %d outside 1..100000", limit_us);
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>((unsigned long long)limit_us * 1000ull, status);
  JQK_CUDA_OK(cudaGetLastError(), "bounded-wait self-test launch");
  return 0;
}
