// Prefill compression, reconstruction and code extraction for packed key pages.
//
// fp32 CUDA-core version: exact fp32 arithmetic for any key dtype (used for fp32 keys and as
// the numerical yardstick of the tensor-core transform).
//
// Reference semantics (experiments/stage1/toolkit/per_coord_quantization.py):
//   x   = keys.float() @ forward_map                       (:132-135)
//   idx = argmin_l |x_j - cb[j, l]|, first index on ties   (:156-157)
//   xh  = cb[j, idx]; k_hat = xh @ inverse_map             (:158-164)
// The argmin is evaluated through exact fp32 decision thresholds prepared on the host.

#include "jqk_common.cuh"

// Tensor-core path (jqk_compress_tc.cu): 0 = launched, 1 = call does not fit it, else an error code.
int32_t jqk_compress_tc_try(const jqk_head_tables* tables, const void* keys, int32_t key_dtype, int64_t seq_stride,
                            int64_t head_stride, int64_t token_stride, int32_t n_seqs, const int32_t* n_tokens,
                            const int32_t* seq_starts, int32_t max_tokens, const int32_t* page_table,
                            int32_t page_table_stride, int32_t n_pages, uint32_t* k_pool, int32_t* status,
                            cudaStream_t st);

namespace jqk {

constexpr int TILE_T = 64;     // keys per thread block
constexpr int XS_STRIDE = 129; // padded row of the transformed tile
constexpr int WS_ROWS = 32;    // rows of the map staged per step

struct PagedArgs {
  const int32_t* n_tokens;
  const int32_t* seq_starts;
  const int32_t* page_table;
  int32_t pt_stride;
  int32_t n_pages;
  int32_t max_tokens;
  int32_t* status;
};

__device__ __forceinline__ int meta_width(int m) { return m & 15; }
__device__ __forceinline__ int meta_bitpos(int m) { return (m >> 4) & 1023; }
__device__ __forceinline__ int meta_coord(int m) { return (m >> 16) & 255; }

// acc[r][m] += sum_i a[4*ty + r][i] * w[i][tx + 16*m], rows of `w` staged through shared memory.
// `a_s` is the [TILE_T][XS_STRIDE] operand tile, `w_g` the [k_dim][128] map in global memory.
__device__ __forceinline__ void tile_gemm(const float* a_s, const float* __restrict__ w_g, int k_dim,
                                          int n_out, float* w_s, float (&acc)[4][8]) {
  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;
  const int m_lim = (n_out + 15) >> 4;
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[r][m] = 0.f;
  for (int i0 = 0; i0 < k_dim; i0 += WS_ROWS) {
    __syncthreads();
    for (int e = tid; e < WS_ROWS * 128; e += blockDim.x) {
      int ii = e >> 7, c = e & 127;
      w_s[e] = (i0 + ii < k_dim) ? w_g[(size_t)(i0 + ii) * 128 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int ii = 0; ii < WS_ROWS; ++ii) {
      float a[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) a[r] = a_s[(4 * ty + r) * XS_STRIDE + i0 + ii];
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        if (m < m_lim) {
          float w = w_s[ii * 128 + tx + 16 * m];
#pragma unroll
          for (int r = 0; r < 4; ++r) acc[r][m] = fmaf(a[r], w, acc[r][m]);
        }
      }
    }
  }
  __syncthreads();
}

// Tokens of sequence `seq` this call handles: n_tokens[seq], cut to the max_tokens the call (its grid
// and its output rows) was sized for, with JQK_STATUS_BAD_LENGTH when it had to be cut.
__device__ __forceinline__ int call_tokens(const PagedArgs& pa, int seq) {
  int n = pa.n_tokens[seq];
  if (n > pa.max_tokens) {
    n = pa.max_tokens;
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && pa.status) atomicOr(pa.status, JQK_STATUS_BAD_LENGTH);
  }
  return n;
}

template <typename KT>
__global__ void __launch_bounds__(256)
compress_simt_kernel(jqk_head_tables tb, const KT* __restrict__ keys, int64_t seq_stride,
                     int64_t head_stride, int64_t token_stride, PagedArgs pa,
                     uint32_t* __restrict__ k_pool) {
  extern __shared__ float smem[];
  float* xs = smem;                        // [TILE_T][XS_STRIDE]
  float* ws = smem + TILE_T * XS_STRIDE;   // [WS_ROWS][128]
  const int head = blockIdx.y, seq = blockIdx.z;
  const int t0 = blockIdx.x * TILE_T;
  const int n_tok = call_tokens(pa, seq);
  if (t0 >= n_tok) return;
  const HeadDesc hd = load_desc(tb.desc, head);
  const int d = hd.d;
  const int tid = threadIdx.x;

  const KT* kbase = keys + (size_t)seq * seq_stride + (size_t)head * head_stride;
  const float* center = tb.center ? tb.center + (size_t)head * d : nullptr;
  for (int e = tid; e < TILE_T * d; e += blockDim.x) {
    int t = e / d, i = e - t * d;
    float v = 0.f;
    if (t0 + t < n_tok) {
      v = to_f32<KT>(kbase[(size_t)(t0 + t) * token_stride + i]);
      if (center) v -= center[i];   // fp32, as the reference's `states - mu` (v_compressor_adapter.py:70)
    }
    xs[t * XS_STRIDE + i] = v;
  }
  float acc[4][8];
  tile_gemm(xs, tb.fwd_cols + (size_t)head * d * 128, d, hd.n_cols, ws, acc);
  {
    const int ty = tid >> 4, tx = tid & 15;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int m = 0; m < 8; ++m) xs[(4 * ty + r) * XS_STRIDE + tx + 16 * m] = acc[r][m];
  }
  __syncthreads();

  const int32_t* wcb = tb.desc + (size_t)head * JQK_DESC_INTS + 8;
  const int32_t* meta = tb.col_meta + (size_t)head * 128;
  const float* thr = tb.thresholds + (size_t)head * 128 * 16;
  const int seq_start = pa.seq_starts ? pa.seq_starts[seq] : 0;
  const int wpr = tb.words_per_record;
  for (int item = tid; item < TILE_T * hd.n_words; item += blockDim.x) {
    const int t = item & (TILE_T - 1), w = item / TILE_T;
    if (t0 + t >= n_tok) continue;
    uint32_t word = 0;
    const int c_end = wcb[w + 1];
    for (int c = wcb[w]; c < c_end; ++c) {
      const int m = meta[c];
      const int width = meta_width(m);
      const float x = xs[t * XS_STRIDE + c];
      const float* wide_row = width > 4 ? tb.wide_thr + ((size_t)head * JQK_MAX_WIDE + (c - hd.wide_first)) * 256 : nullptr;
      const uint32_t code = threshold_code(x, width, thr + c * 16, wide_row);
      word |= code << (meta_bitpos(m) - 32 * w);
    }
    const int tok = seq_start + t0 + t;
    const int page = lookup_page(pa.page_table, pa.pt_stride, seq, tok / JQK_PAGE_TOKENS, pa.n_pages, pa.status);
    if (page < 0) continue;
    k_pool[(((size_t)page * tb.n_heads + head) * wpr + w) * JQK_PAGE_TOKENS + (tok % JQK_PAGE_TOKENS)] = word;
  }
}

// A handful of keys per sequence (the newest token of a generate loop): one block of 128 threads per
// (key, head, sequence), thread = column.  The dot product runs over the dims in ascending order
// with fused multiply-adds, the order of compress_simt_kernel's tile product, so both kernels give
// the same bits; the record is assembled with shared-memory atomics.
constexpr int TOKEN_KERNEL_MAX = 4;
template <typename KT>
__global__ void __launch_bounds__(128)
compress_token_kernel(jqk_head_tables tb, const KT* __restrict__ keys, int64_t seq_stride, int64_t head_stride,
                      int64_t token_stride, PagedArgs pa, uint32_t* __restrict__ k_pool) {
  __shared__ float krow[JQK_MAX_DIM];
  __shared__ uint32_t words[JQK_MAX_WORDS];
  const int t = blockIdx.x, head = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x;
  const int n_tok = call_tokens(pa, seq);
  if (t >= n_tok) return;
  const HeadDesc hd = load_desc(tb.desc, head);
  const int d = hd.d;
  const KT* row = keys + (size_t)seq * seq_stride + (size_t)head * head_stride + (size_t)t * token_stride;
  if (tid < JQK_MAX_DIM) {
    float v = 0.f;
    if (tid < d) {
      v = to_f32<KT>(row[tid]);
      if (tb.center) v -= tb.center[(size_t)head * d + tid];
    }
    krow[tid] = v;
  }
  if (tid < JQK_MAX_WORDS) words[tid] = 0u;
  __syncthreads();
  if (tid < hd.n_active) {
    const float* w = tb.fwd_cols + (size_t)head * d * 128 + tid;
    float x = 0.f;
#pragma unroll 8
    for (int i = 0; i < d; ++i) x = fmaf(krow[i], __ldg(w + (size_t)i * 128), x);
    const int m = tb.col_meta[(size_t)head * 128 + tid];
    const int width = meta_width(m);
    const float* wide_row = width > 4 ? tb.wide_thr + ((size_t)head * JQK_MAX_WIDE + (tid - hd.wide_first)) * 256 : nullptr;
    const uint32_t code = threshold_code(x, width, tb.thresholds + ((size_t)head * 128 + tid) * 16, wide_row);
    const int bp = meta_bitpos(m);
    atomicOr(&words[bp >> 5], code << (bp & 31));
  }
  __syncthreads();
  if (tid < hd.n_words) {
    const int tok = (pa.seq_starts ? pa.seq_starts[seq] : 0) + t;
    const int page = lookup_page(pa.page_table, pa.pt_stride, seq, tok / JQK_PAGE_TOKENS, pa.n_pages, pa.status);
    if (page >= 0)
      k_pool[(((size_t)page * tb.n_heads + head) * tb.words_per_record + tid) * JQK_PAGE_TOKENS + (tok % JQK_PAGE_TOKENS)] = words[tid];
  }
}

// Code of column `c` of the record of key `tok` (absolute position in the sequence).
__device__ __forceinline__ uint32_t fetch_code(const uint32_t* __restrict__ k_pool, size_t rec_base,
                                               int slot, int meta) {
  const int bp = meta_bitpos(meta);
  const uint32_t word = k_pool[rec_base + (size_t)(bp >> 5) * JQK_PAGE_TOKENS + slot];
  return (word >> (bp & 31)) & ((1u << meta_width(meta)) - 1u);
}

__global__ void __launch_bounds__(256)
decompress_simt_kernel(jqk_head_tables tb, PagedArgs pa, const uint32_t* __restrict__ k_pool,
                       float* __restrict__ out) {
  extern __shared__ float smem[];
  float* xs = smem;
  float* ws = smem + TILE_T * XS_STRIDE;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int t0 = blockIdx.x * TILE_T;
  const int n_tok = call_tokens(pa, seq);
  if (t0 >= n_tok) return;
  const HeadDesc hd = load_desc(tb.desc, head);
  const int d = hd.d, tid = threadIdx.x;
  const int32_t* meta = tb.col_meta + (size_t)head * 128;
  const float* cb = tb.cb_cols + (size_t)head * 128 * 16;
  const int seq_start = pa.seq_starts ? pa.seq_starts[seq] : 0;
  const int wpr = tb.words_per_record;

  for (int item = tid; item < TILE_T * 128; item += blockDim.x) {
    const int t = item & (TILE_T - 1), c = item / TILE_T;
    float v = 0.f;
    if (c < hd.n_active && t0 + t < n_tok) {
      const int tok = seq_start + t0 + t;
      const int page = lookup_page(pa.page_table, pa.pt_stride, seq, tok / JQK_PAGE_TOKENS, pa.n_pages, pa.status);
      if (page >= 0) {
        const size_t rec = ((size_t)page * tb.n_heads + head) * wpr * JQK_PAGE_TOKENS;
        const uint32_t code = fetch_code(k_pool, rec, tok % JQK_PAGE_TOKENS, meta[c]);
        v = meta_width(meta[c]) > 4 ? tb.wide_cb[((size_t)head * JQK_MAX_WIDE + (c - hd.wide_first)) * 256 + code]
                                    : cb[c * 16 + code];
      }
    }
    xs[t * XS_STRIDE + c] = v;
  }
  float acc[4][8];
  // inv_rows is [128][d]; tile_gemm expects rows of 128 floats, so d < 128 uses a strided view.
  if (d == 128) {
    tile_gemm(xs, tb.inv_rows + (size_t)head * 128 * 128, hd.n_cols, d, ws, acc);
  } else {
    // Generic path: stage rows of width d into a 128-wide buffer.
    const float* inv = tb.inv_rows + (size_t)head * 128 * d;
    const int ty = tid >> 4, tx = tid & 15;
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int m = 0; m < 8; ++m) acc[r][m] = 0.f;
    for (int c0 = 0; c0 < hd.n_cols; c0 += WS_ROWS) {
      __syncthreads();
      for (int e = tid; e < WS_ROWS * 128; e += blockDim.x) {
        int ii = e >> 7, i = e & 127;
        ws[e] = (c0 + ii < hd.n_cols && i < d) ? inv[(size_t)(c0 + ii) * d + i] : 0.f;
      }
      __syncthreads();
      for (int ii = 0; ii < WS_ROWS; ++ii) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          float a = xs[(4 * ty + r) * XS_STRIDE + c0 + ii];
#pragma unroll
          for (int m = 0; m < 8; ++m) acc[r][m] = fmaf(a, ws[ii * 128 + tx + 16 * m], acc[r][m]);
        }
      }
    }
    __syncthreads();
  }
  const int ty = tid >> 4, tx = tid & 15;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int t = 4 * ty + r;
    if (t0 + t >= n_tok) continue;
    float* o = out + (((size_t)seq * tb.n_heads + head) * pa.max_tokens + t0 + t) * d;
    const float* center = tb.center ? tb.center + (size_t)head * d : nullptr;
#pragma unroll
    for (int m = 0; m < 8; ++m)
      if (tx + 16 * m < d) o[tx + 16 * m] = center ? acc[r][m] + center[tx + 16 * m] : acc[r][m];
  }
}

__global__ void __launch_bounds__(256)
unpack_codes_kernel(jqk_head_tables tb, PagedArgs pa, const uint32_t* __restrict__ k_pool,
                    uint8_t* __restrict__ codes) {
  const int head = blockIdx.y, seq = blockIdx.z;
  const int t0 = blockIdx.x * TILE_T;
  const int n_tok = call_tokens(pa, seq);
  if (t0 >= n_tok) return;
  const HeadDesc hd = load_desc(tb.desc, head);
  const int d = hd.d, tid = threadIdx.x;
  const int32_t* meta = tb.col_meta + (size_t)head * 128;
  const int seq_start = pa.seq_starts ? pa.seq_starts[seq] : 0;
  const int wpr = tb.words_per_record;
  uint8_t* obase = codes + (((size_t)seq * tb.n_heads + head) * pa.max_tokens + t0) * d;
  const int rows = min(TILE_T, n_tok - t0);
  for (int e = tid; e < rows * d; e += blockDim.x) obase[e] = 0;
  __syncthreads();
  for (int item = tid; item < TILE_T * hd.n_active; item += blockDim.x) {
    const int t = item & (TILE_T - 1), c = item / TILE_T;
    if (t >= rows) continue;
    const int tok = seq_start + t0 + t;
    const int page = lookup_page(pa.page_table, pa.pt_stride, seq, tok / JQK_PAGE_TOKENS, pa.n_pages, pa.status);
    if (page < 0) continue;
    const size_t rec = ((size_t)page * tb.n_heads + head) * wpr * JQK_PAGE_TOKENS;
    const int m = meta[c];
    obase[(size_t)t * d + meta_coord(m)] = (uint8_t)fetch_code(k_pool, rec, tok % JQK_PAGE_TOKENS, m);
  }
}

static int32_t check_paged(const jqk_head_tables* tables, int32_t n_seqs, const int32_t* n_tokens,
                           int32_t max_tokens, const int32_t* page_table, int32_t pt_stride,
                           int32_t n_pages, const void* k_pool) {
  int32_t rc = check_tables(tables);
  if (rc) return rc;
  if (n_seqs < 0 || max_tokens < 0) return fail(JQK_E_ARG, "negative n_seqs or max_tokens");
  if (n_seqs > 65535) return fail(JQK_E_UNSUPPORTED, "n_seqs %d exceeds 65535", n_seqs);
  if (n_seqs == 0 || max_tokens == 0) return 0;
  if (!n_tokens || !page_table || !k_pool) return fail(JQK_E_ARG, "null n_tokens, page_table or k_pool");
  if (pt_stride <= 0 || n_pages <= 0) return fail(JQK_E_ARG, "page_table_stride and n_pages must be positive");
  return 0;
}

constexpr size_t kTileSmem = (size_t)(TILE_T * XS_STRIDE + WS_ROWS * 128) * sizeof(float);

}  // namespace jqk

using namespace jqk;

extern "C" int32_t jqk_compress_paged(const jqk_head_tables* tables, const void* keys, int32_t key_dtype,
                                      int64_t seq_stride, int64_t head_stride, int64_t token_stride,
                                      int32_t n_seqs, const int32_t* n_tokens, const int32_t* seq_starts,
                                      int32_t max_tokens, const int32_t* page_table,
                                      int32_t page_table_stride, int32_t n_pages, uint32_t* k_pool,
                                      int32_t* status, void* stream) {
  int32_t rc = check_paged(tables, n_seqs, n_tokens, max_tokens, page_table, page_table_stride, n_pages, k_pool);
  if (rc) return rc;
  if (n_seqs == 0 || max_tokens == 0) return 0;
  if (!keys) return fail(JQK_E_ARG, "null keys");
  if (token_stride < tables->d) return fail(JQK_E_ARG, "token_stride %lld smaller than d", (long long)token_stride);
  cudaStream_t st = (cudaStream_t)stream;
  PagedArgs pa{n_tokens, seq_starts, page_table, page_table_stride, n_pages, max_tokens, status};
  if (max_tokens <= TOKEN_KERNEL_MAX) {
    // a few keys per sequence (the append of a generate loop): one small block per key and head
    dim3 tgrid(max_tokens, tables->n_heads, n_seqs);
    if (key_dtype == JQK_DTYPE_F32)
      compress_token_kernel<float><<<tgrid, 128, 0, st>>>(*tables, (const float*)keys, seq_stride, head_stride, token_stride, pa, k_pool);
    else if (key_dtype == JQK_DTYPE_BF16)
      compress_token_kernel<__nv_bfloat16><<<tgrid, 128, 0, st>>>(*tables, (const __nv_bfloat16*)keys, seq_stride, head_stride, token_stride, pa, k_pool);
    else if (key_dtype == JQK_DTYPE_F16)
      compress_token_kernel<__half><<<tgrid, 128, 0, st>>>(*tables, (const __half*)keys, seq_stride, head_stride, token_stride, pa, k_pool);
    else
      return fail(JQK_E_ARG, "unknown key dtype %d", key_dtype);
    JQK_CUDA_OK(cudaGetLastError(), "token compress launch");
    return 0;
  }
  {
    // bf16 keys of head_dim 128 go to the tensor-core kernel; everything else (fp32 / fp16 keys,
    // other head sizes, unaligned strides, fewer than 128 keys) stays on the exact fp32 kernel.
    const int32_t r = jqk_compress_tc_try(tables, keys, key_dtype, seq_stride, head_stride, token_stride, n_seqs,
                                          n_tokens, seq_starts, max_tokens, page_table, page_table_stride, n_pages,
                                          k_pool, status, st);
    if (r != 1) return r;
  }
  dim3 grid((max_tokens + TILE_T - 1) / TILE_T, tables->n_heads, n_seqs);
#define JQK_LAUNCH_COMPRESS(KT)                                                                       \
  do {                                                                                                 \
    JQK_SMEM_ONCE(compress_simt_kernel<KT>, kTileSmem, "compress smem attribute");                      \
    compress_simt_kernel<KT><<<grid, 256, kTileSmem, st>>>(*tables, (const KT*)keys, seq_stride,        \
                                                           head_stride, token_stride, pa, k_pool);     \
  } while (0)
  if (key_dtype == JQK_DTYPE_F32) JQK_LAUNCH_COMPRESS(float);
  else if (key_dtype == JQK_DTYPE_BF16) JQK_LAUNCH_COMPRESS(__nv_bfloat16);
  else if (key_dtype == JQK_DTYPE_F16) JQK_LAUNCH_COMPRESS(__half);
  else return fail(JQK_E_ARG, "unknown key dtype %d", key_dtype);
#undef JQK_LAUNCH_COMPRESS
  JQK_CUDA_OK(cudaGetLastError(), "compress launch");
  return 0;
}

extern "C" int32_t jqk_decompress_paged(const jqk_head_tables* tables, int32_t n_seqs,
                                        const int32_t* n_tokens, const int32_t* seq_starts, int32_t max_tokens,
                                        const int32_t* page_table, int32_t page_table_stride,
                                        int32_t n_pages, const uint32_t* k_pool, float* out,
                                        int32_t* status, void* stream) {
  int32_t rc = check_paged(tables, n_seqs, n_tokens, max_tokens, page_table, page_table_stride, n_pages, k_pool);
  if (rc) return rc;
  if (n_seqs == 0 || max_tokens == 0) return 0;
  if (!out) return fail(JQK_E_ARG, "null out");
  dim3 grid((max_tokens + TILE_T - 1) / TILE_T, tables->n_heads, n_seqs);
  PagedArgs pa{n_tokens, seq_starts, page_table, page_table_stride, n_pages, max_tokens, status};
  JQK_SMEM_ONCE(decompress_simt_kernel, kTileSmem, "decompress smem attribute");
  decompress_simt_kernel<<<grid, 256, kTileSmem, (cudaStream_t)stream>>>(*tables, pa, k_pool, out);
  JQK_CUDA_OK(cudaGetLastError(), "decompress launch");
  return 0;
}

extern "C" int32_t jqk_unpack_codes(const jqk_head_tables* tables, int32_t n_seqs, const int32_t* n_tokens,
                                    int32_t max_tokens, const int32_t* page_table,
                                    int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                                    uint8_t* codes, int32_t* status, void* stream) {
  int32_t rc = check_paged(tables, n_seqs, n_tokens, max_tokens, page_table, page_table_stride, n_pages, k_pool);
  if (rc) return rc;
  if (n_seqs == 0 || max_tokens == 0) return 0;
  if (!codes) return fail(JQK_E_ARG, "null codes");
  dim3 grid((max_tokens + TILE_T - 1) / TILE_T, tables->n_heads, n_seqs);
  PagedArgs pa{n_tokens, nullptr, page_table, page_table_stride, n_pages, max_tokens, status};
  unpack_codes_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(*tables, pa, k_pool, codes);
  JQK_CUDA_OK(cudaGetLastError(), "unpack launch");
  return 0;
}
