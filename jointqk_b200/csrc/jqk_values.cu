// Values into pages: bf16 V pool, dims-major and swizzled inside a (page, head) block.
//
// The reference keeps values untouched in the HF cache and appends the newest token each step
// (experiments/stage1/toolkit/jointqk_press.py:298-307); here they live in the paged pool the
// decode kernel reads (layout in include/jointqk_b200.h), so prefill and every appended token go
// through this transposition: rows [token][dim] in, blocks [dim][16 key slots] out.
//
// One block moves a tile of 64 destination slots (four pages) of one (sequence, kv head): rows are
// read with 16-byte loads where the strides allow, converted to bf16 and staged in shared memory;
// every 16-byte piece of a page block (8 key slots of one dim) is then written with one store, so a
// warp writes 512 contiguous bytes.  Pages that are only partly covered (an append that starts or
// ends inside a page) are written slot by slot, leaving the other slots as they were.
#include <type_traits>

#include "jqk_common.cuh"

namespace jqk {

constexpr int VS_TILE = 64;                    // destination slots per block
constexpr int VS_THREADS = 256;
constexpr int VS_PITCH = JQK_MAX_DIM * 2 + 16;  // bytes per staged token row

struct ValueArgs {
  const int32_t* n_tokens;
  const int32_t* seq_starts;
  const int32_t* page_table;
  int32_t pt_stride, n_pages, n_heads, d;
  long long seq_stride, head_stride, token_stride;
  int32_t vec_ok;  // rows may be read in 16-byte pieces
  int32_t* status;
};

template <typename T>
__device__ __forceinline__ void load8_as_bf16(const T* src, bool vec, __nv_bfloat16 (&out)[8]) {
  if constexpr (sizeof(T) == 2) {
    if (vec) {
      const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src));
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {   // already the pool's type: no conversion
        *reinterpret_cast<uint4*>(out) = raw;
        return;
      }
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) out[i] = __float2bfloat16(to_f32<T>(e[i]));
      return;
    }
  } else {
    if (vec) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src) + 1);
      out[0] = __float2bfloat16(a.x); out[1] = __float2bfloat16(a.y); out[2] = __float2bfloat16(a.z); out[3] = __float2bfloat16(a.w);
      out[4] = __float2bfloat16(b.x); out[5] = __float2bfloat16(b.y); out[6] = __float2bfloat16(b.z); out[7] = __float2bfloat16(b.w);
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = __float2bfloat16(to_f32<T>(src[i]));
}

template <typename T>
__global__ void __launch_bounds__(VS_THREADS)
store_values_kernel(const T* __restrict__ values, ValueArgs pa, __nv_bfloat16* __restrict__ v_pool) {
  __shared__ __align__(16) unsigned char rows[VS_TILE * VS_PITCH];
  __shared__ int pages[VS_TILE / JQK_PAGE_TOKENS];
  const int tid = threadIdx.x;
  const int head = blockIdx.y, seq = blockIdx.z;
  const int n_tok = pa.n_tokens[seq];
  const int start = pa.seq_starts ? pa.seq_starts[seq] : 0;
  if (n_tok <= 0 || start < 0) return;
  const int pos0 = (start / JQK_PAGE_TOKENS) * JQK_PAGE_TOKENS + blockIdx.x * VS_TILE;  // first slot of the tile
  if (pos0 >= start + n_tok) return;
  const int d = pa.d, chunks = d / 8;
  const T* src = values + (size_t)seq * pa.seq_stride + (size_t)head * pa.head_stride;
  for (int e = tid; e < VS_TILE * chunks; e += VS_THREADS) {
    const int t = e / chunks, c = e - t * chunks;
    const int tok = pos0 + t - start;  // index into this call's rows
    __nv_bfloat16 v8[8];
    if (tok >= 0 && tok < n_tok) {
      load8_as_bf16<T>(src + (size_t)tok * pa.token_stride + 8 * c, pa.vec_ok != 0, v8);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v8[i] = __float2bfloat16(0.f);
    }
    *reinterpret_cast<uint4*>(rows + t * VS_PITCH + c * 16) = *reinterpret_cast<const uint4*>(v8);
  }
  if (tid < VS_TILE / JQK_PAGE_TOKENS) {
    const int first = pos0 + tid * JQK_PAGE_TOKENS;  // a page takes part if any of its slots is written
    const bool touched = first < start + n_tok && first + JQK_PAGE_TOKENS > start;
    pages[tid] = touched ? lookup_page(pa.page_table, pa.pt_stride, seq, first / JQK_PAGE_TOKENS, pa.n_pages, pa.status) : -1;
  }
  __syncthreads();
  // unit = (page of the tile, dim, physical 16-byte half of the dim's row)
  const int units = (VS_TILE / JQK_PAGE_TOKENS) * d * 2;
  for (int u = tid; u < units; u += VS_THREADS) {
    const int p = u / (2 * d), r = u - p * 2 * d;
    const int dim = r >> 1, ph = r & 1;
    const int page = pages[p];
    if (page < 0) continue;
    const int half = ph ^ ((dim >> 2) & 1);                 // key slots 8*half .. 8*half+7 live in this piece
    const int t0 = p * JQK_PAGE_TOKENS + 8 * half;           // row of the tile
    const int tok0 = pos0 + t0 - start;
    __nv_bfloat16 v8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v8[i] = *reinterpret_cast<const __nv_bfloat16*>(rows + (t0 + i) * VS_PITCH + dim * 2);
    __nv_bfloat16* dst = v_pool + ((size_t)page * pa.n_heads + head) * (size_t)(JQK_PAGE_TOKENS * d) + dim * JQK_PAGE_TOKENS + ph * 8;
    if (tok0 >= 0 && tok0 + 8 <= n_tok) {
      *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v8);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (tok0 + i >= 0 && tok0 + i < n_tok) dst[i] = v8[i];
    }
  }
}

}  // namespace jqk

using namespace jqk;

extern "C" int32_t jqk_store_values_paged(const void* values, int32_t dtype, int64_t seq_stride, int64_t head_stride,
                                          int64_t token_stride, int32_t n_seqs, int32_t n_kv_heads, int32_t d,
                                          const int32_t* n_tokens, const int32_t* seq_starts, int32_t max_tokens,
                                          const int32_t* page_table, int32_t page_table_stride, int32_t n_pages,
                                          void* v_pool, int32_t* status, void* stream) {
  if (n_seqs < 0 || max_tokens < 0) return fail(JQK_E_ARG, "negative size");
  if (n_seqs == 0 || max_tokens == 0) return 0;
  if (!values || !n_tokens || !page_table || !v_pool) return fail(JQK_E_ARG, "null pointer argument");
  if (n_kv_heads <= 0 || n_kv_heads > 65535 || n_seqs > 65535) return fail(JQK_E_ARG, "n_kv_heads / n_seqs out of range");
  if (d <= 0 || d > JQK_MAX_DIM || d % 16) return fail(JQK_E_UNSUPPORTED, "head_dim %d must be a multiple of 16 and at most %d", d, JQK_MAX_DIM);
  if (page_table_stride <= 0 || n_pages <= 0) return fail(JQK_E_ARG, "page_table_stride and n_pages must be positive");
  if ((uintptr_t)v_pool % 16) return fail(JQK_E_ARG, "v_pool must be 16-byte aligned");
  const int esz = dtype == JQK_DTYPE_F32 ? 4 : 2;
  const bool vec = (uintptr_t)values % 16 == 0 && (seq_stride * esz) % 16 == 0 && (head_stride * esz) % 16 == 0 &&
                   (token_stride * esz) % 16 == 0;
  ValueArgs pa{n_tokens, seq_starts, page_table, page_table_stride, n_pages, n_kv_heads, d,
               (long long)seq_stride, (long long)head_stride, (long long)token_stride, vec ? 1 : 0, status};
  // a call may start inside a page: up to 15 slots of lead-in before its first row
  dim3 grid((unsigned)((max_tokens + JQK_PAGE_TOKENS - 1 + VS_TILE - 1) / VS_TILE), n_kv_heads, n_seqs);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == JQK_DTYPE_BF16)
    store_values_kernel<__nv_bfloat16><<<grid, VS_THREADS, 0, st>>>((const __nv_bfloat16*)values, pa, (__nv_bfloat16*)v_pool);
  else if (dtype == JQK_DTYPE_F16)
    store_values_kernel<__half><<<grid, VS_THREADS, 0, st>>>((const __half*)values, pa, (__nv_bfloat16*)v_pool);
  else if (dtype == JQK_DTYPE_F32)
    store_values_kernel<float><<<grid, VS_THREADS, 0, st>>>((const float*)values, pa, (__nv_bfloat16*)v_pool);
  else
    return fail(JQK_E_ARG, "unknown dtype %d", dtype);
  JQK_CUDA_OK(cudaGetLastError(), "value store launch");
  return 0;
}
