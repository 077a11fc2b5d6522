// Calibration second moments per kv head:  Sigma_Q (pooled over the group's q heads), Sigma_K
// and C_QK (group-mean query times key), accumulated as fp32 sums over tokens.
//
// Reference: the four einsums of compute_moments_from_tensors
// (experiments/stage1/calibration/compute_stats.py:118-123) and the streaming accumulators of
// experiments/stage1/toolkit/moments.py:68,110.  All three are X^T Y contractions over tokens:
//   sq[h] = sum_g Q_g^T Q_g,  sk[h] = K^T K,  cqk[h] = (1/G) sum_g Q_g^T K.
#include "jqk_common.cuh"

// Tensor-core path (jqk_moments_tc.cu): 0 = launched, 1 = call does not fit it, else an error code.
int32_t jqk_moments_tc_try(const void* q, const void* k, int32_t dtype, int64_t n_tokens, int64_t q_head_stride,
                           int64_t k_head_stride, int32_t n_q_heads, int32_t n_kv_heads, int32_t d, float* sq_sum,
                           float* sk_sum, float* cqk_sum, float* q_sum, float* k_sum, int32_t max_chain_tokens,
                           int32_t* status, cudaStream_t st);

namespace jqk {

constexpr int MOM_TOK = 32;      // tokens staged per step
constexpr int MOM_CHUNK = 512;   // tokens per thread block; short chunks keep the fp32 running sums accurate

// One block: (token chunk, kv head, which matrix).  256 threads, each an 8x8 patch of the
// d x d output (d <= 128); operands staged in shared memory as fp32.  The blocks of the two
// symmetric matrices also add up the first moments of the rows they stage (queries pooled over the
// group, keys), so those need no pass of their own.
template <typename T>
__global__ void __launch_bounds__(256)
moments_simt_kernel(const T* __restrict__ q, const T* __restrict__ k, long long n_tokens, long long q_head_stride,
                    long long k_head_stride, int n_q_heads, int n_kv_heads, int d, float* __restrict__ sq, float* __restrict__ sk,
                    float* __restrict__ cqk, float* __restrict__ q_sum, float* __restrict__ k_sum) {
  __shared__ float xs[MOM_TOK][JQK_MAX_DIM + 4];
  __shared__ float ys[MOM_TOK][JQK_MAX_DIM + 4];
  const int which = blockIdx.z;  // 0: sq, 1: sk, 2: cqk
  float* dst = which == 0 ? sq : (which == 1 ? sk : cqk);
  float* first = which == 0 ? q_sum : (which == 1 ? k_sum : nullptr);
  if (!dst && !first) return;
  float first_acc = 0.f;
  const int head = blockIdx.y;
  const int group = n_q_heads / n_kv_heads;
  const long long t_begin = (long long)blockIdx.x * MOM_CHUNK;
  const long long t_end = min(n_tokens, t_begin + MOM_CHUNK);
  const int tid = threadIdx.x;
  const int ty = tid >> 4, tx = tid & 15;  // rows 8*ty.., cols tx + 16*m
  float acc[8][8];
#pragma unroll
  for (int r = 0; r < 8; ++r)
#pragma unroll
    for (int m = 0; m < 8; ++m) acc[r][m] = 0.f;
  const int n_pass = (which == 1) ? 1 : group;
  for (int g = 0; g < n_pass; ++g) {
    const T* xsrc = (which == 1) ? k + (size_t)head * k_head_stride : q + (size_t)(head * group + g) * q_head_stride;
    const T* ysrc = (which == 0) ? xsrc : k + (size_t)head * k_head_stride;
    for (long long t0 = t_begin; t0 < t_end; t0 += MOM_TOK) {
      __syncthreads();
      for (int e = tid; e < MOM_TOK * d; e += blockDim.x) {
        const int t = e / d, i = e - t * d;
        const bool ok = t0 + t < t_end;
        xs[t][i] = ok ? to_f32<T>(xsrc[(size_t)(t0 + t) * d + i]) : 0.f;
        ys[t][i] = ok ? to_f32<T>(ysrc[(size_t)(t0 + t) * d + i]) : 0.f;
      }
      __syncthreads();
      if (first && tid < d) {
#pragma unroll 8
        for (int t = 0; t < MOM_TOK; ++t) first_acc += xs[t][tid];
      }
      if (!dst) continue;
#pragma unroll 4
      for (int t = 0; t < MOM_TOK; ++t) {
        float a[8], b[8];
#pragma unroll
        for (int r = 0; r < 8; ++r) a[r] = xs[t][8 * ty + r];
#pragma unroll
        for (int m = 0; m < 8; ++m) b[m] = ys[t][tx + 16 * m];
#pragma unroll
        for (int r = 0; r < 8; ++r)
#pragma unroll
          for (int m = 0; m < 8; ++m) acc[r][m] = fmaf(a[r], b[m], acc[r][m]);
      }
    }
  }
  if (first && tid < d) atomicAdd(first + (size_t)head * d + tid, first_acc);
  if (!dst) return;
  const float f = (which == 2) ? 1.0f / (float)group : 1.0f;
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    const int row = 8 * ty + r;
    if (row >= d) continue;
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      const int col = tx + 16 * m;
      if (col < d) atomicAdd(dst + ((size_t)head * d + row) * d + col, acc[r][m] * f);
    }
  }
}

}  // namespace jqk

using namespace jqk;

extern "C" size_t jqk_moments_workspace_bytes(int64_t n_tokens, int32_t n_q_heads, int32_t n_kv_heads, int32_t d) {
  (void)n_tokens; (void)n_q_heads; (void)n_kv_heads; (void)d;
  return sizeof(int32_t);  // one status word
}

extern "C" int32_t jqk_moments_accumulate(const void* q, const void* k, int32_t dtype, int64_t n_tokens,
                                          int64_t q_head_stride, int64_t k_head_stride, int32_t n_q_heads, int32_t n_kv_heads, int32_t d, float* sq_sum,
                                          float* sk_sum, float* cqk_sum, float* q_sum, float* k_sum,
                                          int32_t max_chain_tokens, void* workspace,
                                          size_t workspace_bytes, void* stream) {
  int32_t* status = (workspace && workspace_bytes >= sizeof(int32_t)) ? (int32_t*)workspace : nullptr;
  if (n_tokens < 0) return fail(JQK_E_ARG, "negative n_tokens");
  if (n_kv_heads <= 0 || n_q_heads <= 0 || n_q_heads % n_kv_heads) return fail(JQK_E_ARG, "GQA mismatch: q_heads=%d, kv_heads=%d", n_q_heads, n_kv_heads);
  if (d <= 0 || d > JQK_MAX_DIM || d % 16) return fail(JQK_E_UNSUPPORTED, "head_dim %d must be a multiple of 16 and at most %d", d, JQK_MAX_DIM);
  if (max_chain_tokens < 0) return fail(JQK_E_ARG, "negative max_chain_tokens");
  if (n_tokens == 0) return 0;
  const bool want_q = sq_sum || cqk_sum || q_sum;
  if (k_head_stride < n_tokens * d || (want_q && q_head_stride < n_tokens * d))
    return fail(JQK_E_ARG, "head stride smaller than n_tokens * d");
  if (!k || (want_q && !q)) return fail(JQK_E_ARG, "null q or k");
  if (n_kv_heads > 65535) return fail(JQK_E_UNSUPPORTED, "too many kv heads");
  {
    // bf16 inputs of head_dim 128 with at most 4 q heads per kv head go to the tensor-core kernel
    const int32_t r = jqk_moments_tc_try(q, k, dtype, n_tokens, q_head_stride, k_head_stride, n_q_heads, n_kv_heads, d,
                                         sq_sum, sk_sum, cqk_sum, q_sum, k_sum, max_chain_tokens, status, (cudaStream_t)stream);
    if (r != 1) return r;
  }
  const long long chunks = (n_tokens + MOM_CHUNK - 1) / MOM_CHUNK;
  if (chunks > 0x7fffffffLL) return fail(JQK_E_UNSUPPORTED, "n_tokens too large for one call");
  dim3 grid((unsigned)chunks, n_kv_heads, 3);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == JQK_DTYPE_BF16)
    moments_simt_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)q, (const __nv_bfloat16*)k, n_tokens,
                                                             q_head_stride, k_head_stride, n_q_heads, n_kv_heads, d, sq_sum, sk_sum, cqk_sum, q_sum, k_sum);
  else if (dtype == JQK_DTYPE_F16)
    moments_simt_kernel<__half><<<grid, 256, 0, st>>>((const __half*)q, (const __half*)k, n_tokens, q_head_stride, k_head_stride, n_q_heads,
                                                      n_kv_heads, d, sq_sum, sk_sum, cqk_sum, q_sum, k_sum);
  else if (dtype == JQK_DTYPE_F32)
    moments_simt_kernel<float><<<grid, 256, 0, st>>>((const float*)q, (const float*)k, n_tokens, q_head_stride, k_head_stride, n_q_heads,
                                                     n_kv_heads, d, sq_sum, sk_sum, cqk_sum, q_sum, k_sum);
  else
    return fail(JQK_E_ARG, "unknown dtype %d", dtype);
  JQK_CUDA_OK(cudaGetLastError(), "moments launch");
  return 0;
}
