// Round trip without a packed record: transform, nearest level, reconstruction, for any allocation of
// 0..8 bits per coordinate.
//
// The packed record holds at most 32 coordinates above 4 bits and 512 bits per key; the reference's
// own recipe (water-fill tail capped at 8 bits, experiments/stage1/toolkit/per_coord_quantization.py:365-379)
// goes beyond that from budgets of about 3.5 bits per coordinate on.  Its roundtrip (:123-165: x = k @ F,
// argmin over the coordinate's levels, gather, x_hat @ F^-1) never needs a record, so this kernel
// serves those allocations: codes by binary search over the exact fp32 decision thresholds of each
// coordinate (the same thresholds, and the same order of the dot product, as the packed path's
// CUDA-core kernels, so both give the same codes where both apply).
#include "jqk_common.cuh"

namespace jqk {

constexpr int DENSE_TOK = 8;        // rows per block
constexpr int DENSE_THREADS = 128;  // thread = coordinate

__global__ void __launch_bounds__(DENSE_THREADS)
roundtrip_dense_kernel(const float* __restrict__ fwd, const float* __restrict__ inv, const float* __restrict__ thr,
                       const float* __restrict__ levels, const int32_t* __restrict__ widths,
                       const float* __restrict__ center, int d, const void* __restrict__ rows, int dtype,
                       long long head_stride, long long token_stride, long long n_tokens, float* __restrict__ out,
                       uint8_t* __restrict__ codes) {
  __shared__ float xs[DENSE_TOK][JQK_MAX_DIM];
  const int h = blockIdx.y, j = threadIdx.x;
  const long long t0 = (long long)blockIdx.x * DENSE_TOK;
  const float mu = (center && j < d) ? center[(size_t)h * d + j] : 0.f;
#pragma unroll
  for (int t = 0; t < DENSE_TOK; ++t) {
    float v = 0.f;
    if (j < d && t0 + t < n_tokens)
      v = load_as_f32(rows, dtype, (size_t)h * head_stride + (size_t)(t0 + t) * token_stride + j) - mu;
    xs[t][j] = v;
  }
  __syncthreads();
  float x[DENSE_TOK];
#pragma unroll
  for (int t = 0; t < DENSE_TOK; ++t) x[t] = 0.f;
  if (j < d) {
    const float* F = fwd + (size_t)h * d * d + j;   // column j of the forward map
    for (int i = 0; i < d; ++i) {
      const float f = __ldg(F + (size_t)i * d);
#pragma unroll
      for (int t = 0; t < DENSE_TOK; ++t) x[t] = fmaf(xs[t][i], f, x[t]);
    }
  }
  __syncthreads();
  if (j < d) {
    const int w = widths[(size_t)h * d + j];
    const float* trow = thr + ((size_t)h * d + j) * 255;
    const float* lrow = levels + ((size_t)h * d + j) * 256;
#pragma unroll
    for (int t = 0; t < DENSE_TOK; ++t) {
      uint32_t code = 0;
      for (int step = (1 << w) >> 1; step >= 1; step >>= 1)
        code += (x[t] >= __ldg(trow + code + step - 1)) ? (uint32_t)step : 0u;
      xs[t][j] = __ldg(lrow + code);
      if (codes && t0 + t < n_tokens) codes[((size_t)h * n_tokens + (size_t)(t0 + t)) * d + j] = (uint8_t)code;
    }
  }
  __syncthreads();
  if (out && j < d) {
    const float* I = inv + (size_t)h * d * d + j;   // column j of the inverse map
#pragma unroll
    for (int t = 0; t < DENSE_TOK; ++t) x[t] = 0.f;
    for (int c = 0; c < d; ++c) {
      const float f = __ldg(I + (size_t)c * d);
#pragma unroll
      for (int t = 0; t < DENSE_TOK; ++t) x[t] = fmaf(xs[t][c], f, x[t]);
    }
#pragma unroll
    for (int t = 0; t < DENSE_TOK; ++t)
      if (t0 + t < n_tokens) out[((size_t)h * n_tokens + (size_t)(t0 + t)) * d + j] = x[t] + mu;
  }
}

}  // namespace jqk

using namespace jqk;

extern "C" int32_t jqk_roundtrip_dense(const float* forward_maps, const float* inverse_maps, const float* thresholds,
                                       const float* levels, const int32_t* widths, const float* center,
                                       int32_t n_heads, int32_t d, const void* rows, int32_t dtype,
                                       int64_t head_stride, int64_t token_stride, int64_t n_tokens, float* out,
                                       uint8_t* codes, void* stream) {
  if (!forward_maps || !inverse_maps || !thresholds || !levels || !widths) return fail(JQK_E_ARG, "null table pointer");
  if (n_heads <= 0 || d <= 0 || d > JQK_MAX_DIM) return fail(JQK_E_LAYOUT, "n_heads %d, d %d outside 1.. / 1..%d", n_heads, d, JQK_MAX_DIM);
  if (dtype != JQK_DTYPE_F32 && dtype != JQK_DTYPE_BF16 && dtype != JQK_DTYPE_F16) return fail(JQK_E_ARG, "unknown dtype %d", dtype);
  if (n_tokens < 0) return fail(JQK_E_ARG, "negative n_tokens");
  if (n_tokens == 0) return 0;
  if (!rows) return fail(JQK_E_ARG, "null rows");
  if (!out && !codes) return fail(JQK_E_ARG, "neither out nor codes given");
  if (token_stride < d) return fail(JQK_E_ARG, "token_stride %lld smaller than d", (long long)token_stride);
  const long long blocks = (n_tokens + DENSE_TOK - 1) / DENSE_TOK;
  if (blocks > 0x7fffffffll || n_heads > 65535) return fail(JQK_E_UNSUPPORTED, "too many rows or heads for one launch");
  roundtrip_dense_kernel<<<dim3((unsigned)blocks, (unsigned)n_heads), DENSE_THREADS, 0, (cudaStream_t)stream>>>(
      forward_maps, inverse_maps, thresholds, levels, widths, center, d, rows, dtype, (long long)head_stride,
      (long long)token_stride, (long long)n_tokens, out, codes);
  JQK_CUDA_OK(cudaGetLastError(), "dense roundtrip launch");
  return 0;
}
