// Shared host/device helpers for the jointqk_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/jointqk_b200.h"

namespace jqk {

// ---------------------------------------------------------------------------------------
// Host-side error reporting (thread-local message, integer return codes).
// ---------------------------------------------------------------------------------------
char* error_buffer();  // defined in jqk_api.cu, 512 bytes, thread-local

inline int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int32_t cuda_fail(cudaError_t e, const char* what) {
  snprintf(error_buffer(), 512, "%s: %s", what, cudaGetErrorString(e));
  return (int32_t)e;
}

#define JQK_CUDA_OK(call, what)                      \
  do {                                               \
    cudaError_t e__ = (call);                        \
    if (e__ != cudaSuccess) return ::jqk::cuda_fail(e__, what); \
  } while (0)

// Raises a kernel's dynamic shared-memory limit the first time it is launched on each device
// (a plain attribute call, kept out of the steady-state path and of stream captures).
#define JQK_SMEM_ONCE(kernel, bytes, what)                                                   \
  do {                                                                                       \
    static bool done__[64] = {false};                                                        \
    int dev__ = 0;                                                                           \
    JQK_CUDA_OK(cudaGetDevice(&dev__), "cudaGetDevice");                                     \
    if (dev__ < 0 || dev__ >= 64 || !done__[dev__]) {                                        \
      JQK_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                       (int)(bytes)), what);                                 \
      if (dev__ >= 0 && dev__ < 64) done__[dev__] = true;                                    \
    }                                                                                        \
  } while (0)

// Validates the table struct against the limits the kernels are written for.
int32_t check_tables(const jqk_head_tables* t);
int32_t check_decodable(const jqk_head_tables* t, const char* what);

// ---------------------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------------------
struct HeadDesc {
  int d, n_cols, n_active, n_words, n_a_words, n_c_words, n_tables, payload_bits;
  int wide_first, n_wide;   // columns of 5..8 bits: wide_first .. wide_first + n_wide - 1
};

__device__ __forceinline__ HeadDesc load_desc(const int32_t* desc, int head) {
  const int32_t* p = desc + (size_t)head * JQK_DESC_INTS;
  HeadDesc h;
  h.d = p[0]; h.n_cols = p[1]; h.n_active = p[2]; h.n_words = p[3];
  h.n_a_words = p[4]; h.n_c_words = p[5]; h.n_tables = p[6]; h.payload_bits = p[7];
  h.wide_first = p[30]; h.n_wide = p[31];
  return h;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

__device__ __forceinline__ float load_as_f32(const void* base, int dtype, size_t idx) {
  if (dtype == JQK_DTYPE_F32) return ((const float*)base)[idx];
  if (dtype == JQK_DTYPE_BF16) return __bfloat162float(((const __nv_bfloat16*)base)[idx]);
  return __half2float(((const __half*)base)[idx]);
}

// Physical page of logical page `lp` of sequence `s`, or -1 and a status bit: JQK_STATUS_BAD_LENGTH
// when `lp` lies outside the sequence's page-table row (a length or start the caller did not size
// the table for; the next row is never read), JQK_STATUS_BAD_PAGE when the table holds an index
// outside the pool.  The caller skips the access when -1 is returned.
__device__ __forceinline__ int lookup_page(const int32_t* page_table, int pt_stride, int s, int lp,
                                           int n_pages, int32_t* status) {
  if ((unsigned)lp >= (unsigned)pt_stride) {
    if (status) atomicOr(status, JQK_STATUS_BAD_LENGTH);
    return -1;
  }
  int p = page_table[(size_t)s * pt_stride + lp];
  if ((unsigned)p >= (unsigned)n_pages) {
    if (status) atomicOr(status, JQK_STATUS_BAD_PAGE);
    return -1;
  }
  return p;
}

// code = #{l : x >= thr[l]} over the 2^width - 1 sorted thresholds of a column.  Narrow columns
// (width <= 4) count through their 16-entry row; a wide column (5..8 bits) searches its 256-entry
// row, which gives the same count in 8 steps.
__device__ __forceinline__ uint32_t threshold_code(float x, int width, const float* __restrict__ narrow_row,
                                                   const float* __restrict__ wide_row) {
  uint32_t code = 0;
  if (width <= 4) {
    const int n_thr = (1 << width) - 1;
    for (int l = 0; l < n_thr; ++l) code += (x >= narrow_row[l]) ? 1u : 0u;
  } else {
    for (int step = (1 << width) >> 1; step >= 1; step >>= 1)
      code += (x >= wide_row[code + step - 1]) ? (uint32_t)step : 0u;
  }
  return code;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace jqk
