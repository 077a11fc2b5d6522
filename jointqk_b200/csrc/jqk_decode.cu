// Scoring of packed keys through shared-memory lookup tables, and paged decode attention.
//
// Reference semantics: logits = q . k_hat / sqrt(d) with k_hat = x_hat @ inverse_map
// (experiments/stage1/toolkit/eval.py:20-21, per_coord_quantization.py:158-164), GQA grouping
// of metric_transform.py:21-27, then softmax and a product with V in fp32.
//
// Because k_hat = x_hat @ inverse_map, q . k_hat = q' . x_hat with q' = inverse_map @ q.  The
// query is projected once per thread block; each lookup (nibble slot or sub-byte field of a
// record, see layout.py) owns a 16-entry table holding, for the <=4 query heads of the group,
// the summed contribution q'_c * cb[c][code] of its coordinates.  Entries are 16-bit fixed
// point with one fp32 scale per query head, 8 bytes per entry, 128 bytes per table, so a
// warp-wide 8-byte read of one table never has a bank conflict.  No key is ever dequantised.
#include <math_constants.h>

#include "jqk_common.cuh"

namespace jqk {

constexpr int DEC_THREADS = 256;
constexpr int DEC_WARPS = DEC_THREADS / 32;
constexpr int TILE_TOK = 32;  // keys per warp step (two pages)
constexpr float kLog2e = 1.4426950408889634f;

struct LutView {
  const uint2* lut;  // [n_tables][16] (int16 x 4 heads)
  int n_a_words, n_c_words, n_words;
};

// ---- shared memory carve-up ------------------------------------------------------------
struct DecodeSmem {
  uint2 lut[JQK_MAX_TABLES * 16];        // 26,624 B
  float qraw[JQK_MAX_GROUP][JQK_MAX_DIM];  // 2 KB
  float qproj[2][JQK_MAX_COLS][JQK_MAX_GROUP];  // two partial sums over halves of the dims
  float scale[JQK_MAX_GROUP];
  unsigned int absmax[JQK_MAX_GROUP];
  float pbuf[DEC_WARPS][TILE_TOK][JQK_MAX_GROUP];
  float wm[DEC_WARPS][JQK_MAX_GROUP];
  float wl[DEC_WARPS][JQK_MAX_GROUP];
  float wacc[DEC_WARPS][JQK_MAX_GROUP][JQK_MAX_DIM];
  int is_last;
};

// One table entry in fp32 for the heads of the group.
__device__ __forceinline__ void table_entry(const int32_t* __restrict__ fields, const float* __restrict__ cb,
                                            const float (*qp)[JQK_MAX_GROUP], int e, float (&v)[JQK_MAX_GROUP]) {
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) v[h] = 0.f;
#pragma unroll
  for (int f = 0; f < 4; ++f) {
    const int fld = fields[f];
    if (fld < 0) break;
    const int col = fld & 255, width = (fld >> 8) & 15, shift = (fld >> 12) & 15;
    const float c = cb[col * 16 + ((e >> shift) & ((1 << width) - 1))];
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) v[h] = fmaf(qp[col][h], c, v[h]);
  }
}

// Projects the group's queries into column space and fills the lookup tables.
//   q_rows[h] : pointer to the d values of query head h of the group (h < n_group), q_dtype
template <typename SM>
__device__ void build_tables(SM& sm, const jqk_head_tables& tb, int head, const HeadDesc& hd,
                             const void* q_base, int q_dtype, size_t q_head_stride, int n_group) {
  const int tid = threadIdx.x;
  const int d = hd.d;
  for (int e = tid; e < JQK_MAX_GROUP * JQK_MAX_DIM; e += blockDim.x) {
    const int h = e / JQK_MAX_DIM, i = e % JQK_MAX_DIM;
    sm.qraw[h][i] = (h < n_group && i < d) ? load_as_f32(q_base, q_dtype, (size_t)h * q_head_stride + i) : 0.f;
  }
  if (tid < JQK_MAX_GROUP) sm.absmax[tid] = 0u;
  __syncthreads();
  {
    // thread -> (column c, half of the dims); rows of qproj_cols are contiguous in c
    const int c = tid & 127, half = tid >> 7;
    const float* P = tb.qproj_cols + (size_t)head * d * 128;
    float a[JQK_MAX_GROUP] = {0.f, 0.f, 0.f, 0.f};
    if (half < 2) {
      const int i_lo = half * (d / 2), i_hi = i_lo + d / 2;
#pragma unroll 8
      for (int i = i_lo; i < i_hi; ++i) {
        const float w = P[(size_t)i * 128 + c];
#pragma unroll
        for (int h = 0; h < JQK_MAX_GROUP; ++h) a[h] = fmaf(sm.qraw[h][i], w, a[h]);
      }
#pragma unroll
      for (int h = 0; h < JQK_MAX_GROUP; ++h) sm.qproj[half][c][h] = a[h];
    }
  }
  __syncthreads();
  if (tid < 128) {
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) sm.qproj[0][tid][h] += sm.qproj[1][tid][h];
  }
  __syncthreads();
  const int32_t* fields = tb.table_fields + (size_t)head * JQK_MAX_TABLES * 4;
  const float* cb = tb.cb_cols + (size_t)head * 128 * 16;
  const int n_entries = hd.n_tables * 16;
  float mx[JQK_MAX_GROUP] = {0.f, 0.f, 0.f, 0.f};
  for (int e = tid; e < n_entries; e += blockDim.x) {
    float v[JQK_MAX_GROUP];
    table_entry(fields + (e >> 4) * 4, cb, sm.qproj[0], e & 15, v);
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) mx[h] = fmaxf(mx[h], fabsf(v[h]));
  }
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) {
    const float m = warp_max(mx[h]);
    if ((tid & 31) == 0) atomicMax(&sm.absmax[h], __float_as_uint(m));  // non-negative floats order as uints
  }
  __syncthreads();
  if (tid < JQK_MAX_GROUP) {
    const float m = __uint_as_float(sm.absmax[tid]);
    sm.scale[tid] = (m > 0.f && m < CUDART_INF_F) ? m / 32767.f : 1.f;
  }
  __syncthreads();
  float inv[JQK_MAX_GROUP];
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) inv[h] = 1.f / sm.scale[h];
  for (int e = tid; e < n_entries; e += blockDim.x) {
    float v[JQK_MAX_GROUP];
    table_entry(fields + (e >> 4) * 4, cb, sm.qproj[0], e & 15, v);
    int q[JQK_MAX_GROUP];
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) q[h] = max(-32767, min(32767, __float2int_rn(v[h] * inv[h])));
    uint2 packed;
    packed.x = (uint32_t)(q[0] & 0xffff) | ((uint32_t)q[1] << 16);
    packed.y = (uint32_t)(q[2] & 0xffff) | ((uint32_t)q[3] << 16);
    sm.lut[e] = packed;
  }
  __syncthreads();
}

__device__ __forceinline__ void add_entry(const uint2 e, int (&acc)[JQK_MAX_GROUP]) {
  acc[0] += (int)(short)(e.x & 0xffffu);
  acc[1] += ((int)e.x) >> 16;
  acc[2] += (int)(short)(e.y & 0xffffu);
  acc[3] += ((int)e.y) >> 16;
}

// Integer score sums of one record.  `kp` points at word 0 of the key's slot inside its page
// (words are JQK_PAGE_TOKENS uint32 apart).
__device__ __forceinline__ void score_record(const uint32_t* __restrict__ kp, const LutView& lv,
                                             int (&acc)[JQK_MAX_GROUP]) {
  uint32_t ra[JQK_MAX_WORDS], rc[JQK_MAX_WORDS];
#pragma unroll
  for (int w = 0; w < JQK_MAX_WORDS; ++w) {
    ra[w] = (w < lv.n_a_words) ? __ldg(kp + w * JQK_PAGE_TOKENS) : 0u;
    rc[w] = (w < lv.n_c_words) ? __ldg(kp + (lv.n_words - 1 - w) * JQK_PAGE_TOKENS) : 0u;
  }
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) acc[h] = 0;
#pragma unroll
  for (int w = 0; w < JQK_MAX_WORDS; ++w) {
    if (w < lv.n_a_words) {
      const uint32_t x = ra[w];
#pragma unroll
      for (int k = 0; k < 8; ++k) add_entry(lv.lut[(w * 8 + k) * 16 + ((x >> (4 * k)) & 15u)], acc);
    }
  }
  const uint2* lc = lv.lut + lv.n_a_words * 8 * 16;
#pragma unroll
  for (int w = 0; w < JQK_MAX_WORDS; ++w) {
    if (w < lv.n_c_words) {
      const uint32_t x = rc[w];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const uint32_t y = x >> (8 * b);
        add_entry(lc[((w * 12 + b * 3 + 0) * 16) + (y & 7u)], acc);
        add_entry(lc[((w * 12 + b * 3 + 1) * 16) + ((y >> 3) & 7u)], acc);
        add_entry(lc[((w * 12 + b * 3 + 2) * 16) + ((y >> 6) & 3u)], acc);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Score kernel (evaluation / parity): one block per (token chunk, kv head x q block, seq x query)
// ---------------------------------------------------------------------------------------
constexpr int SCORE_CHUNK = 2048;

struct ScoreSmem {
  uint2 lut[JQK_MAX_TABLES * 16];
  float qraw[JQK_MAX_GROUP][JQK_MAX_DIM];
  float qproj[2][JQK_MAX_COLS][JQK_MAX_GROUP];
  float scale[JQK_MAX_GROUP];
  unsigned int absmax[JQK_MAX_GROUP];
};

__global__ void __launch_bounds__(DEC_THREADS)
score_kernel(jqk_head_tables tb, const void* __restrict__ q, int q_dtype, int n_q_heads, int n_queries,
             const int32_t* __restrict__ seq_lens, int max_tokens, const int32_t* __restrict__ page_table,
             int pt_stride, int n_pages, const uint32_t* __restrict__ k_pool, float* __restrict__ scores,
             int32_t* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  ScoreSmem& sm = *reinterpret_cast<ScoreSmem*>(smem_raw);
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
  build_tables(sm, tb, head, hd, q_ptr, q_dtype, (size_t)n_queries * d, n_group);
  LutView lv{sm.lut, hd.n_a_words, hd.n_c_words, hd.n_words};
  const float inv_sqrt_d = 1.0f / sqrtf((float)d);
  for (int tok = t_begin + threadIdx.x; tok < t_end; tok += blockDim.x) {
    const int page = lookup_page(page_table, pt_stride, seq, tok / JQK_PAGE_TOKENS, n_pages, status);
    if (page < 0) continue;
    const uint32_t* kp = k_pool + ((size_t)page * tb.n_heads + head) * tb.words_per_record * JQK_PAGE_TOKENS +
                         (tok % JQK_PAGE_TOKENS);
    int acc[JQK_MAX_GROUP];
    score_record(kp, lv, acc);
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) {
      if (h < n_group)
        scores[(((size_t)seq * n_q_heads + qh0 + h) * n_queries + qi) * max_tokens + tok] =
            (float)acc[h] * sm.scale[h] * inv_sqrt_d;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Decode attention
// ---------------------------------------------------------------------------------------
struct DecodeWs {
  float* part_m;     // [n_seqs][n_q_heads][max_splits]
  float* part_l;     // [n_seqs][n_q_heads][max_splits]
  float* part_acc;   // [n_seqs][n_q_heads][max_splits][128]
  unsigned int* counters;  // [n_seqs][n_kv_heads * q_blocks]
  int max_splits;
};

__device__ __forceinline__ void store_out(void* out, int out_dtype, size_t idx, float v) {
  if (out_dtype == JQK_DTYPE_F32) ((float*)out)[idx] = v;
  else ((__nv_bfloat16*)out)[idx] = __float2bfloat16(v);
}

__global__ void __launch_bounds__(DEC_THREADS)
decode_kernel(jqk_head_tables tb, const __nv_bfloat16* __restrict__ q, int n_q_heads,
              const int32_t* __restrict__ seq_lens, int tokens_per_split,
              const int32_t* __restrict__ page_table, int pt_stride, int n_pages,
              const uint32_t* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
              void* __restrict__ out, int out_dtype, DecodeWs ws, int32_t* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  DecodeSmem& sm = *reinterpret_cast<DecodeSmem*>(smem_raw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int group = n_q_heads / tb.n_heads;
  const int q_blocks = (group + JQK_MAX_GROUP - 1) / JQK_MAX_GROUP;
  const int head = blockIdx.y / q_blocks, qb = blockIdx.y % q_blocks;
  const int seq = blockIdx.z, split = blockIdx.x;
  const int len = seq_lens[seq];
  const int n_splits = (len + tokens_per_split - 1) / tokens_per_split;
  const HeadDesc hd = load_desc(tb.desc, head);
  const int d = hd.d;
  const int g0 = qb * JQK_MAX_GROUP, n_group = min(JQK_MAX_GROUP, group - g0);
  const int qh0 = head * group + g0;
  if (len <= 0) {  // empty context: defined output (zeros), written by split 0
    if (split == 0)
      for (int e = tid; e < n_group * d; e += blockDim.x)
        store_out(out, out_dtype, ((size_t)seq * n_q_heads + qh0 + e / d) * d + e % d, 0.f);
    return;
  }
  if (split >= n_splits) return;
  const int t_begin = split * tokens_per_split;
  const int t_end = min(len, t_begin + tokens_per_split);

  build_tables(sm, tb, head, hd, q + ((size_t)seq * n_q_heads + qh0) * d, JQK_DTYPE_BF16, (size_t)d, n_group);
  LutView lv{sm.lut, hd.n_a_words, hd.n_c_words, hd.n_words};
  float sc[JQK_MAX_GROUP];
  {
    const float f = kLog2e / sqrtf((float)d);
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) sc[h] = sm.scale[h] * f;
  }

  float m_run[JQK_MAX_GROUP], l_run[JQK_MAX_GROUP], o[JQK_MAX_GROUP][4];
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) {
    m_run[h] = -CUDART_INF_F; l_run[h] = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) o[h][k] = 0.f;
  }
  const size_t k_page_words = (size_t)tb.n_heads * tb.words_per_record * JQK_PAGE_TOKENS;
  const size_t v_page_elems = (size_t)tb.n_heads * JQK_PAGE_TOKENS * d;
  const bool lane_has_dims = 4 * lane < d;

  for (int t0 = t_begin + warp * TILE_TOK; t0 < t_end; t0 += DEC_WARPS * TILE_TOK) {
    const int tok = t0 + lane;
    const bool valid = tok < t_end;
    int page = -1;
    if (valid) page = lookup_page(page_table, pt_stride, seq, tok / JQK_PAGE_TOKENS, n_pages, status);
    float s[JQK_MAX_GROUP];
    if (page >= 0) {
      const uint32_t* kp = k_pool + (size_t)page * k_page_words +
                           (size_t)head * tb.words_per_record * JQK_PAGE_TOKENS + (tok % JQK_PAGE_TOKENS);
      int acc[JQK_MAX_GROUP];
      score_record(kp, lv, acc);
#pragma unroll
      for (int h = 0; h < JQK_MAX_GROUP; ++h) s[h] = (float)acc[h] * sc[h];
    } else {
#pragma unroll
      for (int h = 0; h < JQK_MAX_GROUP; ++h) s[h] = -CUDART_INF_F;
    }
    float p[JQK_MAX_GROUP];
    bool any = false;
#pragma unroll
    for (int h = 0; h < JQK_MAX_GROUP; ++h) {
      const float tmax = warp_max(s[h]);
      const float m_new = fmaxf(m_run[h], tmax);
      if (m_new == -CUDART_INF_F) { p[h] = 0.f; continue; }
      any = true;
      const float alpha = exp2f(m_run[h] - m_new);  // exp2(-inf) = 0 on the first tile
      p[h] = exp2f(s[h] - m_new);
      l_run[h] = l_run[h] * alpha + warp_sum(p[h]);
      m_run[h] = m_new;
#pragma unroll
      for (int k = 0; k < 4; ++k) o[h][k] *= alpha;
    }
    if (!any) continue;  // warp-uniform: every lane sees the same maxima
    *reinterpret_cast<float4*>(&sm.pbuf[warp][lane][0]) = make_float4(p[0], p[1], p[2], p[3]);
    __syncwarp();
    const int page_lo = __shfl_sync(0xffffffffu, page, 0);
    const int page_hi = __shfl_sync(0xffffffffu, page, 16);
    const int n_here = min(TILE_TOK, t_end - t0);
#pragma unroll 8
    for (int t = 0; t < n_here; ++t) {
      const int pg = (t < 16) ? page_lo : page_hi;
      if (pg < 0) continue;
      const float4 pw = *reinterpret_cast<const float4*>(&sm.pbuf[warp][t][0]);
      if (lane_has_dims) {
        const __nv_bfloat16* vp = v_pool + (size_t)pg * v_page_elems +
                                  ((size_t)head * JQK_PAGE_TOKENS + (t & 15)) * d + 4 * lane;
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(vp));
        const float v0 = __uint_as_float(raw.x << 16), v1 = __uint_as_float(raw.x & 0xffff0000u);
        const float v2 = __uint_as_float(raw.y << 16), v3 = __uint_as_float(raw.y & 0xffff0000u);
        o[0][0] = fmaf(pw.x, v0, o[0][0]); o[0][1] = fmaf(pw.x, v1, o[0][1]);
        o[0][2] = fmaf(pw.x, v2, o[0][2]); o[0][3] = fmaf(pw.x, v3, o[0][3]);
        o[1][0] = fmaf(pw.y, v0, o[1][0]); o[1][1] = fmaf(pw.y, v1, o[1][1]);
        o[1][2] = fmaf(pw.y, v2, o[1][2]); o[1][3] = fmaf(pw.y, v3, o[1][3]);
        o[2][0] = fmaf(pw.z, v0, o[2][0]); o[2][1] = fmaf(pw.z, v1, o[2][1]);
        o[2][2] = fmaf(pw.z, v2, o[2][2]); o[2][3] = fmaf(pw.z, v3, o[2][3]);
        o[3][0] = fmaf(pw.w, v0, o[3][0]); o[3][1] = fmaf(pw.w, v1, o[3][1]);
        o[3][2] = fmaf(pw.w, v2, o[3][2]); o[3][3] = fmaf(pw.w, v3, o[3][3]);
      }
    }
    __syncwarp();
  }

  // ---- combine the warps of this block -------------------------------------------------
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) {
    if (lane == 0) { sm.wm[warp][h] = m_run[h]; sm.wl[warp][h] = l_run[h]; }
    if (lane_has_dims)
      *reinterpret_cast<float4*>(&sm.wacc[warp][h][4 * lane]) = make_float4(o[h][0], o[h][1], o[h][2], o[h][3]);
  }
  __syncthreads();
  const bool single = (n_splits == 1);
  for (int e = tid; e < n_group * d; e += blockDim.x) {
    const int h = e / d, i = e % d;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, sm.wm[w][h]);
    float L = 0.f, A = 0.f;
    if (M > -CUDART_INF_F) {
#pragma unroll
      for (int w = 0; w < DEC_WARPS; ++w) {
        const float f = exp2f(sm.wm[w][h] - M);
        L += sm.wl[w][h] * f;
        A += sm.wacc[w][h][i] * f;
      }
    }
    const size_t qrow = (size_t)seq * n_q_heads + qh0 + h;
    if (single) {
      store_out(out, out_dtype, qrow * d + i, L > 0.f ? A / L : 0.f);
    } else {
      const size_t pidx = qrow * ws.max_splits + split;
      ws.part_acc[pidx * JQK_MAX_DIM + i] = A;
      if (i == 0) { ws.part_m[pidx] = M; ws.part_l[pidx] = L; }
    }
  }
  if (single) return;

  // ---- last block of this (sequence, head group) merges the splits -----------------------
  __threadfence();
  __syncthreads();
  unsigned int* counter = ws.counters + (size_t)seq * gridDim.y + blockIdx.y;
  if (tid == 0) {
    const unsigned int prev = atomicAdd(counter, 1u);
    sm.is_last = (prev == (unsigned int)(n_splits - 1));
  }
  __syncthreads();
  if (!sm.is_last) return;
  __threadfence();
  for (int e = tid; e < n_group * d; e += blockDim.x) {
    const int h = e / d, i = e % d;
    const size_t qrow = (size_t)seq * n_q_heads + qh0 + h;
    const size_t p0 = qrow * ws.max_splits;
    float M = -CUDART_INF_F;
    for (int s2 = 0; s2 < n_splits; ++s2) M = fmaxf(M, __ldcg(ws.part_m + p0 + s2));
    float L = 0.f, A = 0.f;
    if (M > -CUDART_INF_F) {
      for (int s2 = 0; s2 < n_splits; ++s2) {
        const float f = exp2f(__ldcg(ws.part_m + p0 + s2) - M);
        L += __ldcg(ws.part_l + p0 + s2) * f;
        A += __ldcg(ws.part_acc + (p0 + s2) * JQK_MAX_DIM + i) * f;
      }
    }
    store_out(out, out_dtype, qrow * d + i, L > 0.f ? A / L : 0.f);
  }
  if (tid == 0) *counter = 0u;  // ready for the next launch that shares this workspace
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
  size_t b = align_up((size_t)n_seqs * n_kv_heads * q_blocks_for(n_q_heads, n_kv_heads) * sizeof(unsigned int), 256);
  b += align_up(rows * sizeof(float), 256) * 2;
  b += align_up(rows * JQK_MAX_DIM * sizeof(float), 256);
  return b;
}

extern "C" int32_t jqk_decode_default_split(int32_t n_seqs, int32_t n_q_heads, int32_t n_kv_heads,
                                            int32_t max_seq_len) {
  if (n_seqs <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_seq_len <= 0) return TILE_TOK * DEC_WARPS;
  const long long items = (long long)n_seqs * n_kv_heads * q_blocks_for(n_q_heads, n_kv_heads);
  const long long target_blocks = 148LL * 2;  // two resident blocks per SM
  long long splits = target_blocks / items;
  if (splits < 1) splits = 1;
  long long tps = (max_seq_len + splits - 1) / splits;
  if (items * 4 >= target_blocks && tps > 2048) tps = 2048;  // many sequences: fixed granularity
  tps = (tps + TILE_TOK - 1) / TILE_TOK * TILE_TOK;
  if (tps < TILE_TOK * DEC_WARPS) tps = TILE_TOK * DEC_WARPS;
  return (int32_t)tps;
}

extern "C" int32_t jqk_score_paged(const jqk_head_tables* tables, const void* q, int32_t q_dtype,
                                   int32_t n_seqs, int32_t n_q_heads, int32_t n_queries,
                                   const int32_t* seq_lens, int32_t max_tokens, const int32_t* page_table,
                                   int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                                   float* scores, int32_t* status, void* stream) {
  int32_t rc = check_tables(tables);
  if (rc) return rc;
  if (n_seqs < 0 || n_queries < 0 || max_tokens < 0) return fail(JQK_E_ARG, "negative size");
  if (n_seqs == 0 || n_queries == 0 || max_tokens == 0) return 0;
  if (!q || !seq_lens || !page_table || !k_pool || !scores) return fail(JQK_E_ARG, "null pointer argument");
  if (n_q_heads <= 0 || n_q_heads % tables->n_heads) return fail(JQK_E_ARG, "n_q_heads %d is not a multiple of the %d kv heads", n_q_heads, tables->n_heads);
  if (q_dtype != JQK_DTYPE_F32 && q_dtype != JQK_DTYPE_BF16 && q_dtype != JQK_DTYPE_F16) return fail(JQK_E_ARG, "unknown q dtype %d", q_dtype);
  if ((long long)n_seqs * n_queries > 65535) return fail(JQK_E_UNSUPPORTED, "n_seqs * n_queries exceeds 65535");
  if (page_table_stride <= 0 || n_pages <= 0) return fail(JQK_E_ARG, "page_table_stride and n_pages must be positive");
  dim3 grid((max_tokens + SCORE_CHUNK - 1) / SCORE_CHUNK, tables->n_heads * q_blocks_for(n_q_heads, tables->n_heads),
            n_seqs * n_queries);
  JQK_SMEM_ONCE(score_kernel, sizeof(ScoreSmem), "score smem attribute");
  score_kernel<<<grid, DEC_THREADS, sizeof(ScoreSmem), (cudaStream_t)stream>>>(
      *tables, q, q_dtype, n_q_heads, n_queries, seq_lens, max_tokens, page_table, page_table_stride, n_pages,
      k_pool, scores, status);
  JQK_CUDA_OK(cudaGetLastError(), "score launch");
  return 0;
}

extern "C" int32_t jqk_decode_attend(const jqk_head_tables* tables, const void* q, int32_t n_seqs,
                                     int32_t n_q_heads, const int32_t* seq_lens, int32_t max_seq_len,
                                     int32_t tokens_per_split, const int32_t* page_table,
                                     int32_t page_table_stride, int32_t n_pages, const uint32_t* k_pool,
                                     const void* v_pool, void* out, int32_t out_dtype, void* workspace,
                                     size_t workspace_bytes, int32_t* status, void* stream) {
  int32_t rc = check_tables(tables);
  if (rc) return rc;
  if (n_seqs < 0 || max_seq_len < 0) return fail(JQK_E_ARG, "negative size");
  if (n_seqs == 0) return 0;
  if (!q || !seq_lens || !out) return fail(JQK_E_ARG, "null q, seq_lens or out");
  if (n_q_heads <= 0 || n_q_heads % tables->n_heads) return fail(JQK_E_ARG, "n_q_heads %d is not a multiple of the %d kv heads", n_q_heads, tables->n_heads);
  if (out_dtype != JQK_DTYPE_F32 && out_dtype != JQK_DTYPE_BF16) return fail(JQK_E_ARG, "out dtype must be f32 or bf16");
  if (n_seqs > 65535) return fail(JQK_E_UNSUPPORTED, "n_seqs %d exceeds 65535", n_seqs);
  if (tables->d % 4) return fail(JQK_E_UNSUPPORTED, "head_dim must be a multiple of 4");
  if (max_seq_len > 0 && (!page_table || !k_pool || !v_pool)) return fail(JQK_E_ARG, "null page_table, k_pool or v_pool");
  if (max_seq_len > 0 && (page_table_stride <= 0 || n_pages <= 0)) return fail(JQK_E_ARG, "page_table_stride and n_pages must be positive");
  if (tokens_per_split == 0) tokens_per_split = jqk_decode_default_split(n_seqs, n_q_heads, tables->n_heads, max_seq_len);
  if (tokens_per_split < 0 || tokens_per_split % TILE_TOK) return fail(JQK_E_ARG, "tokens_per_split %d must be a positive multiple of %d", tokens_per_split, TILE_TOK);
  const int max_splits = max_seq_len > 0 ? (max_seq_len + tokens_per_split - 1) / tokens_per_split : 1;
  const int qbl = q_blocks_for(n_q_heads, tables->n_heads);
  DecodeWs ws{nullptr, nullptr, nullptr, nullptr, max_splits};
  if (max_splits > 1) {
    const size_t need = jqk_decode_workspace_bytes(n_seqs, n_q_heads, tables->n_heads, max_splits);
    if (!workspace || workspace_bytes < need) return fail(JQK_E_WORKSPACE, "decode workspace needs %zu bytes, got %zu", need, workspace_bytes);
    if ((uintptr_t)workspace % 16) return fail(JQK_E_ARG, "workspace must be 16-byte aligned");
    const size_t rows = (size_t)n_seqs * n_q_heads * max_splits;
    char* p = (char*)workspace;
    ws.counters = (unsigned int*)p; p += align_up((size_t)n_seqs * tables->n_heads * qbl * sizeof(unsigned int), 256);
    ws.part_m = (float*)p; p += align_up(rows * sizeof(float), 256);
    ws.part_l = (float*)p; p += align_up(rows * sizeof(float), 256);
    ws.part_acc = (float*)p;
  }
  dim3 grid(max_splits, tables->n_heads * qbl, n_seqs);
  JQK_SMEM_ONCE(decode_kernel, sizeof(DecodeSmem), "decode smem attribute");
  decode_kernel<<<grid, DEC_THREADS, sizeof(DecodeSmem), (cudaStream_t)stream>>>(
      *tables, (const __nv_bfloat16*)q, n_q_heads, seq_lens, tokens_per_split, page_table, page_table_stride,
      n_pages, k_pool, (const __nv_bfloat16*)v_pool, out, out_dtype, ws, status);
  JQK_CUDA_OK(cudaGetLastError(), "decode launch");
  return 0;
}
