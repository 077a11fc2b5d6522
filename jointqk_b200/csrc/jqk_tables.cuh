// Query projection and lookup-table construction shared by the score and decode kernels.
//
// q . k_hat = q' . x_hat with q' = inverse_map @ q (k_hat = x_hat @ inverse_map,
// experiments/stage1/toolkit/per_coord_quantization.py:158-164).  Each lookup of a record owns a
// 16-entry table with, for the <=4 query heads of the group, the summed contribution
// q'_c * cb[c][code] of its coordinates.  Entries are 16-bit fixed point with one fp32 scale
// per query head: 8 bytes per entry, 128 bytes per table, so a warp-wide 8-byte read of one
// table never has a bank conflict.
//
// Fixed-point scale.  Tables of later record words belong to lower-variance coordinates, so a
// single scale would spend most of the 16 bits on a few large tables.  Instead word w (nibble
// words first, then byte words) is quantised at scale_h / 2^K_w with K non-decreasing in w; the
// scoring loop shifts its integer sums left by K_w - K_{w-1} before it adds the lookups of word
// w, which is exact, and the final sum is in units of scale_h / 2^K_last.  K_w is the largest
// shift that keeps every entry of every later-or-equal word inside 16 bits (capped at
// TBL_MAX_SHIFT so that the 32-bit sums cannot overflow).
//
// Columns of 5..8 bits (a byte each, in whole words between the nibble and the byte region) get a
// table of 2^width entries each (2 .. 16 slots of 16 entries), after the 16-entry ones; their words
// are scanned first (they are the highest-variance coordinates), one lookup per column.
#pragma once

#include <math_constants.h>
#include <stddef.h>

#include "jqk_common.cuh"

namespace jqk {

constexpr int TBL_THREADS = 256;  // threads that take part in the query projection (blocks may be larger)
constexpr int TBL_MAX_SHIFT = 7;  // 320 lookups x 2^16 x 2^7 < 2^32: the packed sums stay recoverable
constexpr int TBL_WORDS = 2 * JQK_MAX_WORDS;  // nibble words, then byte words

struct TableSmem {
  uint2 lut[JQK_MAX_TABLES * 16];                // 26,624 B: [table][16] x (int16 x 4 heads)
  float part[8][JQK_MAX_COLS][JQK_MAX_GROUP];    // 16,384 B: projection partial sums
  float qproj[JQK_MAX_COLS][JQK_MAX_GROUP];      //  2,048 B: projected queries, column space
  float qraw[JQK_MAX_GROUP][JQK_MAX_DIM];        //  2,048 B
  float cb[JQK_MAX_COLS * 16];                   //  8,192 B: staged codebooks
  int32_t fields[JQK_MAX_TABLES * 4];            //  3,328 B: staged table composition
  float scale[JQK_MAX_GROUP];                    // value of one unit of the final integer sum
  float wmax[TBL_WORDS][JQK_MAX_GROUP];          // per scan-order word: bound on |entry| per head
  int dshift[TBL_WORDS];                         // K_w - K_{w-1}
  unsigned int bias;                             // what the +32768 offsets of the low halves add up to
  int wcb[JQK_MAX_WORDS + 4];                    // first column of every physical record word
  alignas(8) uint16_t woff[JQK_MAX_WIDE];        // wide column i: byte offset of its 2^width-entry table,
                                                 // counted from the end of the 16-entry tables
  uint8_t wwidth[JQK_MAX_WIDE];                  // wide column i: its code width (5..8)
};

// Scan-order word of table t: nibble word t/8, or n_a_words + byte word.
__device__ __forceinline__ int table_word(int t, int n_a_words) {
  return (t < 8 * n_a_words) ? (t >> 3) : (n_a_words + (t - 8 * n_a_words) / 12);
}

// One table entry in fp32 for the heads of the group (all operands in shared memory).  The four
// possible fields are evaluated side by side (an absent field contributes zero), so their
// dependent shared-memory reads overlap.
__device__ __forceinline__ void table_entry(const TableSmem& sm, int e, float (&v)[JQK_MAX_GROUP]) {
  const int4 f4 = *reinterpret_cast<const int4*>(sm.fields + (e >> 4) * 4);
  const int fl[4] = {f4.x, f4.y, f4.z, f4.w};
  const int idx = e & 15;
  float c[4];
  float4 qp[4];
#pragma unroll
  for (int f = 0; f < 4; ++f) {
    const bool on = fl[f] >= 0;
    const int fld = on ? fl[f] : 0;
    const int col = fld & 255, width = (fld >> 8) & 15, shift = (fld >> 12) & 15;
    const float lv = sm.cb[col * 16 + ((idx >> shift) & ((1 << width) - 1))];
    c[f] = on ? lv : 0.f;
    qp[f] = *reinterpret_cast<const float4*>(sm.qproj[col]);
  }
  v[0] = fmaf(qp[3].x, c[3], fmaf(qp[2].x, c[2], fmaf(qp[1].x, c[1], qp[0].x * c[0])));
  v[1] = fmaf(qp[3].y, c[3], fmaf(qp[2].y, c[2], fmaf(qp[1].y, c[1], qp[0].y * c[0])));
  v[2] = fmaf(qp[3].z, c[3], fmaf(qp[2].z, c[2], fmaf(qp[1].z, c[1], qp[0].z * c[0])));
  v[3] = fmaf(qp[3].w, c[3], fmaf(qp[2].w, c[2], fmaf(qp[1].w, c[1], qp[0].w * c[0])));
}

// The global reads of the table build, issued into registers as early as the caller can: one
// memory round trip covers the projection matrix, the queries, the codebooks and the table
// composition, and it overlaps whatever the caller does before it needs the tables.
struct TableLoads {
  float4 w[JQK_MAX_DIM / 8];
  float qv[2];
  float4 cv[2];
  int4 fv;
  int wv;  // word_col_begin[tid] of the head descriptor (tid <= JQK_MAX_WORDS)
  // tables with wide columns only: warp i holds the 256-entry level row of wide column i (zero beyond
  // the column's levels), lane l the entries l + 32 u; and the descriptor of column tid
  float wl[8];
  int mv;
};

//   q_base + h * q_head_stride : the d values of query head h of the group (h < n_group)
// Needs blockDim.x >= TBL_THREADS.  Codebooks and table composition are read at their full
// per-head extent (both arrays are allocated at it), so the head descriptor is not needed yet.
template <bool WIDE = false>
__device__ __forceinline__ TableLoads issue_table_loads(const jqk_head_tables& tb, int head, int d, const void* q_base,
                                                        int q_dtype, size_t q_head_stride, int n_group) {
  static_assert(JQK_MAX_GROUP * JQK_MAX_DIM <= 2 * TBL_THREADS && JQK_MAX_COLS * 4 <= 2 * TBL_THREADS &&
                JQK_MAX_TABLES <= TBL_THREADS, "staging assumes at most two items per thread");
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int cg = tid & 31, rg = (tid >> 5) & 7;  // columns 4*cg..4*cg+3, rows rg + 8*r
  const bool projector = tid < TBL_THREADS;
  const float4* P4 = reinterpret_cast<const float4*>(tb.qproj_cols + (size_t)head * d * 128);
  const float4* cb4 = reinterpret_cast<const float4*>(tb.cb_cols + (size_t)head * 128 * 16);
  const int4* f4 = reinterpret_cast<const int4*>(tb.table_fields + (size_t)head * JQK_MAX_TABLES * 4);
  TableLoads ld;
#pragma unroll
  for (int r = 0; r < JQK_MAX_DIM / 8; ++r) {
    const int i = rg + 8 * r;
    ld.w[r] = (projector && i < d) ? __ldg(P4 + (size_t)i * 32 + cg) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int e = tid + u * nthr;
    const int h = e / JQK_MAX_DIM, i = e % JQK_MAX_DIM;
    ld.qv[u] = (e < JQK_MAX_GROUP * JQK_MAX_DIM && h < n_group && i < d)
                   ? load_as_f32(q_base, q_dtype, (size_t)h * q_head_stride + i) : 0.f;
    ld.cv[u] = (e < JQK_MAX_COLS * 4) ? __ldg(cb4 + e) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  ld.fv = (tid < JQK_MAX_TABLES) ? __ldg(f4 + tid) : make_int4(-1, -1, -1, -1);
  ld.wv = (tid <= JQK_MAX_WORDS) ? __ldg(tb.desc + (size_t)head * JQK_DESC_INTS + 8 + tid) : 0;
  if constexpr (WIDE) {
    // (the rows are allocated at their full extent for every head, so the head's count is not needed yet)
    const float* row = tb.wide_cb + ((size_t)head * JQK_MAX_WIDE + (tid >> 5)) * 256 + (tid & 31);
#pragma unroll
    for (int u = 0; u < 8; ++u) ld.wl[u] = (tid < 32 * JQK_MAX_WIDE) ? __ldg(row + 32 * u) : 0.f;
    ld.mv = (tid < JQK_MAX_COLS) ? __ldg(tb.col_meta + (size_t)head * JQK_MAX_COLS + tid) : 0;
  }
  return ld;
}

// Projects the group's queries into column space and fills the lookup tables from the reads that
// issue_table_loads() started.  After the block-wide projection every warp owns whole record
// words: it sums the partial projections of its word's columns and bounds that word's tables by
// itself, so only the word maxima cross warps (one barrier); every warp then derives all shifts
// and the entries are quantised by all threads.
// WIDE: the head may have wide columns; `wide_cb`: their 256-entry level rows.  The loads hold the
// rows of the first (number of warps) wide columns; further ones are read here.
template <bool WIDE = false>
__device__ __forceinline__ void build_tables(TableSmem& sm, const HeadDesc& hd, const TableLoads& ld,
                                             const float* __restrict__ wide_cb = nullptr) {
  const int tid = threadIdx.x, nthr = blockDim.x;  // nthr >= TBL_THREADS
  const int cg = tid & 31, rg = (tid >> 5) & 7;  // columns 4*cg..4*cg+3, rows rg + 8*r
  const int lane = tid & 31, warp = tid >> 5, n_warps = nthr >> 5;
  const bool projector = tid < TBL_THREADS;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int e = tid + u * nthr;
    if (e < JQK_MAX_GROUP * JQK_MAX_DIM) (&sm.qraw[0][0])[e] = ld.qv[u];
    if (e < JQK_MAX_COLS * 4) reinterpret_cast<float4*>(sm.cb)[e] = ld.cv[u];
  }
  if (tid < JQK_MAX_TABLES) reinterpret_cast<int4*>(sm.fields)[tid] = ld.fv;
  if (tid <= JQK_MAX_WORDS) sm.wcb[tid] = ld.wv;
  if constexpr (WIDE) {
    const int wi = tid - hd.wide_first;
    if (tid < JQK_MAX_COLS && wi >= 0 && wi < hd.n_wide) sm.wwidth[wi] = (uint8_t)(ld.mv & 15);
  }
  __syncthreads();
  if (projector) {
    float a[4][JQK_MAX_GROUP];
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int h = 0; h < JQK_MAX_GROUP; ++h) a[k][h] = 0.f;
#pragma unroll
    for (int r = 0; r < JQK_MAX_DIM / 8; ++r) {
      const int i = rg + 8 * r;  // beyond d: w[r] is zero and qraw is zero
      const float q0 = sm.qraw[0][i], q1 = sm.qraw[1][i], q2 = sm.qraw[2][i], q3 = sm.qraw[3][i];
      const float wk[4] = {ld.w[r].x, ld.w[r].y, ld.w[r].z, ld.w[r].w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        a[k][0] = fmaf(q0, wk[k], a[k][0]); a[k][1] = fmaf(q1, wk[k], a[k][1]);
        a[k][2] = fmaf(q2, wk[k], a[k][2]); a[k][3] = fmaf(q3, wk[k], a[k][3]);
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
      *reinterpret_cast<float4*>(sm.part[rg][4 * cg + k]) = make_float4(a[k][0], a[k][1], a[k][2], a[k][3]);
  }
  __syncthreads();
  const int n_wide = WIDE ? hd.n_wide : 0, n_w_words = (n_wide + 3) >> 2;
  const int n_a_words = hd.n_a_words, n_scan_words = n_w_words + hd.n_a_words + hd.n_c_words;
  const int n_narrow_tables = 8 * hd.n_a_words + 12 * hd.n_c_words;
  // column bounds |q'_c| * max |level| reuse the raw-query staging, which the projection is done with
  float4* colb = reinterpret_cast<float4*>(&sm.qraw[0][0]);  // [JQK_MAX_COLS]
  // slots of the wide columns' tables: exclusive prefix sum of 2^(width - 4)
  if (n_wide && warp == 0) {
    int slots = (lane < n_wide) ? (1 << ((int)sm.wwidth[lane] - 4)) : 0;
    int incl = slots;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int other = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += other;
    }
    if (lane < n_wide) sm.woff[lane] = (uint16_t)((incl - slots) * 128);
  }
  // wide columns, a warp each: the projected query and the bound |q'_c| * max |level| (the row is
  // zero beyond its levels, so its largest magnitude is that of the levels)
  if constexpr (WIDE) {
    for (int i = warp; i < n_wide; i += n_warps) {
      float big = 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u)
        big = fmaxf(big, fabsf(i < n_warps ? ld.wl[u] : __ldg(wide_cb + (size_t)i * 256 + lane + 32 * u)));
      big = warp_max(big);
      if (lane == 0) {
        const int c = hd.wide_first + i;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const float4 p = *reinterpret_cast<const float4*>(sm.part[r][c]);
          s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
        }
        *reinterpret_cast<float4*>(sm.qproj[c]) = s;
        colb[c] = make_float4(fabsf(s.x) * big, fabsf(s.y) * big, fabsf(s.z) * big, fabsf(s.w) * big);
      }
    }
    if (n_wide) __syncthreads();   // (block-uniform)
  }
  // ---- per warp and scan word: projected queries of the word's columns, bound of its tables ----
  for (int sw = warp; sw < n_scan_words; sw += n_warps) {
    // scan order: wide words (physical words n_a_words ..), nibble words (0 ..), byte words (from the end)
    const bool is_wide = sw < n_w_words;
    const int nw = sw - n_w_words;                                                // index among the narrow scan words
    const int pw = is_wide ? n_a_words + sw : (nw < n_a_words) ? nw : hd.n_words - 1 - (nw - n_a_words);  // physical word
    const int c_first = sm.wcb[pw], n_c = sm.wcb[pw + 1] - c_first;            // <= 32 columns
    if (lane < n_c && !is_wide) {
      const int c = c_first + lane;
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float4 p = *reinterpret_cast<const float4*>(sm.part[r][c]);
        s.x += p.x; s.y += p.y; s.z += p.z; s.w += p.w;
      }
      *reinterpret_cast<float4*>(sm.qproj[c]) = s;
      // levels are sorted and padded with zeros: the largest magnitude of a row is its largest |level|
      float big = 0.f;
#pragma unroll
      for (int l4 = 0; l4 < 4; ++l4) {
        const float4 lv = *reinterpret_cast<const float4*>(sm.cb + c * 16 + 4 * l4);
        big = fmaxf(fmaxf(big, fmaxf(fabsf(lv.x), fabsf(lv.y))), fmaxf(fabsf(lv.z), fabsf(lv.w)));
      }
      colb[c] = make_float4(fabsf(s.x) * big, fabsf(s.y) * big, fabsf(s.z) * big, fabsf(s.w) * big);
    }
    __syncwarp();
    // The fields of a table take their codes independently, so the largest |entry| of a table is at
    // most the sum of its columns' bounds; lane k owns table k of the word.  (A wide word: one
    // single-column table per column.)
    const int t_first = (nw < n_a_words) ? 8 * nw : 8 * n_a_words + 12 * (nw - n_a_words);
    const int n_t = is_wide ? 0 : (nw < n_a_words) ? 8 : 12;
    float4 m = make_float4(0.f, 0.f, 0.f, 0.f);
    if (is_wide && lane < n_c) m = colb[c_first + lane];
    if (lane < n_t) {
      const int4 f4 = *reinterpret_cast<const int4*>(sm.fields + (t_first + lane) * 4);
      const int fl[4] = {f4.x, f4.y, f4.z, f4.w};
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        if (fl[f] >= 0) {
          const float4 cbd = colb[fl[f] & 255];
          m.x += cbd.x; m.y += cbd.y; m.z += cbd.z; m.w += cbd.w;
        }
      }
    }
    m.x = warp_max(m.x); m.y = warp_max(m.y); m.z = warp_max(m.z); m.w = warp_max(m.w);
    if (lane == 0) *reinterpret_cast<float4*>(sm.wmax[sw]) = make_float4(m.x, m.y, m.z, m.w);
  }
  __syncthreads();
  // ---- every warp derives the per-word shifts from the word maxima (lane w owns scan word w) ----
  float wm[JQK_MAX_GROUP], gm[JQK_MAX_GROUP];
  int fit = TBL_MAX_SHIFT;
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) {
    wm[h] = (lane < n_scan_words) ? sm.wmax[lane][h] : 0.f;
    gm[h] = warp_max(wm[h]);
    if (!(gm[h] < CUDART_INF_F)) gm[h] = 0.f;
    // largest shift that keeps this word inside 16 bits for head h: floor(log2(gm / wm)), which for
    // positive floats is the difference of their bit patterns shifted down by the mantissa width
    if (gm[h] > 0.f && wm[h] > 0.f) fit = min(fit, max(0, (__float_as_int(gm[h]) - __float_as_int(wm[h])) >> 23));
  }
  // K_w = min over later-or-equal words (suffix minimum): non-decreasing along the scan
  int kw = (lane < n_scan_words) ? fit : TBL_MAX_SHIFT;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int other = __shfl_down_sync(0xffffffffu, kw, o);
    if (lane + o < 32) kw = min(kw, other);
  }
  const int k_last = __shfl_sync(0xffffffffu, kw, max(n_scan_words - 1, 0));
  if (warp == 0) {
    const int prev = __shfl_up_sync(0xffffffffu, kw, 1);
    unsigned int term = 0u;
    if (lane < n_scan_words) {
      sm.dshift[lane] = kw - (lane ? prev : 0);
      const int lookups = lane < n_w_words ? min(4, n_wide - 4 * lane) : (lane - n_w_words < n_a_words ? 8 : 12);
      term = (unsigned int)(lookups * 32768) << (k_last - kw);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) term += __shfl_xor_sync(0xffffffffu, term, o);
    if (lane == 0) sm.bias = term;
  }
  // One unit at shift 0.  The bound on |entry| maps to 32750, not 32767: the quantising pass rounds
  // with a magic-number add that must never leave the signed 16-bit range.
  float inv[JQK_MAX_GROUP];
#pragma unroll
  for (int h = 0; h < JQK_MAX_GROUP; ++h) {
    const float base = (gm[h] > 0.f) ? gm[h] * (1.f / 32750.f) : 1.f;
    inv[h] = __frcp_rn(base);
    if (tid == h) sm.scale[h] = base * __int_as_float((127 - (n_scan_words ? k_last : 0)) << 23);  // base / 2^k_last
  }
  // ---- all threads: quantise the entries (every warp knows every word's shift) ----
  const int n_entries = n_narrow_tables * 16;
  for (int e0 = warp * 32; e0 < n_entries; e0 += nthr) {
    const int e = e0 + lane;  // n_entries is a multiple of 16: the second half-warp may be past the end
    const int sw = n_w_words + table_word(min(e, n_entries - 1) >> 4, n_a_words);
    const float up = (float)(1 << __shfl_sync(0xffffffffu, kw, sw));
    if (e < n_entries) {
      float v[JQK_MAX_GROUP];
      table_entry(sm, e, v);
      // round to nearest by adding 1.5 * 2^23: the low 16 bits of the sum are the two's complement
      // value (even heads: plus 32768, the offset of the low halves)
      const uint32_t q0 = __float_as_uint(fmaf(v[0], inv[0] * up, 12582912.f + 32768.f));
      const uint32_t q1 = __float_as_uint(fmaf(v[1], inv[1] * up, 12582912.f));
      const uint32_t q2 = __float_as_uint(fmaf(v[2], inv[2] * up, 12582912.f + 32768.f));
      const uint32_t q3 = __float_as_uint(fmaf(v[3], inv[3] * up, 12582912.f));
      // high half: signed value of the odd head; low half: value of the even head plus 32768
      sm.lut[e] = make_uint2(__byte_perm(q0, q1, 0x5410), __byte_perm(q2, q3, 0x5410));
    }
  }
  // the tables of the wide columns: entry = q'_c * level, behind the 16-entry tables; a warp per column
  if constexpr (WIDE) {
    for (int i = warp; i < n_wide; i += n_warps) {
      const int levels = 1 << (int)sm.wwidth[i];
      const float up = (float)(1 << __shfl_sync(0xffffffffu, kw, i >> 2));
      const float4 qp = *reinterpret_cast<const float4*>(sm.qproj[hd.wide_first + i]);
      uint2* dst = sm.lut + n_entries + ((int)sm.woff[i] >> 3);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int e = lane + 32 * u;
        const float lv = i < n_warps ? ld.wl[u] : __ldg(wide_cb + (size_t)i * 256 + e);
        const uint32_t q0 = __float_as_uint(fmaf(qp.x * lv, inv[0] * up, 12582912.f + 32768.f));
        const uint32_t q1 = __float_as_uint(fmaf(qp.y * lv, inv[1] * up, 12582912.f));
        const uint32_t q2 = __float_as_uint(fmaf(qp.z * lv, inv[2] * up, 12582912.f + 32768.f));
        const uint32_t q3 = __float_as_uint(fmaf(qp.w * lv, inv[3] * up, 12582912.f));
        if (e < levels) dst[e] = make_uint2(__byte_perm(q0, q1, 0x5410), __byte_perm(q2, q3, 0x5410));
      }
    }
  }
  __syncthreads();
}

// Running sums of one record.  An entry word holds a signed 16-bit value in its high half and an
// offset (unsigned) one in its low half.  `hi` accumulates floor(word / 65536), which is exactly
// the high value (one IMAD.HI); `raw` accumulates the whole word modulo 2^32 (one IADD).  The low
// sum is recovered at the end as raw - 65536 * hi - bias, exact because it stays below 2^32.
struct ScoreAcc {
  int hi[2];
  unsigned int raw[2];
  __device__ __forceinline__ void clear() { hi[0] = hi[1] = 0; raw[0] = raw[1] = 0u; }
  __device__ __forceinline__ void shift(int sh) { hi[0] <<= sh; hi[1] <<= sh; raw[0] <<= sh; raw[1] <<= sh; }
  __device__ __forceinline__ void add(const uint2 e) {
    asm("mad.hi.s32 %0, %1, 65536, %0;" : "+r"(hi[0]) : "r"(e.x));
    raw[0] += e.x;
    asm("mad.hi.s32 %0, %1, 65536, %0;" : "+r"(hi[1]) : "r"(e.y));
    raw[1] += e.y;
  }
  // integer sums of the four heads, in units of scale[h]
  __device__ __forceinline__ void finish(unsigned int bias, int (&out)[JQK_MAX_GROUP]) const {
    out[1] = hi[0];
    out[0] = (int)(raw[0] - ((unsigned int)hi[0] << 16) - bias);
    out[3] = hi[1];
    out[2] = (int)(raw[1] - ((unsigned int)hi[1] << 16) - bias);
  }
};

// Scores one record.  `word(w)` returns physical word w of the record.  Nibble words are scanned
// from the start of the record, (3,3,2)-byte words from its end; lookups that fall on the other
// region hit all-zero tables.  The word loops are not unrolled: the body of one word (8 or 12
// lookups) is what has to stay in the instruction cache.
// What the scoring loop reads, wherever it lives (the builder's TableSmem or a copy of the record).
struct TableView {
  const uint2* lut;
  const int* dshift;
  unsigned int bias;
  const uint16_t* woff = nullptr;
};

// Finished tables of one (sequence, kv head, q-head block) in global memory: written by the table
// kernel, copied into shared memory by every decode block of that group.
struct TableRecord {
  uint2 lut[JQK_MAX_TABLES * 16];
  int dshift[TBL_WORDS];
  float scale[JQK_MAX_GROUP];
  unsigned int bias;
  alignas(8) uint16_t woff[JQK_MAX_WIDE];
  unsigned int pad[26 - JQK_MAX_WIDE / 2];
};
static_assert(sizeof(TableRecord) % 16 == 0 && offsetof(TableRecord, dshift) % 16 == 0, "bulk copies need 16-byte pieces");
constexpr uint32_t TABLE_RECORD_META_BYTES = sizeof(TableRecord) - offsetof(TableRecord, dshift);  // 256

// WIDE: the record also holds `n_wide` byte-wide codes in the words after the nibble words; their
// 256-entry tables lie behind the 16-entry ones and their words come first in the scan.
template <bool WIDE = false, typename WordFn>
__device__ __forceinline__ void score_record(WordFn word, const TableView& sm, int n_a_words, int n_c_words,
                                             int n_words, int (&out)[JQK_MAX_GROUP], int n_wide = 0) {
  ScoreAcc acc;
  acc.clear();
  const char* lb = reinterpret_cast<const char*>(sm.lut);
  const int* dshift = sm.dshift;
  if constexpr (WIDE) {
    const char* lw = lb + (size_t)(8 * n_a_words + 12 * n_c_words) * 128;
    const int n_full = n_wide >> 2, rest = n_wide & 3;
#pragma unroll 1
    for (int j = 0; j < n_full; ++j) {
      const uint32_t x = word(n_a_words + j);
      const uint2 wo = reinterpret_cast<const uint2*>(sm.woff)[j];  // table offsets of the word's four columns
      acc.shift(dshift[j]);
      acc.add(*reinterpret_cast<const uint2*>(lw + (wo.x & 0xffffu) + ((x << 3) & 0x7f8u)));
      acc.add(*reinterpret_cast<const uint2*>(lw + (wo.x >> 16) + ((x >> 5) & 0x7f8u)));
      acc.add(*reinterpret_cast<const uint2*>(lw + (wo.y & 0xffffu) + ((x >> 13) & 0x7f8u)));
      acc.add(*reinterpret_cast<const uint2*>(lw + (wo.y >> 16) + ((x >> 21) & 0x7f8u)));
    }
    if (rest) {  // the last word holds one to three columns
      const uint32_t x = word(n_a_words + n_full);
      const uint2 wo = reinterpret_cast<const uint2*>(sm.woff)[n_full];
      acc.shift(dshift[n_full]);
      acc.add(*reinterpret_cast<const uint2*>(lw + (wo.x & 0xffffu) + ((x << 3) & 0x7f8u)));
      if (rest > 1) acc.add(*reinterpret_cast<const uint2*>(lw + (wo.x >> 16) + ((x >> 5) & 0x7f8u)));
      if (rest > 2) acc.add(*reinterpret_cast<const uint2*>(lw + (wo.y & 0xffffu) + ((x >> 13) & 0x7f8u)));
    }
    dshift += (n_wide + 3) >> 2;
  }
#pragma unroll 4
  for (int w = 0; w < n_a_words; ++w) {
    const uint32_t x = word(w);
    acc.shift(dshift[w]);
    const char* lw = lb + w * 1024;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t off = (k == 0) ? ((x << 3) & 0x78u) : ((x >> (4 * k - 3)) & 0x78u);
      acc.add(*reinterpret_cast<const uint2*>(lw + k * 128 + off));
    }
  }
  const char* lc = lb + n_a_words * 1024;
#pragma unroll 2
  for (int w = 0; w < n_c_words; ++w) {
    const uint32_t x = word(n_words - 1 - w);
    acc.shift(dshift[n_a_words + w]);
    const char* lw = lc + w * 1536;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t o0 = (b == 0) ? ((x << 3) & 0x38u) : ((x >> (8 * b - 3)) & 0x38u);
      const uint32_t o1 = (x >> (8 * b)) & 0x38u;      // bits 3..5 of the byte, already times 8
      const uint32_t o2 = (x >> (8 * b + 3)) & 0x18u;  // bits 6..7 of the byte, times 8
      acc.add(*reinterpret_cast<const uint2*>(lw + (b * 3 + 0) * 128 + o0));
      acc.add(*reinterpret_cast<const uint2*>(lw + (b * 3 + 1) * 128 + o1));
      acc.add(*reinterpret_cast<const uint2*>(lw + (b * 3 + 2) * 128 + o2));
    }
  }
  acc.finish(sm.bias, out);
}

}  // namespace jqk
