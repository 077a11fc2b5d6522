// Prefill compression on the tensor cores (bf16 keys, head_dim 128).
//
// Same result as compress_simt_kernel (jqk_compress.cu); reference semantics
// experiments/stage1/toolkit/per_coord_quantization.py:132-157.  The basis transform
// x = k @ forward_map runs as tcgen05.mma with the fp32 map split into three bf16 limbs
// (F = F0 + F1 + F2 to ~2^-24): bf16 x bf16 products are exact in fp32, the limbs are added
// smallest first into one fp32 TMEM accumulator, so the transform keeps fp32 accuracy, which
// the bit-exact code requirement needs (one bf16 or TF32 pass would flip ~1e-3 of the codes).
//
// One thread block walks a run of 128-key tiles of one (sequence, head):
//   warp 0      TMA producer: key tiles [128 keys][128 dims] bf16 into a 3-stage ring (128B swizzle)
//   warp 1      allocates TMEM, loads the three limb matrices once, issues 24 MMAs per tile
//               (8 K-steps x 3 limbs, M=128, N=columns, K=16) into one of two accumulators
//   warps 2..17 epilogue: a thread owns one key (TMEM lane) and a quarter of the record's words; it
//               reads 16 columns at a time, finds each code (a cell lookup plus one comparison with
//               the exact fp32 decision threshold, or a binary search over the thresholds when the
//               cell tables do not apply), appends the bits and stores finished words to the page
//               (word-major pages: 64-byte segments per warp store).
// Every mbarrier wait is bounded in time; on expiry the block flags JQK_STATUS_WAIT_EXPIRED,
// drains its copies, frees TMEM and returns.
#include <math_constants.h>

#include "jqk_common.cuh"
#include "jqk_sm100.cuh"

namespace jqk {

using namespace sm100;

constexpr int TC_TILE = 128;
constexpr int TC_STAGES = 3;
constexpr int CH = 16;  // accumulator columns an epilogue thread handles per TMEM load
constexpr int TC_PARTS = 4;        // parts of the record's words; one epilogue warp per TMEM lane quarter and part (five measured no faster)
constexpr int TC_EPI_WARPS = 4 * TC_PARTS;
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS;
constexpr uint32_t TC_A_BYTES = TC_TILE * 128 * 2;   // one key tile
constexpr uint32_t TC_B_BYTES = 3 * 128 * 128 * 2;   // three limb matrices
constexpr uint32_t TC_TMEM_COLS = 512;               // two fp32 accumulators of 128 columns; the rest is only
                                                     // there so that a 16-column read may start at any column
constexpr int TC_COL_PAD = 128 + CH;                 // per-column tables cover a read that starts at column 127
constexpr int TC_PART_WORDS = 4;                     // words a part's registers hold (more: generic path)
constexpr unsigned long long TC_WAIT_NS = 2000000000ull;

struct TcSmem {
  uint8_t a[TC_STAGES][TC_A_BYTES];  // [k half][128 keys][64 dims], 128B swizzle
  uint8_t b[3][128 * 128 * 2];       // limb l: [k half][128 columns][64 dims], 128B swizzle
  float thr[TC_COL_PAD * 16];
  uint8_t pre[TC_COL_PAD * 128];  // coarse-to-exact quantiser: lower bound of the code per cell
  float2 aff[TC_COL_PAD];         // cell = round(127 * saturate(x * aff.x + aff.y))
  uint4 mult[TC_COL_PAD];         // 1 << bit position in word j of the column's part (one of four is non-zero)
  int32_t meta[128];
  int32_t wcb[JQK_MAX_WORDS + 4];
  int32_t cut[TC_PARTS + 1];      // word ranges of the parts
  uint64_t full[TC_STAGES], empty[TC_STAGES], acc_full[2], acc_empty[2], b_full;
  uint32_t tmem_base;
  volatile int abort;
};

struct TcArgs {
  const int32_t* n_tokens;
  const int32_t* seq_starts;
  const int32_t* page_table;
  int32_t pt_stride;
  int32_t n_pages;
  int32_t tiles_per_block;
  int32_t* status;
};

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: false (and the abort flag) after TC_WAIT_NS or when another role gave up.
__device__ __forceinline__ bool tc_wait(TcSmem& sm, uint64_t* bar, uint32_t parity, int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = now_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      __nanosleep(40);  // waiting roles must not eat the issue slots of the working warps
    }
    if (sm.abort) return false;
    if (now_ns() - t0 > TC_WAIT_NS) {
      sm.abort = 1;
      if (status) atomicOr(status, JQK_STATUS_WAIT_EXPIRED);
      return false;
    }
  }
}

// code = #{l : x >= thr[l]} for sorted thresholds, by binary search over 2^width - 1 entries.
__device__ __forceinline__ uint32_t search_code(float x, const float* __restrict__ thr, int width) {
  uint32_t code = 0;
  for (int step = (1 << width) >> 1; step >= 1; step >>= 1)
    code += (x >= thr[code + step - 1]) ? step : 0;
  return code;
}

#ifdef JQK_COMPRESS_PROFILE
// Development aid: clock totals of the MMA thread (wait full, wait acc_empty, issue) and of epilogue
// warp 2 (wait acc_full, tmem load, quantise+pack, other).  Not part of the product build.
__device__ long long g_tc_prof[8];
#define TCP_MARK(i) do { const long long n__ = clock64(); atomicAdd((unsigned long long*)&g_tc_prof[i], (unsigned long long)(n__ - tp)); tp = n__; } while (0)
#else
#define TCP_MARK(i) do {} while (0)
#endif

// Codes of 16 consecutive columns (first column c0, any alignment) of one key, added at their bit
// positions into the registers of the part's words.  Branch-free, so the 16 dependent chains
// (cell, lower bound, exact comparison) overlap.  TAIL: only the first n_here columns belong to
// the part; J: words of the part.  The cell tables give code 0 for columns past the head's last column.
template <bool USE_BUCKETS, bool TAIL, int J>
__device__ __forceinline__ void quant_chunk(const TcSmem& sm, const float (&v)[CH], int c0, int n_here,
                                            uint32_t (&cur)[TC_PART_WORDS]) {
  uint32_t code[CH];
  if constexpr (USE_BUCKETS) {
    // two fused multiply-adds find the cell (the first one saturates to [0, 1], which is the clamp),
    // a byte table gives a lower bound of the code that is at most one short, one exact comparison
    // with the fp32 decision threshold settles it
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const float2 af = sm.aff[c0 + i];
      const float y = __saturatef(fmaf(v[i], af.x, af.y));
      const uint32_t cell = __float_as_uint(fmaf(y, 127.f, 8388608.f)) - 0x4B000000u;
      const uint32_t k = sm.pre[(c0 + i) * 128 + cell];
      code[i] = k + ((v[i] >= sm.thr[(c0 + i) * 16 + k]) ? 1u : 0u);
    }
  } else {
    // 16 independent four-step searches (rows are +inf padded, so narrower codes never pass
    // their last level)
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const float* th = sm.thr + (c0 + i) * 16;
      uint32_t k = (v[i] >= th[7]) ? 8u : 0u;
      k += (v[i] >= th[k + 3]) ? 4u : 0u;
      k += (v[i] >= th[k + 1]) ? 2u : 0u;
      k += (v[i] >= th[k]) ? 1u : 0u;
      code[i] = k;
    }
  }
#pragma unroll
  for (int i = 0; i < CH; ++i) {
    if (!TAIL || i < n_here) {  // warp-uniform
      const uint4 m = sm.mult[c0 + i];
      cur[0] += code[i] * m.x;
      if constexpr (J > 1) cur[1] += code[i] * m.y;
      if constexpr (J > 2) cur[2] += code[i] * m.z;
      if constexpr (J > 3) cur[3] += code[i] * m.w;
    }
  }
}

template <bool USE_BUCKETS>
__global__ void __launch_bounds__(TC_THREADS, 1)
compress_tc_kernel(const __grid_constant__ CUtensorMap key_map, const __grid_constant__ CUtensorMap limb_map,
                   jqk_head_tables tb, TcArgs pa, uint32_t* __restrict__ k_pool) {
  extern __shared__ uint8_t smem_raw[];
  // align by pointer arithmetic on the __shared__ array (an integer round trip would turn every access into a generic load)
  TcSmem& sm = *reinterpret_cast<TcSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef JQK_COMPRESS_PROFILE
  const long long t_block0 = clock64();
#endif
  const int head = blockIdx.y, seq = blockIdx.z;
  const int n_tok = pa.n_tokens[seq];
  const int n_tiles = (n_tok + TC_TILE - 1) / TC_TILE;
  const int tile_lo = blockIdx.x * pa.tiles_per_block;
  const int tile_hi = min(n_tiles, tile_lo + pa.tiles_per_block);
  if (tile_lo >= tile_hi) return;
  const HeadDesc hd = load_desc(tb.desc, head);

  // ---- set-up ----
  // per-column tables; columns past n_cols (reachable by the last 16-column read of a part) quantise to code 0
  for (int e = tid; e < TC_COL_PAD * 16; e += TC_THREADS)
    sm.thr[e] = (e < hd.n_cols * 16) ? tb.thresholds[(size_t)head * 128 * 16 + e] : CUDART_INF_F;
  for (int e = tid; e < 128; e += TC_THREADS) sm.meta[e] = tb.col_meta[(size_t)head * 128 + e];
  {
    const uint4* src = reinterpret_cast<const uint4*>(tb.bucket_pre + (size_t)head * 128 * 128);
    uint4* dst = reinterpret_cast<uint4*>(sm.pre);
    for (int e = tid; e < TC_COL_PAD * 8; e += TC_THREADS)
      dst[e] = (USE_BUCKETS && e < hd.n_cols * 8) ? src[e] : make_uint4(0u, 0u, 0u, 0u);
    for (int e = tid; e < TC_COL_PAD; e += TC_THREADS) {
      float2 af = make_float2(0.f, 0.f);
      if (USE_BUCKETS && e < hd.n_cols) {
        // host form: cell = clamp(round(x * inv_step + off), 0, 127) with 2^23 folded into off
        const float2 h2 = reinterpret_cast<const float2*>(tb.bucket_aff)[(size_t)head * 128 + e];
        af = make_float2(h2.x * (1.f / 127.f), (h2.y - 8388608.f) * (1.f / 127.f));
      }
      sm.aff[e] = af;
    }
  }
  for (int e = tid; e <= hd.n_words; e += TC_THREADS) sm.wcb[e] = tb.desc[(size_t)head * JQK_DESC_INTS + 8 + e];
  if (tid == 0) {
    for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&sm.acc_full[a], 1); mbar_init(&sm.acc_empty[a], TC_EPI_WARPS); }
    mbar_init(&sm.b_full, 1);
    sm.abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&sm.tmem_base, TC_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0) {
    // ================= TMA producer =================
    if (lane == 0) {
      tma_prefetch_desc(&key_map);
      int issued = 0;
      for (int t = tile_lo; t < tile_hi; ++t, ++issued) {
        const int s = issued % TC_STAGES;
        const uint32_t ph = (issued / TC_STAGES) & 1;
        if (issued >= TC_STAGES && !tc_wait(sm, &sm.empty[s], ph ^ 1, pa.status)) break;
        mbar_arrive_expect_tx(&sm.full[s], TC_A_BYTES);
        tma_load_4d(sm.a[s], &key_map, &sm.full[s], 0, t * TC_TILE, head, seq);
        tma_load_4d(sm.a[s] + TC_A_BYTES / 2, &key_map, &sm.full[s], 64, t * TC_TILE, head, seq);
      }
      if (sm.abort) {  // let the copies that were issued land before the block goes away
        for (int i = max(0, issued - TC_STAGES); i < issued; ++i)
          tc_wait(sm, &sm.full[i % TC_STAGES], (i / TC_STAGES) & 1, nullptr);
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      tma_prefetch_desc(&limb_map);
      mbar_arrive_expect_tx(&sm.b_full, TC_B_BYTES);
      for (int l = 0; l < 3; ++l)
        for (int kh = 0; kh < 2; ++kh)
          tma_load_2d(sm.b[l] + kh * (128 * 64 * 2), &limb_map, &sm.b_full, 64 * kh, (head * 3 + l) * 128);
      const uint32_t idesc = make_idesc_bf16(128, hd.n_cols, false, false);
      bool ok = tc_wait(sm, &sm.b_full, 0, pa.status);
      int it = 0;
#ifdef JQK_COMPRESS_PROFILE
      long long tp = clock64();
#endif
      for (int t = tile_lo; ok && t < tile_hi; ++t, ++it) {
        const int s = it % TC_STAGES, a = it & 1;
        if (!tc_wait(sm, &sm.full[s], (it / TC_STAGES) & 1, pa.status)) break;
        TCP_MARK(0);
        if (it >= 2 && !tc_wait(sm, &sm.acc_empty[a], ((it >> 1) & 1) ^ 1, pa.status)) break;
        TCP_MARK(1);
        tc_fence_after();
        const uint32_t d_tmem = tmem + a * 128;
        const uint32_t a_base = smem_u32(sm.a[s]);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * (128 * 64 * 2) + (ks & 3) * 32;
          const uint64_t a_desc = make_smem_desc_sw128(a_base + off, 16, 1024);
#pragma unroll
          for (int l = 2; l >= 0; --l) {
            const uint64_t b_desc = make_smem_desc_sw128(smem_u32(sm.b[l]) + off, 16, 1024);
            umma_bf16(d_tmem, a_desc, b_desc, idesc, !(ks == 0 && l == 2));
          }
        }
        umma_commit(&sm.empty[s]);     // the key tile may be overwritten
        umma_commit(&sm.acc_full[a]);  // the accumulator may be read
        TCP_MARK(2);
      }
    }
  } else {
    // ================= epilogue =================
    const int ew = warp - 2;
    const int row = 32 * (warp & 3) + lane;          // TMEM lane = key inside the tile
    const int part = ew >> 2;
    // word ranges of the parts, cut where the column counts are closest to even (low-bit
    // words hold up to four times as many columns as 4-bit words)
    if (ew == 0 && lane == 0) {
      int cut[TC_PARTS + 1];
      cut[0] = 0; cut[TC_PARTS] = hd.n_words;
#pragma unroll
      for (int q = 1; q < TC_PARTS; ++q) {
        const int target = (hd.n_active * q + TC_PARTS / 2) / TC_PARTS;
        int w = cut[q - 1];
        while (w < hd.n_words && sm.wcb[w] < target) ++w;
        if (w > cut[q - 1] && w < hd.n_words && target - sm.wcb[w - 1] < sm.wcb[w] - target) --w;
        cut[q] = max(w, cut[q - 1]);
      }
#pragma unroll
      for (int q = 0; q <= TC_PARTS; ++q) sm.cut[q] = cut[q];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
    {  // bit position of every column as a multiplier for the word registers of its part
      const int et = tid - 64;
      if (et < TC_COL_PAD) {
        uint4 m = make_uint4(0u, 0u, 0u, 0u);
        if (et < hd.n_active) {
          const int bp = (sm.meta[et] >> 4) & 1023;
          const int w = bp >> 5;
          int p = 0;
          while (p < TC_PARTS - 1 && w >= sm.cut[p + 1]) ++p;
          const int j = w - sm.cut[p];
          const uint32_t one = 1u << (bp & 31);
          m.x = (j == 0) ? one : 0u; m.y = (j == 1) ? one : 0u;
          m.z = (j == 2) ? one : 0u; m.w = (j == 3) ? one : 0u;
        }
        sm.mult[et] = m;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
    const int w_lo = sm.cut[part], w_hi = sm.cut[part + 1];
    const int n_part_words = w_hi - w_lo;
    const bool in_regs = n_part_words <= TC_PART_WORDS;  // otherwise: the generic word-by-word path
    const int c_lo = sm.wcb[w_lo], c_hi = sm.wcb[w_hi];
    const int seq_start = pa.seq_starts ? pa.seq_starts[seq] : 0;
    const int wpr = tb.words_per_record;
    int it = 0;
#ifdef JQK_COMPRESS_PROFILE
    long long tp = clock64();
    const bool prof_on = (warp == 2 && lane == 0);
#undef TCP_MARK
#define TCP_MARK(i) do { const long long n__ = clock64(); if (prof_on) atomicAdd((unsigned long long*)&g_tc_prof[i], (unsigned long long)(n__ - tp)); tp = n__; } while (0)
#endif
    for (int t = tile_lo; t < tile_hi; ++t, ++it) {
      const int a = it & 1;
      if (!tc_wait(sm, &sm.acc_full[a], (it >> 1) & 1, pa.status)) break;
      TCP_MARK(3);
      tc_fence_after();
      const int key = t * TC_TILE + row;
      const bool valid = key < n_tok;
      uint32_t* dst = nullptr;
      if (valid) {
        const int tok = seq_start + key;
        const int page = lookup_page(pa.page_table, pa.pt_stride, seq, tok / JQK_PAGE_TOKENS, pa.n_pages, pa.status);
        if (page >= 0)
          dst = k_pool + ((size_t)page * tb.n_heads + head) * wpr * JQK_PAGE_TOKENS + (tok % JQK_PAGE_TOKENS);
      }
      const uint32_t t_lane = tmem + a * 128 + ((uint32_t)(32 * (warp & 3)) << 16);
      if (in_regs) {
        uint32_t cur[TC_PART_WORDS] = {0u, 0u, 0u, 0u};
        for (int c0 = c_lo; c0 < c_hi; c0 += CH) {
          float v[CH];
          tmem_ld16(t_lane + c0, v);
          TCP_MARK(4);
          const int n_here = c_hi - c0;
          if (n_part_words <= 2) {
            if (n_here >= CH) quant_chunk<USE_BUCKETS, false, 2>(sm, v, c0, CH, cur);
            else quant_chunk<USE_BUCKETS, true, 2>(sm, v, c0, n_here, cur);
          } else {
            if (n_here >= CH) quant_chunk<USE_BUCKETS, false, 4>(sm, v, c0, CH, cur);
            else quant_chunk<USE_BUCKETS, true, 4>(sm, v, c0, n_here, cur);
          }
          TCP_MARK(5);
        }
        if (dst) {
#pragma unroll
          for (int j = 0; j < TC_PART_WORDS; ++j)
            if (w_lo + j < w_hi) dst[(w_lo + j) * JQK_PAGE_TOKENS] = cur[j];
        }
      } else {
        int cur_w = w_lo;
        uint32_t cur = 0;
        for (int c0 = c_lo; c0 < c_hi; c0 += CH) {
          float v[CH];
          tmem_ld16(t_lane + c0, v);
          for (int i = 0; i < CH && c0 + i < c_hi; ++i) {
            const int m = sm.meta[c0 + i];
            const int bp = (m >> 4) & 1023;
            while (cur_w < (bp >> 5)) {  // finished words (and pad words) leave in order
              if (dst) dst[cur_w * JQK_PAGE_TOKENS] = cur;
              cur = 0;
              ++cur_w;
            }
            float x = v[0];  // v[i] without dynamic register indexing
#pragma unroll
            for (int u = 1; u < CH; ++u) x = (u == i) ? v[u] : x;
            cur |= search_code(x, sm.thr + (c0 + i) * 16, m & 15) << (bp & 31);
          }
        }
        while (cur_w < w_hi) {
          if (dst) dst[cur_w * JQK_PAGE_TOKENS] = cur;
          cur = 0;
          ++cur_w;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sm.acc_empty[a]);
      TCP_MARK(6);
    }
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
#ifdef JQK_COMPRESS_PROFILE
  if (tid == 64) atomicAdd((unsigned long long*)&g_tc_prof[7], (unsigned long long)(clock64() - t_block0));
#endif
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TC_TMEM_COLS);
  }
}

}  // namespace jqk

using namespace jqk;

#ifdef JQK_COMPRESS_PROFILE
extern "C" int32_t jqk_debug_compress_profile(long long* out8, int32_t reset) {
  if (cudaMemcpyFromSymbol(out8, g_tc_prof, sizeof(long long) * 8) != cudaSuccess) return 1;
  if (reset) {
    long long z[8] = {0};
    if (cudaMemcpyToSymbol(g_tc_prof, z, sizeof(z)) != cudaSuccess) return 1;
  }
  return 0;
}
#endif

// Launches the tensor-core kernel when the call fits it (bf16 keys, head_dim 128, 16-byte aligned
// strides); returns 1 when the caller should use the fp32 CUDA-core kernel instead.
int32_t jqk_compress_tc_try(const jqk_head_tables* tables, const void* keys, int32_t key_dtype,
                            int64_t seq_stride, int64_t head_stride, int64_t token_stride, int32_t n_seqs,
                            const int32_t* n_tokens, const int32_t* seq_starts, int32_t max_tokens,
                            const int32_t* page_table, int32_t page_table_stride, int32_t n_pages,
                            uint32_t* k_pool, int32_t* status, cudaStream_t st) {
  if (key_dtype != JQK_DTYPE_BF16 || tables->d != 128 || !tables->fwd_limbs) return 1;
  if ((uintptr_t)keys % 16 || (token_stride * 2) % 16 || (head_stride * 2) % 16 || (seq_stride * 2) % 16) return 1;
  if ((uintptr_t)tables->fwd_limbs % 16 || max_tokens < TC_TILE) return 1;
  CUtensorMap key_map, limb_map;
  char err[256];
  {
    // dims innermost first: (dim, key, head, sequence); a stride of one sequence / head may be 0
    // bytes for a single-entry dimension, which the encoder rejects, so give it the row pitch.
    const uint64_t row = (uint64_t)token_stride * 2;
    const uint64_t dims[4] = {128, (uint64_t)max_tokens, (uint64_t)tables->n_heads, (uint64_t)n_seqs};
    const uint64_t strides[3] = {row, head_stride ? (uint64_t)head_stride * 2 : row * max_tokens,
                                 seq_stride ? (uint64_t)seq_stride * 2 : row * max_tokens * tables->n_heads};
    const uint32_t box[4] = {64, TC_TILE, 1, 1};
    if (!encode_bf16_map(&key_map, keys, 4, dims, strides, box, err, sizeof(err))) return fail(JQK_E_ARG, "key tensor map: %s", err);
  }
  {
    const uint64_t dims[2] = {128, (uint64_t)tables->n_heads * 3 * 128};
    const uint64_t strides[1] = {256};
    const uint32_t box[2] = {64, 128};
    if (!encode_bf16_map(&limb_map, tables->fwd_limbs, 2, dims, strides, box, err, sizeof(err))) return fail(JQK_E_ARG, "limb tensor map: %s", err);
  }
  const int max_tiles = (max_tokens + TC_TILE - 1) / TC_TILE;
  // at most one wave of blocks over 148 SMs (a block's set-up loads 120 KB of tables), each block a
  // contiguous run of tiles of one head
  const long long pairs = (long long)n_seqs * tables->n_heads;
  long long blocks_per_pair = 148 / pairs;
  if (blocks_per_pair < 1) blocks_per_pair = 1;
  int tiles_per_block = (int)((max_tiles + blocks_per_pair - 1) / blocks_per_pair);
  if (tiles_per_block < 4) tiles_per_block = 4;
  dim3 grid((max_tiles + tiles_per_block - 1) / tiles_per_block, tables->n_heads, n_seqs);
  TcArgs pa{n_tokens, seq_starts, page_table, page_table_stride, n_pages, tiles_per_block, status};
  const size_t smem = sizeof(TcSmem) + 1024;
  if (tables->bucket_pre && tables->bucket_aff) {
    JQK_SMEM_ONCE(compress_tc_kernel<true>, smem, "tensor-core compress smem attribute");
    compress_tc_kernel<true><<<grid, TC_THREADS, smem, st>>>(key_map, limb_map, *tables, pa, k_pool);
  } else {
    JQK_SMEM_ONCE(compress_tc_kernel<false>, smem, "tensor-core compress smem attribute");
    compress_tc_kernel<false><<<grid, TC_THREADS, smem, st>>>(key_map, limb_map, *tables, pa, k_pool);
  }
  JQK_CUDA_OK(cudaGetLastError(), "tensor-core compress launch");
  return 0;
}
