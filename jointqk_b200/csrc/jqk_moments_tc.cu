// Calibration moments on the tensor cores (bf16 inputs, head_dim 128, group size <= 4).
//
// Same sums as moments_simt_kernel (jqk_moments.cu); reference:
// experiments/stage1/calibration/compute_stats.py:118-123.  For one kv head
//   sq  = sum_g Q_g^T Q_g,   sk = K^T K,   cqk = (1/G) sum_g Q_g^T K
// are X^T Y contractions over tokens.  A token tile [64 tokens][128 dims] that TMA drops into
// shared memory with the 128-byte swizzle is, as it stands, an MN-major tcgen05 operand (the
// 128 dims are the M or N index, tokens are K), so one copy of a tile serves as A and as B:
// nothing is transposed or staged twice.  Per 16 tokens the block issues 1 + 2G MMAs
// (M = N = 128, K = 16, bf16 in, fp32 accumulate) into three 128-column TMEM accumulators.
//
// A block owns a chunk of at most 2048 tokens of one kv head; at the end of the chunk the epilogue
// warps read the accumulators and add them to the outputs with reductions that a warp issues
// over 32 consecutive floats (red.global.add.f32).  Short chunks bound the length of each fp32 running sum, which keeps
// the result as accurate as a blocked CPU summation.
//
//   warp 0  TMA producer (G + 1 tiles per stage, 2 stages)     warp 1  TMEM owner + MMA issuer
//   warps 2..5  epilogue (TMEM lane quarter = warp & 3)
// Every mbarrier wait is bounded in time (see tc_wait in jqk_compress_tc.cu for the policy).
#include "jqk_common.cuh"
#include "jqk_sm100.cuh"

namespace jqk {

using namespace sm100;

constexpr int MT_TOK = 64;             // tokens per tile
constexpr int MT_STAGES = 2;
constexpr int MT_CHUNK = 2048;         // default tokens per block
constexpr int MT_EPI_WARPS = 4;          // one per TMEM lane quarter (eight, two per quarter, measured no faster)
constexpr int MT_THREADS = 64 + 32 * MT_EPI_WARPS;
constexpr uint32_t MT_TILE_BYTES = MT_TOK * 128 * 2;  // one head's tile: two boxes of [64 tokens][64 dims]
constexpr uint32_t MT_TMEM_COLS = 512;
constexpr unsigned long long MT_WAIT_NS = 2000000000ull;

struct MtSmem {
  uint8_t tile[MT_STAGES][JQK_MAX_GROUP + 1][MT_TILE_BYTES];  // [stage][q_0..q_{G-1}, k]
  uint8_t ones[2048];  // bf16 1.0 throughout: 16 tokens x 16 columns of ones as an MN-major operand (any swizzle)
  uint64_t full[MT_STAGES], empty[MT_STAGES], done;
  uint32_t tmem_base;
  volatile int abort;
};

__device__ __forceinline__ bool mt_wait(MtSmem& sm, uint64_t* bar, uint32_t parity) {
  if (mbar_wait_timed<0, 1024>(bar, parity, MT_WAIT_NS, &sm.abort)) return true;
  sm.abort = 1;
  return false;
}

// G: q heads per kv head when known at compile time (0 = read `group`); MODE 1: all three second
// moments, no first moments; MODE 2: all three plus both first moments; MODE 0: whatever the
// pointers say.  The one thread that issues the MMAs is the pace-setter of the kernel: with the
// common cases fixed at compile time its loop is straight-line code (run-time tests of the output
// pointers inside it cost 12 % of the kernel time).
template <int G, int MODE>
__global__ void __launch_bounds__(MT_THREADS, 1)
moments_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                  long long n_tokens, int chunk, int group, float* __restrict__ sq, float* __restrict__ sk,
                  float* __restrict__ cqk, float* __restrict__ q_sum, float* __restrict__ k_sum, int32_t* wait_flag) {
  extern __shared__ uint8_t smem_raw[];
  MtSmem& sm = *reinterpret_cast<MtSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;
  const long long t_begin = (long long)blockIdx.x * chunk;
  const long long t_end = min(n_tokens, t_begin + chunk);
  const int n_tiles = (int)((t_end - t_begin + MT_TOK - 1) / MT_TOK);
  const bool want_q = (sq != nullptr) || (cqk != nullptr) || (q_sum != nullptr);

  // the all-ones operand of the first-moment products (written before the barrier below; the MMA
  // reads it through the async proxy, hence the fence)
  for (int e = tid; e < 2048 / 4; e += MT_THREADS) reinterpret_cast<uint32_t*>(sm.ones)[e] = 0x3F803F80u;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (tid == 0) {
    for (int s = 0; s < MT_STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
    mbar_init(&sm.done, 1);
    sm.abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&sm.tmem_base, MT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&k_map);
      if (want_q) tma_prefetch_desc(&q_map);
      const uint32_t bytes = (want_q ? group + 1 : 1) * MT_TILE_BYTES;
      int issued = 0;
      for (int t = 0; t < n_tiles; ++t, ++issued) {
        const int s = issued % MT_STAGES;
        if (issued >= MT_STAGES && !mt_wait(sm, &sm.empty[s], ((issued / MT_STAGES) & 1) ^ 1)) break;
        const int tok = (int)(t_begin + (long long)t * MT_TOK);
        mbar_arrive_expect_tx(&sm.full[s], bytes);
        for (int half = 0; half < 2; ++half) {
          if (want_q)
            for (int g = 0; g < group; ++g)
              tma_load_3d(sm.tile[s][g] + half * (MT_TILE_BYTES / 2), &q_map, &sm.full[s], 64 * half, tok, head * group + g);
          tma_load_3d(sm.tile[s][JQK_MAX_GROUP] + half * (MT_TILE_BYTES / 2), &k_map, &sm.full[s], 64 * half, tok, head);
        }
      }
      if (sm.abort)
        for (int i = max(0, issued - MT_STAGES); i < issued; ++i) mt_wait(sm, &sm.full[i % MT_STAGES], (i / MT_STAGES) & 1);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(128, 128, true, true);
      // First moments ride on the same operands: X^T [128 dims x 16 tokens] times a [16 tokens x 16]
      // block of ones leaves sum_t x_t in each of 16 accumulator columns (columns 384.. for the key,
      // 400.. for the queries of the group, pooled).  No second pass over the inputs.
      const uint32_t idesc_sum = make_idesc_bf16(128, 16, true, true);
      const uint64_t ones_desc = make_smem_desc_sw128(smem_u32(sm.ones), 16, 1024);
      const bool do_sq = MODE ? true : sq != nullptr, do_sk = MODE ? true : sk != nullptr, do_cqk = MODE ? true : cqk != nullptr;
      const bool do_ksum = MODE == 2 ? true : MODE == 1 ? false : k_sum != nullptr;
      const bool do_qsum = MODE == 2 ? true : MODE == 1 ? false : q_sum != nullptr;
      const int n_group = G ? G : group;
      // descriptors of a stage's tiles at token 0; 16 tokens further along is +2048 bytes = +128 in the
      // address field (the second 64-dim block is half a tile away: the leading-dimension offset)
      uint64_t k_desc0[MT_STAGES], q_desc0[MT_STAGES][JQK_MAX_GROUP];
#pragma unroll
      for (int s = 0; s < MT_STAGES; ++s) {
        k_desc0[s] = make_smem_desc_sw128(smem_u32(sm.tile[s][JQK_MAX_GROUP]), MT_TILE_BYTES / 2, 1024);
#pragma unroll
        for (int g = 0; g < JQK_MAX_GROUP; ++g)
          q_desc0[s][g] = make_smem_desc_sw128(smem_u32(sm.tile[s][g]), MT_TILE_BYTES / 2, 1024);
      }
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % MT_STAGES;
        if (!mt_wait(sm, &sm.full[s], (t / MT_STAGES) & 1)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < MT_TOK / 16; ++ks) {
          const bool first = (t == 0 && ks == 0);
          const uint64_t k_desc = (s ? k_desc0[1] : k_desc0[0]) + (uint64_t)(ks * 128);
          if (do_sk) umma_bf16(tmem + 128, k_desc, k_desc, idesc, !first);
          if (do_ksum) umma_bf16(tmem + 384, k_desc, ones_desc, idesc_sum, !first);
          if (want_q) {
#pragma unroll
            for (int g = 0; g < JQK_MAX_GROUP; ++g) {
              if (g < n_group) {
                const uint64_t q_desc = (s ? q_desc0[1][g] : q_desc0[0][g]) + (uint64_t)(ks * 128);
                if (do_sq) umma_bf16(tmem + 0, q_desc, q_desc, idesc, !(first && g == 0));
                if (do_cqk) umma_bf16(tmem + 256, k_desc, q_desc, idesc, !(first && g == 0));  // transposed: lane = k dim
                if (do_qsum) umma_bf16(tmem + 400, q_desc, ones_desc, idesc_sum, !(first && g == 0));
              }
            }
          }
        }
        umma_commit(&sm.empty[s]);
      }
      umma_commit(&sm.done);
    }
  } else {
    // Epilogue.  A thread owns TMEM lane r.  For the two symmetric matrices entry (r, c) is also entry
    // (c, r); the cross moment is accumulated transposed (lane = k dim, column = q dim).  Either way
    // the thread adds its value for column c to out[c][r], so the 32 lanes of a warp hit 32
    // consecutive floats: one 128-byte reduction per instruction instead of 32 scattered ones.
    if (mt_wait(sm, &sm.done, 0) && !sm.abort) {
      tc_fence_after();
      const int row = 32 * (warp & 3) + lane;
      const int col_lo = ((warp - 2) >> 2) * (128 / (MT_EPI_WARPS / 4));
      const uint32_t t_lane = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
      float* outs[3] = {sq, sk, cqk};
      const float scale[3] = {1.f, 1.f, 1.f / (float)group};
#pragma unroll 1
      for (int m = 0; m < 3; ++m) {
        if (!outs[m]) continue;
        float* dst = outs[m] + (size_t)head * 128 * 128 + row;
#pragma unroll 1
        for (int c0 = col_lo; c0 < col_lo + 128 / (MT_EPI_WARPS / 4); c0 += 16) {
          float v[16];
          tmem_ld16(t_lane + m * 128 + c0, v);
#pragma unroll
          for (int i = 0; i < 16; ++i)
            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + (size_t)(c0 + i) * 128), "f"(v[i] * scale[m]) : "memory");
        }
      }
      if (warp - 2 < 4) {  // first moments: lane = dim, every one of the 16 columns holds the same sum
        float* firsts[2] = {k_sum, q_sum};
#pragma unroll 1
        for (int m = 0; m < 2; ++m) {
          if (!firsts[m]) continue;
          float v[16];
          tmem_ld16(t_lane + 384 + 16 * m, v);
          asm volatile("red.global.add.f32 [%0], %1;" ::"l"(firsts[m] + (size_t)head * 128 + row), "f"(v[0]) : "memory");
        }
      }
    }
  }
  if (sm.abort && tid == 0 && wait_flag) atomicOr(wait_flag, JQK_STATUS_WAIT_EXPIRED);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, MT_TMEM_COLS);
  }
}

}  // namespace jqk

using namespace jqk;

// Launches the tensor-core kernel when the call fits it; returns 1 when the caller should use the
// CUDA-core kernel (other dtypes, head sizes, group sizes, unaligned strides, key-only calls).
int32_t jqk_moments_tc_try(const void* q, const void* k, int32_t dtype, int64_t n_tokens, int64_t q_head_stride,
                           int64_t k_head_stride, int32_t n_q_heads, int32_t n_kv_heads, int32_t d, float* sq_sum,
                           float* sk_sum, float* cqk_sum, float* q_sum, float* k_sum, int32_t max_chain_tokens,
                           int32_t* status, cudaStream_t st) {
  const int group = n_q_heads / n_kv_heads;
  if (dtype != JQK_DTYPE_BF16 || d != 128 || group > JQK_MAX_GROUP || n_tokens < MT_TOK || n_tokens > 0x7fffffffLL) return 1;
  const bool want_q = sq_sum || cqk_sum || q_sum;
  if ((uintptr_t)k % 16 || (k_head_stride * 2) % 16) return 1;
  if (want_q && (!q || (uintptr_t)q % 16 || (q_head_stride * 2) % 16)) return 1;
  for (float* o : {sq_sum, sk_sum, cqk_sum})
    if (o && (uintptr_t)o % 16) return 1;
  if (!sq_sum && !sk_sum && !cqk_sum) return 1;  // first moments alone: not worth a tensor-core launch
  CUtensorMap q_map, k_map;
  char err[256];
  const uint32_t box[3] = {64, MT_TOK, 1};
  {
    const uint64_t dims[3] = {128, (uint64_t)n_tokens, (uint64_t)n_kv_heads};
    const uint64_t strides[2] = {256, n_kv_heads > 1 ? (uint64_t)k_head_stride * 2 : 256ull * n_tokens};
    if (!encode_bf16_map(&k_map, k, 3, dims, strides, box, err, sizeof(err))) return fail(JQK_E_ARG, "k tensor map: %s", err);
  }
  if (want_q) {
    const uint64_t dims[3] = {128, (uint64_t)n_tokens, (uint64_t)n_q_heads};
    const uint64_t strides[2] = {256, n_q_heads > 1 ? (uint64_t)q_head_stride * 2 : 256ull * n_tokens};
    if (!encode_bf16_map(&q_map, q, 3, dims, strides, box, err, sizeof(err))) return fail(JQK_E_ARG, "q tensor map: %s", err);
  } else {
    q_map = k_map;
  }
  // One block per SM is resident (160 KB of operand stages), so blocks run in waves of 148.  The
  // chunk is the largest one not above the chain bound (the length of an fp32 running sum in tensor
  // memory: MT_CHUNK unless the caller asks for less) whose block count fills whole waves:
  // 131072 tokens x 8 heads -> 1792 tokens, 592 blocks, 4 waves.
  int cap = MT_CHUNK;
  if (max_chain_tokens > 0 && max_chain_tokens < MT_CHUNK) cap = max(MT_TOK, max_chain_tokens / MT_TOK * MT_TOK);
  int chunk = cap;
  for (long long waves = 1; waves <= 65536; ++waves) {
    const long long per_head = (148LL * waves) / n_kv_heads;
    if (per_head <= 0) continue;
    long long c = (n_tokens + per_head - 1) / per_head;
    c = (c + MT_TOK - 1) / MT_TOK * MT_TOK;
    if (c <= cap) { chunk = (int)(c < MT_TOK ? MT_TOK : c); break; }
  }
  dim3 grid((unsigned)((n_tokens + chunk - 1) / chunk), n_kv_heads);
  const size_t smem = sizeof(MtSmem) + 1024;
  const int mode = (sq_sum && sk_sum && cqk_sum) ? ((q_sum && k_sum) ? 2 : (!q_sum && !k_sum) ? 1 : 0) : 0;
#define JQK_LAUNCH_MOMENTS(GG, MM)                                                                              \
  do {                                                                                                          \
    JQK_SMEM_ONCE((moments_tc_kernel<GG, MM>), smem, "tensor-core moments smem attribute");                     \
    moments_tc_kernel<GG, MM><<<grid, MT_THREADS, smem, st>>>(q_map, k_map, (long long)n_tokens, chunk, group,  \
                                                              sq_sum, sk_sum, cqk_sum, q_sum, k_sum, status);   \
  } while (0)
  if (mode == 1 && group == 4) JQK_LAUNCH_MOMENTS(4, 1);
  else if (mode == 2 && group == 4) JQK_LAUNCH_MOMENTS(4, 2);
  else if (mode == 1 && group == 2) JQK_LAUNCH_MOMENTS(2, 1);
  else if (mode == 2 && group == 2) JQK_LAUNCH_MOMENTS(2, 2);
  else if (mode == 1 && group == 1) JQK_LAUNCH_MOMENTS(1, 1);
  else if (mode == 2 && group == 1) JQK_LAUNCH_MOMENTS(1, 2);
  else JQK_LAUNCH_MOMENTS(0, 0);
#undef JQK_LAUNCH_MOMENTS
  JQK_CUDA_OK(cudaGetLastError(), "tensor-core moments launch");
  return 0;
}
