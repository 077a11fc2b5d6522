// Prefill compression on the tensor cores (bf16 keys, head_dim 128).
//
// Same result as compress_simt_kernel (jqk_compress.cu); reference semantics
// experiments/stage1/toolkit/per_coord_quantization.py:132-157.  The basis transform
// x = k @ forward_map runs as tcgen05.mma with the fp32 map split into three bf16 limbs
// (F = F0 + F1 + F2 to ~2^-24): bf16 x bf16 products are exact in fp32, the limbs are added
// smallest first into one fp32 TMEM accumulator, so the transform keeps fp32 accuracy, which
// the bit-exact code requirement needs (one bf16 or TF32 pass would flip ~1e-3 of the codes).
//
// The map's columns are scaled by 1 / sigma of their coordinate (on the host, before the split), so a
// transformed value is in units of its coordinate's standard deviation and the nearest level of its
// codebook (unit Lloyd-Max levels x sigma) is found against the UNIT levels of its width: one shared
// set of thresholds and cell tables for every column, as compile-time constants in the code for reads
// whose widths are regular.  The rescaling moves a code only when the value lies within ~1e-7
// (relative) of a decision threshold: 1e-7 .. 5e-7 of the coordinates, the size of the difference
// between two fp32 summation orders of the reference's own transform.
//
// One thread block walks a run of 128-key tiles of one head (the head's tiles of all sequences form
// one list, cut into equal runs, so that a batch fills every SM whatever its shape):
//   warp 0      TMA producer: key tiles [128 keys][128 dims] bf16 into a 3-stage ring (128B swizzle)
//   warp 1      allocates TMEM, loads the three limb matrices once, issues 24 MMAs per tile
//               (8 K-steps x 3 limbs, M=128, N=columns, K=16) into one of two accumulators
//   warps 2..17 epilogue: a thread owns one key (TMEM lane); the record's words are dealt to the four
//               warps of a lane quarter as units of one or two words, and a unit is quantised in
//               16-column reads.  A column's code is a cell lookup plus one comparison with the exact
//               fp32 decision threshold (a binary search over the thresholds when the cell tables do
//               not apply; plain comparisons for 1- and 2-bit columns); its bit position and cell
//               scale come from a constant row per column of each read.  Finished words go to the
//               page (word-major pages: 64-byte segments per warp store).
// Every mbarrier wait is bounded in time; on expiry the block flags JQK_STATUS_WAIT_EXPIRED,
// drains its copies, frees TMEM and returns.
#include <math_constants.h>

#include <type_traits>

#include "jqk_common.cuh"
#include "jqk_sm100.cuh"

namespace jqk {

using namespace sm100;

constexpr int TC_TILE = 128;
constexpr int TC_STAGES = 3;
constexpr int CH = 16;  // accumulator columns an epilogue thread handles per TMEM load
constexpr int TC_PARTS = 4;        // parts of the record's words; one epilogue warp per TMEM lane quarter and part (three and five measured no faster)
constexpr int TC_EPI_WARPS = 4 * TC_PARTS;
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS;
constexpr uint32_t TC_A_BYTES = TC_TILE * 128 * 2;   // one key tile
constexpr uint32_t TC_B_BYTES = 3 * 128 * 128 * 2;   // three limb matrices
constexpr uint32_t TC_TMEM_COLS = 512;               // two fp32 accumulators of 128 columns; the rest is only
                                                     // there so that a 16-column read may start at any column
constexpr int TC_MAX_UNITS = JQK_MAX_WORDS;          // a unit is one record word, or two neighbouring ones
constexpr int TC_MAX_SLOTS = 20;                     // 16-column reads of all units (more: generic path)
constexpr unsigned long long TC_WAIT_NS = 2000000000ull;

// Classes of a 16-column read.  A column of known width needs no per-column constant to be quantised
// (its thresholds are the unit thresholds of the width); a column whose width is only known at run
// time reads one word, the address of its width's cell table.  Every class but the two regular ones
// reads per-column multipliers that put a code at its bit position.
enum : int {
  TC_CLS_GENERAL = 0,  // any widths: width word + multipliers per column
  TC_CLS_ODD1 = 1,     // odd columns are 1-bit (or unused): one comparison; even columns as in the general class
  TC_CLS_ALL1 = 2,     // every column 1-bit (or unused): one comparison each
  TC_CLS_ALL2 = 3,     // every column 2-bit (or unused), one word: three comparisons each
  TC_CLS_REG4 = 4,     // sixteen 4-bit columns filling two words in order: no constants read at all
  TC_CLS_REG31 = 5,    // eight (3-bit, 1-bit) pairs filling one word in order: no constants read at all
  TC_CLS_WIDE = 6,     // columns of 5..8 bits (a byte each): binary search over the unit thresholds of the width
};
// The multiplier row of a read holds 8 bytes per column (first word, second word) when the unit has two
// words, else 4 bytes (first word).

// Unit thresholds and the cell grid, passed by value: the comparisons of the regular classes take them
// straight from the constant bank.
struct UnitConsts {
  float thr[64];  // [width - 1][16], +inf padded
  float cs, co;   // cell = round(127 * saturate(x * cs + co))
};

// How the epilogue warps share a head's record: units (one record word, or two neighbouring ones) are
// dealt to the parts, and each unit is quantised in 16-column reads ("slots").
struct TcPlan {
  // reads of each part in the order they run: x = first column | slot << 8,
  // y = first word of the unit | words << 8 | first read of the unit << 16 | last read << 17 | class << 18
  int2 step[TC_PARTS][TC_MAX_SLOTS];
  int32_t n_steps[TC_PARTS];
  int32_t n_slots;                  // n_slots > TC_MAX_SLOTS: the generic path runs
  int32_t slot_step[TC_MAX_SLOTS];  // part * 32 + position in the part's list
  int32_t cut[TC_PARTS + 1];        // word ranges of the parts (generic path)
};

struct TcSmem {
  uint8_t a[TC_STAGES][TC_A_BYTES];  // [k half][128 keys][64 dims], 128B swizzle
  uint8_t b[3][128 * 128 * 2];       // limb l: [k half][128 columns][64 dims], 128B swizzle
  float c0[128];          // centred tables: the mean in column space, subtracted from every transformed value
  float uthr[64];         // unit decision thresholds, [width - 1][16]
  float uwide[4 * 256];   // unit decision thresholds of the widths 5..8, +inf padded rows (tables with wide columns)
  uint8_t upre[4 * 128];  // per width and cell: 16 * (width - 1) + a lower bound of the code (at most one short),
                          // i.e. the index into uthr at which the one exact comparison is made
  // one entry per column of every 16-column read: crow_w = the bit pattern of the shared-memory address
  // of the cell row of the column's width (classes with run-time widths); crow_m = 1 << bit position
  // when the column's code belongs to the first / second word of the unit that issues the read (both 0
  // for columns the read merely passes over)
  float crow_w[TC_MAX_SLOTS * CH];
  uint2 crow_m[TC_MAX_SLOTS * CH];
  TcPlan plan;
  int32_t meta[128];
  int32_t wcb[JQK_MAX_WORDS + 4];
  uint64_t full[TC_STAGES], empty[TC_STAGES], acc_full[2], acc_empty[2], b_full;
  uint32_t tmem_base;
  volatile int abort;
};

static_assert(TC_MAX_UNITS * sizeof(int4) <= sizeof(TcSmem::crow_m), "the planner's scratch lies in the row table");
static_assert(sizeof(TcSmem) + 1024 <= 232448, "shared memory of the tensor-core compress kernel");

struct TcArgs {
  const int32_t* n_tokens;
  const int32_t* seq_starts;
  const int32_t* page_table;
  int32_t pt_stride;
  int32_t n_pages;
  int32_t tiles_per_block;
  int32_t max_tiles;   // tile slots per sequence: the block's run is a range of sequence * max_tiles + tile
  int32_t n_seqs;
  int32_t* status;
};

// A block's run of key tiles: slots [f, f_hi) of the head's tile list, slot = sequence * max_tiles +
// tile.  Slots past a sequence's last key are passed over, the same way by every role.
struct TileWalk {
  int f, f_hi, seq, t, max_tiles, n_tok;
  const int32_t* n_tokens;
  __device__ TileWalk(int f_lo, int f_hi_, int max_tiles_, const int32_t* n_tokens_)
      : f(f_lo), f_hi(f_hi_), max_tiles(max_tiles_), n_tokens(n_tokens_) {
    seq = f / max_tiles;
    t = f - seq * max_tiles;
    n_tok = (f < f_hi) ? n_tokens[seq] : 0;
  }
  // moves to the next slot that holds keys; false at the end of the run
  __device__ bool valid() {
    while (f < f_hi && t * TC_TILE >= n_tok) {
      f += max_tiles - t;
      t = 0;
      ++seq;
      if (f < f_hi) n_tok = n_tokens[seq];
    }
    return f < f_hi;
  }
  __device__ void advance() {
    ++f;
    if (++t == max_tiles) {
      t = 0;
      ++seq;
      if (f < f_hi) n_tok = n_tokens[seq];
    }
  }
};

// Bounded wait: false (and the abort flag) after TC_WAIT_NS or when another role gave up.
__device__ __forceinline__ bool tc_wait(TcSmem& sm, uint64_t* bar, uint32_t parity, int32_t* status) {
  if (mbar_wait_timed<40>(bar, parity, TC_WAIT_NS, &sm.abort)) return true;
  if (!sm.abort) {
    sm.abort = 1;
    if (status) atomicOr(status, JQK_STATUS_WAIT_EXPIRED);
  }
  return false;
}

// code = #{l : x >= thr[l]} for sorted thresholds, by binary search over 2^width - 1 entries.
__device__ __forceinline__ uint32_t search_code(float x, const float* __restrict__ thr, int width) {
  uint32_t code = 0;
  for (int step = (1 << width) >> 1; step >= 1; step >>= 1)
    code += (x >= thr[code + step - 1]) ? step : 0;
  return code;
}


// Run by one whole warp (a single thread took 9 us over it, which every launch paid before its first
// tile could leave).  `wcb[w]` is the first column of record word w (n_words + 1 entries, shared
// memory), `units` a scratch of TC_MAX_UNITS int4 in shared memory.  Lane 0 lists the units, the
// lanes classify one 16-column read each, then all lanes deal the units to the parts in step (the
// same decisions in every lane; lane 0 writes).
__device__ void tc_make_plan(TcPlan& pl, const int32_t* wcb, const int32_t* meta, int n_words, int n_active, int4* units) {
  const int lane = threadIdx.x & 31;
  // Units: every record word on its own, or together with its neighbour where that saves a
  // 16-column read (two 4-bit words hold 16 columns) or one of the two has no column.
  int n_units = 0, n_slots = 0;
  if (lane == 0) {
    for (int w = 0; w < n_words;) {
      const int ca = wcb[w + 1] - wcb[w];
      int nw = 1;
      if (w + 1 < n_words) {
        const int cb = wcb[w + 2] - wcb[w + 1];
        // (a word of byte-wide codes never shares a unit with a word of narrow ones: their reads differ in kind)
        const bool same_kind = ca == 0 || cb == 0 || ((meta[wcb[w]] & 15) > 4) == ((meta[wcb[w + 1]] & 15) > 4);
        if (same_kind && (ca == 0 || cb == 0 || (ca + cb + CH - 1) / CH < (ca + CH - 1) / CH + (cb + CH - 1) / CH)) nw = 2;
      }
      // (a unit without columns still writes its zero words: one read that places nothing)
      const int reads = max(1, (wcb[w + nw] - wcb[w] + CH - 1) / CH);
      units[n_units] = make_int4(w | (nw << 8), wcb[w], reads, n_slots);
      n_slots += reads;
      ++n_units;
      w += nw;
    }
    pl.n_slots = n_slots;
  }
  n_units = __shfl_sync(0xffffffffu, n_units, 0);
  n_slots = __shfl_sync(0xffffffffu, n_slots, 0);
  __syncwarp();
  const bool planned = n_slots <= TC_MAX_SLOTS;   // at most 20: one read per lane
  // class of read `lane` from the widths of its columns (columns past the unit count as unused)
  int my_cls = TC_CLS_GENERAL;
  if (planned && lane < n_slots) {
    int4 un = units[0];
    for (int u = 1; u < n_units; ++u) {
      const int4 cand = units[u];
      if (cand.w <= lane) un = cand;
    }
    const int r = lane - un.w;
    const int c_end = wcb[(un.x & 255) + (un.x >> 8)];
    const bool one_word = (un.x >> 8) == 1;
    const bool full = un.y + r * CH + CH <= c_end;
    bool all1 = true, all2 = true, odd1 = true, reg4 = !one_word && full, reg31 = one_word && full, wide = false;
#pragma unroll 4
    for (int i = 0; i < CH; ++i) {
      const int col = un.y + r * CH + i;
      const int mt = (col < c_end) ? meta[col] : 0;
      const int width = mt & 15, bp = (mt >> 4) & 1023;
      wide = wide || width > 4;
      all1 = all1 && (width == 0 || width == 1);
      all2 = all2 && (width == 0 || width == 2);
      if (i & 1) odd1 = odd1 && (width == 0 || width == 1);
      reg4 = reg4 && width == 4 && bp == 32 * (un.x & 255) + 4 * i;
      reg31 = reg31 && width == ((i & 1) ? 1 : 3) && bp == 32 * (un.x & 255) + 4 * (i / 2) + 3 * (i & 1);
    }
    my_cls = wide ? TC_CLS_WIDE : reg4 ? TC_CLS_REG4 : reg31 ? TC_CLS_REG31 : (all1 && one_word) ? TC_CLS_ALL1 : (all2 && one_word) ? TC_CLS_ALL2
           : odd1 ? TC_CLS_ODD1 : TC_CLS_GENERAL;
  }
  // units to parts: largest first (ties: the earlier unit), each to the part with the least work so far
  int load[TC_PARTS], n_steps[TC_PARTS];
#pragma unroll
  for (int q = 0; q < TC_PARTS; ++q) { load[q] = 0; n_steps[q] = 0; }
  const int4 mine = (lane < n_units) ? units[lane] : make_int4(0, 0, 0, 0);
  bool taken = lane >= n_units;
  for (int k = 0; k < n_units && planned; ++k) {
    const int key = taken ? -1 : ((mine.z << 5) | (31 - lane));
    const int best_key = __reduce_max_sync(0xffffffffu, key);
    const int best = 31 - (best_key & 31);
    if (lane == best) taken = true;
    const int un_x = __shfl_sync(0xffffffffu, mine.x, best), un_y = __shfl_sync(0xffffffffu, mine.y, best);
    const int un_z = __shfl_sync(0xffffffffu, mine.z, best), un_w = __shfl_sync(0xffffffffu, mine.w, best);
    int q_min = 0;
#pragma unroll
    for (int q = 1; q < TC_PARTS; ++q)
      if (load[q] < load[q_min]) q_min = q;
    int pos = 0;
#pragma unroll
    for (int q = 0; q < TC_PARTS; ++q)
      if (q == q_min) { load[q] += un_z * CH + 4; pos = n_steps[q]; n_steps[q] += un_z; }
    for (int r = 0; r < un_z; ++r) {
      const int cls = __shfl_sync(0xffffffffu, my_cls, un_w + r);
      if (lane == 0) {
        pl.slot_step[un_w + r] = q_min * 32 + pos + r;
        pl.step[q_min][pos + r] = make_int2((un_y + r * CH) | ((un_w + r) << 8),
                                            un_x | ((r == 0) << 16) | ((r == un_z - 1) << 17) | (cls << 18));
      }
    }
  }
  if (lane == 0) {
#pragma unroll
    for (int q = 0; q < TC_PARTS; ++q) pl.n_steps[q] = planned ? n_steps[q] : 0;
    // generic path only: word ranges cut where the column counts are closest to even
    int cut[TC_PARTS + 1];
#pragma unroll
    for (int q = 0; q < TC_PARTS; ++q) cut[q] = 0;
    cut[TC_PARTS] = n_words;
#pragma unroll
    for (int q = 1; q < TC_PARTS && !planned; ++q) {
      const int target = (n_active * q + TC_PARTS / 2) / TC_PARTS;
      int w = cut[q - 1];
      while (w < n_words && wcb[w] < target) ++w;
      if (w > cut[q - 1] && w < n_words && target - wcb[w - 1] < wcb[w] - target) --w;
      cut[q] = max(w, cut[q - 1]);
    }
#pragma unroll
    for (int q = 0; q <= TC_PARTS; ++q) pl.cut[q] = cut[q];
  }
  __syncwarp();
}

// Constants of entry e (slot e / 16, column e % 16 of the read) of a planned head: x = the bit pattern
// of the address of the cell row of the column's width (`pre_addr`: shared-memory address of the four
// cell rows; `uwide_addr`: of the threshold rows of the widths 5..8), y / z = multipliers for the first / second word of the unit.
__device__ __forceinline__ uint3 tc_const_row(const TcPlan& pl, const int32_t* wcb, const int32_t* meta, uint32_t pre_addr,
                                              uint32_t uwide_addr, int e) {
  const int ss = pl.slot_step[e >> 4];
  const int2 st = pl.step[ss >> 5][ss & 31];
  const int w_first = st.y & 255, nw = (st.y >> 8) & 255;
  const int col = (st.x & 255) + (e & 15);
  const bool mine = col < wcb[w_first + nw];  // the column belongs to the unit that issues the read
  uint32_t m_lo = 0u, m_hi = 0u;
  int width = 1;
  if (mine) {
    const int bp = (meta[col] >> 4) & 1023;
    if ((bp >> 5) == w_first) m_lo = 1u << (bp & 31);
    else m_hi = 1u << (bp & 31);
    width = max(1, meta[col] & 15);
  }
  // a read of byte-wide columns: the address of the threshold row of the column's width instead
  if (((st.y >> 18) & 7) == TC_CLS_WIDE) return make_uint3(uwide_addr + (uint32_t)(max(width, 5) - 5) * 1024u, m_lo, m_hi);
  return make_uint3(pre_addr + (uint32_t)(width - 1) * 128u, m_lo, m_hi);
}

// Shared-space loads at a register address plus a compile-time offset (the address register of the
// cell read is a float's bit pattern, so these cannot go through C++ pointers).
template <int OFF>
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr) {
  uint32_t r;
  asm("ld.shared.u8 %0, [%1+%2];" : "=r"(r) : "r"(addr), "n"(OFF));
  return r;
}
template <int OFF>
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float r;
  asm("ld.shared.f32 %0, [%1+%2];" : "=f"(r) : "r"(addr), "n"(OFF));
  return r;
}

// f(integral_constant<int, I>) for I = 0 .. N-1, unrolled at compile time.
template <int I, int N, class F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}

// Codes of 16 consecutive columns of one key, added at their bit positions into the one or two word
// registers of the unit.  Written stage by stage over all 16 columns (cells, lower bounds, thresholds,
// comparison, placement) so that the dependent shared-memory reads of a column overlap with those of
// the other fifteen.  A column of width W is quantised against the unit levels of W: a cell of the
// common grid gives, through the cell row of W, the index j of the one threshold that still has to be
// compared exactly; code = (j & 15) + (v >= uthr[j]).  1- and 2-bit columns of known width compare
// with their one or three thresholds directly (operands from the constant bank).  `rw` / `rm`: the
// read's width words and multipliers; `pre_base[W - 1]`: bit pattern (as a float) of the address of
// the cell row of width W; `uthr_addr`: address of the unit thresholds.  The cell index is formed in
// the subnormal range, where a float's bit pattern is its integer value: fma(y, 127 * 2^-149, base)
// has the bit pattern base + round(127 y), the address of the cell.
template <int CLS, int J>
__device__ __forceinline__ void quant16(const UnitConsts& uc, const float* __restrict__ rw, const uint2* __restrict__ rm,
                                        const float (&v)[CH], const float (&pre_base)[4], uint32_t uthr_addr, uint32_t& lo,
                                        uint32_t& hi) {
  constexpr bool all2 = CLS == TC_CLS_ALL2, all1 = CLS == TC_CLS_ALL1;
  uint32_t k[CH];
  float t[CH];
  // stage 1: cell addresses (or the finished code of a directly compared column)
  static_for<0, CH / 4>([&](auto qc) {
    constexpr int Q = decltype(qc)::value;
    [[maybe_unused]] float4 w4;
    if constexpr (CLS == TC_CLS_GENERAL || CLS == TC_CLS_ODD1) w4 = reinterpret_cast<const float4*>(rw)[Q];
    static_for<0, 4>([&](auto hc) {
      constexpr int H = decltype(hc)::value, I = 4 * Q + H;
      constexpr bool direct1 = all1 || ((CLS == TC_CLS_ODD1 || CLS == TC_CLS_REG31) && (I & 1));
      if constexpr (all2) {
        k[I] = ((v[I] >= uc.thr[16]) ? 1u : 0u) + ((v[I] >= uc.thr[17]) ? 1u : 0u) + ((v[I] >= uc.thr[18]) ? 1u : 0u);
      } else if constexpr (direct1) {
        k[I] = (v[I] >= uc.thr[0]) ? 1u : 0u;
      } else {
        const float y = __saturatef(fmaf(v[I], uc.cs, uc.co));
        float base;
        if constexpr (CLS == TC_CLS_REG4) base = pre_base[3];
        else if constexpr (CLS == TC_CLS_REG31) base = pre_base[2];
        else base = (H == 0 ? w4.x : H == 1 ? w4.y : H == 2 ? w4.z : w4.w);
        k[I] = __float_as_uint(fmaf(y, __uint_as_float(127u), base));  // address of the cell
      }
    });
  });
  // stage 2: j = lower bound of the code with the width's offset; stage 3: the exact threshold at j
  static_for<0, CH>([&](auto ic) {
    constexpr int I = decltype(ic)::value;
    constexpr bool direct = all2 || all1 || ((CLS == TC_CLS_ODD1 || CLS == TC_CLS_REG31) && (I & 1));
    if constexpr (!direct) k[I] = lds_u8<0>(k[I]);
  });
  static_for<0, CH>([&](auto ic) {
    constexpr int I = decltype(ic)::value;
    constexpr bool direct = all2 || all1 || ((CLS == TC_CLS_ODD1 || CLS == TC_CLS_REG31) && (I & 1));
    if constexpr (!direct) t[I] = lds_f32<0>(uthr_addr + 4u * k[I]);
  });
  // stage 4: the one exact comparison, and the code at its bit position
  if constexpr (CLS == TC_CLS_REG31) {
    static_for<0, CH>([&](auto ic) {
      constexpr int I = decltype(ic)::value;
      if constexpr (!(I & 1)) k[I] = (k[I] & 15u) + ((v[I] >= t[I]) ? 1u : 0u);
      lo += k[I] * (1u << (4 * (I / 2) + 3 * (I & 1)));
    });
  } else if constexpr (CLS == TC_CLS_REG4) {
    static_for<0, CH>([&](auto ic) {
      constexpr int I = decltype(ic)::value;
      k[I] = (k[I] & 15u) + ((v[I] >= t[I]) ? 1u : 0u);
      if constexpr (I < 8) lo += k[I] * (1u << (4 * I));
      else hi += k[I] * (1u << (4 * (I - 8)));
    });
  } else if constexpr (J > 1) {
    static_for<0, CH / 2>([&](auto pc) {
      constexpr int P = decltype(pc)::value;
      const uint4 m2 = reinterpret_cast<const uint4*>(rm)[P];
      static_for<0, 2>([&](auto hc) {
        constexpr int I = 2 * P + decltype(hc)::value;
        constexpr bool direct = all2 || all1 || (CLS == TC_CLS_ODD1 && (I & 1));
        const uint2 m = (I & 1) ? make_uint2(m2.z, m2.w) : make_uint2(m2.x, m2.y);
        if constexpr (!direct) k[I] = (k[I] & 15u) + ((v[I] >= t[I]) ? 1u : 0u);
        lo += k[I] * m.x;
        hi += k[I] * m.y;
      });
    });
  } else {
    static_for<0, CH / 4>([&](auto qc) {
      constexpr int Q = decltype(qc)::value;
      const uint4 m4 = reinterpret_cast<const uint4*>(rm)[Q];  // four columns' first-word multipliers
      static_for<0, 4>([&](auto hc) {
        constexpr int H = decltype(hc)::value, I = 4 * Q + H;
        constexpr bool direct = all2 || all1 || (CLS == TC_CLS_ODD1 && (I & 1));
        if constexpr (!direct) k[I] = (k[I] & 15u) + ((v[I] >= t[I]) ? 1u : 0u);
        lo += k[I] * (H == 0 ? m4.x : H == 1 ? m4.y : H == 2 ? m4.z : m4.w);
      });
    });
  }
}

// Codes of the byte-wide columns of one read (a unit of one or two words of four such columns: the
// first eight columns of the read at most), by binary search over the +inf padded threshold row of
// each column's width; `rw`: bit patterns of the rows' shared-memory addresses.  The eight searches
// run side by side, a step of all of them before the next.
template <int J>
__device__ __forceinline__ void quant_wide(const float* __restrict__ rw, const uint2* __restrict__ rm, const float (&v)[CH],
                                           uint32_t& lo, uint32_t& hi) {
  constexpr int NW = 8;
  uint32_t a[NW];
  const float4 w0 = reinterpret_cast<const float4*>(rw)[0], w1 = reinterpret_cast<const float4*>(rw)[1];
  a[0] = __float_as_uint(w0.x); a[1] = __float_as_uint(w0.y); a[2] = __float_as_uint(w0.z); a[3] = __float_as_uint(w0.w);
  a[4] = __float_as_uint(w1.x); a[5] = __float_as_uint(w1.y); a[6] = __float_as_uint(w1.z); a[7] = __float_as_uint(w1.w);
  static_for<0, 8>([&](auto sc) {
    constexpr int STEP = 128 >> decltype(sc)::value;
    static_for<0, NW>([&](auto ic) {
      constexpr int I = decltype(ic)::value;
      a[I] += (v[I] >= lds_f32<4 * (STEP - 1)>(a[I])) ? 4u * STEP : 0u;   // a = row address + 4 * code so far
    });
  });
  static_for<0, NW>([&](auto ic) {
    constexpr int I = decltype(ic)::value;
    const uint32_t row = __float_as_uint(I < 4 ? (I == 0 ? w0.x : I == 1 ? w0.y : I == 2 ? w0.z : w0.w)
                                                : (I == 4 ? w1.x : I == 5 ? w1.y : I == 6 ? w1.z : w1.w));
    const uint32_t code = (a[I] - row) >> 2;
    if constexpr (J > 1) {
      const uint2 m = rm[I];
      lo += code * m.x;
      hi += code * m.y;
    } else {
      lo += code * reinterpret_cast<const uint32_t*>(rm)[I];
    }
  });
}

template <bool CENTERED, bool WIDE>
__global__ void __launch_bounds__(TC_THREADS, 1)
compress_tc_kernel(const __grid_constant__ CUtensorMap key_map, const __grid_constant__ CUtensorMap limb_map,
                   const __grid_constant__ UnitConsts uc, jqk_head_tables tb, TcArgs pa, uint32_t* __restrict__ k_pool) {
  extern __shared__ uint8_t smem_raw[];
  // align by pointer arithmetic on the __shared__ array (an integer round trip would turn every access into a generic load)
  TcSmem& sm = *reinterpret_cast<TcSmem*>(smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int head = blockIdx.y;
  const int f_lo = blockIdx.x * pa.tiles_per_block;
  const int f_hi = min(pa.n_seqs * pa.max_tiles, f_lo + pa.tiles_per_block);
  if (f_lo >= f_hi) return;
  // Launched as a programmatic dependent: the set-up below (the head's static tables, barriers,
  // tensor memory, the limb matrices, the read plan) may overlap the tail of the previous kernel on
  // the stream; every role waits for that kernel (griddepcontrol.wait) before it first touches what
  // a call passes in or out: token counts, keys, page table, pages.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const HeadDesc hd = load_desc(tb.desc, head);

  // ---- set-up ----
  // the shared quantiser tables (the same for every head and column) and this head's column descriptors
  for (int e = tid; e < 64; e += TC_THREADS) sm.uthr[e] = uc.thr[e];
  for (int e = tid; e < 4 * 128 / 4; e += TC_THREADS)
    reinterpret_cast<uint32_t*>(sm.upre)[e] = reinterpret_cast<const uint32_t*>(tb.unit_pre)[e];
  for (int e = tid; e < 128; e += TC_THREADS) sm.meta[e] = tb.col_meta[(size_t)head * 128 + e];
  if constexpr (CENTERED)
    for (int e = tid; e < 128; e += TC_THREADS) sm.c0[e] = tb.center_cols[(size_t)head * 128 + e];
  if constexpr (WIDE)
    for (int e = tid; e < 4 * 256; e += TC_THREADS) sm.uwide[e] = tb.unit_wide_thr[e];
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
      asm volatile("griddepcontrol.wait;" ::: "memory");
      int issued = 0;
      for (TileWalk w(f_lo, f_hi, pa.max_tiles, pa.n_tokens); w.valid(); w.advance(), ++issued) {
        const int s = issued % TC_STAGES;
        const uint32_t ph = (issued / TC_STAGES) & 1;
        if (issued >= TC_STAGES && !tc_wait(sm, &sm.empty[s], ph ^ 1, pa.status)) break;
        mbar_arrive_expect_tx(&sm.full[s], TC_A_BYTES);
        tma_load_4d(sm.a[s], &key_map, &sm.full[s], 0, w.t * TC_TILE, head, w.seq);
        tma_load_4d(sm.a[s] + TC_A_BYTES / 2, &key_map, &sm.full[s], 64, w.t * TC_TILE, head, w.seq);
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
      asm volatile("griddepcontrol.wait;" ::: "memory");
      bool ok = tc_wait(sm, &sm.b_full, 0, pa.status);
      int it = 0;
      for (TileWalk w(f_lo, f_hi, pa.max_tiles, pa.n_tokens); ok && w.valid(); w.advance(), ++it) {
        const int s = it % TC_STAGES, a = it & 1;
        if (!tc_wait(sm, &sm.full[s], (it / TC_STAGES) & 1, pa.status)) break;
        if (it >= 2 && !tc_wait(sm, &sm.acc_empty[a], ((it >> 1) & 1) ^ 1, pa.status)) break;
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
      }
    }
  } else {
    // ================= epilogue =================
    const int ew = warp - 2;
    const int row = 32 * (warp & 3) + lane;          // TMEM lane = key inside the tile
    const int part = ew >> 2;
    if (ew == 0) tc_make_plan(sm.plan, sm.wcb, sm.meta, hd.n_words, hd.n_active, reinterpret_cast<int4*>(sm.crow_m));
    asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
    const bool planned = sm.plan.n_slots <= TC_MAX_SLOTS;
    const uint32_t pre_addr = smem_u32(sm.upre), uthr_addr = smem_u32(sm.uthr);
    if (planned) {  // constants of every read: width words and multipliers
      const int et = tid - 64;
      if (et < sm.plan.n_slots * CH) {
        const uint3 cr = tc_const_row(sm.plan, sm.wcb, sm.meta, pre_addr, smem_u32(sm.uwide), et);
        const int2 st = sm.plan.step[sm.plan.slot_step[et >> 4] >> 5][sm.plan.slot_step[et >> 4] & 31];
        asm volatile("" ::: "memory");  // the planner's scratch (units) lies in crow_m: every plan read above comes first
        sm.crow_w[et] = __uint_as_float(cr.x);
        if (((st.y >> 8) & 255) > 1)
          sm.crow_m[et] = make_uint2(cr.y, cr.z);
        else
          reinterpret_cast<uint32_t*>(sm.crow_m + (et & ~15))[et & 15] = cr.y;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(TC_EPI_WARPS * 32) : "memory");
    const int w_lo = sm.plan.cut[part], w_hi = sm.plan.cut[part + 1];
    const int c_lo = sm.wcb[w_lo], c_hi = sm.wcb[w_hi];
    const int my_steps = sm.plan.n_steps[part];
    float pre_base[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) pre_base[w] = __uint_as_float(pre_addr + 128u * w);
    const int wpr = tb.words_per_record;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    int it = 0;
    int seq_of_start = -1, seq_start = 0;
    for (TileWalk w(f_lo, f_hi, pa.max_tiles, pa.n_tokens); w.valid(); w.advance(), ++it) {
      const int a = it & 1, seq = w.seq;
      if (seq != seq_of_start) {
        seq_start = pa.seq_starts ? pa.seq_starts[seq] : 0;
        seq_of_start = seq;
      }
      if (!tc_wait(sm, &sm.acc_full[a], (it >> 1) & 1, pa.status)) break;
      tc_fence_after();
      const int key = w.t * TC_TILE + row;
      const bool valid = key < w.n_tok;
      uint32_t* dst = nullptr;
      if (valid) {
        const int tok = seq_start + key;
        const int page = lookup_page(pa.page_table, pa.pt_stride, seq, tok / JQK_PAGE_TOKENS, pa.n_pages, pa.status);
        if (page >= 0)
          dst = k_pool + ((size_t)page * tb.n_heads + head) * wpr * JQK_PAGE_TOKENS + (tok % JQK_PAGE_TOKENS);
      }
      const uint32_t t_lane = tmem + a * 128 + ((uint32_t)(32 * (warp & 3)) << 16);
      if (planned) {
        // (blocking reads: a second register buffer for a read ahead costs more than its wait)
        float v[CH];
        uint32_t lo = 0u, hi = 0u;
#pragma unroll 1
        for (int s = 0; s < my_steps; ++s) {
          const int2 cur = sm.plan.step[part][s];
          tmem_ld16(t_lane + (cur.x & 255), v);
          if constexpr (CENTERED) {
            const float* cc = sm.c0 + (cur.x & 255);   // the same address in every lane: one broadcast read each
#pragma unroll
            for (int i = 0; i < CH; ++i) v[i] -= (((cur.x & 255) + i) < 128) ? cc[i] : 0.f;
          }
          const float* rw = sm.crow_w + (cur.x >> 8) * CH;
          const uint2* rm = sm.crow_m + (cur.x >> 8) * CH;
          if (cur.y & (1 << 16)) lo = hi = 0u;
          const bool two = (cur.y & 0xff00) == 0x200;
          const int cls = (cur.y >> 18) & 7;  // warp-uniform
          if (WIDE && cls == TC_CLS_WIDE) {
            if (two) quant_wide<2>(rw, rm, v, lo, hi);
            else quant_wide<1>(rw, rm, v, lo, hi);
          } else switch (cls) {
            case TC_CLS_REG4: quant16<TC_CLS_REG4, 2>(uc, rw, rm, v, pre_base, uthr_addr, lo, hi); break;
            case TC_CLS_REG31: quant16<TC_CLS_REG31, 1>(uc, rw, rm, v, pre_base, uthr_addr, lo, hi); break;
            case TC_CLS_ALL2: quant16<TC_CLS_ALL2, 1>(uc, rw, rm, v, pre_base, uthr_addr, lo, hi); break;
            case TC_CLS_ALL1: quant16<TC_CLS_ALL1, 1>(uc, rw, rm, v, pre_base, uthr_addr, lo, hi); break;
            case TC_CLS_ODD1:
              if (two) quant16<TC_CLS_ODD1, 2>(uc, rw, rm, v, pre_base, uthr_addr, lo, hi);
              else quant16<TC_CLS_ODD1, 1>(uc, rw, rm, v, pre_base, uthr_addr, lo, hi);
              break;
            default:
              if (two) quant16<TC_CLS_GENERAL, 2>(uc, rw, rm, v, pre_base, uthr_addr, lo, hi);
              else quant16<TC_CLS_GENERAL, 1>(uc, rw, rm, v, pre_base, uthr_addr, lo, hi);
          }
          if ((cur.y & (1 << 17)) && dst) {
            dst[(cur.y & 255) * JQK_PAGE_TOKENS] = lo;
            if (two) dst[((cur.y & 255) + 1) * JQK_PAGE_TOKENS] = hi;
          }
        }
      } else {
        int cur_w = w_lo;
        uint32_t cur = 0;
        for (int c0 = c_lo; c0 < c_hi; c0 += CH) {
          float v[CH];
          tmem_ld16(t_lane + c0, v);
          if constexpr (CENTERED) {
#pragma unroll
            for (int i = 0; i < CH; ++i) v[i] -= (c0 + i < 128) ? sm.c0[c0 + i] : 0.f;
          }
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
            const int wd = m & 15;
            const float* thr_row = (WIDE && wd > 4) ? sm.uwide + (wd - 5) * 256 : sm.uthr + (wd - 1) * 16;
            cur |= search_code(x, thr_row, wd) << (bp & 31);
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
    }
  }

  // ---- teardown ----
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, TC_TMEM_COLS);
  }
}

}  // namespace jqk

using namespace jqk;


// Launches the tensor-core kernel when the call fits it (bf16 keys, head_dim 128, 16-byte aligned
// strides); returns 1 when the caller should use the fp32 CUDA-core kernel instead.
int32_t jqk_compress_tc_try(const jqk_head_tables* tables, const void* keys, int32_t key_dtype,
                            int64_t seq_stride, int64_t head_stride, int64_t token_stride, int32_t n_seqs,
                            const int32_t* n_tokens, const int32_t* seq_starts, int32_t max_tokens,
                            const int32_t* page_table, int32_t page_table_stride, int32_t n_pages,
                            uint32_t* k_pool, int32_t* status, cudaStream_t st) {
  if (key_dtype != JQK_DTYPE_BF16 || tables->d != 128 || !tables->fwd_limbs || (tables->n_wide > 0 && !tables->unit_wide_thr) ||
      (tables->center && !tables->center_cols))
    return 1;
  if ((uintptr_t)keys % 16 || (token_stride * 2) % 16 || (head_stride * 2) % 16 || (seq_stride * 2) % 16) return 1;
  if ((uintptr_t)tables->fwd_limbs % 16 || max_tokens < TC_TILE || !tables->unit_pre) return 1;
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
  // At most one wave of blocks over 148 SMs (a block's set-up loads 120 KB of tables): the tile
  // slots of a head, all sequences one after the other, are cut into equal runs.
  long long blocks_per_head = 148 / tables->n_heads;
  if (blocks_per_head < 1) blocks_per_head = 1;
  const long long slots = (long long)n_seqs * max_tiles;
  if (slots > 0x7fffffffll) return 1;
  int tiles_per_block = (int)((slots + blocks_per_head - 1) / blocks_per_head);
  if (tiles_per_block < 4) tiles_per_block = 4;
  dim3 grid((unsigned)((slots + tiles_per_block - 1) / tiles_per_block), tables->n_heads, 1);
  TcArgs pa{n_tokens, seq_starts, page_table, page_table_stride, n_pages, tiles_per_block, max_tiles, n_seqs, status};
  const size_t smem = sizeof(TcSmem) + 1024;
  UnitConsts uc;
  for (int i = 0; i < 64; ++i) uc.thr[i] = tables->unit_thr[i];
  // host form of the grid: cell = clamp(round(x * aff[0] + aff[1] - 2^23), 0, 127)
  uc.cs = tables->unit_aff[0] * (1.f / 127.f);
  uc.co = (tables->unit_aff[1] - 8388608.f) * (1.f / 127.f);
  JQK_SMEM_ONCE((compress_tc_kernel<false, false>), smem, "tensor-core compress smem attribute");
  JQK_SMEM_ONCE((compress_tc_kernel<true, false>), smem, "tensor-core compress smem attribute");
  JQK_SMEM_ONCE((compress_tc_kernel<false, true>), smem, "tensor-core compress smem attribute");
  JQK_SMEM_ONCE((compress_tc_kernel<true, true>), smem, "tensor-core compress smem attribute");
  const bool wide = tables->n_wide > 0;
  cudaLaunchAttribute pdl_attr[1];
  pdl_attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl_attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(TC_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = pdl_attr;
  cfg.numAttrs = 1;
#define JQK_LAUNCH_TC(CEN, WID)                                                                                   \
  JQK_CUDA_OK(cudaLaunchKernelEx(&cfg, compress_tc_kernel<CEN, WID>, key_map, limb_map, uc, *tables, pa, k_pool), \
              "tensor-core compress launch")
  if (tables->center && wide) JQK_LAUNCH_TC(true, true);
  else if (tables->center) JQK_LAUNCH_TC(true, false);
  else if (wide) JQK_LAUNCH_TC(false, true);
  else JQK_LAUNCH_TC(false, false);
#undef JQK_LAUNCH_TC
  JQK_CUDA_OK(cudaGetLastError(), "tensor-core compress launch");
  return 0;
}
