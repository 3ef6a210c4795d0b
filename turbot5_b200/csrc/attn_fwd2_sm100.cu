// Fused relative-position-bias flash attention, forward, head dim 64, for sm_100a:
// the two-tile kernel for sequences of more than 128 query rows.
//
// One thread block per SM owns 256 query rows of one (batch, head) -- or of one packed
// sequence -- as two 128-row tiles A and B that share every K/V tile brought into shared
// memory (half the L2 -> SM traffic of one tile per block):
//
//   warps 8-11  a warpgroup of its own.  Lane 0 of warp 8 loads (Q twice, then K/V tiles into a
//               ring; cp.async.bulk.tensor, 128-byte swizzle, completion on mbarriers) and issues
//               the matrix products of tile A; lane 0 of warp 9 issues those of tile B
//               (tcgen05.mma, S = Q K^T from shared memory, O += P V with P read from tensor
//               memory; tcgen05.commit -> mbarriers).  The warpgroup gives its registers away
//               (setmaxnreg): with 12 warps every scheduler holds three, and 88 + 2 x 208
//               registers per thread fill a scheduler's 16384
//   warps 0-3   softmax of tile A, warps 4-7 softmax of tile B: ONE thread per query row.  A
//               thread copies the 128 scores of its row from tensor memory to registers
//               (tcgen05.ld) and hands the S buffer back at once, so the next Q K^T of its tile
//               runs during the softmax; row maximum, then the exponentials in four chunks
//               of 32 columns, each packed to bf16/fp16 and stored to tensor memory
//               (tcgen05.st) as soon as it is complete.
//
// Against the one-tile kernel (attn_fwd_sm100.cu: two threads per row, two blocks per SM) a
// thread handles twice the columns per tile, so the per-tile bookkeeping (barrier waits,
// fences, tile classification, maximum update) is paid once per 128 exponentials instead of
// once per 64, the two threads of a row no longer have to agree on the running maximum, and
// 208 registers per thread leave nothing to spill.  With the instruction stream that lean
// the exponential unit (16 ex2 per clock per SM) becomes the real limit, and moving a share
// of the exponentials to the FMA pipe (PolyExp) pays; see kPoly.
//
// Tensor memory: per tile S 128 + P 64 + O 64 columns (2 x 256 = all 512).  Shared memory:
// Q 2 x 16 KB, K/V ring 3 x 32 KB.
//
// Semantics follow flash_attention_with_fusing_bias
// (src/turbot5/ops/fused_bias_attention.py:184-365) and its packed-sequence counterpart
// (src/turbot5/ops/varlen_fused_bias_attn.py:211-375) with positions as in the reference's
// `basic` path: delta = n - (q_pos_offset + m).
#include "t5b_common.cuh"
#include "attn_params.cuh"
#include "attn_sm100_util.cuh"

#include <atomic>
#include <type_traits>

namespace t5b {
namespace sm100w {

using sm100::pack2;
using sm100::PolyExp;
using sm100::poly_pair;
using sm100::pow2_neg;
using sm100::kRescaleThreshold;
using sm100::make_tmap;

// Issue-order-pinned forms of the softmax arithmetic (volatile: the compiler keeps volatile asm
// statements in program order, which is how pass 2 lays out its software pipeline).
__device__ __forceinline__ void vfma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm volatile("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
               "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
               "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
               : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ float vex2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void vadd2(float& acc0, float& acc1, float x0, float x1) {
  asm volatile("{\n\t.reg .b64 ra, rx;\n\t"
               "mov.b64 ra, {%0, %1};\n\tmov.b64 rx, {%2, %3};\n\t"
               "add.rn.f32x2 ra, ra, rx;\n\tmov.b64 {%0, %1}, ra;\n\t}"
               : "+f"(acc0), "+f"(acc1) : "f"(x0), "f"(x1));
}
template <bool kBf16>
__device__ __forceinline__ uint32_t vpack2(float lo, float hi) {
  uint32_t r;
  if (kBf16) asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  else asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

constexpr int HD = 64;
constexpr int BM = 128;              // query rows per tile
constexpr int TILES = 2;             // tiles per block
constexpr int BLOCK_M = BM * TILES;  // query rows per block
constexpr int BN = 128;              // keys per tile
constexpr int STAGES = 3;            // K/V ring depth
constexpr int NUM_THREADS = 384;
constexpr int REGS_IO = 88, REGS_SOFTMAX = 208;   // per thread after setmaxnreg: (88 + 2 * 208) * 32 = 16128 per scheduler
constexpr int WARP_IO = 8;
constexpr int TMEM_COLS = 512;
constexpr int TILE_COLS = 256;       // tensor-memory columns per query tile
constexpr int COL_S = 0, COL_P = 128, COL_O = 192;
constexpr int Q_BYTES = BM * HD * 2;     // one query tile
constexpr int KV_BYTES = BN * HD * 2;    // one K or V tile
constexpr int SMEM_TILES = TILES * Q_BYTES + 2 * STAGES * KV_BYTES;
constexpr int LUT_PAD = BM + BN;         // bias table padding on each side (entries)

#ifndef T5B_FWD2_POLY
#define T5B_FWD2_POLY 0              // column pairs of every 8 whose exponentials run on the FMA pipe
#endif

enum {
  BAR_Q_FULL = 0,
  BAR_K_FULL = 1,                      // [STAGES]
  BAR_V_FULL = BAR_K_FULL + STAGES,
  BAR_K_EMPTY = BAR_V_FULL + STAGES,
  BAR_V_EMPTY = BAR_K_EMPTY + STAGES,
  BAR_S_FULL = BAR_V_EMPTY + STAGES,   // [TILES]
  BAR_S_FREE = BAR_S_FULL + TILES,
  BAR_P_FULL = BAR_S_FREE + TILES,
  BAR_O_DONE = BAR_P_FULL + TILES,
  NUM_BARS = BAR_O_DONE + TILES
};

struct __align__(8) Control {
  unsigned long long bars[NUM_BARS];
  uint32_t tmem_base;
  int abort_flag;
  int work[6];   // a TileWork, broadcast from warp 0 for packed sequences
};

__host__ __device__ inline size_t smem_bytes(int lut_entries) {
  return 1024 /*alignment slack*/ + SMEM_TILES + sizeof(Control) + 16 + (size_t)lut_entries * 4;
}

// kPoly: of every 8 column pairs of an unmasked tile, this many take their exponentials on the FMA
// pipe (PolyExp) instead of the exponential unit; 8 = all of them (used by the parity tests).
template <bool kBf16, int kPoly>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmap_q,
                 const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v,
                 const __grid_constant__ AttnParams p,
                 const __grid_constant__ BucketSpec spec) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sQ = base;
  const uint32_t sK = base + TILES * Q_BYTES;
  const uint32_t sV = sK + STAGES * KV_BYTES;
  Control* ctl = reinterpret_cast<Control*>(smem + SMEM_TILES);
  float* lut = reinterpret_cast<float*>(smem + SMEM_TILES + ((sizeof(Control) + 15) / 16) * 16);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---------------------------------------------------------------- work item
  // dense: 1-D grid over (256-row tile, head, batch), heaviest causal tiles first; blocks at or
  //        beyond p.tail_first share a tile `parts` ways along the keys (last-wave balancing)
  // packed: blockIdx.x indexes the concatenated per-sequence lists of 256-row tiles, blockIdx.y = head
  TileWork* shared_work = reinterpret_cast<TileWork*>(&ctl->work[0]);
  TileWork w;
  int h, batch_idx = 0, part = 0, parts = 1, tail_slot = 0;
  if (p.cu_q == nullptr) {
    int tile_lin = (int)blockIdx.x;
    if (tile_lin >= p.tail_first) {
      const int e = tile_lin - p.tail_first;
      parts = p.tail_parts;
      tail_slot = e / parts;
      part = e - tail_slot * parts;
      tile_lin = p.tail_first + tail_slot;
    }
    const int tx = tile_lin % p.tiles_x;
    const int hb = tile_lin / p.tiles_x;
    h = hb % p.H;
    batch_idx = hb / p.H;
    w = dense_tile<BLOCK_M>(p, tx, batch_idx);
  } else {
    h = blockIdx.y;
    if (warp == 0) {
      TileWork f = find_varlen_tile<BLOCK_M>(p, (int)blockIdx.x);
      if (lane == 0) *shared_work = f;
    }
    __syncthreads();
    w = *shared_work;
    if (w.b < 0) return;   // block beyond the last tile: uniform exit, nothing allocated yet
  }
  const int b = w.b, q_row0 = w.q_row0, rows_in_block = w.rows_in_tile;
  const int k_row0 = w.k_row0, qpos0 = w.qpos0, len_k = w.len_k;

  // key tiles each query tile walks: [kv_first, kv_first + n_t)
  int n_tile[TILES];
  int kv_first = 0;
  #pragma unroll
  for (int t = 0; t < TILES; ++t) {
    const int rows_t = min(BM, max(0, rows_in_block - t * BM));
    int kv_end = len_k;
    if (p.causal) kv_end = min(len_k, qpos0 + t * BM + rows_t);
    n_tile[t] = (rows_t > 0 && kv_end > 0) ? (kv_end + BN - 1) / BN : 0;
  }
  if (parts > 1) {     // dense, not causal: both tiles see all keys; this block takes one share of them
    const int n_all = n_tile[0];
    const int kv_per = (n_all + parts - 1) / parts;
    kv_first = min(part * kv_per, n_all);
    const int n_mine = min(n_all, kv_first + kv_per) - kv_first;
    n_tile[0] = n_mine;
    n_tile[1] = n_tile[1] > 0 ? n_mine : 0;
  }
  const int n_max = max(n_tile[0], n_tile[1]);
  const int n_first = kv_first * BN;       // first key of this block's first tile

  // ---------------------------------------------------------------- set-up
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  auto load_k = [&](int j) {
    const int s = j % STAGES;
    mbar_expect_tx(bar(BAR_K_FULL + s), KV_BYTES);
    tma_load_4d(sK + s * KV_BYTES, &tmap_k, bar(BAR_K_FULL + s), 0, k_row0 + n_first + j * BN, h, b);
  };
  auto load_v = [&](int j) {
    const int s = j % STAGES;
    mbar_expect_tx(bar(BAR_V_FULL + s), KV_BYTES);
    tma_load_4d(sV + s * KV_BYTES, &tmap_v, bar(BAR_V_FULL + s), 0, k_row0 + n_first + j * BN, h, b);
  };
  // The loading thread sets up the barriers itself and requests Q and the first STAGES key/value
  // tiles at once: they are in flight while the other threads build the bias table below.
  if (warp == WARP_IO && lane == 0) {
    ctl->abort_flag = 0;
    mbar_init(bar(BAR_Q_FULL), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(BAR_K_FULL + s), 1);
      mbar_init(bar(BAR_V_FULL + s), 1);
      mbar_init(bar(BAR_K_EMPTY + s), TILES);    // one arrival per issuing thread
      mbar_init(bar(BAR_V_EMPTY + s), TILES);
    }
    for (int t = 0; t < TILES; ++t) {
      mbar_init(bar(BAR_S_FULL + t), 1);
      mbar_init(bar(BAR_S_FREE + t), 4);     // one arrival per softmax warp of the tile
      mbar_init(bar(BAR_P_FULL + t), 4);
      mbar_init(bar(BAR_O_DONE + t), 1);
    }
    fence_barrier_init();
    fence_proxy_async();
    if (n_max > 0) {
      mbar_expect_tx(bar(BAR_Q_FULL), TILES * Q_BYTES);
      for (int t = 0; t < TILES; ++t)
        tma_load_4d(sQ + t * Q_BYTES, &tmap_q, bar(BAR_Q_FULL), 0, q_row0 + t * BM, h, b);
      for (int j = 0; j < STAGES && j < n_max; ++j) { load_k(j); load_v(j); }
    }
  }
  __syncwarp();
  if (warp == WARP_IO) {
    tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  // delta -> bias (log2 domain) for this head.  Entry i holds delta = i - md - LUT_PAD; the table is
  // constant beyond +-md, and the padding lets a tile that straddles the +-md boundary index it
  // without clamping.
  const int md = spec.max_distance;
  if (p.table != nullptr) {
    for (int i = tid; i <= 2 * md; i += NUM_THREADS) {
      const int bucket = bucket_of_delta_counted(spec, i - md);
      lut[LUT_PAD + i] = load_table(p.table, p.table_dtype, (int64_t)bucket * p.table_stride0 + h) * kLog2e;
    }
    __syncthreads();
    const float lo_v = lut[LUT_PAD], hi_v = lut[LUT_PAD + 2 * md];
    for (int i = tid; i < LUT_PAD; i += NUM_THREADS) {
      lut[i] = lo_v;
      lut[LUT_PAD + 2 * md + 1 + i] = hi_v;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  int fail_code = 0;

  if (warp >= WARP_IO) {
    // ============================================================ loads and matrix products
    // Two issuing threads, one per query tile (lane 0 of warps 8 and 9); the first also refills the
    // K/V ring.  A tcgen05.mma costs its issuing thread tens of cycles (descriptors travel through
    // the uniform registers), and a tile step is twelve of them: one thread for both tiles was
    // busy four fifths of the time and the softmax warps waited for their scores.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_IO));
    const int t = warp - WARP_IO;                 // query tile of this issuing thread
    if (t < TILES && lane == 0 && n_max > 0) {
      constexpr uint32_t IDESC_QK = make_idesc_f16(kBf16, kBf16, BM, BN, false, false);
      constexpr uint32_t IDESC_PV = make_idesc_f16(kBf16, kBf16, BM, HD, false, true);
      const int n_t = t == 0 ? n_tile[0] : n_tile[1];
      const uint32_t tm = tmem + t * TILE_COLS;
      // One ring slot per instantiation: the shared-memory descriptors of a step are then constants
      // of the loop (kept in uniform registers), not values recomputed from j % STAGES per product.
      auto issue_qk = [&](auto slot) {
        constexpr int s = decltype(slot)::value;
        const uint64_t da = make_smem_desc_sw128(sQ + t * Q_BYTES, 16, 1024);
        const uint64_t db = make_smem_desc_sw128(sK + s * KV_BYTES, 16, 1024);
        #pragma unroll
        for (int k = 0; k < 4; ++k)   // 32 bytes of the 128-byte swizzle row per step
          umma_ss(tm + COL_S, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC_QK, k > 0);
        tc_commit(bar(BAR_S_FULL + t));
      };
      bool ok = mbar_wait_bounded(bar(BAR_Q_FULL), 0, abort_flag);
      if (!ok) fail_code = 20;
      if (ok && !mbar_wait_bounded(bar(BAR_K_FULL), 0, abort_flag)) { ok = false; fail_code = 21; }
      if (ok) {
        tc_fence_after();
        if (n_t > 0) issue_qk(std::integral_constant<int, 0>{});
        tc_commit(bar(BAR_K_EMPTY));          // (arrives at once when this thread issued nothing)
      }
      // step j with j % STAGES == slot; returns false when a wait gave up
      auto step = [&](int j, auto slot) -> bool {
        constexpr int s = decltype(slot)::value;
        constexpr int s1 = (s + 1) % STAGES;
        constexpr int sp = (s + STAGES - 1) % STAGES;       // slot of step j - 1
        const uint32_t ph = (uint32_t)((j / STAGES) & 1);
        if (j + 1 < n_max) {
          // S of the tile has been copied to registers: its next Q K^T overlaps this step's softmax
          if (!mbar_wait_bounded(bar(BAR_K_FULL + s1), (uint32_t)(((j + 1) / STAGES) & 1), abort_flag)) { fail_code = 23; return false; }
          tc_fence_after();
          if (j + 1 < n_t) {
            if (!mbar_wait_bounded(bar(BAR_S_FREE + t), (uint32_t)(j & 1), abort_flag)) { fail_code = 25; return false; }
            tc_fence_after();
            issue_qk(std::integral_constant<int, s1>{});
          }
          tc_commit(bar(BAR_K_EMPTY + s1));
        }
        if (t == 0) {
          // refill the ring: K(j+STAGES) into the slot of K(j) (the Q K^T of step j were issued a
          // step ago), V(j-1+STAGES) into the slot of V(j-1) (its products were issued a step ago)
          if (j + STAGES < n_max) {
            if (!mbar_wait_bounded(bar(BAR_K_EMPTY + s), ph, abort_flag)) { fail_code = 10; return false; }
            load_k(j + STAGES);
          }
          if (j >= 1 && j - 1 + STAGES < n_max) {
            if (!mbar_wait_bounded(bar(BAR_V_EMPTY + sp), (uint32_t)(((j - 1) / STAGES) & 1), abort_flag)) { fail_code = 11; return false; }
            load_v(j - 1 + STAGES);
          }
        }
        if (!mbar_wait_bounded(bar(BAR_V_FULL + s), ph, abort_flag)) { fail_code = 24; return false; }
        tc_fence_after();
        if (j < n_t) {
          if (!mbar_wait_bounded(bar(BAR_P_FULL + t), (uint32_t)(j & 1), abort_flag)) { fail_code = 22; return false; }
          tc_fence_after();
          // V tile is [BN keys][64 dims], dims contiguous: an MN-major B operand.  8 keys x 128 B
          // per swizzle group (1024 B, the stride byte offset); each K=16 step covers two groups.
          #pragma unroll
          for (int k = 0; k < BN / 16; ++k) {
            const uint64_t dv = make_smem_desc_sw128(sV + s * KV_BYTES + k * 2048, 16, 1024);
            umma_ts(tm + COL_O, tm + COL_P + k * 8, dv, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(bar(BAR_O_DONE + t));
        }
        tc_commit(bar(BAR_V_EMPTY + s));
        return true;
      };
      static_assert(STAGES == 3, "the loop below is written out for three ring slots");
      for (int j = 0; ok && j < n_max; j += STAGES) {
        ok = step(j, std::integral_constant<int, 0>{});
        if (ok && j + 1 < n_max) ok = step(j + 1, std::integral_constant<int, 1>{});
        if (ok && j + 2 < n_max) ok = step(j + 2, std::integral_constant<int, 2>{});
      }
    }
  } else {
    // ============================================================ softmax warps, one thread per row
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
    const int t = warp >> 2;                       // query tile of this warp
    const int quarter = warp & 3;                  // TMEM lane quarter this warp may touch
    const int r = quarter * 32 + lane;             // query row inside the tile
    const int n_kv = t == 0 ? n_tile[0] : n_tile[1];
    const int qpos_t = qpos0 + t * BM;             // key-coordinate position of the tile's first row
    const int qpos = qpos_t + r;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_base + t * TILE_COLS + COL_S;
    const uint32_t tP = tmem + lane_base + t * TILE_COLS + COL_P;
    const uint32_t tO = tmem + lane_base + t * TILE_COLS + COL_O;
    const float scale = p.scale_log2;
    const float inv_scale = 1.f / scale;
    const bool has_bias = p.table != nullptr;
    float m_use = 0.f;          // maximum the exponentials are taken against (finite)
    float l_sum = 0.f;          // row sum
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const int n0 = n_first + j * BN;             // first key of the tile
      if (!mbar_wait_bounded_warp(bar(BAR_S_FULL + t), (uint32_t)(j & 1), abort_flag)) { ok = false; fail_code = 30; break; }
      tc_fence_after();

      // the row's scores -> registers, then give the S buffer back to the issuing thread
      uint32_t sv[4][32];
      #pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_x32(tS + 32 * c, sv[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_S_FREE + t));

      // tile classification (uniform over the tile's warps)
      const bool need_mask = (n0 + BN > len_k) || (p.causal && (n0 + BN - 1 > qpos_t));
      int bias_mode = 0;            // 0 none, 1 constant over the tile, 2 per element
      float bias_const = 0.f;
      if (has_bias) {
        const int dmin = n0 - (qpos_t + BM - 1), dmax = n0 + BN - 1 - qpos_t;
        if (dmin >= md) { bias_mode = 1; bias_const = lut[2 * md + LUT_PAD]; }
        else if (dmax <= -md) { bias_mode = 1; bias_const = lut[LUT_PAD]; }
        else bias_mode = 2;
      }
      const bool fast = !need_mask && bias_mode != 2 && scale > 0.f;

      // ---- pass 1: row maximum, four independent chains.  Fast tiles (no mask, constant bias):
      // over the raw scores, transformed once.  Other tiles: x = s*scale + bias(delta) (+ mask)
      // is computed in place first.
      float mx, top_raw;     // top_raw: the largest value pass 2 will exponentiate (before e_mul, e_add)
      {
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
        if (fast) {
          // eight independent chains of two-input maxima (the three-input form is no faster per
          // element on this pipe and its chains are half as many)
          float m4 = -INFINITY, m5 = -INFINITY, m6 = -INFINITY, m7 = -INFINITY;
          #pragma unroll
          for (int c = 0; c < 4; ++c)
            #pragma unroll
            for (int i = 0; i < 32; i += 8) {
              m0 = fmaxf(m0, __uint_as_float(sv[c][i]));     m1 = fmaxf(m1, __uint_as_float(sv[c][i + 1]));
              m2 = fmaxf(m2, __uint_as_float(sv[c][i + 2])); m3 = fmaxf(m3, __uint_as_float(sv[c][i + 3]));
              m4 = fmaxf(m4, __uint_as_float(sv[c][i + 4])); m5 = fmaxf(m5, __uint_as_float(sv[c][i + 5]));
              m6 = fmaxf(m6, __uint_as_float(sv[c][i + 6])); m7 = fmaxf(m7, __uint_as_float(sv[c][i + 7]));
            }
          top_raw = fmaxf(fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)), fmaxf(fmaxf(m4, m5), fmaxf(m6, m7)));
          mx = fmaf(top_raw, scale, bias_const);
        } else {
          // per-row window into the padded table: column c of this tile reads brow[c]
          const float* brow = lut + (n0 - qpos + md + LUT_PAD);
          const int n_valid = (p.causal ? min(len_k, qpos + 1) : len_k) - n0;   // columns < n_valid are visible
          #pragma unroll
          for (int c = 0; c < 4; ++c) {
            #pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float bias = bias_mode == 2 ? brow[c * 32 + i] : bias_const;
              float x = fmaf(__uint_as_float(sv[c][i]), scale, bias);
              if (need_mask && (c * 32 + i >= n_valid)) x = -INFINITY;
              sv[c][i] = __float_as_uint(x);
              if ((i & 3) == 0) m0 = fmaxf(m0, x); else if ((i & 3) == 1) m1 = fmaxf(m1, x);
              else if ((i & 3) == 2) m2 = fmaxf(m2, x); else m3 = fmaxf(m3, x);
            }
            asm volatile("" ::: "memory");   // keep the table reads of one chunk from piling up in registers
          }
          mx = max3(fmaxf(m0, m1), m2, m3);
          top_raw = mx;
        }
      }
      // The value the exponentials are taken against moves only when the row maximum outgrew it
      // by more than the threshold, and then by a whole number of powers of two (O and the row
      // sum are then rescaled exactly).  First tile: the row maximum itself.
      float k_step = 0.f;
      if (j == 0) {
        m_use = (mx == -INFINITY) ? 0.f : mx;     // a row without keys keeps l = 0
      } else {
        const float g = mx - m_use;
        if (g > kRescaleThreshold<kBf16>) k_step = fminf(ceilf(g), 1.0e6f);
        // the previous P V must have finished before O is rescaled or P is overwritten
        if (!mbar_wait_bounded_warp(bar(BAR_O_DONE + t), (uint32_t)((j - 1) & 1), abort_flag)) { ok = false; fail_code = 31; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, k_step > 0.f)) {
          const float alpha = pow2_neg(k_step);
          l_sum *= alpha;
          m_use += k_step;
          #pragma unroll 1
          for (int c = 0; c < HD / 16; ++c) {
            uint32_t ov[16];
            tmem_ld_x16(tO + c * 16, ov);
            tmem_ld_wait();
            #pragma unroll
            for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_x16(tO + c * 16, ov);
          }
        }
      }
      // fast tiles: p = 2^(s*scale + (bias - m)); others: p = 2^(x - m) = 2^(x*1 + (-m))
      const float e_mul = fast ? scale : 1.f;
      const float e_add = fast ? bias_const - m_use : -m_use;

      // ---- pass 2: the exponentials, software-pipelined by hand.  A warp issues in order, and with
      // two softmax warps per scheduler nothing else hides the latency of a dependent chain
      // (FFMA2 -> ex2 -> pack -> add), so the three stages of DIFFERENT column pairs are interleaved
      // in program order (volatile asm keeps that order): scale+shift of pair g, exponentials of
      // pair g - kDist, pack + row sum of pair g - 2 kDist.  Pairs that take the FMA-pipe
      // exponential do all of it in the first stage, between the ex2 of their neighbours.  Each
      // chunk of 32 columns is stored to tensor memory as soon as it is packed.
      float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
      const bool poly_ok = kPoly > 0 && !need_mask && scale > 0.f;
      PolyExp pe;
      if (poly_ok) pe.setup(e_mul, fast ? inv_scale : 1.f, e_add);
      {
        constexpr int kDist = 4;
        uint32_t pk[4][16];
        auto run = [&](auto use_poly) {
          constexpr bool kUsePoly = decltype(use_poly)::value;
          #pragma unroll
          for (int g = 0; g < 64 + 2 * kDist; ++g) {
            if (g < 64) {
              const int c = g >> 4, i = g & 15;
              float a0 = __uint_as_float(sv[c][2 * i]), a1 = __uint_as_float(sv[c][2 * i + 1]);
              if (kUsePoly && poly_pair(i, kPoly)) pe.eval(a0, a1, a0, a1);
              else vfma2(a0, a1, a0, a1, e_mul, e_add);
              sv[c][2 * i] = __float_as_uint(a0);
              sv[c][2 * i + 1] = __float_as_uint(a1);
            }
            if (g >= kDist && g - kDist < 64) {
              const int c = (g - kDist) >> 4, i = (g - kDist) & 15;
              if (!(kUsePoly && poly_pair(i, kPoly))) {
                sv[c][2 * i] = __float_as_uint(vex2(__uint_as_float(sv[c][2 * i])));
                sv[c][2 * i + 1] = __float_as_uint(vex2(__uint_as_float(sv[c][2 * i + 1])));
              }
            }
            if (g >= 2 * kDist) {
              const int c = (g - 2 * kDist) >> 4, i = (g - 2 * kDist) & 15;
              const float p0 = __uint_as_float(sv[c][2 * i]), p1 = __uint_as_float(sv[c][2 * i + 1]);
              pk[c][i] = vpack2<kBf16>(p0, p1);
              if (i & 1) vadd2(t2, t3, p0, p1); else vadd2(t0, t1, p0, p1);
              if (i == 15) tmem_st_x16(tP + 16 * c, pk[c]);
            }
          }
        };
        if (poly_ok) run(std::true_type{}); else run(std::false_type{});
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(BAR_P_FULL + t));

      float t_sum = (t0 + t1) + (t2 + t3);
      if (kBf16) {
        // The tensor core multiplies V by the ROUNDED probabilities.  With lazy rescaling the
        // largest one is not exactly 1, so when one key dominates a row its rounding error
        // (up to 2^-9 relative) would pass straight into the output.  Count that element in
        // the row sum as the tensor core sees it.
        float p_top = fast_exp2(fmaf(top_raw, e_mul, e_add)), p_dup;
        if (kPoly == 8 && poly_ok) pe.eval(top_raw, top_raw, p_top, p_dup);
        t_sum += __bfloat162float(__float2bfloat16_rn(p_top)) - p_top;
      }
      l_sum += t_sum;
    }

    // ---- epilogue: O / l -> global, one row (64 columns, 128 bytes) per thread
    if (ok && n_kv > 0) {
      if (!mbar_wait_bounded_warp(bar(BAR_O_DONE + t), (uint32_t)((n_kv - 1) & 1), abort_flag)) { ok = false; fail_code = 32; }
      tc_fence_after();
    }
    const int row_in_block = t * BM + r;
    if (ok) {
      const bool row_ok = row_in_block < rows_in_block;
      const int64_t row = (int64_t)q_row0 + row_in_block;
      float o[HD];
      #pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t v[32];
        if (n_kv > 0) {
          tmem_ld_x32(tO + 32 * c, v);
          tmem_ld_wait();
        } else {
          #pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        #pragma unroll
        for (int i = 0; i < 32; ++i) o[32 * c + i] = __uint_as_float(v[i]);
      }
      bool write_out = row_ok;
      if (parts > 1 && row_ok) {
        // This block saw only part of the keys.  Publish (max, sum, unnormalised O) for this row;
        // the last of the `parts` blocks to arrive merges them (no waiting).
        const int64_t slot = (int64_t)tail_slot * parts + part;
        float* my_o = p.ws_o + (slot * BLOCK_M + row_in_block) * HD;
        #pragma unroll
        for (int i = 0; i < HD / 4; ++i)
          reinterpret_cast<float4*>(my_o)[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        float* my_ml = p.ws_ml + (slot * BLOCK_M + row_in_block) * 2;
        my_ml[0] = l_sum > 0.f ? m_use : -INFINITY;
        my_ml[1] = l_sum;
        __threadfence();
        int* counter = p.ws_counters + (int64_t)tail_slot * BLOCK_M + row_in_block;
        const int arrived = atomicAdd(counter, 1);
        write_out = (arrived == parts - 1);
        if (write_out) {
          __threadfence();
          float m_all = -INFINITY;
          for (int s2 = 0; s2 < parts; ++s2)
            m_all = fmaxf(m_all, __ldcg(p.ws_ml + (((int64_t)tail_slot * parts + s2) * BLOCK_M + row_in_block) * 2));
          const float m_ref = (m_all == -INFINITY) ? 0.f : m_all;
          float l_all = 0.f;
          #pragma unroll
          for (int i = 0; i < HD; ++i) o[i] = 0.f;
          for (int s2 = 0; s2 < parts; ++s2) {
            const int64_t sl = (int64_t)tail_slot * parts + s2;
            const float* ml = p.ws_ml + (sl * BLOCK_M + row_in_block) * 2;
            const float sc = fast_exp2(__ldcg(ml) - m_ref);
            l_all = fmaf(__ldcg(ml + 1), sc, l_all);
            const float4* po = reinterpret_cast<const float4*>(p.ws_o + (sl * BLOCK_M + row_in_block) * HD);
            #pragma unroll
            for (int i = 0; i < HD / 4; ++i) {
              const float4 t4 = __ldcg(po + i);
              o[4 * i] = fmaf(t4.x, sc, o[4 * i]);         o[4 * i + 1] = fmaf(t4.y, sc, o[4 * i + 1]);
              o[4 * i + 2] = fmaf(t4.z, sc, o[4 * i + 2]); o[4 * i + 3] = fmaf(t4.w, sc, o[4 * i + 3]);
            }
          }
          m_use = m_all;
          l_sum = l_all;
          *counter = 0;     // leave the scratch ready for the next launch
        }
      }
      if (write_out) {
        const float inv_l = l_sum > 0.f ? 1.f / l_sum : 0.f;
        const int64_t o_off = (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + row * p.o_stride_m;
        uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) + 2 * o_off;
        if (p.out_f32) {
          float4* of = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o_off);
          #pragma unroll
          for (int i = 0; i < HD / 4; ++i)
            of[i] = make_float4(o[4 * i] * inv_l, o[4 * i + 1] * inv_l, o[4 * i + 2] * inv_l, o[4 * i + 3] * inv_l);
        } else
        #pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
          uint4 w4;
          w4.x = pack2<kBf16>(o[8 * i + 0] * inv_l, o[8 * i + 1] * inv_l);
          w4.y = pack2<kBf16>(o[8 * i + 2] * inv_l, o[8 * i + 3] * inv_l);
          w4.z = pack2<kBf16>(o[8 * i + 4] * inv_l, o[8 * i + 5] * inv_l);
          w4.w = pack2<kBf16>(o[8 * i + 6] * inv_l, o[8 * i + 7] * inv_l);
          *reinterpret_cast<uint4*>(orow + i * 16) = w4;
        }
        if (p.lse != nullptr) {
          const float lse = l_sum > 0.f ? (m_use + log2f(l_sum)) * kLn2 : -INFINITY;
          if (p.cu_q == nullptr) p.lse[((int64_t)batch_idx * p.H + h) * p.M + row] = lse;
          else p.lse[row * p.H + h] = lse;
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, 2000 + fail_code);
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_IO) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace sm100w

// ------------------------------------------------------------------ host side

// True when the two-tile kernel was asked for and applies: head dim 64, full (not block-local)
// attention, and more than one 128-row query tile per sequence.
bool sm100w_prefers(const t5b_attn_args& a) {
  if (a.kernel != T5B_KERNEL_TCGEN05_2TILE || a.D != 64 || a.local_block != 0 || a.window != 0) return false;
  return a.M > sm100w::BM;      // packed calls: M is the caller's max_seqlen_q
}

static int sm_count(int dev) {
  static std::atomic<int> sms[64];     // 0 = not asked yet (any thread may get here first)
  if (dev < 0 || dev >= 64) return 0;
  int n = sms[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); return 0; }
    sms[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Last-wave balancing for dense, non-causal launches: one block per SM, so the grid runs in waves
// of `SMs` equal blocks; the 256-row tiles of a partially filled last wave are split along the
// keys so that the wave finishes in a fraction of a block time.
TailPlan sm100w_tail_plan(const t5b_attn_args& a) {
  using namespace sm100w;
  TailPlan t;
  t.tiles_x = (a.M + BLOCK_M - 1) / BLOCK_M;
  const long long n_total = (long long)t.tiles_x * a.H * a.B;
  t.n_total = (int)(n_total > 0x7fffffffLL ? 0x7fffffff : n_total);
  t.tail_first = t.n_total;
  t.parts = 1;
  t.counters_bytes = t.ml_bytes = t.o_bytes = 0;
  if (a.cu_seqlens_q != nullptr || a.causal || n_total > 0x3fffffffLL) return t;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return t; }
  const int slots = sm_count(dev);
  if (slots <= 0) return t;
  const int rem = (int)(n_total % slots);
  const int n_kv = (a.N + BN - 1) / BN;
  if (rem == 0) return t;
  int parts = slots / rem;
  if (parts > n_kv / 4) parts = n_kv / 4;     // at least four key tiles per part
  if (parts > 8) parts = 8;
  if (parts < 2) return t;
  t.parts = parts;
  t.tail_first = t.n_total - rem;
  auto al = [](int64_t x) { return (x + 255) / 256 * 256; };
  // the counter area has one fixed size per device, so that launches with different splits
  // sharing a scratch buffer never see each other's partial results as counters
  t.counters_bytes = al((int64_t)2 * slots * BLOCK_M * 4);
  t.ml_bytes = al((int64_t)rem * parts * BLOCK_M * 2 * 4);
  t.o_bytes = al((int64_t)rem * parts * BLOCK_M * HD * 4);
  return t;
}

int sm100w_attention_fwd(const t5b_attn_args& a, const BucketSpec& spec, cudaStream_t stream) {
  using namespace sm100w;
  const bool varlen = a.cu_seqlens_q != nullptr;
  const bool bf16 = a.dtype == T5B_BF16;
  CUtensorMap mq, mk, mv;
  int st;
  if (varlen) {
    if ((st = make_tmap(&mq, a.q, bf16, HD, BM, a.total_q, a.H, 1, a.q_stride_m, a.q_stride_h, 0)) != T5B_OK) return st;
    if ((st = make_tmap(&mk, a.k, bf16, HD, BN, a.total_k, a.H, 1, a.k_stride_n, a.k_stride_h, 0)) != T5B_OK) return st;
    if ((st = make_tmap(&mv, a.v, bf16, HD, BN, a.total_k, a.H, 1, a.v_stride_n, a.v_stride_h, 0)) != T5B_OK) return st;
  } else {
    if ((st = make_tmap(&mq, a.q, bf16, HD, BM, a.M, a.H, a.B, a.q_stride_m, a.q_stride_h, a.q_stride_b)) != T5B_OK) return st;
    if ((st = make_tmap(&mk, a.k, bf16, HD, BN, a.N, a.H, a.B, a.k_stride_n, a.k_stride_h, a.k_stride_b)) != T5B_OK) return st;
    if ((st = make_tmap(&mv, a.v, bf16, HD, BN, a.N, a.H, a.B, a.v_stride_n, a.v_stride_h, a.v_stride_b)) != T5B_OK) return st;
  }
  AttnParams p = make_attn_params(a);
  const int lut_n = a.table ? 2 * spec.max_distance + 1 + 2 * LUT_PAD : 0;
  const size_t smem = smem_bytes(lut_n);
  dim3 grid;
  if (varlen) {
    // upper bound on sum_b ceil(len_b / 256) known without reading cu_seqlens
    const long long ub = (long long)a.total_q / BLOCK_M + a.B;
    grid = dim3((unsigned)ub, (unsigned)a.H, 1);
  } else {
    TailPlan plan = sm100w_tail_plan(a);
    p.tiles_x = plan.tiles_x;
    p.tail_first = plan.n_total;
    long long blocks = plan.n_total;
    if (plan.parts > 1 && a.workspace != nullptr && a.workspace_bytes >= plan.bytes() &&
        ((uintptr_t)a.workspace & 255) == 0) {
      char* ws = (char*)a.workspace;
      p.ws_counters = (int32_t*)ws;
      p.ws_ml = (float*)(ws + plan.counters_bytes);
      p.ws_o = (float*)(ws + plan.counters_bytes + plan.ml_bytes);
      p.tail_first = plan.tail_first;
      p.tail_parts = plan.parts;
      blocks = plan.tail_first + (long long)(plan.n_total - plan.tail_first) * plan.parts;
    }
    if (blocks > 0x7fffffffLL) return T5B_ERR_SHAPE;
    grid = dim3((unsigned)blocks, 1, 1);
  }
  if (grid.y > 65535 || grid.z > 65535) return T5B_ERR_SHAPE;
  using KernelFn = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, AttnParams, BucketSpec);
  static const KernelFn kernels[2][2] = {
      {attn_fwd2_kernel<false, T5B_FWD2_POLY>, attn_fwd2_kernel<false, 8>},
      {attn_fwd2_kernel<true, T5B_FWD2_POLY>, attn_fwd2_kernel<true, 8>}};
  const int all_poly = a.kernel == T5B_KERNEL_TCGEN05_POLYEXP ? 1 : 0;
  const KernelFn kern = kernels[bf16 ? 1 : 0][all_poly];
  // opt in to > 48 KB of dynamic shared memory once per device and kernel (any thread may get here first)
  static std::atomic<bool> attr_set[64][4];
  int dev = 0;
  cudaGetDevice(&dev);
  const int which = (bf16 ? 1 : 0) + 2 * all_poly;
  if (dev < 0 || dev >= 64 || !attr_set[dev][which].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem_bytes(2 * 2048 + 1 + 2 * LUT_PAD)) != cudaSuccess) {
      cudaGetLastError();
      return T5B_ERR_LAUNCH;
    }
    if (dev >= 0 && dev < 64) attr_set[dev][which].store(true, std::memory_order_release);
  }
  kern<<<grid, NUM_THREADS, smem, stream>>>(mq, mk, mv, p, spec);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

}  // namespace t5b
