// Backward of the fused relative-position-bias attention for sm_100a (bf16/fp16, head dim 64 or 128;
// head dims 16 and 32 run as 64 with the missing columns zero-filled by the tensor maps).
//
// Three launches, as the reference's backward (src/turbot5/ops/fused_bias_attention.py:62-147):
//
//   bwd_delta_kernel      delta[row] = sum_d dO[row,d] * O[row,d]           (:398-437)
//   attn_bwd_dq_kernel    one block per 128-row query tile, streaming 64-key tiles:
//                           S = Q K^T, dP = dO V^T           (tcgen05.mma, both operands in shared memory)
//                           P = exp2(S*scale + bias - lse),  dS = P o (dP - delta)   (softmax warps)
//                           dQ += dS K                       (dS from tensor memory, K as MN-major operand)
//                         and the gradient of the bias table: dtable[bucket(delta), h] += dS   (:635-820)
//   attn_bwd_dkv_kernel   one block per 128-key tile, streaming 64-query tiles, everything transposed
//                         so that the keys are the rows (TMEM lanes):
//                           S^T = K Q^T, dP^T = V dO^T
//                           P^T, dS^T written over S^T, dP^T in place (16-bit)
//                           dV += P^T dO,  dK += dS^T Q                                  (:440-632)
//                         (head dim 128; head dim 64 when built with T5B_BWD_DKV_WIDE=0)
//   attn_bwd_dkv_wide_kernel   head dim 64: the same products over 128-query steps, one block per SM,
//                         P^T and dS^T in tensor-memory columns of their own, the two 64-query halves
//                         of a step as independent pipelines
//
// S and dP are recomputed in both kernels (7 matrix products per tile pair instead of 5): no
// atomics on dQ, every output tile has one owner, results are deterministic except the few
// atomics on the small bias-table gradient.  Warp roles, barriers, bounded waits and the
// shared-memory bias table are those of the forward kernel (attn_fwd_sm100.cu); the saved
// log-sum-exp replaces the running maximum, so the softmax warps have no rendezvous at all.
#include "t5b_common.cuh"
#include "attn_params.cuh"
#include "attn_sm100_util.cuh"

#include <atomic>

namespace t5b {
namespace sm100b {

using sm100::make_tmap;
using sm100::pack2;

constexpr int BM = 128;            // rows of the tile a block owns (MMA M)
constexpr int BT = 64;             // rows of a streamed tile
constexpr int STAGES = 3;            // the streamed tiles stay resident until the LAST product of their step
constexpr int NUM_THREADS = 320;
constexpr int WARP_TMA = 8, WARP_MMA = 9;
constexpr int LUT_PAD = BM + BT;
constexpr int MAX_BUCKETS = 2 * kMaxBucketsPerSide;
// dq kernel, bias-table gradient of the tiles near the diagonal: a warp owns a 32 x 32 piece of
// the tile (lane = row, register = column) whose elements fall on 63 diagonals.  Each warp sums
// them in a private window of shared memory with plain 128-bit read-modify-writes: the lanes are
// split into four groups by (lane & 3), each with its own copy of the window, so that within a
// batch of four columns no two lanes touch the same word; __syncwarp() orders the batches.  The
// copies start at word offsets whose banks make every quarter-warp access conflict-free, and
// each is shifted by ((group + 1) & 3) words so that the four words of a batch are 16-byte aligned.
constexpr int DIAG_GROUP_WORDS = 68;
constexpr int DIAG_WARP_WORDS = 220 + DIAG_GROUP_WORDS;      // group bases 0, 72, 144, 220
constexpr int DIAG_BYTES = 8 * DIAG_WARP_WORDS * 4;
__device__ __forceinline__ int diag_group_base(int g) { return g == 3 ? 220 : 72 * g; }

// Geometry per head dim.  A row of 128 dims is two 128-byte-swizzled sub-tiles of 64 dims (two TMA
// boxes; the K loop of the first products walks both; an MN-major operand spans two swizzle atoms,
// leading byte offset = one sub-tile).  Head dim 64: 80 KB of tiles and <= 256 TMEM columns, two
// blocks per SM.  Head dim 128: 160 KB and up to 384 columns, one block per SM.
template <int HD_>
struct BGeo {
  static constexpr int HD = HD_;
  static constexpr int NSUB = HD_ / 64;
  static constexpr int SUB_BIG = BM * 128, SUB_SMALL = BT * 128;
  static constexpr int BIG_BYTES = NSUB * SUB_BIG, SMALL_BYTES = NSUB * SUB_SMALL;
  static constexpr int SMEM_TILES = 2 * BIG_BYTES + 2 * STAGES * SMALL_BYTES;
  static constexpr int TMEM_COLS = HD_ == 64 ? 256 : 512;
  static constexpr int OH = HD_ / 2;                      // output columns per softmax thread
  static constexpr int BLOCKS_PER_SM = HD_ == 64 ? 2 : 1;
};

struct BwdExtra {
  const void* dout;
  int64_t do_stride_b, do_stride_h, do_stride_m;
  void* dq; void* dk; void* dv;
  float* dtable;
  float* delta;
  float sm_scale;
  // Last-wave balancing (dense, non-causal launches): blocks at or beyond *_tail_first share a
  // tile *_parts ways along the streamed dimension; their partial gradients are additive (the
  // log-sum-exp is global), so they meet in float32 scratch rows through atomics, and the last
  // part to arrive (a counter per row half) rounds the row to the output and zeroes the scratch.
  int32_t q_tail_first, q_parts, k_tail_first, k_parts;
  int32_t* ws_cnt_q; float* ws_dq;
  int32_t* ws_cnt_k; float* ws_dk; float* ws_dv;
};

struct __align__(16) Control {
  unsigned long long bars[24];
  uint32_t tmem_base;
  int abort_flag;
  int work[6];
  float vec[STAGES][2][BT];     // dkv kernel: -lse (log2 domain) and -delta of the streamed query tile
  float hist[MAX_BUCKETS];      // dq kernel: bias-table gradient of this block
};

template <int HD>
__host__ __device__ inline size_t smem_bytes(int lut_entries) {
  // float bias per delta, float gradient per delta, int16 bucket per delta
  return 1024 + BGeo<HD>::SMEM_TILES + sizeof(Control) + 16 + (size_t)lut_entries * 10 + 16 + DIAG_BYTES;
}

// ---------------------------------------------------------------- delta = rowsum(dO o O)
// HD / 8 lanes per row, one 16-byte load of O and of dO each (rows and strides are 16-byte
// aligned: both tensors are also read or written 16 bytes at a time by the other kernels).
template <typename T, int HD>
__global__ void __launch_bounds__(256) bwd_delta_kernel(const AttnParams p, const BwdExtra e, long long n_rows) {
  constexpr int LPR = HD / 8, RPW = 32 / LPR;          // lanes per row, rows per warp
  const int lane = threadIdx.x & 31, sub = lane % LPR;
  const long long group0 = ((blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5) * RPW + lane / LPR;
  const long long stride = (((long long)gridDim.x * blockDim.x) >> 5) * RPW;
  // whole warps iterate together (the shuffles below are warp-wide); rows past the end add zeros
  const long long n_iter = (n_rows + stride - 1) / stride;
  for (long long it = 0; it < n_iter; ++it) {
    const long long i = group0 + it * stride;
    const bool valid = i < n_rows;
    float s = 0.f;
    if (valid) {
      int64_t o_off, do_off;
      if (p.cu_q == nullptr) {
        const int m = (int)(i % p.M);
        const long long bh = i / p.M;
        const int h = (int)(bh % p.H), b = (int)(bh / p.H);
        o_off = (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + (int64_t)m * p.o_stride_m;
        do_off = (int64_t)b * e.do_stride_b + (int64_t)h * e.do_stride_h + (int64_t)m * e.do_stride_m;
      } else {
        const int h = (int)(i % p.H);
        const long long row = i / p.H;
        o_off = (int64_t)h * p.o_stride_h + row * p.o_stride_m;
        do_off = (int64_t)h * e.do_stride_h + row * e.do_stride_m;
      }
      const uint4 ov = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.out) + o_off) + sub);
      const uint4 dv = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(e.dout) + do_off) + sub);
      const T* o8 = reinterpret_cast<const T*>(&ov);
      const T* d8 = reinterpret_cast<const T*>(&dv);
      #pragma unroll
      for (int c = 0; c < 8; ++c) s = fmaf(to_float(o8[c]), to_float(d8[c]), s);
    }
    #pragma unroll
    for (int off = LPR / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (valid && sub == 0) e.delta[i] = s;      // same indexing as lse: (b,h,m) dense, (row,h) packed
  }
}

enum {
  B_RES_FULL = 0,                    // the block's resident tiles (Q,dO | K,V)
  B_A_FULL = 1,                      // [STAGES] streamed tile A (K | Q)
  B_B_FULL = B_A_FULL + STAGES,      // [STAGES] streamed tile B (V | dO)
  B_A_EMPTY = B_B_FULL + STAGES,
  B_B_EMPTY = B_A_EMPTY + STAGES,
  B_S_FULL = B_B_EMPTY + STAGES,
  B_S_FREE,
  B_P_FULL,
  B_O_DONE,
  B_P_FULL1,
  B_DP_FULL,                         // dkv kernel: dP^T of a tile (S^T has its own barrier)
  B_DP_FULL1,
  B_PT_FULL,                         // dkv kernel, one S^T/dP^T pair: P^T of a tile is stored (dS^T follows on P_FULL)
  B_NUM
};
static_assert(B_NUM <= 24, "barrier slots");

// ======================================================================== dQ and dtable
// kWindow (all three kernels): the sliding-window mode is compiled into kernels of its own, so that
// its extra per-row values do not cost the plain kernels registers.
template <bool kBf16, int HD, bool kWindow>
__global__ void __launch_bounds__(NUM_THREADS, (HD == 64 ? 2 : 1))
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                   const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                   const __grid_constant__ AttnParams p, const __grid_constant__ BwdExtra e,
                   const __grid_constant__ BucketSpec spec) {
  const int window = kWindow ? p.window : 0;
  using G = BGeo<HD>;
  constexpr int NSUB = G::NSUB, SUB_BIG = G::SUB_BIG, SUB_SMALL = G::SUB_SMALL;
  constexpr int BIG_BYTES = G::BIG_BYTES, SMALL_BYTES = G::SMALL_BYTES, SMEM_TILES = G::SMEM_TILES;
  constexpr int TMEM_COLS = G::TMEM_COLS, OH = G::OH;
  constexpr int COL_S = 0, COL_DP = 64, COL_DS = 128, COL_DQ = 160;      // dQ: HD columns from 160
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sQ = base, sDO = base + BIG_BYTES;
  const uint32_t sK = base + 2 * BIG_BYTES, sV = sK + STAGES * SMALL_BYTES;
  Control* ctl = reinterpret_cast<Control*>(smem + SMEM_TILES);
  float* lut = reinterpret_cast<float*>(smem + SMEM_TILES + ((sizeof(Control) + 15) / 16) * 16);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- work item: as the forward kernel (query tile of a (batch, head) or packed sequence)
  TileWork* shared_work = reinterpret_cast<TileWork*>(&ctl->work[0]);
  TileWork w;
  int h, batch_idx = 0, part = 0, parts = 1, tail_slot = 0;
  if (p.cu_q == nullptr) {
    int tile_lin = (int)blockIdx.x;
    if (tile_lin >= e.q_tail_first) {
      const int ee = tile_lin - e.q_tail_first;
      parts = e.q_parts;
      tail_slot = ee / parts;
      part = ee - tail_slot * parts;
      tile_lin = e.q_tail_first + tail_slot;
    }
    const int tx = tile_lin % p.tiles_x;
    const int hb = tile_lin / p.tiles_x;
    h = hb % p.H;
    batch_idx = hb / p.H;
    w = dense_tile<BM>(p, tx, batch_idx);
  } else {
    h = blockIdx.y;
    if (warp == 0) {
      TileWork f = find_varlen_tile<BM>(p, (int)blockIdx.x);
      if (lane == 0) *shared_work = f;
    }
    __syncthreads();
    w = *shared_work;
    if (w.b < 0) return;
  }
  const int b = w.b, q_row0 = w.q_row0, rows_in_tile = w.rows_in_tile;
  const int k_row0 = w.k_row0, qpos0 = w.qpos0;
  int len_k = w.len_k, n_base = 0;
  if (p.local_block > 0) {
    // block-local attention: the keys of the three neighbouring blocks, the zero padding blocks
    // beyond either end included and unmasked (see attn_fwd_sm100.cu)
    const int bl = p.M < p.local_block ? p.M : p.local_block;
    const int blk = q_row0 / bl;
    n_base = (blk - 1) * bl;
    len_k = (blk + 2) * bl;
  }
  int kv_end = len_k;
  if (p.causal) kv_end = min(len_k, qpos0 + rows_in_tile);
  if (window > 0) {
    // sliding window |key - query position| < window: the key tiles that hold a visible key of any row
    n_base = max(0, qpos0 - window + 1) / BT * BT;
    kv_end = min(kv_end, qpos0 + rows_in_tile - 1 + window);
  }
  const int n_kv_all = kv_end > n_base ? (kv_end - n_base + BT - 1) / BT : 0;
  const int kv_per = (n_kv_all + parts - 1) / parts;
  const int kv_first = min(part * kv_per, n_kv_all);      // this block's key tiles: [kv_first, kv_first + n_kv)
  const int n_kv = min(n_kv_all, kv_first + kv_per) - kv_first;
  const int n_first = n_base + kv_first * BT;

  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  // this thread's row statistics, requested before the set-up below so that the latency of the
  // two reads is over by the time the first scores arrive
  float lse_raw = 0.f, delta_r = 0.f;
  if (warp < 8) {
    const int r_ = (warp & 3) * 32 + lane;
    if (r_ < rows_in_tile) {
      const int64_t row_ = (int64_t)q_row0 + r_;
      const int64_t idx_ = p.cu_q == nullptr ? ((int64_t)batch_idx * p.H + h) * p.M + row_ : row_ * p.H + h;
      lse_raw = p.lse[idx_];
      delta_r = e.delta[idx_];
    }
  }
  auto load_kv_tile = [&](int j) {
    const int s = j % STAGES;
    mbar_expect_tx(bar(B_A_FULL + s), SMALL_BYTES);
    #pragma unroll
    for (int u = 0; u < NSUB; ++u)
      tma_load_4d(sK + s * SMALL_BYTES + u * SUB_SMALL, &tmap_k, bar(B_A_FULL + s), 64 * u, k_row0 + n_first + j * BT, h, b);
    mbar_expect_tx(bar(B_B_FULL + s), SMALL_BYTES);
    #pragma unroll
    for (int u = 0; u < NSUB; ++u)
      tma_load_4d(sV + s * SMALL_BYTES + u * SUB_SMALL, &tmap_v, bar(B_B_FULL + s), 64 * u, k_row0 + n_first + j * BT, h, b);
  };
  if (warp == WARP_TMA && lane == 0) {
    // the loading thread sets up the barriers itself and starts the block's first loads at once:
    // they are in flight while the other threads build the bias tables below
    ctl->abort_flag = 0;
    mbar_init(bar(B_RES_FULL), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(B_A_FULL + s), 1);
      mbar_init(bar(B_B_FULL + s), 1);
      mbar_init(bar(B_A_EMPTY + s), 1);
      mbar_init(bar(B_B_EMPTY + s), 1);
    }
    mbar_init(bar(B_S_FULL), 1);
    mbar_init(bar(B_S_FREE), 8);
    mbar_init(bar(B_P_FULL), 8);
    mbar_init(bar(B_O_DONE), 1);
    fence_barrier_init();
    fence_proxy_async();
    if (n_kv > 0) {
      mbar_expect_tx(bar(B_RES_FULL), 2 * BIG_BYTES);
      #pragma unroll
      for (int u = 0; u < NSUB; ++u) {
        tma_load_4d(sQ + u * SUB_BIG, &tmap_q, bar(B_RES_FULL), 64 * u, q_row0, h, b);
        tma_load_4d(sDO + u * SUB_BIG, &tmap_do, bar(B_RES_FULL), 64 * u, q_row0, h, b);
      }
      for (int j = 0; j < STAGES && j < n_kv; ++j) load_kv_tile(j);
    }
  }
  if (warp == WARP_MMA) {
    tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  // delta -> bias (log2 domain) and delta -> bucket for this head
  const int md = spec.max_distance;
  const int lut_n = 2 * md + 1 + 2 * LUT_PAD;
  // gradient per delta: element (row r, column c) of a tile adds to entry (c - r + const), so
  // the 32 lanes of a warp instruction hit 32 consecutive words: conflict-free shared atomics.
  // Folded into buckets once, at the end of the block.
  float* dlut = lut + lut_n;
  int16_t* lutb = reinterpret_cast<int16_t*>(dlut + lut_n);
  float* diag = reinterpret_cast<float*>((reinterpret_cast<uintptr_t>(lutb + lut_n) + 15) & ~uintptr_t(15));
  const bool has_bias = p.table != nullptr;
  if (has_bias) {
    // one bucket search and one table load per delta in [-md, md]; beyond, the bucket no longer
    // changes and the padding is filled with the two end values
    for (int i = tid; i <= 2 * md; i += NUM_THREADS) {
      const int bucket = bucket_of_delta_counted(spec, i - md);
      lut[LUT_PAD + i] = load_table(p.table, p.table_dtype, (int64_t)bucket * p.table_stride0 + h) * kLog2e;
      lutb[LUT_PAD + i] = (int16_t)bucket;
    }
    for (int i = tid; i < lut_n; i += NUM_THREADS) dlut[i] = 0.f;
    __syncthreads();
    {
      const float lo_v = lut[LUT_PAD], hi_v = lut[LUT_PAD + 2 * md];
      const int16_t lo_b = lutb[LUT_PAD], hi_b = lutb[LUT_PAD + 2 * md];
      for (int i = tid; i < LUT_PAD; i += NUM_THREADS) {
        lut[i] = lo_v; lutb[i] = lo_b;
        lut[LUT_PAD + 2 * md + 1 + i] = hi_v; lutb[LUT_PAD + 2 * md + 1 + i] = hi_b;
      }
    }
    for (int i = tid; i < 8 * DIAG_WARP_WORDS; i += NUM_THREADS) diag[i] = 0.f;
    for (int i = tid; i < MAX_BUCKETS; i += NUM_THREADS) ctl->hist[i] = 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  int fail_code = 0;

  if (warp == WARP_TMA) {
    if (lane == 0) {
      for (int j = STAGES; j < n_kv; ++j) {        // the first STAGES tiles were requested above
        const int s = j % STAGES;
        const uint32_t ph = (uint32_t)((j / STAGES) & 1);
        if (!mbar_wait_bounded(bar(B_A_EMPTY + s), ph ^ 1u, abort_flag)) { fail_code = 10; break; }
        if (!mbar_wait_bounded(bar(B_B_EMPTY + s), ph ^ 1u, abort_flag)) { fail_code = 11; break; }
        load_kv_tile(j);
      }
    }
  } else if (warp == WARP_MMA) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t IDESC_SS = make_idesc_f16(kBf16, kBf16, BM, BT, false, false);   // 128 x 64 keys
      constexpr uint32_t IDESC_DQ = make_idesc_f16(kBf16, kBf16, BM, HD, false, true);    // K as MN-major B
      auto issue_s = [&](int j) -> bool {
        const int s = j % STAGES;
        const uint32_t ph = (uint32_t)((j / STAGES) & 1);
        if (!mbar_wait_bounded(bar(B_A_FULL + s), ph, abort_flag)) return false;
        if (!mbar_wait_bounded(bar(B_B_FULL + s), ph, abort_flag)) return false;
        tc_fence_after();
        #pragma unroll
        for (int u = 0; u < NSUB; ++u) {
          const uint64_t dq_ = make_smem_desc_sw128(sQ + u * SUB_BIG, 16, 1024);
          const uint64_t dk = make_smem_desc_sw128(sK + s * SMALL_BYTES + u * SUB_SMALL, 16, 1024);
          #pragma unroll
          for (int k = 0; k < 4; ++k) umma_ss(tmem + COL_S, dq_ + (uint64_t)(2 * k), dk + (uint64_t)(2 * k), IDESC_SS, (u | k) > 0);
        }
        #pragma unroll
        for (int u = 0; u < NSUB; ++u) {
          const uint64_t ddo = make_smem_desc_sw128(sDO + u * SUB_BIG, 16, 1024);
          const uint64_t dv = make_smem_desc_sw128(sV + s * SMALL_BYTES + u * SUB_SMALL, 16, 1024);
          #pragma unroll
          for (int k = 0; k < 4; ++k) umma_ss(tmem + COL_DP, ddo + (uint64_t)(2 * k), dv + (uint64_t)(2 * k), IDESC_SS, (u | k) > 0);
        }
        tc_commit(bar(B_S_FULL));
        tc_commit(bar(B_B_EMPTY + s));      // V is not needed again
        return true;
      };
      bool ok = mbar_wait_bounded(bar(B_RES_FULL), 0, abort_flag);
      if (!ok) fail_code = 20;
      if (ok && !issue_s(0)) { ok = false; fail_code = 21; }
      for (int j = 0; ok && j < n_kv; ++j) {
        if (j + 1 < n_kv) {
          if (!mbar_wait_bounded(bar(B_S_FREE), (uint32_t)(j & 1), abort_flag)) { fail_code = 25; break; }
          tc_fence_after();
          if (!issue_s(j + 1)) { fail_code = 23; break; }
        }
        if (!mbar_wait_bounded(bar(B_P_FULL), (uint32_t)(j & 1), abort_flag)) { fail_code = 22; break; }
        tc_fence_after();
        const int s = j % STAGES;
        // dQ += dS K: the K tile [64 keys][64 dims] read as an MN-major B operand
        #pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint64_t dkm = make_smem_desc_sw128(sK + s * SMALL_BYTES + k * 2048, NSUB > 1 ? SUB_SMALL : 16, 1024);
          umma_ts(tmem + COL_DQ, tmem + COL_DS + k * 8, dkm, IDESC_DQ, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar(B_O_DONE));
        tc_commit(bar(B_A_EMPTY + s));
      }
    }
  } else if (warp < 8) {
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_base + COL_S + half * 32;
    const uint32_t tDP = tmem + lane_base + COL_DP + half * 32;
    const uint32_t tDS = tmem + lane_base + COL_DS + half * 16;
    const uint32_t tDQ = tmem + lane_base + COL_DQ + half * OH;
    const float scale = p.scale_log2;
    const int qpos = qpos0 + r;
    const bool row_ok = r < rows_in_tile;
    const int64_t row = (int64_t)q_row0 + r;
    const float lse2 = lse_to_log2(lse_raw, row_ok);
    // bias-table gradient of tiles that lie entirely beyond +-max_distance: one bucket each
    float far_neg = 0.f, far_pos = 0.f;
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const int n0 = n_first + j * BT;
      const int c0 = half * 32;
      if (!mbar_wait_warp_fast(bar(B_S_FULL), (uint32_t)(j & 1), abort_flag)) { ok = false; fail_code = 30; break; }
      tc_fence_after();
      uint32_t sv[32], dp[32];
      tmem_ld_x32(tS, sv);
      tmem_ld_x32(tDP, dp);
      tmem_ld_wait();
      tc_fence_before();
      // (tcgen05.wait is warp-wide: every lane's accesses are complete, no __syncwarp before the arrival)
      if (lane == 0) mbar_arrive(bar(B_S_FREE));

      const bool need_mask = (n0 + BT > len_k) || (p.causal && (n0 + BT - 1 > qpos0)) ||
                             (window > 0 && (n0 <= qpos0 + BM - 1 - window || n0 + BT - 1 >= qpos0 + window));
      int bias_mode = 0;
      float bias_const = 0.f;
      if (has_bias) {
        const int dmin = n0 - (qpos0 + BM - 1), dmax = n0 + BT - 1 - qpos0;
        if (dmin >= md) { bias_mode = 1; bias_const = lut[2 * md + LUT_PAD]; }
        else if (dmax <= -md) { bias_mode = 3; bias_const = lut[LUT_PAD]; }
        else bias_mode = 2;
      }
      const int lut0 = n0 + c0 - qpos + md + LUT_PAD;      // table index of column 0 of this thread
      int n_valid = (p.causal ? min(len_k, qpos + 1) : len_k) - n0 - c0;     // columns < n_valid are visible
      int n_lo = -(1 << 30);                                                 // ... from column n_lo on
      if (window > 0) {
        n_valid = min(n_valid, qpos + window - n0 - c0);
        n_lo = qpos - window + 1 - n0 - c0;
      }
      uint32_t pk[16];
      float ds_sum = 0.f;
      if (!need_mask && bias_mode != 2) {
        // whole tile visible, one bias value: two elements per instruction
        const float add = bias_const - lse2, nd = -delta_r;
        float a0 = 0.f, a1 = 0.f;
        #pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0, x1, g0, g1, d0, d1;
          fma2(x0, x1, __uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]), scale, add);
          fma2(g0, g1, __uint_as_float(dp[2 * i]), __uint_as_float(dp[2 * i + 1]), 1.f, nd);
          mul2(d0, d1, fast_exp2(x0), fast_exp2(x1), g0, g1);
          add2(a0, a1, d0, d1);
          pk[i] = pack2<kBf16>(d0, d1);
        }
        ds_sum = a0 + a1;
      } else if (!need_mask) {
        // whole tile visible, bias per element (near the diagonal); dS stays in sv for the
        // bias-table gradient below
        const float nl = -lse2, nd = -delta_r;
        const float* lrow = lut + lut0;
        #pragma unroll
        for (int i = 0; i < 16; ++i) {
          float x0 = lrow[2 * i], x1 = lrow[2 * i + 1], g0, g1, d0, d1;
          add2(x0, x1, nl, nl);
          fma2v(x0, x1, __uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1]), scale, x0, x1);
          fma2(g0, g1, __uint_as_float(dp[2 * i]), __uint_as_float(dp[2 * i + 1]), 1.f, nd);
          mul2(d0, d1, fast_exp2(x0), fast_exp2(x1), g0, g1);
          sv[2 * i] = __float_as_uint(d0); sv[2 * i + 1] = __float_as_uint(d1);
          pk[i] = pack2<kBf16>(d0, d1);
        }
      } else {
        #pragma unroll
        for (int i = 0; i < 16; ++i) {
          float dsv[2];
          #pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int c = 2 * i + u;
            const float bias = bias_mode == 2 ? lut[lut0 + c] : bias_const;
            float x = fmaf(__uint_as_float(sv[c]), scale, bias) - lse2;
            if (need_mask && (c >= n_valid || c < n_lo)) x = -INFINITY;
            const float pr = fast_exp2(x);
            const float d = pr * (__uint_as_float(dp[c]) - delta_r);
            dsv[u] = d;
            if (bias_mode == 2) sv[c] = __float_as_uint(d);
            else ds_sum += d;
          }
          pk[i] = pack2<kBf16>(dsv[0], dsv[1]);
        }
      }
      if (bias_mode == 1) far_pos += ds_sum;
      if (bias_mode == 3) far_neg += ds_sum;
      if (j > 0) {
        if (!mbar_wait_warp_fast(bar(B_O_DONE), (uint32_t)((j - 1) & 1), abort_flag)) { ok = false; fail_code = 31; break; }
        tc_fence_after();
      }
      tmem_st_x16(tDS, pk);
      tmem_st_wait();
      tc_fence_before();
      if (lane == 0) mbar_arrive(bar(B_P_FULL));
      // (after dS is published: the matrix product runs while the warp does its bookkeeping)
      if (bias_mode == 2) {
        // element (lane, c) lies on diagonal t = c - lane + 31 of this warp's piece
        float* wdiag = diag + warp * DIAG_WARP_WORDS;
        const int g = lane & 3;
        float* mine = wdiag + diag_group_base(g) + ((g + 1) & 3) + 31 - lane;
        #pragma unroll
        for (int bq = 0; bq < 8; ++bq) {
          float4 a4 = *reinterpret_cast<float4*>(mine + 4 * bq);
          a4.x += __uint_as_float(sv[4 * bq]);     a4.y += __uint_as_float(sv[4 * bq + 1]);
          a4.z += __uint_as_float(sv[4 * bq + 2]); a4.w += __uint_as_float(sv[4 * bq + 3]);
          *reinterpret_cast<float4*>(mine + 4 * bq) = a4;
          __syncwarp();
        }
        // fold the four copies, clear them, and add the 63 sums to the block's table of deltas
        #pragma unroll
        for (int tt = 0; tt < 2; ++tt) {
          const int t = lane + 32 * tt;
          float sum = 0.f;
          #pragma unroll
          for (int gg = 0; gg < 4; ++gg) {
            float* w_ = wdiag + diag_group_base(gg) + ((gg + 1) & 3) + t;
            sum += *w_;
            *w_ = 0.f;
          }
          // lane 31 of the second round (t = 63) holds no diagonal: its words are never written
          if (t < 63 && sum != 0.f) atomicAdd(&dlut[lut0 + lane - 31 + t], sum);
        }
        __syncwarp();
      }
    }

    if (ok && n_kv > 0) {
      if (!mbar_wait_bounded_warp(bar(B_O_DONE), (uint32_t)((n_kv - 1) & 1), abort_flag)) { ok = false; fail_code = 32; }
      tc_fence_after();
    }
    if (ok) {          // warp-uniform: tcgen05.ld is a whole-warp instruction; only the stores depend on the row
      const float sc = e.sm_scale;
      float o[OH];
      #pragma unroll
      for (int c = 0; c < OH / 32; ++c) {
        uint32_t v[32];
        if (n_kv > 0) {
          tmem_ld_x32(tDQ + 32 * c, v);
          tmem_ld_wait();
        } else {
          #pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        #pragma unroll
        for (int i = 0; i < 32; ++i) o[32 * c + i] = __uint_as_float(v[i]) * sc;
      }
      uint8_t* drow = reinterpret_cast<uint8_t*>(e.dq) + half * OH * 2 +
                      2 * ((int64_t)b * p.q_stride_b + (int64_t)h * p.q_stride_h + row * p.q_stride_m);
      // head dims 16 and 32 run zero-filled to 64 (see the tensor maps): only the real columns are written
      const int d_cols = p.D - half * OH;
      bool write_out = row_ok && d_cols > 0;
      if (parts > 1 && write_out) {
        float* acc = e.ws_dq + ((int64_t)tail_slot * BM + r) * HD + half * OH;
        #pragma unroll
        for (int i = 0; i < OH; ++i) atomicAdd(acc + i, o[i]);
        __threadfence();
        int* counter = e.ws_cnt_q + ((int64_t)tail_slot * BM + r) * 2 + half;
        write_out = (atomicAdd(counter, 1) == parts - 1);
        if (write_out) {
          __threadfence();
          #pragma unroll
          for (int i = 0; i < OH / 4; ++i) {
            const float4 t4 = __ldcg(reinterpret_cast<const float4*>(acc) + i);
            o[4 * i] = t4.x; o[4 * i + 1] = t4.y; o[4 * i + 2] = t4.z; o[4 * i + 3] = t4.w;
            reinterpret_cast<float4*>(acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
          *counter = 0;        // scratch and counter are left as they were found: zero
        }
      }
      if (write_out) {
        #pragma unroll
        for (int i = 0; i < OH / 8; ++i) {
          uint4 w4;
          w4.x = pack2<kBf16>(o[8 * i + 0], o[8 * i + 1]);
          w4.y = pack2<kBf16>(o[8 * i + 2], o[8 * i + 3]);
          w4.z = pack2<kBf16>(o[8 * i + 4], o[8 * i + 5]);
          w4.w = pack2<kBf16>(o[8 * i + 6], o[8 * i + 7]);
          if (8 * i < d_cols) *reinterpret_cast<uint4*>(drow + i * 16) = w4;
        }
      }
    }
    if (has_bias) {
      #pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        far_pos += __shfl_xor_sync(0xffffffffu, far_pos, off);
        far_neg += __shfl_xor_sync(0xffffffffu, far_neg, off);
      }
      if (lane == 0) {
        if (far_pos != 0.f) atomicAdd(&ctl->hist[lutb[2 * md + LUT_PAD]], far_pos);
        if (far_neg != 0.f) atomicAdd(&ctl->hist[lutb[LUT_PAD]], far_neg);
      }
    }
  }

  if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, 2000 + fail_code);
  tc_fence_before();
  __syncthreads();
  if (has_bias && e.dtable != nullptr) {
    // deltas -> buckets: a bucket covers a run of consecutive deltas, so each warp sums the runs
    // inside its 32 entries with shuffles and only the first lane of a run touches the histogram
    // (one shared-memory atomic per run instead of 32 lanes retrying on the same word)
    for (int i0 = warp * 32; i0 < lut_n; i0 += NUM_THREADS) {
      const int i = i0 + lane;
      float g = i < lut_n ? dlut[i] : 0.f;
      const int bk = i < lut_n ? (int)lutb[i] : -1;
      const int prev = __shfl_up_sync(0xffffffffu, bk, 1);
      const bool head = lane == 0 || prev != bk;
      const unsigned heads = __ballot_sync(0xffffffffu, head);
      const int run = __popc(heads & (0xffffffffu >> (31 - lane)));      // index of this lane's run
      #pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float v = __shfl_down_sync(0xffffffffu, g, off);
        const int r2 = __shfl_down_sync(0xffffffffu, run, off);
        if (lane + off < 32 && r2 == run) g += v;
      }
      if (head && bk >= 0 && g != 0.f) atomicAdd(&ctl->hist[bk], g);
    }
    __syncthreads();
    const int nb = spec.bidirectional ? 2 * spec.n_side : spec.n_side;
    for (int i = tid; i < nb; i += NUM_THREADS) {
      const float g = ctl->hist[i];
      if (g != 0.f) atomicAdd(&e.dtable[(int64_t)i * p.H + h], g);
    }
  }
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ======================================================================== dK and dV
template <bool kBf16, int HD, bool kWindow>
__global__ void __launch_bounds__(NUM_THREADS, (HD == 64 ? 2 : 1))
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                    const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                    const __grid_constant__ AttnParams p, const __grid_constant__ BwdExtra e,
                    const __grid_constant__ BucketSpec spec) {
  const int window = kWindow ? p.window : 0;
  // tensor memory: S^T and dP^T (64 fp32 columns each, keys in the lanes); P^T and dS^T are
  // written over them in place: the 32 query columns of row half q sit, packed, in the first
  // 16 columns of that half's own 32 (a K=16 step of the second MMA takes any column address)
  using G = BGeo<HD>;
  constexpr int NSUB = G::NSUB, SUB_BIG = G::SUB_BIG, SUB_SMALL = G::SUB_SMALL;
  constexpr int BIG_BYTES = G::BIG_BYTES, SMALL_BYTES = G::SMALL_BYTES, SMEM_TILES = G::SMEM_TILES;
  constexpr int TMEM_COLS = G::TMEM_COLS, OH = G::OH;
  constexpr int COL_ST = 0, COL_DPT = 64, COL_DV = 128, COL_DK = 128 + HD;
  // Head dim 128 owns the SM alone (512 columns): the 128 spare columns hold a second S^T / dP^T
  // pair, so the first products of tile i+1 run while the softmax warps work on tile i.
  constexpr int NBUF = HD == 128 ? 2 : 1;
  constexpr int COL_BUF1 = 128 + 2 * HD;        // 384: offset of the second pair
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sK = base, sV = base + BIG_BYTES;
  const uint32_t sQ = base + 2 * BIG_BYTES, sDO = sQ + STAGES * SMALL_BYTES;
  Control* ctl = reinterpret_cast<Control*>(smem + SMEM_TILES);
  float* lut = reinterpret_cast<float*>(smem + SMEM_TILES + ((sizeof(Control) + 15) / 16) * 16);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- work item: a 128-key tile of one (batch, head) or packed sequence
  int h, b = 0, batch_idx = 0, part = 0, parts = 1, tail_slot = 0;
  int key0;            // first key of the tile inside its sequence
  int k_row0 = 0, len_k, q_row0 = 0, len_q, q_off;
  if (p.cu_k == nullptr) {
    const int tiles_k = (p.N + BM - 1) / BM;
    int tile_lin = (int)blockIdx.x;
    if (tile_lin >= e.k_tail_first) {
      const int ee = tile_lin - e.k_tail_first;
      parts = e.k_parts;
      tail_slot = ee / parts;
      part = ee - tail_slot * parts;
      tile_lin = e.k_tail_first + tail_slot;
    }
    const int tx = tile_lin % tiles_k;
    const int hb = tile_lin / tiles_k;
    h = hb % p.H;
    batch_idx = b = hb / p.H;
    key0 = tx * BM;
    len_k = p.N; len_q = p.M; q_off = p.q_pos_offset;
  } else {
    h = blockIdx.y;
    if (warp == 0) {
      int seq = -1, t = 0;
      const bool found = find_seq_tile(p.cu_k, p.B, BM, (int)blockIdx.x, seq, t);
      if (lane == 0) { ctl->work[0] = found ? seq : -1; ctl->work[1] = t; }
    }
    __syncthreads();
    const int seq = ctl->work[0];
    if (seq < 0) return;
    key0 = ctl->work[1] * BM;
    k_row0 = min(p.cu_k[seq], p.total_k); len_k = min(p.cu_k[seq + 1], p.total_k) - k_row0;
    q_row0 = min(p.cu_q[seq], p.total_q); len_q = min(p.cu_q[seq + 1], p.total_q) - q_row0;
    q_off = len_k - len_q;
  }
  const int keys_in_tile = min(BM, len_k - key0);
  // query tiles that can see a key of this tile: causal keeps q_off + m >= key
  int i_first = 0;
  if (p.causal) i_first = max(0, key0 - q_off) / BT;
  int n_qt_all = (len_q + BT - 1) / BT;
  if (p.local_block > 0) {
    // block-local attention: only the queries of the three neighbouring blocks see this key tile
    const int bl = p.M < p.local_block ? p.M : p.local_block;
    const int kb = key0 / bl;
    i_first = max(0, (kb - 1) * bl) / BT;
    n_qt_all = (min(len_q, (kb + 2) * bl) + BT - 1) / BT;
  }
  if (window > 0) {
    // sliding window: the queries within (key - window, key + window) of a key of this tile
    i_first = max(0, key0 - window + 1 - q_off) / BT;
    n_qt_all = (min(len_q, max(0, key0 + BM - 1 + window - q_off)) + BT - 1) / BT;
  }
  int n_qt = max(0, n_qt_all - i_first);
  if (parts > 1) {       // this block's share of the query tiles
    const int per = (n_qt + parts - 1) / parts;
    const int first = min(part * per, n_qt);
    n_qt = min(n_qt, first + per) - first;
    i_first += first;
  }

  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  // producer warp: lse / delta of the first query tile, requested before the set-up below
  float pre_l[2] = {0.f, 0.f}, pre_d[2] = {0.f, 0.f};
  auto stat_index = [&](int m) -> int64_t {
    return p.cu_q == nullptr ? ((int64_t)batch_idx * p.H + h) * p.M + m : ((int64_t)q_row0 + m) * p.H + h;
  };
  if (warp == WARP_TMA && n_qt > 0) {
    #pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int m = i_first * BT + lane + 32 * u;
      if (m < len_q) { pre_l[u] = p.lse[stat_index(m)]; pre_d[u] = e.delta[stat_index(m)]; }
    }
  }
  auto load_q_tile = [&](int i) {
    const int s = i % STAGES;
    const int m0 = (i_first + i) * BT;
    mbar_expect_tx(bar(B_A_FULL + s), SMALL_BYTES);
    #pragma unroll
    for (int u = 0; u < NSUB; ++u)
      tma_load_4d(sQ + s * SMALL_BYTES + u * SUB_SMALL, &tmap_q, bar(B_A_FULL + s), 64 * u, q_row0 + m0, h, b);
    mbar_expect_tx(bar(B_B_FULL + s), SMALL_BYTES);
    #pragma unroll
    for (int u = 0; u < NSUB; ++u)
      tma_load_4d(sDO + s * SMALL_BYTES + u * SUB_SMALL, &tmap_do, bar(B_B_FULL + s), 64 * u, q_row0 + m0, h, b);
  };
  if (warp == WARP_TMA && lane == 0) {       // as in the dQ kernel: barriers, then the first loads at once
    ctl->abort_flag = 0;
    mbar_init(bar(B_RES_FULL), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(B_A_FULL + s), 2);       // TMA transaction + the lse/delta vectors written by the producer warp
      mbar_init(bar(B_B_FULL + s), 1);
      mbar_init(bar(B_A_EMPTY + s), 1);
      mbar_init(bar(B_B_EMPTY + s), 1);
    }
    mbar_init(bar(B_S_FULL), 1);
    mbar_init(bar(B_DP_FULL), 1);
    mbar_init(bar(B_DP_FULL1), 1);
    mbar_init(bar(B_P_FULL), 8);
    mbar_init(bar(B_P_FULL1), 8);
    mbar_init(bar(B_PT_FULL), 8);
    mbar_init(bar(B_O_DONE), 1);
    fence_barrier_init();
    fence_proxy_async();
    if (n_qt > 0) {
      mbar_expect_tx(bar(B_RES_FULL), 2 * BIG_BYTES);
      #pragma unroll
      for (int u = 0; u < NSUB; ++u) {
        tma_load_4d(sK + u * SUB_BIG, &tmap_k, bar(B_RES_FULL), 64 * u, k_row0 + key0, h, b);
        tma_load_4d(sV + u * SUB_BIG, &tmap_v, bar(B_RES_FULL), 64 * u, k_row0 + key0, h, b);
      }
      for (int i = 0; i < STAGES && i < n_qt; ++i) load_q_tile(i);
    }
  }
  if (warp == WARP_MMA) {
    tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  const int md = spec.max_distance;
  const int lut_n = 2 * md + 1 + 2 * LUT_PAD;
  const bool has_bias = p.table != nullptr;
  if (has_bias) {
    for (int i = tid; i <= 2 * md; i += NUM_THREADS) {       // as in the dQ kernel
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

  if (warp == WARP_TMA) {
    // whole warp: lane 0 drives the TMA, all lanes fetch the lse / delta of the query tile
    if (n_qt > 0) {
      bool okp = true;
      for (int i = 0; i < n_qt; ++i) {
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)((i / STAGES) & 1);
        const int m0 = (i_first + i) * BT;
        if (i >= STAGES) {
          // every lane waits: the vectors of this stage are rewritten below
          if (!mbar_wait_bounded(bar(B_A_EMPTY + s), ph ^ 1u, abort_flag)) { okp = false; }
          if (okp && !mbar_wait_bounded(bar(B_B_EMPTY + s), ph ^ 1u, abort_flag)) { okp = false; }
          if (!__all_sync(0xffffffffu, okp)) { fail_code = 10; break; }
        }
        if (lane == 0 && i >= STAGES) load_q_tile(i);      // the first STAGES tiles were requested above
        #pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int c = lane + 32 * u;
          const int m = m0 + c;
          const bool valid = m < len_q;
          const int64_t idx = stat_index(m);
          const float l_ = i == 0 ? pre_l[u] : (valid ? p.lse[idx] : 0.f);
          const float d_ = i == 0 ? pre_d[u] : (valid ? e.delta[idx] : 0.f);
          // stored negated: the softmax warps add them with packed adds
          ctl->vec[s][0][c] = -lse_to_log2(l_, valid);
          ctl->vec[s][1][c] = valid ? -d_ : 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_A_FULL + s));
      }
    }
  } else if (warp == WARP_MMA) {
    if (lane == 0 && n_qt > 0) {
      constexpr uint32_t IDESC_SS = make_idesc_f16(kBf16, kBf16, BM, BT, false, false);   // 128 keys x 64 queries
      constexpr uint32_t IDESC_TS = make_idesc_f16(kBf16, kBf16, BM, HD, false, true);    // dO / Q as MN-major B
      // S^T and dP^T of a tile are queued separately, each behind the product that still reads the
      // columns it overwrites (dV reads P^T, dK reads dS^T), and each with its own barrier: the
      // softmax warps start on the exponentials while dK and dP^T are still running
      auto issue_st = [&](int i) -> bool {
        const uint32_t boff = (NBUF == 2 && (i & 1)) ? (uint32_t)COL_BUF1 : 0u;
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)((i / STAGES) & 1);
        if (!mbar_wait_bounded(bar(B_A_FULL + s), ph, abort_flag)) return false;
        tc_fence_after();
        #pragma unroll
        for (int u = 0; u < NSUB; ++u) {
          const uint64_t dk = make_smem_desc_sw128(sK + u * SUB_BIG, 16, 1024);
          const uint64_t dq_ = make_smem_desc_sw128(sQ + s * SMALL_BYTES + u * SUB_SMALL, 16, 1024);
          #pragma unroll
          for (int k = 0; k < 4; ++k) umma_ss(tmem + COL_ST + boff, dk + (uint64_t)(2 * k), dq_ + (uint64_t)(2 * k), IDESC_SS, (u | k) > 0);
        }
        // with two pairs the softmax warps take S^T and dP^T together: one barrier, after dP^T
        if (NBUF == 1) tc_commit(bar(B_S_FULL));
        return true;
      };
      auto issue_dpt = [&](int i) -> bool {
        const uint32_t boff = (NBUF == 2 && (i & 1)) ? (uint32_t)COL_BUF1 : 0u;
        const int s = i % STAGES;
        const uint32_t ph = (uint32_t)((i / STAGES) & 1);
        if (!mbar_wait_bounded(bar(B_B_FULL + s), ph, abort_flag)) return false;
        tc_fence_after();
        #pragma unroll
        for (int u = 0; u < NSUB; ++u) {
          const uint64_t dv = make_smem_desc_sw128(sV + u * SUB_BIG, 16, 1024);
          const uint64_t ddo = make_smem_desc_sw128(sDO + s * SMALL_BYTES + u * SUB_SMALL, 16, 1024);
          #pragma unroll
          for (int k = 0; k < 4; ++k) umma_ss(tmem + COL_DPT + boff, dv + (uint64_t)(2 * k), ddo + (uint64_t)(2 * k), IDESC_SS, (u | k) > 0);
        }
        tc_commit(bar((NBUF == 2 && (i & 1)) ? B_DP_FULL1 : B_DP_FULL));
        return true;
      };
      bool ok = mbar_wait_bounded(bar(B_RES_FULL), 0, abort_flag);
      if (!ok) fail_code = 20;
      if (ok && !(issue_st(0) && issue_dpt(0))) { ok = false; fail_code = 21; }
      if (ok && NBUF == 2 && n_qt > 1 && !(issue_st(1) && issue_dpt(1))) { ok = false; fail_code = 21; }
      for (int i = 0; ok && i < n_qt; ++i) {
        const int s = i % STAGES;
        const uint32_t boff = (NBUF == 2 && (i & 1)) ? (uint32_t)COL_BUF1 : 0u;
        // With two S^T/dP^T pairs the softmax warps can finish tile i+1 without anything further from
        // this thread (its products were queued a tile ago), so a barrier shared by all tiles could
        // complete two phases between two looks of this thread and the parity test would then wait
        // for ever.  One barrier per pair: its next phase needs S^T(i+2), queued below this wait.
        // One pair: dV(i) and S^T(i+1) are queued as soon as P^T(i) is stored (B_PT_FULL), while the
        // softmax warps still form dS^T(i); dK(i) and dP^T(i+1) follow on P_FULL.  The next phase of
        // either barrier needs a product that is queued after the wait on its current phase.
        if (!mbar_wait_bounded(bar(NBUF == 1 ? B_PT_FULL : ((i & 1) ? B_P_FULL1 : B_P_FULL)), (uint32_t)((i / NBUF) & 1), abort_flag)) { fail_code = 22; break; }
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < BT / 16; ++k) {       // 16 queries per step
          const uint32_t a_off = (uint32_t)(k < 2 ? 8 * k : 32 + 8 * (k - 2));
          const uint64_t ddo = make_smem_desc_sw128(sDO + s * SMALL_BYTES + k * 2048, NSUB > 1 ? SUB_SMALL : 16, 1024);
          umma_ts(tmem + COL_DV, tmem + COL_ST + boff + a_off, ddo, IDESC_TS, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar(B_B_EMPTY + s));
        // the tensor core runs MMAs in issue order: S^T / dP^T may be overwritten once the
        // products that read P^T / dS^T from the same columns are queued
        if (NBUF == 1 && i + 1 < n_qt && !issue_st(i + 1)) { fail_code = 23; break; }
        if (NBUF == 1) {
          if (!mbar_wait_bounded(bar(B_P_FULL), (uint32_t)(i & 1), abort_flag)) { fail_code = 26; break; }
          tc_fence_after();
        }
        #pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          const uint32_t a_off = (uint32_t)(k < 2 ? 8 * k : 32 + 8 * (k - 2));
          const uint64_t dq_ = make_smem_desc_sw128(sQ + s * SMALL_BYTES + k * 2048, NSUB > 1 ? SUB_SMALL : 16, 1024);
          umma_ts(tmem + COL_DK, tmem + COL_DPT + boff + a_off, dq_, IDESC_TS, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar(B_A_EMPTY + s));
        if (NBUF == 2 && i + 2 < n_qt && !issue_st(i + 2)) { fail_code = 23; break; }
        if (i + NBUF < n_qt && !issue_dpt(i + NBUF)) { fail_code = 24; break; }
        if (i + 1 == n_qt) tc_commit(bar(B_O_DONE));
      }
    }
  } else if (warp < 8) {
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;               // key row inside the tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tST0 = tmem + lane_base + COL_ST + half * 32;
    const uint32_t tDPT0 = tmem + lane_base + COL_DPT + half * 32;
    const float scale = p.scale_log2;
    const int key = key0 + r;
    const bool key_ok = r < keys_in_tile;
    bool ok = true;

    for (int i = 0; i < n_qt; ++i) {
      const int s = i % STAGES;
      const int m0 = (i_first + i) * BT + half * 32;     // first query of this thread's columns
      const uint32_t boff = (NBUF == 2 && (i & 1)) ? (uint32_t)COL_BUF1 : 0u;
      const uint32_t tST = tST0 + boff, tDPT = tDPT0 + boff;
      if (!mbar_wait_bounded_warp(bar(NBUF == 1 ? B_S_FULL : ((i & 1) ? B_DP_FULL1 : B_DP_FULL)), (uint32_t)((i / NBUF) & 1), abort_flag)) { ok = false; fail_code = 30; break; }
      tc_fence_after();
      uint32_t sv[32];
      tmem_ld_x32(tST, sv);
      // the lse / delta vectors of this stage were published on the same barrier as the Q tile
      // (long complete: the matrix products above needed it); observing it here orders the reads
      if (!mbar_wait_bounded_warp(bar(B_A_FULL + s), (uint32_t)((i / STAGES) & 1), abort_flag)) { ok = false; fail_code = 33; break; }
      tmem_ld_wait();

      const int qp0 = q_off + m0;                        // key-coordinate position of column 0
      // column c has delta = key - (qp0 + c): table index falls as c grows
      const int lut0 = key - qp0 + md + LUT_PAD;
      int bias_mode = 0;
      float bias_const = 0.f;
      if (has_bias) {
        const int dmin = key0 - (q_off + (i_first + i) * BT + BT - 1), dmax = key0 + BM - 1 - (q_off + (i_first + i) * BT);
        if (dmin >= md) { bias_mode = 1; bias_const = lut[2 * md + LUT_PAD]; }
        else if (dmax <= -md) { bias_mode = 1; bias_const = lut[LUT_PAD]; }
        else bias_mode = 2;
      }
      const float* vl = &ctl->vec[s][0][half * 32];
      const float* vd = &ctl->vec[s][1][half * 32];
      // fast path (uniform over the block): every key of the tile is inside the sequence, no
      // causal boundary crosses the tile, one bias value.  Two halves of 16 columns: each is
      // stored as soon as it is packed, which keeps the live registers below the limit.
      const int q_lo = q_off + (i_first + i) * BT;      // position of the tile's first query
      const bool tile_masked = (key0 + BM > len_k) || (p.causal && key0 + BM - 1 > q_lo) ||
                               (window > 0 && (key0 + BM - 1 - q_lo >= window || q_lo + BT - 1 - key0 >= window));
      if constexpr (NBUF == 1) {
        // pass 1: P^T = exp2(S^T scale + bias - lse), kept in sv as float32 and stored as the A
        // operand of the dV product.  Two halves of 16 columns, each stored as soon as it is packed.
        #pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t pp[8];
          if (!tile_masked && bias_mode != 2) {
            #pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              const int c = 16 * hh + 2 * ii;
              const float2 l2 = *reinterpret_cast<const float2*>(vl + c);
              float x0, x1;
              fma2(x0, x1, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), scale, bias_const);
              add2(x0, x1, l2.x, l2.y);          // - lse
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              sv[c] = __float_as_uint(p0); sv[c + 1] = __float_as_uint(p1);
              pp[ii] = pack2<kBf16>(p0, p1);
            }
          } else if (!tile_masked) {
            // whole tile visible, bias per element (near the diagonal)
            const float* lrow = lut + lut0;
            #pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              const int c = 16 * hh + 2 * ii;
              const float2 l2 = *reinterpret_cast<const float2*>(vl + c);
              float x0 = lrow[-c], x1 = lrow[-c - 1];
              add2(x0, x1, l2.x, l2.y);          // bias - lse
              fma2v(x0, x1, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), scale, x0, x1);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              sv[c] = __float_as_uint(p0); sv[c + 1] = __float_as_uint(p1);
              pp[ii] = pack2<kBf16>(p0, p1);
            }
          } else {
            #pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              float pv[2];
              #pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int c = 16 * hh + 2 * ii + u;
                const float bias = bias_mode == 2 ? lut[lut0 - c] : bias_const;
                float x = fmaf(__uint_as_float(sv[c]), scale, bias) + vl[c];
                // masked: key outside the sequence, or (causal) after the query
                if (!key_ok || (p.causal && key > qp0 + c) ||
                    (window > 0 && (key - (qp0 + c) >= window || (qp0 + c) - key >= window))) x = -INFINITY;
                pv[u] = fast_exp2(x);
                sv[c] = __float_as_uint(pv[u]);
              }
              pp[ii] = pack2<kBf16>(pv[0], pv[1]);
            }
          }
          tmem_st_x8(tST + 8 * hh, pp);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_PT_FULL));
        // pass 2: dS^T = P^T o (dP^T - delta), once dP^T has arrived
        if (!mbar_wait_bounded_warp(bar((NBUF == 2 && (i & 1)) ? B_DP_FULL1 : B_DP_FULL), (uint32_t)((i / NBUF) & 1), abort_flag)) { ok = false; fail_code = 34; break; }
        tc_fence_after();
        {
          uint32_t dp[32];
          tmem_ld_x32(tDPT, dp);
          tmem_ld_wait();
          #pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t pd[8];
            #pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              const int c = 16 * hh + 2 * ii;
              const float2 d2 = *reinterpret_cast<const float2*>(vd + c);
              float g0 = __uint_as_float(dp[c]), g1 = __uint_as_float(dp[c + 1]), e0, e1;
              add2(g0, g1, d2.x, d2.y);          // dP - delta
              mul2(e0, e1, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), g0, g1);
              pd[ii] = pack2<kBf16>(e0, e1);
            }
            tmem_st_x8(tDPT + 8 * hh, pd);
          }
        }
      } else {
        // two S^T/dP^T pairs (head dim 128): both products of this tile were queued a tile ago, one pass
        uint32_t dp[32];
        tmem_ld_x32(tDPT, dp);
        tmem_ld_wait();
        #pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          uint32_t pp[8], pd[8];
          if (!tile_masked && bias_mode != 2) {
            #pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              const int c = 16 * hh + 2 * ii;
              const float2 l2 = *reinterpret_cast<const float2*>(vl + c);
              const float2 d2 = *reinterpret_cast<const float2*>(vd + c);
              float x0, x1, g0 = __uint_as_float(dp[c]), g1 = __uint_as_float(dp[c + 1]), e0, e1;
              fma2(x0, x1, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), scale, bias_const);
              add2(x0, x1, l2.x, l2.y);          // - lse
              add2(g0, g1, d2.x, d2.y);          // dP - delta
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              mul2(e0, e1, p0, p1, g0, g1);
              pp[ii] = pack2<kBf16>(p0, p1);
              pd[ii] = pack2<kBf16>(e0, e1);
            }
          } else if (!tile_masked) {
            // whole tile visible, bias per element (near the diagonal)
            const float* lrow = lut + lut0;
            #pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              const int c = 16 * hh + 2 * ii;
              const float2 l2 = *reinterpret_cast<const float2*>(vl + c);
              const float2 d2 = *reinterpret_cast<const float2*>(vd + c);
              float x0 = lrow[-c], x1 = lrow[-c - 1], g0 = __uint_as_float(dp[c]), g1 = __uint_as_float(dp[c + 1]), e0, e1;
              add2(x0, x1, l2.x, l2.y);          // bias - lse
              fma2v(x0, x1, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), scale, x0, x1);
              add2(g0, g1, d2.x, d2.y);          // dP - delta
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              mul2(e0, e1, p0, p1, g0, g1);
              pp[ii] = pack2<kBf16>(p0, p1);
              pd[ii] = pack2<kBf16>(e0, e1);
            }
          } else {
            #pragma unroll
            for (int ii = 0; ii < 8; ++ii) {
              float pv[2], dv2[2];
              #pragma unroll
              for (int u = 0; u < 2; ++u) {
                const int c = 16 * hh + 2 * ii + u;
                const float bias = bias_mode == 2 ? lut[lut0 - c] : bias_const;
                float x = fmaf(__uint_as_float(sv[c]), scale, bias) + vl[c];
                // masked: key outside the sequence, or (causal) after the query
                if (!key_ok || (p.causal && key > qp0 + c) ||
                    (window > 0 && (key - (qp0 + c) >= window || (qp0 + c) - key >= window))) x = -INFINITY;
                const float pr = fast_exp2(x);
                pv[u] = pr;
                dv2[u] = pr * (__uint_as_float(dp[c]) + vd[c]);
              }
              pp[ii] = pack2<kBf16>(pv[0], pv[1]);
              pd[ii] = pack2<kBf16>(dv2[0], dv2[1]);
            }
          }
          tmem_st_x8(tST + 8 * hh, pp);
          tmem_st_x8(tDPT + 8 * hh, pd);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar((NBUF == 2 && (i & 1)) ? B_P_FULL1 : B_P_FULL));
    }

    if (ok && n_qt > 0) {
      if (!mbar_wait_bounded_warp(bar(B_O_DONE), 0, abort_flag)) { ok = false; fail_code = 32; }
      tc_fence_after();
    }
    if (ok) {          // warp-uniform (see the dQ kernel); only the stores depend on the key row
      const int64_t krow = (int64_t)k_row0 + key;
      uint8_t* dvrow = reinterpret_cast<uint8_t*>(e.dv) + half * OH * 2 +
                       2 * ((int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h + krow * p.v_stride_n);
      uint8_t* dkrow = reinterpret_cast<uint8_t*>(e.dk) + half * OH * 2 +
                       2 * ((int64_t)b * p.k_stride_b + (int64_t)h * p.k_stride_h + krow * p.k_stride_n);
      #pragma unroll 1
      for (int t = 0; t < 2; ++t) {
        const float sc = t == 0 ? 1.f : e.sm_scale;
        uint8_t* dst = t == 0 ? dvrow : dkrow;
        float o[OH];
        #pragma unroll
        for (int c = 0; c < OH / 32; ++c) {
          uint32_t v[32];
          if (n_qt > 0) {
            tmem_ld_x32(tmem + lane_base + (t == 0 ? COL_DV : COL_DK) + half * OH + 32 * c, v);
            tmem_ld_wait();
          } else {
            #pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0u;
          }
          #pragma unroll
          for (int i = 0; i < 32; ++i) o[32 * c + i] = __uint_as_float(v[i]) * sc;
        }
        const int d_cols = p.D - half * OH;      // head dims 16 and 32: only the real columns are written
        bool write_out = key_ok && d_cols > 0;
        if (parts > 1 && write_out) {
          float* acc = (t == 0 ? e.ws_dv : e.ws_dk) + ((int64_t)tail_slot * BM + r) * HD + half * OH;
          #pragma unroll
          for (int i = 0; i < OH; ++i) atomicAdd(acc + i, o[i]);
          __threadfence();
          int* counter = e.ws_cnt_k + (((int64_t)tail_slot * BM + r) * 2 + half) * 2 + t;
          write_out = (atomicAdd(counter, 1) == parts - 1);
          if (write_out) {
            __threadfence();
            #pragma unroll
            for (int i = 0; i < OH / 4; ++i) {
              const float4 t4 = __ldcg(reinterpret_cast<const float4*>(acc) + i);
              o[4 * i] = t4.x; o[4 * i + 1] = t4.y; o[4 * i + 2] = t4.z; o[4 * i + 3] = t4.w;
              reinterpret_cast<float4*>(acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            *counter = 0;
          }
        }
        if (write_out) {
          #pragma unroll
          for (int i = 0; i < OH / 8; ++i) {
            uint4 w4;
            w4.x = pack2<kBf16>(o[8 * i + 0], o[8 * i + 1]);
            w4.y = pack2<kBf16>(o[8 * i + 2], o[8 * i + 3]);
            w4.z = pack2<kBf16>(o[8 * i + 4], o[8 * i + 5]);
            w4.w = pack2<kBf16>(o[8 * i + 6], o[8 * i + 7]);
            if (8 * i < d_cols) *reinterpret_cast<uint4*>(dst + i * 16) = w4;
          }
        }
      }
    }
  }

  if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, 3000 + fail_code);
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ======================================================================== dK and dV, head dim 64
// One block per SM owns a 128-key tile and streams 128-query tiles.  Tensor memory (all 512
// columns): S^T and dP^T (128 float32 columns each), P^T and dS^T (64 columns each: 128 queries in
// 16 bits) in columns of their OWN, dV and dK (64 each).  Because P^T and dS^T do not overwrite
// S^T and dP^T, the products of the next query tile are queued as soon as the softmax warps have
// READ the current ones into registers; sixteen softmax warps (lane quarter x 32-column group)
// then never wait for the tensor core in steady state, and the 128-wide products run at the full
// tensor rate instead of the shared-memory rate of the 64-wide ones.  Two issuing threads: one
// for the products with both operands in shared memory (S^T, dP^T), one for those that read
// P^T / dS^T from tensor memory (dV, dK).
namespace wide {
constexpr int BQ = 128;                 // rows of a streamed query tile
constexpr int ST = 4;                   // stages of the Q / dO ring
constexpr int TILE = BM * 128;          // bytes of a 128-row x 64-dim tile
constexpr int SOFTMAX_WARPS = 16;
constexpr int WARP_LOAD = 16, WARP_SS = 17, WARP_TS = 18;
constexpr int THREADS = 19 * 32;
constexpr int PAD = 2 * BM;             // table padding: |key - query| of a near-diagonal tile stays below max_distance + 255
constexpr int COL_ST = 0, COL_DPT = 128, COL_PT = 256, COL_DST = 320, COL_DV = 384, COL_DK = 448;
enum {
  W_RES_FULL = 0,
  W_Q_FULL = 1,                         // [ST] Q tile (TMA) + its lse / delta vectors (loading warp)
  W_DO_FULL = W_Q_FULL + ST,            // [ST]
  W_EMPTY = W_DO_FULL + ST,             // [ST] both tiles of a stage: after dK of that step
  // per half of a query tile (queries 0-63 | 64-127; two barriers each):
  W_FULL = W_EMPTY + ST,                // S^T and dP^T of the half are complete
  W_FREE = W_FULL + 2,                  // ... and read into registers by its eight softmax warps
  W_PDS_FULL = W_FREE + 2,              // P^T and dS^T of the half are stored
  W_TS_DONE = W_PDS_FULL + 2,           // ... and read by the dV and dK products
  W_O_DONE = W_TS_DONE + 2,
  W_NUM
};
static_assert(W_NUM <= 24, "barrier slots");
struct __align__(16) WControl {
  unsigned long long bars[24];
  uint32_t tmem_base;
  int abort_flag;
  int work[6];
  float vec[ST][2][BQ];                 // (bias of a far tile) - lse in the log2 domain, and -delta
};
__host__ __device__ inline size_t smem_bytes(int lut_entries) {
  return 1024 + (size_t)(2 + 2 * ST) * TILE + sizeof(WControl) + 16 + (size_t)lut_entries * 4 + 16;
}
}  // namespace wide

template <bool kBf16, bool kWindow>
__global__ void __launch_bounds__(wide::THREADS, 1)
attn_bwd_dkv_wide_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                         const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                         const __grid_constant__ AttnParams p, const __grid_constant__ BwdExtra e,
                         const __grid_constant__ BucketSpec spec) {
  const int window = kWindow ? p.window : 0;
  using namespace wide;
  constexpr int HD = 64;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sK = base, sV = base + TILE, sQ = base + 2 * TILE, sDO = sQ + ST * TILE;
  WControl* ctl = reinterpret_cast<WControl*>(smem + (2 + 2 * ST) * TILE);
  float* lut = reinterpret_cast<float*>(smem + (2 + 2 * ST) * TILE + ((sizeof(WControl) + 15) / 16) * 16);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- work item: a 128-key tile of one (batch, head) or packed sequence
  int h, b = 0, batch_idx = 0, part = 0, parts = 1, tail_slot = 0;
  int key0, k_row0 = 0, len_k, q_row0 = 0, len_q, q_off;
  if (p.cu_k == nullptr) {
    const int tiles_k = (p.N + BM - 1) / BM;
    int tile_lin = (int)blockIdx.x;
    if (tile_lin >= e.k_tail_first) {
      const int ee = tile_lin - e.k_tail_first;
      parts = e.k_parts;
      tail_slot = ee / parts;
      part = ee - tail_slot * parts;
      tile_lin = e.k_tail_first + tail_slot;
    }
    const int tx = tile_lin % tiles_k;
    const int hb = tile_lin / tiles_k;
    h = hb % p.H;
    batch_idx = b = hb / p.H;
    key0 = tx * BM;
    len_k = p.N; len_q = p.M; q_off = p.q_pos_offset;
  } else {
    h = blockIdx.y;
    if (warp == 0) {
      int seq = -1, t = 0;
      const bool found = find_seq_tile(p.cu_k, p.B, BM, (int)blockIdx.x, seq, t);
      if (lane == 0) { ctl->work[0] = found ? seq : -1; ctl->work[1] = t; }
    }
    __syncthreads();
    const int seq = ctl->work[0];
    if (seq < 0) return;
    key0 = ctl->work[1] * BM;
    k_row0 = min(p.cu_k[seq], p.total_k); len_k = min(p.cu_k[seq + 1], p.total_k) - k_row0;
    q_row0 = min(p.cu_q[seq], p.total_q); len_q = min(p.cu_q[seq + 1], p.total_q) - q_row0;
    q_off = len_k - len_q;
  }
  const int keys_in_tile = min(BM, len_k - key0);
  // query tiles that can see a key of this tile: causal keeps q_off + m >= key
  int i_first = 0;
  if (p.causal) i_first = max(0, key0 - q_off) / BQ;
  int n_qt_all = (len_q + BQ - 1) / BQ;
  if (p.local_block > 0) {
    // block-local attention: only the queries of the three neighbouring blocks see this key tile
    const int bl = p.M < p.local_block ? p.M : p.local_block;
    const int kb = key0 / bl;
    i_first = max(0, (kb - 1) * bl) / BQ;
    n_qt_all = (min(len_q, (kb + 2) * bl) + BQ - 1) / BQ;
  }
  if (window > 0) {
    // sliding window: the queries within (key - window, key + window) of a key of this tile
    i_first = max(0, key0 - window + 1 - q_off) / BQ;
    n_qt_all = (min(len_q, max(0, key0 + BM - 1 + window - q_off)) + BQ - 1) / BQ;
  }
  int n_qt = max(0, n_qt_all - i_first);
  if (parts > 1) {       // this block's share of the query tiles
    const int per = (n_qt + parts - 1) / parts;
    const int first = min(part * per, n_qt);
    n_qt = min(n_qt, first + per) - first;
    i_first += first;
  }

  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  const int md = spec.max_distance;
  const bool has_bias = p.table != nullptr;
  auto stat_index = [&](int m) -> int64_t {
    return p.cu_q == nullptr ? ((int64_t)batch_idx * p.H + h) * p.M + m : ((int64_t)q_row0 + m) * p.H + h;
  };
  // loading warp: lse / delta of the first query tile, requested before the set-up below
  float pre_l[4] = {0.f, 0.f, 0.f, 0.f}, pre_d[4] = {0.f, 0.f, 0.f, 0.f};
  if (warp == WARP_LOAD && n_qt > 0) {
    #pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int m = i_first * BQ + lane + 32 * u;
      if (m < len_q) { pre_l[u] = p.lse[stat_index(m)]; pre_d[u] = e.delta[stat_index(m)]; }
    }
  }
  auto load_q_tile = [&](int i) {
    const int s = i % ST;
    const int m0 = (i_first + i) * BQ;
    mbar_expect_tx(bar(W_Q_FULL + s), TILE);
    tma_load_4d(sQ + s * TILE, &tmap_q, bar(W_Q_FULL + s), 0, q_row0 + m0, h, b);
    mbar_expect_tx(bar(W_DO_FULL + s), TILE);
    tma_load_4d(sDO + s * TILE, &tmap_do, bar(W_DO_FULL + s), 0, q_row0 + m0, h, b);
  };
  if (warp == WARP_LOAD && lane == 0) {
    ctl->abort_flag = 0;
    mbar_init(bar(W_RES_FULL), 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(bar(W_Q_FULL + s), 2);       // TMA transaction + the vectors written by the loading warp
      mbar_init(bar(W_DO_FULL + s), 1);
      mbar_init(bar(W_EMPTY + s), 1);
    }
    for (int hf = 0; hf < 2; ++hf) {
      mbar_init(bar(W_FULL + hf), 1);
      mbar_init(bar(W_FREE + hf), SOFTMAX_WARPS / 2);
      mbar_init(bar(W_PDS_FULL + hf), SOFTMAX_WARPS / 2);
      mbar_init(bar(W_TS_DONE + hf), 1);
    }
    mbar_init(bar(W_O_DONE), 1);
    fence_barrier_init();
    fence_proxy_async();
    if (n_qt > 0) {
      mbar_expect_tx(bar(W_RES_FULL), 2 * TILE);
      tma_load_4d(sK, &tmap_k, bar(W_RES_FULL), 0, k_row0 + key0, h, b);
      tma_load_4d(sV, &tmap_v, bar(W_RES_FULL), 0, k_row0 + key0, h, b);
      for (int i = 0; i < ST && i < n_qt; ++i) load_q_tile(i);
    }
  }
  if (warp == WARP_SS) {
    tmem_alloc(smem_u32(&ctl->tmem_base), 512);
    tmem_relinquish();
  }
  if (has_bias) {
    for (int i = tid; i <= 2 * md; i += THREADS) {
      const int bucket = bucket_of_delta_counted(spec, i - md);
      lut[PAD + i] = load_table(p.table, p.table_dtype, (int64_t)bucket * p.table_stride0 + h) * kLog2e;
    }
    __syncthreads();
    const float lo_v = lut[PAD], hi_v = lut[PAD + 2 * md];
    for (int i = tid; i < PAD; i += THREADS) {
      lut[i] = lo_v;
      lut[PAD + 2 * md + 1 + i] = hi_v;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl->tmem_base;
  volatile int* abort_flag = &ctl->abort_flag;
  int fail_code = 0;
  // bias of a query tile that lies entirely beyond +-max_distance of this key tile (one value for
  // the whole 128 x 128 tile): the loading warp folds it into the lse vector
  auto far_tile_bias = [&](int q_lo, bool& is_far) -> float {
    is_far = false;
    if (!has_bias) { is_far = true; return 0.f; }
    const int dmin = key0 - (q_lo + BQ - 1), dmax = key0 + BM - 1 - q_lo;
    if (dmin >= md) { is_far = true; return lut[2 * md + PAD]; }
    if (dmax <= -md) { is_far = true; return lut[PAD]; }
    return 0.f;
  };

  if (warp == WARP_LOAD) {
    // whole warp: lane 0 drives the TMA, all lanes fetch the lse / delta of the query tile
    bool okp = true;
    for (int i = 0; i < n_qt; ++i) {
      const int s = i % ST;
      const uint32_t ph = (uint32_t)((i / ST) & 1);
      const int m0 = (i_first + i) * BQ;
      // the statistics of the next tile are requested a whole iteration before they are used
      float cur_l[4], cur_d[4];
      #pragma unroll
      for (int u = 0; u < 4; ++u) {
        cur_l[u] = pre_l[u]; cur_d[u] = pre_d[u];
        const int m = m0 + BQ + lane + 32 * u;
        if (i + 1 < n_qt && m < len_q) { pre_l[u] = p.lse[stat_index(m)]; pre_d[u] = e.delta[stat_index(m)]; }
      }
      if (i >= ST) {
        // every lane waits: the vectors of this stage are rewritten below
        if (!mbar_wait_bounded(bar(W_EMPTY + s), ph ^ 1u, abort_flag)) okp = false;
        if (!__all_sync(0xffffffffu, okp)) { fail_code = 10; break; }
        if (lane == 0) load_q_tile(i);        // the first ST tiles were requested above
      }
      bool is_far;
      const float fold = far_tile_bias(q_off + m0, is_far);
      #pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = lane + 32 * u;
        const int m = m0 + c;
        const bool valid = m < len_q;
        const float l_ = valid ? cur_l[u] : 0.f;
        const float d_ = valid ? cur_d[u] : 0.f;
        // stored negated: the softmax warps add them with packed operations
        ctl->vec[s][0][c] = fold - lse_to_log2(l_, valid);
        ctl->vec[s][1][c] = valid ? -d_ : 0.f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(W_Q_FULL + s));
    }
  } else if (warp == WARP_SS) {
    if (lane == 0 && n_qt > 0) {
      constexpr uint32_t IDESC = make_idesc_f16(kBf16, kBf16, BM, BQ / 2, false, false);   // 128 keys x 64 queries
      bool ok = mbar_wait_bounded(bar(W_RES_FULL), 0, abort_flag);
      if (!ok) fail_code = 20;
      for (int i = 0; ok && i < n_qt; ++i) {
        const int s = i % ST;
        const uint32_t ph = (uint32_t)((i / ST) & 1);
        if (!mbar_wait_bounded(bar(W_Q_FULL + s), ph, abort_flag)) { fail_code = 21; break; }
        if (!mbar_wait_bounded(bar(W_DO_FULL + s), ph, abort_flag)) { fail_code = 23; break; }
        #pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          // S^T(i) = K Q^T and dP^T(i) = V dO^T of this half once its warps hold those of tile i-1 in registers
          if (i > 0 && !mbar_wait_bounded(bar(W_FREE + hf), (uint32_t)((i - 1) & 1), abort_flag)) { ok = false; fail_code = 22; break; }
          tc_fence_after();
          {
            const uint64_t da = make_smem_desc_sw128(sK, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sQ + s * TILE + hf * (TILE / 2), 16, 1024);
            #pragma unroll
            for (int k = 0; k < 4; ++k) umma_ss(tmem + COL_ST + 64 * hf, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, k > 0);
          }
          {
            const uint64_t da = make_smem_desc_sw128(sV, 16, 1024);
            const uint64_t db = make_smem_desc_sw128(sDO + s * TILE + hf * (TILE / 2), 16, 1024);
            #pragma unroll
            for (int k = 0; k < 4; ++k) umma_ss(tmem + COL_DPT + 64 * hf, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC, k > 0);
          }
          tc_commit(bar(W_FULL + hf));
        }
      }
    }
  } else if (warp == WARP_TS) {
    if (lane == 0 && n_qt > 0) {
      constexpr uint32_t IDESC = make_idesc_f16(kBf16, kBf16, BM, HD, false, true);    // dO / Q as MN-major B
      bool ok = true;
      for (int i = 0; ok && i < n_qt; ++i) {
        const int s = i % ST;
        #pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          // P^T(i) and dS^T(i) of this half are stored.  (Their stage was loaded long ago: S^T(i)
          // needed it, and the softmax warps saw S^T(i) before they arrived here.)
          if (!mbar_wait_bounded(bar(W_PDS_FULL + hf), (uint32_t)(i & 1), abort_flag)) { ok = false; fail_code = 25; break; }
          tc_fence_after();
          // dV += P^T(i) dO, dK += dS^T(i) Q: 16 queries per step, the first operand from tensor memory
          #pragma unroll
          for (int k = 4 * hf; k < 4 * hf + 4; ++k) {
            const uint64_t db = make_smem_desc_sw128(sDO + s * TILE + k * 2048, 16, 1024);
            umma_ts(tmem + COL_DV, tmem + COL_PT + 8 * k, db, IDESC, (i > 0 || k > 0) ? 1u : 0u);
          }
          #pragma unroll
          for (int k = 4 * hf; k < 4 * hf + 4; ++k) {
            const uint64_t db = make_smem_desc_sw128(sQ + s * TILE + k * 2048, 16, 1024);
            umma_ts(tmem + COL_DK, tmem + COL_DST + 8 * k, db, IDESC, (i > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(bar(W_TS_DONE + hf));   // P^T and dS^T of the half may be overwritten
        }
        if (!ok) break;
        // S^T(i) and dP^T(i), the other readers of this stage, completed before P^T(i) could be formed
        tc_commit(bar(W_EMPTY + s));
        if (i + 1 == n_qt) tc_commit(bar(W_O_DONE));
      }
    }
  } else {
    const int quarter = warp & 3, cg = warp >> 2;      // tensor-memory lane quarter, 32-column group
    const int r = quarter * 32 + lane;                 // key row inside the tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tST = tmem + lane_base + COL_ST + cg * 32;
    const uint32_t tDPT = tmem + lane_base + COL_DPT + cg * 32;
    const uint32_t tPT = tmem + lane_base + COL_PT + cg * 16;
    const uint32_t tDST = tmem + lane_base + COL_DST + cg * 16;
    const float scale = p.scale_log2;
    const int key = key0 + r;
    const bool key_ok = r < keys_in_tile;
    const int wkey0 = key0 + quarter * 32;             // first key of this warp
    bool ok = true;

    // One probe per wait in the common case: the vote makes the branch uniform.  A wait that ran
    // out leaves `ok` false for the whole warp; the tile is finished with whatever the registers
    // hold (nothing below can fault) and the loop ends at the bottom of the tile.
    auto wait = [&](int which, uint32_t parity, int code) {
      if (__all_sync(0xffffffffu, mbar_try_wait(bar(which), parity))) return;
      if (!mbar_wait_bounded_warp(bar(which), parity, abort_flag) && ok) { ok = false; fail_code = code; }
    };
    // every arrival follows a warp-wide tcgen05.wait: all lanes' accesses are complete, no __syncwarp
    auto arrive = [&](int which) {
      tc_fence_before();
      if (lane == 0) mbar_arrive(bar(which));
    };
    const bool warp_beyond_keys = wkey0 + 32 > len_k;
    const int hf = cg >> 1;                            // half of the query tile this warp works on
    // One pass per tile, as in the dQ kernel: S^T and dP^T are read together, P^T and dS^T stored
    // together: two probes, one load and one store round trip, two arrivals per tile.  The lse /
    // delta vectors of a stage are ordered by the chain loading warp -> Q_FULL -> issuing thread
    // -> FULL (commit) -> here.
    for (int i = 0; i < n_qt; ++i) {
      const int s = i % ST;
      const int q_lo = q_off + (i_first + i) * BQ;       // key-coordinate position of the tile's first query
      const int qp0 = q_lo + cg * 32;                    // ... of this warp's column 0
      // a tile entirely beyond +-max_distance has one bias value, folded into the vector by the
      // loading warp; otherwise the bias is looked up per element (the table is padded with its
      // end values, so any key - query of such a tile is inside it)
      const bool per_element = has_bias && !(key0 - (q_lo + BQ - 1) >= md || key0 + BM - 1 - q_lo <= -md);
      const bool masked = warp_beyond_keys || (p.causal && wkey0 + 31 > qp0) ||
                          (window > 0 && (wkey0 + 31 - qp0 >= window || qp0 + 31 - wkey0 >= window));
      const float* vl = &ctl->vec[s][0][cg * 32];
      const float* vd = &ctl->vec[s][1][cg * 32];
      // column c has delta = key - (qp0 + c): the table index falls as c grows
      const float* lrow = lut + (key - qp0 + md + PAD);
      wait(W_FULL + hf, (uint32_t)(i & 1), 30);
      tc_fence_after();
      uint32_t sv[32], dp[32];
      tmem_ld_x32(tST, sv);
      tmem_ld_x32(tDPT, dp);
      tmem_ld_wait();
      arrive(W_FREE + hf);                                   // S^T(i+1) and dP^T(i+1) may be formed now

      // P^T = exp2(S^T scale + bias - lse), dS^T = P^T o (dP^T - delta); both rounded to 16 bits as
      // the first operands of the dV and dK products
      // (all 32 columns before the first store: a version that stored each half of 16 as soon as it
      // was packed had fewer live registers and was 9 % slower over the whole backward)
      uint32_t pp[16], pd[16];
      if (!masked && !per_element) {
        #pragma unroll
        for (int g = 0; g < 8; ++g) {
          const int c = 4 * g;
          const float4 l4 = *reinterpret_cast<const float4*>(vl + c);
          const float4 d4 = *reinterpret_cast<const float4*>(vd + c);
          float x0, x1, x2, x3;
          fma2v(x0, x1, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), scale, l4.x, l4.y);
          fma2v(x2, x3, __uint_as_float(sv[c + 2]), __uint_as_float(sv[c + 3]), scale, l4.z, l4.w);
          float g0 = __uint_as_float(dp[c]), g1 = __uint_as_float(dp[c + 1]);
          float g2 = __uint_as_float(dp[c + 2]), g3 = __uint_as_float(dp[c + 3]), e0, e1, e2, e3;
          add2(g0, g1, d4.x, d4.y);          // dP - delta
          add2(g2, g3, d4.z, d4.w);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);
          mul2(e0, e1, p0, p1, g0, g1);
          mul2(e2, e3, p2, p3, g2, g3);
          pp[2 * g] = pack2<kBf16>(p0, p1);
          pp[2 * g + 1] = pack2<kBf16>(p2, p3);
          pd[2 * g] = pack2<kBf16>(e0, e1);
          pd[2 * g + 1] = pack2<kBf16>(e2, e3);
        }
      } else if (!masked) {
        #pragma unroll
        for (int g = 0; g < 16; ++g) {
          const int c = 2 * g;
          const float2 l2 = *reinterpret_cast<const float2*>(vl + c);
          const float2 d2 = *reinterpret_cast<const float2*>(vd + c);
          float x0 = lrow[-c], x1 = lrow[-c - 1], g0 = __uint_as_float(dp[c]), g1 = __uint_as_float(dp[c + 1]), e0, e1;
          add2(x0, x1, l2.x, l2.y);          // bias - lse
          fma2v(x0, x1, __uint_as_float(sv[c]), __uint_as_float(sv[c + 1]), scale, x0, x1);
          add2(g0, g1, d2.x, d2.y);          // dP - delta
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          mul2(e0, e1, p0, p1, g0, g1);
          pp[g] = pack2<kBf16>(p0, p1);
          pd[g] = pack2<kBf16>(e0, e1);
        }
      } else {
        #pragma unroll
        for (int g = 0; g < 16; ++g) {
          float pv[2], dv2[2];
          #pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int c = 2 * g + u;
            const float bias = per_element ? lrow[-c] : 0.f;
            float x = fmaf(__uint_as_float(sv[c]), scale, bias) + vl[c];
            // masked: key outside the sequence, or (causal) after the query
            if (!key_ok || (p.causal && key > qp0 + c) ||
                (window > 0 && (key - (qp0 + c) >= window || (qp0 + c) - key >= window))) x = -INFINITY;
            pv[u] = fast_exp2(x);
            dv2[u] = pv[u] * (__uint_as_float(dp[c]) + vd[c]);
          }
          pp[g] = pack2<kBf16>(pv[0], pv[1]);
          pd[g] = pack2<kBf16>(dv2[0], dv2[1]);
        }
      }
      if (i > 0) {
        wait(W_TS_DONE + hf, (uint32_t)((i - 1) & 1), 32);    // dV(i-1) and dK(i-1) have read P^T(i-1) and dS^T(i-1)
        tc_fence_after();
      }
      tmem_st_x16(tPT, pp);
      tmem_st_x16(tDST, pd);
      tmem_st_wait();
      arrive(W_PDS_FULL + hf);
      if (!ok) break;                                    // warp-uniform: every wait ends in a vote
    }


    if (ok && n_qt > 0) {
      if (!mbar_wait_bounded_warp(bar(W_O_DONE), 0, abort_flag)) { ok = false; fail_code = 35; }
      tc_fence_after();
    }
    if (ok) {          // warp-uniform; only the stores depend on the key row
      const int64_t krow = (int64_t)k_row0 + key;
      uint8_t* dvrow = reinterpret_cast<uint8_t*>(e.dv) + cg * 32 +
                       2 * ((int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h + krow * p.v_stride_n);
      uint8_t* dkrow = reinterpret_cast<uint8_t*>(e.dk) + cg * 32 +
                       2 * ((int64_t)b * p.k_stride_b + (int64_t)h * p.k_stride_h + krow * p.k_stride_n);
      #pragma unroll 1
      for (int t = 0; t < 2; ++t) {
        const float sc = t == 0 ? 1.f : e.sm_scale;
        uint8_t* dst = t == 0 ? dvrow : dkrow;
        float o[16];
        uint32_t v[16];
        if (n_qt > 0) {
          tmem_ld_x16(tmem + lane_base + (t == 0 ? COL_DV : COL_DK) + cg * 16, v);
          tmem_ld_wait();
        } else {
          #pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0u;
        }
        #pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = __uint_as_float(v[i]) * sc;
        bool write_out = key_ok && cg * 16 < p.D;   // head dims 16 and 32: only the real columns are written
        if (parts > 1 && write_out) {
          float* acc = (t == 0 ? e.ws_dv : e.ws_dk) + ((int64_t)tail_slot * BM + r) * HD + cg * 16;
          #pragma unroll
          for (int i = 0; i < 16; ++i) atomicAdd(acc + i, o[i]);
          __threadfence();
          int* counter = e.ws_cnt_k + (((int64_t)tail_slot * BM + r) * 4 + cg) * 2 + t;
          write_out = (atomicAdd(counter, 1) == parts - 1);
          if (write_out) {
            __threadfence();
            #pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 t4 = __ldcg(reinterpret_cast<const float4*>(acc) + i);
              o[4 * i] = t4.x; o[4 * i + 1] = t4.y; o[4 * i + 2] = t4.z; o[4 * i + 3] = t4.w;
              reinterpret_cast<float4*>(acc)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            *counter = 0;
          }
        }
        if (write_out) {
          #pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint4 w4;
            w4.x = pack2<kBf16>(o[8 * i + 0], o[8 * i + 1]);
            w4.y = pack2<kBf16>(o[8 * i + 2], o[8 * i + 3]);
            w4.z = pack2<kBf16>(o[8 * i + 4], o[8 * i + 5]);
            w4.w = pack2<kBf16>(o[8 * i + 6], o[8 * i + 7]);
            *reinterpret_cast<uint4*>(dst + i * 16) = w4;
          }
        }
      }
    }
  }

  if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, 3100 + fail_code);
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_SS) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace sm100b

// Last-wave plan of the two backward kernels (see BwdExtra).  The counter areas have a fixed
// size per device; the float32 rows follow.  Everything in the scratch is zero between launches.
struct BwdPlan {
  int q_tail_first, q_parts, q_rem, k_tail_first, k_parts, k_rem;
  int64_t cnt_bytes, dq_bytes, dk_bytes;
  int64_t bytes() const { return (q_parts > 1 || k_parts > 1) ? 2 * cnt_bytes + dq_bytes + 2 * dk_bytes : 0; }
};

// Head dim 64 takes the 128-query dK/dV kernel (one block per SM); T5B_BWD_DKV_WIDE=0 builds
// the library with the 64-query kernel (two blocks per SM) for every head dim.
#ifndef T5B_BWD_DKV_WIDE
#define T5B_BWD_DKV_WIDE 1
#endif
static bool dkv_wide(const t5b_attn_args& a) { return T5B_BWD_DKV_WIDE != 0 && a.D <= 64; }

static BwdPlan sm100_bwd_plan(const t5b_attn_args& a) {
  using namespace sm100b;
  const int HD = a.D <= 64 ? 64 : 128;      // width the kernels compute in
  BwdPlan t;
  const long long nq = (long long)((a.M + BM - 1) / BM) * a.H * a.B;
  const long long nk = (long long)((a.N + BM - 1) / BM) * a.H * a.B;
  t.q_tail_first = (int)(nq > 0x7fffffffLL ? 0x7fffffff : nq);
  t.k_tail_first = (int)(nk > 0x7fffffffLL ? 0x7fffffff : nk);
  t.q_parts = t.k_parts = 1;
  t.q_rem = t.k_rem = 0;
  t.cnt_bytes = t.dq_bytes = t.dk_bytes = 0;
  if (a.cu_seqlens_q != nullptr || a.causal || a.local_block > 0 || a.window > 0 || nq > 0x3fffffffLL || nk > 0x3fffffffLL) return t;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    return t;
  }
  const int slots = (HD == 64 ? 2 : 1) * sms;
  auto al = [](int64_t x) { return (x + 255) / 256 * 256; };
  auto split = [&](long long n_total, int n_stream, int& tail_first, int& parts, int& rem) {
    rem = (int)(n_total % slots);
    if (rem == 0) return;
    int pp = slots / rem;
    if (pp > n_stream / 16) pp = n_stream / 16;   // at least 16 streamed tiles (1024 rows) per part
    if (pp > 8) pp = 8;
    if (pp < 2) { rem = 0; return; }
    parts = pp;
    tail_first = (int)(n_total - rem);
  };
  split(nq, (a.N + BT - 1) / BT, t.q_tail_first, t.q_parts, t.q_rem);
  if (dkv_wide(a)) {
    // one block per SM, 128-query steps: at least 8 of them (1024 rows) per part
    auto split_wide = [&](long long n_total, int n_stream, int& tail_first, int& parts, int& rem) {
      rem = (int)(n_total % sms);
      if (rem == 0) return;
      int pp = sms / rem;
      if (pp > n_stream / 8) pp = n_stream / 8;
      if (pp > 8) pp = 8;
      if (pp < 2) { rem = 0; return; }
      parts = pp;
      tail_first = (int)(n_total - rem);
    };
    split_wide(nk, (a.M + wide::BQ - 1) / wide::BQ, t.k_tail_first, t.k_parts, t.k_rem);
  } else {
    split(nk, (a.M + BT - 1) / BT, t.k_tail_first, t.k_parts, t.k_rem);
  }
  // counters: (row, half, tensor) per slot of the 64-query kernels = (row, 16-column group, tensor)
  // per SM of the 128-query kernel: the same size
  t.cnt_bytes = al((int64_t)(HD == 64 ? 2 : 1) * sms * BM * 2 * 2 * 4);
  t.dq_bytes = al((int64_t)t.q_rem * BM * HD * 4);
  t.dk_bytes = al((int64_t)t.k_rem * BM * HD * 4);
  return t;
}

int64_t sm100_bwd_workspace_bytes(const t5b_attn_bwd_args& g) {
  if (!sm100_bwd_supports(g)) return 0;
  return sm100_bwd_plan(g.fwd).bytes();
}

// True when the tensor-core backward can take this problem.
bool sm100_bwd_supports(const t5b_attn_bwd_args& g) {
  const t5b_attn_args& a = g.fwd;
  if (!sm100_supports(a)) return false;       // bf16/fp16, aligned; head dims 16 and 32 run zero-filled to 64
  auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (!al16(g.dout) || !al16(g.dq) || !al16(g.dk) || !al16(g.dv)) return false;
  const int64_t s[] = {g.do_stride_b, g.do_stride_h, g.do_stride_m};
  for (int64_t x : s) if (x < 0 || (x % 8) != 0) return false;
  return true;
}

int sm100_attention_bwd(const t5b_attn_bwd_args& g, const BucketSpec& spec, cudaStream_t stream) {
  using namespace sm100b;
  const t5b_attn_args& a = g.fwd;
  const bool varlen = a.cu_seqlens_q != nullptr;
  const bool bf16 = a.dtype == T5B_BF16;
  const int HD = a.D <= 64 ? 64 : 128;      // width the kernels compute in; the tensor maps zero-fill columns past a.D
  AttnParams p = make_attn_params(a);
  p.tiles_x = (a.M + BM - 1) / BM;
  BwdExtra e;
  e.dout = g.dout;
  e.do_stride_b = g.do_stride_b; e.do_stride_h = g.do_stride_h; e.do_stride_m = g.do_stride_m;
  e.dq = g.dq; e.dk = g.dk; e.dv = g.dv;
  e.dtable = g.dtable; e.delta = g.delta; e.sm_scale = a.sm_scale;
  BwdPlan plan = sm100_bwd_plan(a);
  const bool use_ws = plan.bytes() > 0 && g.workspace != nullptr && g.workspace_bytes >= plan.bytes() &&
                      ((uintptr_t)g.workspace & 255) == 0;
  if (!use_ws) {
    plan.q_parts = plan.k_parts = 1;
    plan.q_tail_first = plan.k_tail_first = 0x7fffffff;
    plan.q_rem = plan.k_rem = 0;
  }
  if (plan.q_parts <= 1) plan.q_tail_first = 0x7fffffff;
  if (plan.k_parts <= 1) plan.k_tail_first = 0x7fffffff;
  e.q_tail_first = plan.q_tail_first; e.q_parts = plan.q_parts;
  e.k_tail_first = plan.k_tail_first; e.k_parts = plan.k_parts;
  {
    char* ws = use_ws ? (char*)g.workspace : nullptr;
    e.ws_cnt_q = (int32_t*)ws;
    e.ws_cnt_k = (int32_t*)(ws ? ws + plan.cnt_bytes : nullptr);
    e.ws_dq = (float*)(ws ? ws + 2 * plan.cnt_bytes : nullptr);
    e.ws_dk = (float*)(ws ? ws + 2 * plan.cnt_bytes + plan.dq_bytes : nullptr);
    e.ws_dv = (float*)(ws ? ws + 2 * plan.cnt_bytes + plan.dq_bytes + plan.dk_bytes : nullptr);
  }

  const long long rows_q = varlen ? (long long)a.total_q : (long long)a.B * a.M;
  const long long rows_k = varlen ? (long long)a.total_k : (long long)a.B * a.N;
  // 1. delta
  {
    const long long n_rows = rows_q * a.H;
    const int rows_per_block = 8 * (32 / (a.D / 8));
    long long blocks = (n_rows + rows_per_block - 1) / rows_per_block;
    if (blocks > 148LL * 16) blocks = 148LL * 16;
    if (blocks > 0) {
      const unsigned nb = (unsigned)blocks;
      if (a.D == 16) {
        if (bf16) bwd_delta_kernel<__nv_bfloat16, 16><<<nb, 256, 0, stream>>>(p, e, n_rows);
        else bwd_delta_kernel<__half, 16><<<nb, 256, 0, stream>>>(p, e, n_rows);
      } else if (a.D == 32) {
        if (bf16) bwd_delta_kernel<__nv_bfloat16, 32><<<nb, 256, 0, stream>>>(p, e, n_rows);
        else bwd_delta_kernel<__half, 32><<<nb, 256, 0, stream>>>(p, e, n_rows);
      } else if (a.D == 64) {
        if (bf16) bwd_delta_kernel<__nv_bfloat16, 64><<<nb, 256, 0, stream>>>(p, e, n_rows);
        else bwd_delta_kernel<__half, 64><<<nb, 256, 0, stream>>>(p, e, n_rows);
      } else {
        if (bf16) bwd_delta_kernel<__nv_bfloat16, 128><<<nb, 256, 0, stream>>>(p, e, n_rows);
        else bwd_delta_kernel<__half, 128><<<nb, 256, 0, stream>>>(p, e, n_rows);
      }
      if (cudaGetLastError() != cudaSuccess) return T5B_ERR_LAUNCH;
    }
  }
  (void)rows_k;   // > 0: checked by the caller
  int st;
  CUtensorMap q128, do128, k64, v64, k128, v128, q64, do64;
  const int64_t Mr = varlen ? a.total_q : a.M, Nr = varlen ? a.total_k : a.N;
  const int Bm = varlen ? 1 : a.B;
  const int64_t qsb = varlen ? 0 : a.q_stride_b, ksb = varlen ? 0 : a.k_stride_b, vsb = varlen ? 0 : a.v_stride_b;
  const int64_t dsb = varlen ? 0 : g.do_stride_b;
  if ((st = make_tmap(&q128, a.q, bf16, a.D, BM, Mr, a.H, Bm, a.q_stride_m, a.q_stride_h, qsb)) != T5B_OK) return st;
  if ((st = make_tmap(&do128, g.dout, bf16, a.D, BM, Mr, a.H, Bm, g.do_stride_m, g.do_stride_h, dsb)) != T5B_OK) return st;
  if ((st = make_tmap(&k64, a.k, bf16, a.D, BT, Nr, a.H, Bm, a.k_stride_n, a.k_stride_h, ksb)) != T5B_OK) return st;
  if ((st = make_tmap(&v64, a.v, bf16, a.D, BT, Nr, a.H, Bm, a.v_stride_n, a.v_stride_h, vsb)) != T5B_OK) return st;
  if ((st = make_tmap(&k128, a.k, bf16, a.D, BM, Nr, a.H, Bm, a.k_stride_n, a.k_stride_h, ksb)) != T5B_OK) return st;
  if ((st = make_tmap(&v128, a.v, bf16, a.D, BM, Nr, a.H, Bm, a.v_stride_n, a.v_stride_h, vsb)) != T5B_OK) return st;
  if ((st = make_tmap(&q64, a.q, bf16, a.D, BT, Mr, a.H, Bm, a.q_stride_m, a.q_stride_h, qsb)) != T5B_OK) return st;
  if ((st = make_tmap(&do64, g.dout, bf16, a.D, BT, Mr, a.H, Bm, g.do_stride_m, g.do_stride_h, dsb)) != T5B_OK) return st;

  const int lut_n = a.table ? 2 * spec.max_distance + 1 + 2 * LUT_PAD : 0;
  const size_t smem = HD == 64 ? smem_bytes<64>(lut_n) : smem_bytes<128>(lut_n);
  const bool win = a.window > 0;
  using KernelFn = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, AttnParams, BwdExtra, BucketSpec);
  static const KernelFn kq_all[2][2][2] = {
      {{attn_bwd_dq_kernel<false, 64, false>, attn_bwd_dq_kernel<false, 64, true>},
       {attn_bwd_dq_kernel<true, 64, false>, attn_bwd_dq_kernel<true, 64, true>}},
      {{attn_bwd_dq_kernel<false, 128, false>, attn_bwd_dq_kernel<false, 128, true>},
       {attn_bwd_dq_kernel<true, 128, false>, attn_bwd_dq_kernel<true, 128, true>}}};
  static const KernelFn kkv_all[2][2][2] = {
      {{attn_bwd_dkv_kernel<false, 64, false>, attn_bwd_dkv_kernel<false, 64, true>},
       {attn_bwd_dkv_kernel<true, 64, false>, attn_bwd_dkv_kernel<true, 64, true>}},
      {{attn_bwd_dkv_kernel<false, 128, false>, attn_bwd_dkv_kernel<false, 128, true>},
       {attn_bwd_dkv_kernel<true, 128, false>, attn_bwd_dkv_kernel<true, 128, true>}}};
  const KernelFn kq = kq_all[HD == 64 ? 0 : 1][bf16 ? 1 : 0][win ? 1 : 0];
  const KernelFn kkv = kkv_all[HD == 64 ? 0 : 1][bf16 ? 1 : 0][win ? 1 : 0];
  static std::atomic<bool> attr_set[64][8];   // any thread may get here first
  int dev = 0;
  cudaGetDevice(&dev);
  const int which = (bf16 ? 1 : 0) + (HD == 64 ? 0 : 2) + (win ? 4 : 0);
  if (dev < 0 || dev >= 64 || !attr_set[dev][which].load(std::memory_order_acquire)) {
    const int lut_max = 2 * 2048 + 1 + 2 * LUT_PAD;
    const int smem_max = (int)(HD == 64 ? smem_bytes<64>(lut_max) : smem_bytes<128>(lut_max));
    if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max) != cudaSuccess ||
        cudaFuncSetAttribute(kkv, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max) != cudaSuccess) {
      cudaGetLastError();
      return T5B_ERR_LAUNCH;
    }
    if (dev >= 0 && dev < 64) attr_set[dev][which].store(true, std::memory_order_release);
  }
  dim3 gq, gk;
  if (varlen) {
    gq = dim3((unsigned)((long long)a.total_q / BM + a.B), (unsigned)a.H, 1);
    gk = dim3((unsigned)((long long)a.total_k / BM + a.B), (unsigned)a.H, 1);
  } else {
    long long nq = (long long)p.tiles_x * a.H * a.B;
    long long nk = (long long)((a.N + BM - 1) / BM) * a.H * a.B;
    if (plan.q_parts > 1) nq = plan.q_tail_first + (long long)plan.q_rem * plan.q_parts;
    if (plan.k_parts > 1) nk = plan.k_tail_first + (long long)plan.k_rem * plan.k_parts;
    if (nq > 0x7fffffffLL || nk > 0x7fffffffLL) return T5B_ERR_SHAPE;
    gq = dim3((unsigned)nq, 1, 1);
    gk = dim3((unsigned)nk, 1, 1);
  }
  if (gq.y > 65535 || gk.y > 65535) return T5B_ERR_SHAPE;
  if (gq.x > 0) {
    kq<<<gq, NUM_THREADS, smem, stream>>>(q128, do128, k64, v64, p, e, spec);
    if (cudaGetLastError() != cudaSuccess) return T5B_ERR_LAUNCH;
  }
  if (gk.x > 0 && dkv_wide(a)) {
    const KernelFn kw = bf16 ? (win ? attn_bwd_dkv_wide_kernel<true, true> : attn_bwd_dkv_wide_kernel<true, false>)
                             : (win ? attn_bwd_dkv_wide_kernel<false, true> : attn_bwd_dkv_wide_kernel<false, false>);
    static std::atomic<bool> wide_attr_set[64][4];
    const int which_w = (bf16 ? 1 : 0) + (win ? 2 : 0);
    if (dev < 0 || dev >= 64 || !wide_attr_set[dev][which_w].load(std::memory_order_acquire)) {
      const int smem_max = (int)wide::smem_bytes(2 * 2048 + 1 + 2 * wide::PAD);
      if (cudaFuncSetAttribute(kw, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_max) != cudaSuccess) {
        cudaGetLastError();
        return T5B_ERR_LAUNCH;
      }
      if (dev >= 0 && dev < 64) wide_attr_set[dev][which_w].store(true, std::memory_order_release);
    }
    const size_t smem_w = wide::smem_bytes(a.table ? 2 * spec.max_distance + 1 + 2 * wide::PAD : 0);
    kw<<<gk, wide::THREADS, smem_w, stream>>>(k128, v128, q128, do128, p, e, spec);
    if (cudaGetLastError() != cudaSuccess) return T5B_ERR_LAUNCH;
  } else if (gk.x > 0) {
    kkv<<<gk, NUM_THREADS, smem, stream>>>(k128, v128, q64, do64, p, e, spec);
    if (cudaGetLastError() != cudaSuccess) return T5B_ERR_LAUNCH;
  }
  return T5B_OK;
}

}  // namespace t5b
