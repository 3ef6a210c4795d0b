// Fused relative-position-bias flash attention, forward, for sm_100a.
//
// One thread block owns one 128-row query tile of one (batch, head) -- or of one
// packed sequence when cu_seqlens are given -- and walks the key/value tiles:
//
//   warp 8      TMA producer: Q once, then K/V tiles into a shared-memory ring
//               (cp.async.bulk.tensor, 128-byte swizzle, completion on mbarriers)
//   warp 9      tensor-core issuer: S = Q K^T and O += P V with tcgen05.mma,
//               accumulators in tensor memory, tcgen05.commit -> mbarriers
//   warps 0-7   softmax: two threads share a query row (warp w and warp w+4 see the
//               same 32 TMEM lanes; one takes the first half of the tile's key columns,
//               the other the second half, and the matching half of the O columns).  A
//               thread copies its scores from tensor memory to registers at once
//               (tcgen05.ld) and the S buffer is handed back immediately, so the next
//               QK^T runs while this tile's softmax is computed.  The T5 bias is added
//               from a shared-memory copy of delta -> table[bucket(delta), head] (no
//               L x L tensor exists, no 1/sqrt(d) unless asked).  Two passes over the
//               registers: maximum, then all exponentials (packed to bf16/fp16) and the
//               row sum; P goes back to tensor memory (tcgen05.st) where the second MMA
//               reads it as its A operand.  O and the row sum are rescaled lazily: the
//               value the exponentials are taken against moves only when a maximum has
//               outgrown it by 2^40 (bf16; 2^10 for fp16), and then by a whole number of
//               powers of two, which lets the two threads of a row agree after the
//               exponentials instead of before them (see the loop).
//
// At head dim 64 one thread (warp 8) both loads and issues the matrix products -- every refill of
// the K/V ring waits on an event at least half a tile old, so it never blocks -- and the block has
// nine warps; at head dim 128 the loads keep warp 8 and the products move to warp 9.
//
// Head dim 64 uses 128-key tiles, head dim 128 uses 64-key tiles whose rows are two
// 128-byte-swizzled sub-tiles; either way two blocks fit on an SM (<= 256 TMEM columns and
// 80-96 KB of tiles each), so one block's softmax overlaps the other block's matrix products.
// The exponential unit (16 ex2 per clock per SM) is the scarcest resource at head dim 64: it
// needs twice the time of the tensor core for the same tile.
//
// Semantics follow flash_attention_with_fusing_bias
// (src/turbot5/ops/fused_bias_attention.py:184-365) with positions as in the
// reference's `basic` path: delta = n - (q_pos_offset + m).
#include "t5b_common.cuh"
#include "attn_params.cuh"
#include "attn_sm100_util.cuh"

#include <atomic>

namespace t5b {

namespace sm100 {

// Head dim 64: column pairs of every 8 whose exponentials run on the FMA pipe.  Measured on B200 at
// B2 H12 L8192: 0 -> 0.594 ms, 2 -> 0.648 ms, i.e. in THIS kernel (two threads per row, 96 registers,
// bound by issue slots and latency rather than by the exponential unit alone) the extra FMA-pipe
// instructions cost more than the freed ex2 slots give back, so the default is 0.  More registers do
// not help either: 18 warps per SM put 5 on one scheduler, 16384 / (5 x 32) = 102 registers is the
// ceiling for two blocks per SM (a 104- or 112-register build runs one block per SM: 0.88-0.97 ms).
#ifndef T5B_FWD_POLY64
#define T5B_FWD_POLY64 0
#endif
constexpr int BM = 128;            // query rows per block
constexpr int STAGES = 2;          // K/V ring depth
constexpr int MAX_THREADS = 320;
constexpr int SOFTMAX_THREADS = 256;
constexpr int WARP_TMA = 8;
constexpr int TMEM_COLS = 256;

// Tile geometry per head dim.  Head dim 64: 128 keys per tile.  Head dim 128: 64 keys per tile,
// so that two blocks still fit on an SM (96 KB of tiles, 224 TMEM columns each).  A tile row of
// 128 dims is two 128-byte-swizzled sub-tiles of 64 dims, loaded by two TMA boxes.
template <int HD_>
struct Geo {
  static constexpr int HD = HD_;
  static constexpr int BN = HD_ == 64 ? 128 : 64;     // keys per tile
  static constexpr int NSUB = HD_ / 64;                 // 64-dim sub-tiles per row
  static constexpr int SUB_Q = BM * 128;                // bytes of one Q sub-tile  [128 rows][64 dims]
  static constexpr int SUB_KV = BN * 128;               // bytes of one K/V sub-tile [BN rows][64 dims]
  static constexpr int Q_BYTES = NSUB * SUB_Q;
  static constexpr int KV_BYTES = NSUB * SUB_KV;
  static constexpr int SMEM_TILES = Q_BYTES + 2 * STAGES * KV_BYTES;
  // tensor memory: S = BN fp32 columns, P = BN/2 (packed 16-bit pairs), O = HD fp32 columns
  static constexpr int COL_S = 0, COL_P = BN, COL_O = BN + BN / 2;
  static constexpr int NH = BN / 2;                     // score columns per softmax thread
  static constexpr int NCH = NH / 32;                   // ... in chunks of 32
  static constexpr int OH = HD_ / 2;                    // output columns per softmax thread
  static constexpr int LUT_PAD = BM + BN;               // bias table padding on each side (entries)
  static_assert(COL_O + HD_ <= TMEM_COLS, "tensor memory layout");
};

// barrier slots
enum {
  BAR_Q_FULL = 0,
  BAR_K_FULL = 1,                    // [STAGES]
  BAR_V_FULL = BAR_K_FULL + STAGES,  // [STAGES]
  BAR_K_EMPTY = BAR_V_FULL + STAGES, // [STAGES]
  BAR_V_EMPTY = BAR_K_EMPTY + STAGES,
  BAR_S_FULL = BAR_V_EMPTY + STAGES,
  BAR_S_FREE,
  BAR_P_FULL,
  BAR_O_DONE,
  BAR_PAIR,                          // [4]: the two warps sharing a TMEM lane quarter (one arrival each)
  NUM_BARS = BAR_PAIR + 4
};

struct __align__(8) Control {
  unsigned long long bars[NUM_BARS];
  uint32_t tmem_base;
  int abort_flag;
  int work[6];   // a TileWork, broadcast from warp 0 for packed sequences
  float xchg[2][2][BM];   // [tile parity][column half][row]: row maxima; at the end: row sums
};

template <int HD>
__host__ __device__ inline size_t smem_bytes(int lut_entries) {
  return 1024 /*alignment slack*/ + Geo<HD>::SMEM_TILES + sizeof(Control) + 16 + (size_t)lut_entries * 4;
}


// kPoly: of every 8 column pairs of an unmasked tile, this many take their exponentials on the FMA
// pipe (PolyExp above) instead of the exponential unit; 8 = all of them (used by the parity tests).
// kWindow: the sliding-window mode is compiled into a kernel of its own (with it in the plain kernel
// the two extra per-row values of the masked path raised the spills of the softmax loop from 108 to
// 264 bytes and the 8k forward went from 0.577 to 0.67 ms).
// kNarrow: head dims 16 and 32 (run as head dim 64, see the epilogue) have kernels of their own for the
// same reason: the column test in the epilogue, outside every loop, cost the plain kernel 3 %.
template <bool kBf16, int HD, int kPoly, bool kWindow = false, bool kNarrow = false>
__global__ void __launch_bounds__(HD == 64 ? 288 : MAX_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q,
                const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v,
                const __grid_constant__ AttnParams p,
                const __grid_constant__ BucketSpec spec) {
  using G = Geo<HD>;
  // head dim 64: warp 8 does the loads and the matrix products (288 threads); head dim 128: the
  // loads keep a warp of their own (its tiles are shorter, the refill has less slack)
  constexpr bool kOneIoThread = HD == 64;
  constexpr int NUM_THREADS = kOneIoThread ? 288 : MAX_THREADS;
  constexpr int WARP_MMA = kOneIoThread ? 8 : 9;
  constexpr int BN = G::BN, NSUB = G::NSUB, SUB_Q = G::SUB_Q, SUB_KV = G::SUB_KV;
  constexpr int Q_BYTES = G::Q_BYTES, KV_BYTES = G::KV_BYTES, SMEM_TILES = G::SMEM_TILES;
  constexpr int COL_S = G::COL_S, COL_P = G::COL_P, COL_O = G::COL_O;
  constexpr int NH = G::NH, NCH = G::NCH, OH = G::OH, LUT_PAD = G::LUT_PAD;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sQ = base;
  const uint32_t sK = base + Q_BYTES;
  const uint32_t sV = sK + STAGES * KV_BYTES;
  Control* ctl = reinterpret_cast<Control*>(smem + SMEM_TILES);
  float* lut = reinterpret_cast<float*>(smem + SMEM_TILES + ((sizeof(Control) + 15) / 16) * 16);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // ---------------------------------------------------------------- work item
  // dense: 1-D grid over (query tile, head, batch), heaviest causal tiles first; blocks at or
  //        beyond p.tail_first share a tile `parts` ways along the keys (last-wave balancing)
  // varlen: blockIdx.x indexes the concatenated per-sequence tile lists, blockIdx.y = head
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
    w = dense_tile<BM>(p, tx, batch_idx);
  } else {
    h = blockIdx.y;
    if (warp == 0) {
      TileWork f = find_varlen_tile<BM>(p, (int)blockIdx.x);
      if (lane == 0) *shared_work = f;
    }
    __syncthreads();
    w = *shared_work;
    if (w.b < 0) return;   // block beyond the last tile: uniform exit, nothing allocated yet
  }
  const int b = w.b, q_row0 = w.q_row0, rows_in_tile = w.rows_in_tile;
  const int k_row0 = w.k_row0, qpos0 = w.qpos0;
  int len_k = w.len_k;
  // Block-local attention (T5LocalAttention, src/turbot5/model/attentions.py:523-650): the rows of
  // block i of `local_block` queries see the keys of blocks i-1, i, i+1 and nothing else.  Keys
  // before 0 or after the end are the reference's zero padding blocks: they are NOT masked (their
  // scores are the bare bias) and the TMA zero fill supplies them.  So the key range becomes
  // [n_base, len_k) with a negative n_base for the first block and len_k past the tensor's end.
  int n_base = 0;
  if (p.local_block > 0) {
    const int bl = p.M < p.local_block ? p.M : p.local_block;      // a shorter sequence is one block
    const int blk = q_row0 / bl;
    n_base = (blk - 1) * bl;
    len_k = (blk + 2) * bl;
  }

  const int window = kWindow ? p.window : 0;
  // keys this tile can see
  int kv_end = len_k;
  if (p.causal) kv_end = min(len_k, qpos0 + rows_in_tile);
  // Sliding window (T5LocalAttention with its padding mask: |n - query| < window over the valid keys):
  // the tile walks the key tiles that hold a visible key for any of its rows.
  if (window > 0) {
    n_base = max(0, qpos0 - window + 1) / BN * BN;
    kv_end = min(kv_end, qpos0 + rows_in_tile - 1 + window);
  }
  const int n_kv_all = kv_end > n_base ? (kv_end - n_base + BN - 1) / BN : 0;
  // this block's share of the key tiles: [kv_first, kv_first + n_kv)
  const int kv_per = (n_kv_all + parts - 1) / parts;
  const int kv_first = min(part * kv_per, n_kv_all);
  const int n_kv = min(n_kv_all, kv_first + kv_per) - kv_first;
  const int n_first = n_base + kv_first * BN;       // first key of this block's first tile

  // ---------------------------------------------------------------- set-up
  const uint32_t bar0 = smem_u32(&ctl->bars[0]);
  auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };
  auto load_k = [&](int j) {
    const int s = j % STAGES;
    mbar_expect_tx(bar(BAR_K_FULL + s), KV_BYTES);
    #pragma unroll
    for (int u = 0; u < NSUB; ++u)
      tma_load_4d(sK + s * KV_BYTES + u * SUB_KV, &tmap_k, bar(BAR_K_FULL + s), 64 * u, k_row0 + n_first + j * BN, h, b);
  };
  auto load_v = [&](int j) {
    const int s = j % STAGES;
    mbar_expect_tx(bar(BAR_V_FULL + s), KV_BYTES);
    #pragma unroll
    for (int u = 0; u < NSUB; ++u)
      tma_load_4d(sV + s * KV_BYTES + u * SUB_KV, &tmap_v, bar(BAR_V_FULL + s), 64 * u, k_row0 + n_first + j * BN, h, b);
  };
  // The loading thread sets up the barriers itself and requests Q and the first STAGES key/value
  // tiles at once: they are in flight while the other threads build the bias table below.
  if (warp == (kOneIoThread ? WARP_MMA : WARP_TMA) && lane == 0) {
    ctl->abort_flag = 0;
    mbar_init(bar(BAR_Q_FULL), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(BAR_K_FULL + s), 1);
      mbar_init(bar(BAR_V_FULL + s), 1);
      mbar_init(bar(BAR_K_EMPTY + s), 1);
      mbar_init(bar(BAR_V_EMPTY + s), 1);
    }
    mbar_init(bar(BAR_S_FULL), 1);
    // one arrival per softmax warp (lane 0, after the warp has converged): 32 lanes arriving
    // on one barrier word are 32 serialised shared-memory atomics
    mbar_init(bar(BAR_S_FREE), SOFTMAX_THREADS / 32);
    mbar_init(bar(BAR_P_FULL), SOFTMAX_THREADS / 32);
    mbar_init(bar(BAR_O_DONE), 1);
    for (int qd = 0; qd < 4; ++qd) mbar_init(bar(BAR_PAIR + qd), 2);
    fence_barrier_init();
    fence_proxy_async();
    if (n_kv > 0) {
      mbar_expect_tx(bar(BAR_Q_FULL), Q_BYTES);
      #pragma unroll
      for (int u = 0; u < NSUB; ++u) tma_load_4d(sQ + u * SUB_Q, &tmap_q, bar(BAR_Q_FULL), 64 * u, q_row0, h, b);
      for (int j = 0; j < STAGES && j < n_kv; ++j) { load_k(j); load_v(j); }
    }
  }
  __syncwarp();
  if (warp == WARP_MMA) {
    tmem_alloc(smem_u32(&ctl->tmem_base), TMEM_COLS);
    tmem_relinquish();
  }
  // delta -> bias (log2 domain) for this head.  Entry i holds delta = i - md - LUT_PAD;
  // the table is constant beyond +-md, and the padding lets a tile that straddles
  // the +-md boundary index it without clamping.
  const int md = spec.max_distance;
  const int lut_n = 2 * md + 1 + 2 * LUT_PAD;
  if (p.table != nullptr) {
    // one bucket search and one table load per delta in [-md, md]; beyond, the bucket no longer
    // changes and the padding is filled with the two end values
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

  if (kOneIoThread && warp == WARP_MMA) {
    // ============================================================ loads and matrix products, one thread
    // (head dim 64).  Every ring refill waits on an event that lies at least half a tile back, so
    // the thread never blocks on them, and the block has one warp less to schedule and poll.
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t IDESC_QK = make_idesc_f16(kBf16, kBf16, BM, BN, false, false);
      constexpr uint32_t IDESC_PV = make_idesc_f16(kBf16, kBf16, BM, HD, false, true);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % STAGES;
        if (!mbar_wait_bounded(bar(BAR_K_FULL + s), (uint32_t)((j / STAGES) & 1), abort_flag)) return false;
        tc_fence_after();
        #pragma unroll
        for (int u = 0; u < NSUB; ++u) {
          const uint64_t da = make_smem_desc_sw128(sQ + u * SUB_Q, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sK + s * KV_BYTES + u * SUB_KV, 16, 1024);
          #pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_ss(tmem + COL_S, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC_QK, (u | k) > 0);
        }
        tc_commit(bar(BAR_S_FULL));
        tc_commit(bar(BAR_K_EMPTY + s));
        return true;
      };
      static_assert(STAGES == 2, "the refills below assume the two tiles requested during set-up");
      bool ok = mbar_wait_bounded(bar(BAR_Q_FULL), 0, abort_flag);
      if (!ok) fail_code = 20;
      if (ok && !issue_qk(0)) { ok = false; fail_code = 21; }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int s = j % STAGES;
        if (j + 1 < n_kv) {
          if (!mbar_wait_bounded(bar(BAR_S_FREE), (uint32_t)(j & 1), abort_flag)) { fail_code = 25; break; }
          tc_fence_after();
          if (!issue_qk(j + 1)) { fail_code = 23; break; }
        }
        // refill the ring: K(j+2) into the slot of K(j) (QK(j) finished before S(j) could be copied),
        // V(j+1) into the slot of V(j-1) (PV(j-1) was issued a tile ago)
        if (j + 2 < n_kv) {
          if (!mbar_wait_bounded(bar(BAR_K_EMPTY + s), (uint32_t)((j / STAGES) & 1), abort_flag)) { fail_code = 10; break; }
          load_k(j + 2);
        }
        if (j >= 1 && j + 1 < n_kv) {
          if (!mbar_wait_bounded(bar(BAR_V_EMPTY + ((j - 1) % STAGES)), (uint32_t)(((j - 1) / STAGES) & 1), abort_flag)) { fail_code = 11; break; }
          load_v(j + 1);
        }
        if (!mbar_wait_bounded(bar(BAR_P_FULL), (uint32_t)(j & 1), abort_flag)) { fail_code = 22; break; }
        tc_fence_after();
        if (!mbar_wait_bounded(bar(BAR_V_FULL + s), (uint32_t)((j / STAGES) & 1), abort_flag)) { fail_code = 24; break; }
        tc_fence_after();
        #pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint64_t dv = make_smem_desc_sw128(sV + s * KV_BYTES + k * 2048, NSUB > 1 ? SUB_KV : 16, 1024);
          umma_ts(tmem + COL_O, tmem + COL_P + k * 8, dv, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar(BAR_O_DONE));
        tc_commit(bar(BAR_V_EMPTY + s));
      }
    }
  } else if (!kOneIoThread && warp == WARP_TMA) {
    // ============================================================ TMA producer
    if (lane == 0) {
      for (int j = STAGES; j < n_kv; ++j) {        // the first STAGES tiles were requested during set-up
        const int s = j % STAGES;
        const uint32_t ph = (uint32_t)((j / STAGES) & 1);
        if (!mbar_wait_bounded(bar(BAR_K_EMPTY + s), ph ^ 1u, abort_flag)) { fail_code = 10; break; }
        load_k(j);
        if (!mbar_wait_bounded(bar(BAR_V_EMPTY + s), ph ^ 1u, abort_flag)) { fail_code = 11; break; }
        load_v(j);
      }
    }
  } else if (!kOneIoThread && warp == WARP_MMA) {
    // ============================================================ MMA issuer
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t IDESC_QK = make_idesc_f16(kBf16, kBf16, BM, BN, false, false);
      constexpr uint32_t IDESC_PV = make_idesc_f16(kBf16, kBf16, BM, HD, false, true);
      auto issue_qk = [&](int j) -> bool {
        const int s = j % STAGES;
        if (!mbar_wait_bounded(bar(BAR_K_FULL + s), (uint32_t)((j / STAGES) & 1), abort_flag)) return false;
        tc_fence_after();
        #pragma unroll
        for (int u = 0; u < NSUB; ++u) {
          const uint64_t da = make_smem_desc_sw128(sQ + u * SUB_Q, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sK + s * KV_BYTES + u * SUB_KV, 16, 1024);
          #pragma unroll
          for (int k = 0; k < 4; ++k)   // 32 bytes of the 128-byte swizzle row per step
            umma_ss(tmem + COL_S, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), IDESC_QK, (u | k) > 0);
        }
        tc_commit(bar(BAR_S_FULL));
        tc_commit(bar(BAR_K_EMPTY + s));
        return true;
      };
      bool ok = mbar_wait_bounded(bar(BAR_Q_FULL), 0, abort_flag);
      if (!ok) fail_code = 20;
      if (ok && !issue_qk(0)) { ok = false; fail_code = 21; }
      for (int j = 0; ok && j < n_kv; ++j) {
        if (j + 1 < n_kv) {
          // S has been copied to registers: the next QK^T overlaps this tile's softmax
          if (!mbar_wait_bounded(bar(BAR_S_FREE), (uint32_t)(j & 1), abort_flag)) { fail_code = 25; break; }
          tc_fence_after();
          if (!issue_qk(j + 1)) { fail_code = 23; break; }
        }
        if (!mbar_wait_bounded(bar(BAR_P_FULL), (uint32_t)(j & 1), abort_flag)) { fail_code = 22; break; }
        tc_fence_after();
        const int s = j % STAGES;
        if (!mbar_wait_bounded(bar(BAR_V_FULL + s), (uint32_t)((j / STAGES) & 1), abort_flag)) { fail_code = 24; break; }
        tc_fence_after();
        // V tile is [BN keys][HD dims], dims contiguous: an MN-major B operand.  8 keys x 128 B
        // per swizzle group (1024 B, the stride byte offset); each K=16 step covers two groups;
        // dims 64-127 live in the second sub-tile, SUB_KV bytes on (the leading byte offset).
        #pragma unroll
        for (int k = 0; k < BN / 16; ++k) {
          const uint64_t dv = make_smem_desc_sw128(sV + s * KV_BYTES + k * 2048, NSUB > 1 ? SUB_KV : 16, 1024);
          umma_ts(tmem + COL_O, tmem + COL_P + k * 8, dv, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(bar(BAR_O_DONE));
        tc_commit(bar(BAR_V_EMPTY + s));
      }
    }
  } else if (warp < 8) {
    // ============================================================ softmax warps
    const int quarter = warp & 3;                  // TMEM lane quarter this warp may touch
    const int half = warp >> 2;                    // which 64 key columns / 32 output columns
    const int r = quarter * 32 + lane;             // query row inside the tile
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_base + COL_S + half * NH;
    const uint32_t tP = tmem + lane_base + COL_P + half * (NH / 2);
    const uint32_t tO = tmem + lane_base + COL_O + half * OH;
    const float scale = p.scale_log2;
    const float inv_scale = 1.f / scale;
    const bool has_bias = p.table != nullptr;
    const int qpos = qpos0 + r;
    // Rendezvous of the two warps that share this lane quarter: an mbarrier with a bounded
    // wait, so that a partner that gave up can never leave this warp waiting for ever.
    const uint32_t pair_bar = bar(BAR_PAIR + quarter);
    uint32_t pair_uses = 0;
    auto pair_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(pair_bar);
      const bool done = mbar_wait_bounded_warp(pair_bar, pair_uses & 1u, abort_flag);
      ++pair_uses;
      return done;
    };
    float m_use = -INFINITY;    // maximum the exponentials are taken against
    float l_sum = 0.f;          // this thread's half of the row sum
    bool ok = true;

    for (int j = 0; j < n_kv; ++j) {
      const int n0 = n_first + j * BN;             // first key of the tile
      const int c0 = half * NH;                    // first column of this thread inside the tile
      if (!mbar_wait_warp_fast(bar(BAR_S_FULL), (uint32_t)(j & 1), abort_flag)) { ok = false; fail_code = 30; break; }
      tc_fence_after();

      // this thread's scores -> registers, then give the S buffer back to the MMA warp
      uint32_t sv[NCH][32];
      #pragma unroll
      for (int c = 0; c < NCH; ++c) tmem_ld_x32(tS + 32 * c, sv[c]);
      tmem_ld_wait();                                // warp-wide: every lane's loads are complete
      tc_fence_before();
      if (lane == 0) mbar_arrive(bar(BAR_S_FREE));

      // tile classification (uniform over the block)
      const bool need_mask = (n0 + BN > len_k) || (p.causal && (n0 + BN - 1 > qpos0)) ||
                             (window > 0 && (n0 <= qpos0 + BM - 1 - window || n0 + BN - 1 >= qpos0 + window));
      int bias_mode = 0;            // 0 none, 1 constant over the tile, 2 per element
      float bias_const = 0.f;
      if (has_bias) {
        const int dmin = n0 - (qpos0 + BM - 1), dmax = n0 + BN - 1 - qpos0;
        if (dmin >= md) { bias_mode = 1; bias_const = lut[2 * md + LUT_PAD]; }
        else if (dmax <= -md) { bias_mode = 1; bias_const = lut[LUT_PAD]; }
        else bias_mode = 2;
      }
      const bool fast = !need_mask && bias_mode != 2 && scale > 0.f;

      // ---- pass 1: maximum of this thread's half row, four independent chains.  Fast tiles
      // (no mask, constant bias): over the raw scores, transformed once.  Other tiles:
      // x = s*scale + bias(delta) (+ mask) is computed in place first.
      float mx, top_raw;     // top_raw: the largest value pass 2 will exponentiate (before e_mul, e_add)
      {
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
        if (fast) {
          // eight independent chains of two-input maxima (the three-input form is no faster per
          // element on this pipe and its chains are half as many)
          float m4 = -INFINITY, m5 = -INFINITY, m6 = -INFINITY, m7 = -INFINITY;
          #pragma unroll
          for (int c = 0; c < NCH; ++c)
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
          const float* brow = lut + (n0 + c0 - qpos + md + LUT_PAD);
          int n_valid = (p.causal ? min(len_k, qpos + 1) : len_k) - n0 - c0;   // columns < n_valid are visible
          int n_lo = -(1 << 30);                                               // ... from column n_lo on
          if (window > 0) {
            n_valid = min(n_valid, qpos + window - n0 - c0);
            n_lo = qpos - window + 1 - n0 - c0;
          }
          #pragma unroll
          for (int c = 0; c < NCH; ++c) {
            #pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float bias = bias_mode == 2 ? brow[c * 32 + i] : bias_const;
              float x = fmaf(__uint_as_float(sv[c][i]), scale, bias);
              if (need_mask && (c * 32 + i >= n_valid || c * 32 + i < n_lo)) x = -INFINITY;
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
      // The maximum the exponentials are taken against, m_use, is the same in both threads of a
      // row.  First tile: the two halves exchange their maxima and wait for each other.  Later
      // tiles: m_use only moves when a half grew past the threshold, and then by a whole number
      // of powers of two, k.  Each thread publishes its k (almost always 0), computes its
      // exponentials against m_use + k without waiting, and reads the partner's k afterwards;
      // if the two differ, the smaller side rescales its packed P by 2^-(difference), which is
      // exact.  The rendezvous latency so hides behind the exponentials.
      float k_me = 0.f;
      if (j == 0) {
        ctl->xchg[0][half][r] = mx;
        if (!pair_sync()) { ok = false; fail_code = 33; break; }
        const float m0 = fmaxf(mx, ctl->xchg[0][half ^ 1][r]);
        m_use = (m0 == -INFINITY) ? 0.f : m0;     // finite from here on; a row without keys keeps l = 0
      } else {
        const float g = mx - m_use;
        if (g > kRescaleThreshold<kBf16>) k_me = fminf(ceilf(g), 1.0e6f);
        ctl->xchg[j & 1][half][r] = k_me;
        __syncwarp();
        if (lane == 0) mbar_arrive(pair_bar);
      }
      const float m_prov = m_use + k_me;
      // fast tiles: p = 2^(s*scale + (bias - m)); others: p = 2^(x - m) = 2^(x*1 + (-m))
      const float e_mul = fast ? scale : 1.f;
      const float e_add = fast ? bias_const - m_prov : -m_prov;

      // ---- pass 2: all exponentials of the tile into registers (packed P) and the row sum.
      // The scores die as they are consumed.
      uint32_t pk[NCH][16];
      float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
      const bool poly_ok = kPoly > 0 && !need_mask && scale > 0.f;
      PolyExp pe;
      if (poly_ok) {
        // unmasked tile: kPoly of every 8 column pairs on the FMA pipe, the rest on the exponential unit
        pe.setup(e_mul, fast ? inv_scale : 1.f, e_add);
        #pragma unroll
        for (int c = 0; c < NCH; ++c) {
          #pragma unroll
          for (int i = 0; i < 16; ++i) {
            float p0, p1;
            if (poly_pair(i, kPoly)) {
              pe.eval(__uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1]), p0, p1);
            } else {
              float x0, x1;
              fma2(x0, x1, __uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1]), e_mul, e_add);
              p0 = fast_exp2(x0);
              p1 = fast_exp2(x1);
            }
            pk[c][i] = pack2<kBf16>(p0, p1);
            if (i & 1) add2(t2, t3, p0, p1); else add2(t0, t1, p0, p1);
          }
        }
      } else {
        #pragma unroll
        for (int c = 0; c < NCH; ++c) {
          #pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0, x1;
            fma2(x0, x1, __uint_as_float(sv[c][2 * i]), __uint_as_float(sv[c][2 * i + 1]), e_mul, e_add);
            const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
            pk[c][i] = pack2<kBf16>(p0, p1);
            if (i & 1) add2(t2, t3, p0, p1); else add2(t0, t1, p0, p1);
          }
        }
      }
      float t_sum = (t0 + t1) + (t2 + t3);
      if (kBf16) {
        // The tensor core multiplies V by the ROUNDED probabilities.  With lazy rescaling the
        // largest one is not exactly 1, so when one key dominates a row its rounding error
        // (up to 2^-9 relative) would pass straight into the output.  Count that element in
        // the row sum as the tensor core sees it: same arithmetic as pass 2, then rounded.
        // (the same arithmetic as the element itself: with every pair on the FMA pipe that is the polynomial)
        float p_top = fast_exp2(fmaf(top_raw, e_mul, e_add)), p_dup;
        if (kPoly == 8 && poly_ok) pe.eval(top_raw, top_raw, p_top, p_dup);
        t_sum += __bfloat162float(__float2bfloat16_rn(p_top)) - p_top;
      }

      // ---- partner's step; rescale O, l and (if the steps differ) this tile's P.  Rare.
      bool o_done_seen = (j == 0);
      if (j > 0) {
        const bool met = mbar_wait_warp_fast(pair_bar, pair_uses & 1u, abort_flag);
        ++pair_uses;
        if (!met) { ok = false; fail_code = 33; break; }
        const float k_max = fmaxf(k_me, ctl->xchg[j & 1][half ^ 1][r]);
        if (__any_sync(0xffffffffu, k_max > 0.f)) {
          if (!mbar_wait_bounded_warp(bar(BAR_O_DONE), (uint32_t)((j - 1) & 1), abort_flag)) { ok = false; fail_code = 31; break; }
          tc_fence_after();
          o_done_seen = true;
          const float alpha = pow2_neg(k_max);
          l_sum *= alpha;
          m_use += k_max;
          #pragma unroll 1
          for (int c = 0; c < OH / 16; ++c) {      // this thread's columns of O
            uint32_t ov[16];
            tmem_ld_x16(tO + c * 16, ov);
            tmem_ld_wait();
            #pragma unroll
            for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st_x16(tO + c * 16, ov);
          }
          if (k_max > k_me) {
            const float beta = pow2_neg(k_max - k_me);
            t_sum *= beta;
            #pragma unroll
            for (int c = 0; c < NCH; ++c)
              #pragma unroll
              for (int i = 0; i < 16; ++i) pk[c][i] = scale_packed<kBf16>(pk[c][i], beta);
          }
        }
      }
      l_sum += t_sum;
      if (!o_done_seen) {
        if (!mbar_wait_warp_fast(bar(BAR_O_DONE), (uint32_t)((j - 1) & 1), abort_flag)) { ok = false; fail_code = 31; break; }
        tc_fence_after();
      }
      #pragma unroll
      for (int c = 0; c < NCH; ++c) tmem_st_x16(tP + 16 * c, pk[c]);
      tmem_st_wait();                                // warp-wide: every lane's stores are complete
      tc_fence_before();
      if (lane == 0) mbar_arrive(bar(BAR_P_FULL));
    }

    // ---- epilogue: O / l -> global (each thread its 32 output columns)
    if (ok && n_kv > 0) {
      if (!mbar_wait_bounded_warp(bar(BAR_O_DONE), (uint32_t)((n_kv - 1) & 1), abort_flag)) { ok = false; fail_code = 32; }
      tc_fence_after();
    }
    // total row sum = this half + the other half (slot parity distinct from the last tile's maxima)
    const int slot = n_kv & 1;
    ctl->xchg[slot][half][r] = l_sum;
    if (ok && !pair_sync()) { ok = false; fail_code = 33; }
    l_sum += ctl->xchg[slot][half ^ 1][r];
    // Head dims 16 and 32 run as head dim 64: the tensor maps fill the missing columns of Q, K and
    // V with zeros, so S is unchanged and the extra columns of O are zero; only the real ones
    // (p.D) are written.
    const int d_cols = kNarrow ? p.D - half * OH : OH;
    if (ok && d_cols > 0) {
      const bool row_ok = r < rows_in_tile;
      const int64_t row = (int64_t)q_row0 + r;
      const int64_t o_off = (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + row * p.o_stride_m + half * OH;
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) + 2 * o_off;
      float o[OH];
      #pragma unroll
      for (int c = 0; c < OH / 32; ++c) {
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
        // This block saw only part of the keys.  Publish (max, sum, unnormalised O) for this
        // row half; the last of the `parts` blocks to arrive merges them (no waiting).
        const int64_t slot = (int64_t)tail_slot * parts + part;
        float* my_o = p.ws_o + (slot * BM + r) * HD + half * OH;
        #pragma unroll
        for (int i = 0; i < OH / 4; ++i)
          reinterpret_cast<float4*>(my_o)[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        float* my_ml = p.ws_ml + ((slot * BM + r) * 2 + half) * 2;
        my_ml[0] = l_sum > 0.f ? m_use : -INFINITY;
        my_ml[1] = l_sum;
        __threadfence();
        int* counter = p.ws_counters + ((int64_t)tail_slot * BM + r) * 2 + half;
        const int arrived = atomicAdd(counter, 1);
        write_out = (arrived == parts - 1);
        if (write_out) {
          __threadfence();
          float m_all = -INFINITY;
          for (int s2 = 0; s2 < parts; ++s2)
            m_all = fmaxf(m_all, __ldcg(p.ws_ml + ((((int64_t)tail_slot * parts + s2) * BM + r) * 2 + half) * 2));
          const float m_ref = (m_all == -INFINITY) ? 0.f : m_all;
          float l_all = 0.f;
          #pragma unroll
          for (int i = 0; i < OH; ++i) o[i] = 0.f;
          for (int s2 = 0; s2 < parts; ++s2) {
            const int64_t sl = (int64_t)tail_slot * parts + s2;
            const float* ml = p.ws_ml + ((sl * BM + r) * 2 + half) * 2;
            const float sc = fast_exp2(__ldcg(ml) - m_ref);
            l_all = fmaf(__ldcg(ml + 1), sc, l_all);
            const float4* po = reinterpret_cast<const float4*>(p.ws_o + (sl * BM + r) * HD + half * OH);
            #pragma unroll
            for (int i = 0; i < OH / 4; ++i) {
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
        if (p.out_f32) {
          float4* of = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o_off);
          #pragma unroll
          for (int i = 0; i < OH / 4; ++i)
            if (!kNarrow || 4 * i < d_cols)
              of[i] = make_float4(o[4 * i] * inv_l, o[4 * i + 1] * inv_l, o[4 * i + 2] * inv_l, o[4 * i + 3] * inv_l);
        } else
        #pragma unroll
        for (int i = 0; i < OH / 8; ++i) {
          uint4 w4;
          w4.x = pack2<kBf16>(o[8 * i + 0] * inv_l, o[8 * i + 1] * inv_l);
          w4.y = pack2<kBf16>(o[8 * i + 2] * inv_l, o[8 * i + 3] * inv_l);
          w4.z = pack2<kBf16>(o[8 * i + 4] * inv_l, o[8 * i + 5] * inv_l);
          w4.w = pack2<kBf16>(o[8 * i + 6] * inv_l, o[8 * i + 7] * inv_l);
          if (!kNarrow || 8 * i < d_cols) *reinterpret_cast<uint4*>(orow + i * 16) = w4;
        }
        if (p.lse != nullptr && half == 0) {
          const float lse = l_sum > 0.f ? (m_use + log2f(l_sum)) * kLn2 : -INFINITY;
          if (p.cu_q == nullptr) p.lse[((int64_t)batch_idx * p.H + h) * p.M + row] = lse;
          else p.lse[row * p.H + h] = lse;
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, 1000 + fail_code);
  tc_fence_before();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
}  // namespace sm100

// True when the tcgen05 kernel can take this problem.
bool sm100_supports(const t5b_attn_args& a) {
  if (a.dtype != T5B_BF16 && a.dtype != T5B_F16) return false;
  if (a.D != 16 && a.D != 32 && a.D != 64 && a.D != 128) return false;    // 16 and 32 run zero-padded to 64
  if (a.max_distance > 2048 && a.table) return false;
  if (a.local_block < 0 || a.window < 0) return false;
  if (a.window > 0 && (a.causal || a.local_block > 0)) return false;
  if (a.local_block > 0) {
    // block-local attention: dense self-attention without a causal mask; a 128-row query tile
    // must lie inside one block
    if (a.cu_seqlens_q != nullptr || a.causal || a.M != a.N || a.q_pos_offset != 0) return false;
    if (a.M > a.local_block && (a.local_block % 128) != 0) return false;
  }
  auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (!al16(a.q) || !al16(a.k) || !al16(a.v) || !al16(a.out)) return false;
  const int64_t s[] = {a.q_stride_b, a.q_stride_h, a.q_stride_m, a.k_stride_b, a.k_stride_h, a.k_stride_n,
                       a.v_stride_b, a.v_stride_h, a.v_stride_n, a.o_stride_b, a.o_stride_h, a.o_stride_m};
  for (int64_t x : s) if (x < 0 || (x % 8) != 0) return false;   // 16-byte multiples
  return true;
}

// Last-wave balancing for dense, non-causal launches: with two blocks per SM the grid runs in
// waves of 2 x SMs equal-sized blocks; the tiles of a partially filled last wave are split along
// the keys so that the wave finishes in a fraction of a block time.
TailPlan sm100_tail_plan(const t5b_attn_args& a) {
  using namespace sm100;
  if (sm100w_prefers(a)) return sm100w_tail_plan(a);
  const int HD = a.D <= 64 ? 64 : 128, BN = HD == 64 ? Geo<64>::BN : Geo<128>::BN;
  TailPlan t;
  t.tiles_x = (a.M + BM - 1) / BM;
  const long long n_total = (long long)t.tiles_x * a.H * a.B;
  t.n_total = (int)(n_total > 0x7fffffffLL ? 0x7fffffff : n_total);
  t.tail_first = t.n_total;
  t.parts = 1;
  t.counters_bytes = t.ml_bytes = t.o_bytes = 0;
  if (a.cu_seqlens_q != nullptr || a.causal || a.local_block > 0 || a.window > 0 || n_total > 0x3fffffffLL) return t;
  static std::atomic<int> sms[64];     // SM count per device, 0 = not asked yet (any thread may get here first)
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return t; }
  int n_sm = sms[dev].load(std::memory_order_relaxed);
  if (n_sm == 0) {
    if (cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sm <= 0) { cudaGetLastError(); return t; }
    sms[dev].store(n_sm, std::memory_order_relaxed);
  }
  const int slots = 2 * n_sm;
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
  t.counters_bytes = al((int64_t)slots * BM * 2 * 4);
  t.ml_bytes = al((int64_t)rem * parts * BM * 2 * 2 * 4);
  t.o_bytes = al((int64_t)rem * parts * BM * HD * 4);
  return t;
}

int sm100_attention_fwd(const t5b_attn_args& a, const BucketSpec& spec, cudaStream_t stream) {
  using namespace sm100;
  if (sm100w_prefers(a)) return sm100w_attention_fwd(a, spec, stream);
  const bool varlen = a.cu_seqlens_q != nullptr;
  const bool bf16 = a.dtype == T5B_BF16;
  const int HD = a.D <= 64 ? 64 : 128;    // width the kernel computes in; the tensor maps zero-fill columns past a.D
  const int BN = HD == 64 ? Geo<64>::BN : Geo<128>::BN;
  const int LUT_PAD = BM + BN;
  CUtensorMap mq, mk, mv;
  int st;
  if (varlen) {
    if ((st = make_tmap(&mq, a.q, bf16, a.D, BM, a.total_q, a.H, 1, a.q_stride_m, a.q_stride_h, 0)) != T5B_OK) return st;
    if ((st = make_tmap(&mk, a.k, bf16, a.D, BN, a.total_k, a.H, 1, a.k_stride_n, a.k_stride_h, 0)) != T5B_OK) return st;
    if ((st = make_tmap(&mv, a.v, bf16, a.D, BN, a.total_k, a.H, 1, a.v_stride_n, a.v_stride_h, 0)) != T5B_OK) return st;
  } else {
    if ((st = make_tmap(&mq, a.q, bf16, a.D, BM, a.M, a.H, a.B, a.q_stride_m, a.q_stride_h, a.q_stride_b)) != T5B_OK) return st;
    if ((st = make_tmap(&mk, a.k, bf16, a.D, BN, a.N, a.H, a.B, a.k_stride_n, a.k_stride_h, a.k_stride_b)) != T5B_OK) return st;
    if ((st = make_tmap(&mv, a.v, bf16, a.D, BN, a.N, a.H, a.B, a.v_stride_n, a.v_stride_h, a.v_stride_b)) != T5B_OK) return st;
  }
  AttnParams p = make_attn_params(a);
  const int lut_n = a.table ? 2 * spec.max_distance + 1 + 2 * LUT_PAD : 0;
  const size_t smem = HD == 64 ? smem_bytes<64>(lut_n) : smem_bytes<128>(lut_n);
  dim3 grid;
  if (varlen) {
    // upper bound on sum_b ceil(len_b / BM) known without reading cu_seqlens
    const long long ub = (long long)a.total_q / BM + a.B;
    grid = dim3((unsigned)ub, (unsigned)a.H, 1);
  } else {
    TailPlan plan = sm100_tail_plan(a);
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
  // kernel variant: [head dim 128][bf16][0: default, 1: every exponential on the FMA pipe, 2: sliding window,
  // 3: default for head dims 16 and 32].  At head dim 64 the variants 1 and 2 also take the narrow heads.
  using KernelFn = void (*)(CUtensorMap, CUtensorMap, CUtensorMap, AttnParams, BucketSpec);
  static const KernelFn kernels[2][2][4] = {
      {{attn_fwd_kernel<false, 64, T5B_FWD_POLY64>, attn_fwd_kernel<false, 64, 8, false, true>,
        attn_fwd_kernel<false, 64, 0, true, true>, attn_fwd_kernel<false, 64, T5B_FWD_POLY64, false, true>},
       {attn_fwd_kernel<true, 64, T5B_FWD_POLY64>, attn_fwd_kernel<true, 64, 8, false, true>,
        attn_fwd_kernel<true, 64, 0, true, true>, attn_fwd_kernel<true, 64, T5B_FWD_POLY64, false, true>}},
      {{attn_fwd_kernel<false, 128, 0>, attn_fwd_kernel<false, 128, 8>, attn_fwd_kernel<false, 128, 0, true>, nullptr},
       {attn_fwd_kernel<true, 128, 0>, attn_fwd_kernel<true, 128, 8>, attn_fwd_kernel<true, 128, 0, true>, nullptr}}};
  int all_poly = a.window > 0 ? 2 : (a.kernel == T5B_KERNEL_TCGEN05_POLYEXP ? 1 : 0);
  if (all_poly == 0 && a.D < 64) all_poly = 3;
  const KernelFn kern = kernels[HD == 64 ? 0 : 1][bf16 ? 1 : 0][all_poly];
  // opt in to > 48 KB of dynamic shared memory once per device and kernel (any thread may get here first)
  static std::atomic<bool> attr_set[64][16];
  int dev = 0;
  cudaGetDevice(&dev);
  const int which = (bf16 ? 1 : 0) + (HD == 64 ? 0 : 2) + 4 * all_poly;
  const size_t smem_max = HD == 64 ? smem_bytes<64>(2 * 2048 + 1 + 2 * LUT_PAD) : smem_bytes<128>(2 * 2048 + 1 + 2 * LUT_PAD);
  if (dev < 0 || dev >= 64 || !attr_set[dev][which].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_max) != cudaSuccess) {
      cudaGetLastError();
      return T5B_ERR_LAUNCH;
    }
    if (dev >= 0 && dev < 64) attr_set[dev][which].store(true, std::memory_order_release);
  }
  kern<<<grid, HD == 64 ? 288 : MAX_THREADS, smem, stream>>>(mq, mk, mv, p, spec);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

}  // namespace t5b
