// Kernel-side view of a forward attention call (both kernel families).
#pragma once

#include "t5b_common.cuh"

namespace t5b {

struct AttnParams {
  const void* q; const void* k; const void* v; void* out;
  float* lse;
  const void* table;
  const int32_t* cu_q; const int32_t* cu_k;
  int32_t* status;
  int64_t q_stride_b, q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_h, k_stride_n;
  int64_t v_stride_b, v_stride_h, v_stride_n;
  int64_t o_stride_b, o_stride_h, o_stride_m;
  int64_t table_stride0;
  int32_t table_dtype;
  int32_t B, H, M, N, D;
  int32_t total_q, total_k;   // packed tensors: rows of q / of k and v (cu_seqlens beyond them are cut: nothing past a tensor is touched)
  int32_t causal;
  int32_t q_pos_offset;
  int32_t local_block;   // > 0: block-local attention (tensor-core forward only)
  int32_t out_f32;       // != 0: out is float32 (a partial result for the merge kernel)
  int32_t window;        // > 0: keys with |n - query position| < window only (one-tile tensor-core forward)
  float scale_log2;   // sm_scale * log2(e): softmax runs in the base-2 domain
  // Dense tensor-core launches use a 1-D grid over (query tile, head, batch).  Blocks at or
  // beyond `tail_first` share a query tile `tail_parts` ways along the keys and merge through
  // the scratch arrays (tail_first = number of tiles when nothing is split).
  int32_t tiles_x, tail_first, tail_parts;
  int32_t* ws_counters;   // [tail tiles][128 rows][2 halves]
  float* ws_ml;           // [tail tiles * parts][128][2][2]  (max, sum) per row half
  float* ws_o;            // [tail tiles * parts][128][64]    unnormalised O
};

// How the last wave of a dense launch is split (host side).
struct TailPlan {
  int tiles_x, n_total, tail_first, parts;
  int64_t counters_bytes, ml_bytes, o_bytes;
  int64_t bytes() const { return counters_bytes + ml_bytes + o_bytes; }
};
TailPlan sm100_tail_plan(const t5b_attn_args& a);

inline AttnParams make_attn_params(const t5b_attn_args& a) {
  AttnParams p;
  p.q = a.q; p.k = a.k; p.v = a.v; p.out = a.out;
  p.lse = a.lse; p.table = a.table;
  p.cu_q = a.cu_seqlens_q; p.cu_k = a.cu_seqlens_k;
  p.status = a.device_status;
  p.q_stride_b = a.q_stride_b; p.q_stride_h = a.q_stride_h; p.q_stride_m = a.q_stride_m;
  p.k_stride_b = a.k_stride_b; p.k_stride_h = a.k_stride_h; p.k_stride_n = a.k_stride_n;
  p.v_stride_b = a.v_stride_b; p.v_stride_h = a.v_stride_h; p.v_stride_n = a.v_stride_n;
  p.o_stride_b = a.o_stride_b; p.o_stride_h = a.o_stride_h; p.o_stride_m = a.o_stride_m;
  p.table_stride0 = a.table_stride0;
  p.table_dtype = a.table_dtype;
  p.B = a.B; p.H = a.H; p.M = a.M; p.N = a.N; p.D = a.D;
  p.total_q = (int32_t)a.total_q; p.total_k = (int32_t)a.total_k;
  p.causal = a.causal;
  p.q_pos_offset = a.q_pos_offset;
  p.local_block = a.local_block;
  p.out_f32 = a.out_f32;
  p.window = a.window;
  p.scale_log2 = a.sm_scale * kLog2e;
  p.tiles_x = 0; p.tail_first = 0x7fffffff; p.tail_parts = 1;
  p.ws_counters = nullptr; p.ws_ml = nullptr; p.ws_o = nullptr;
  return p;
}

// Work item of one thread block: a tile of query rows of one (batch | sequence).
struct TileWork {
  int b;             // batch index (0 for packed tensors); -1: block has no work
  int q_row0;        // first query row of the tile (global row for packed tensors)
  int rows_in_tile;
  int k_row0;        // first key row of the sequence (0 for dense)
  int len_k;
  int qpos0;         // key-coordinate position of the tile's first query row
};

#ifdef __CUDACC__
// Packed sequences: block `blk` walks the concatenation of the per-sequence tile
// lists (ceil(len_q / TILE_M) tiles each).  Called by ONE full warp; the result
// is valid in every lane.  No host-built work list, no host synchronisation.
template <int TILE_M>
__device__ __noinline__ TileWork find_varlen_tile(const AttnParams& p, int blk) {
  const int lane = threadIdx.x & 31;
  int found_b = -1, tile_in_seq = 0, acc = 0;
  // Longest sequences first: a tile's work grows with its sequence's key count, and a long tile
  // scheduled last leaves the GPU mostly idle while it finishes.
  if (p.B <= 128) {
    // Exact order (key count descending, index ascending) without sorting anything: a lane owns up
    // to four sequences and counts, for each, the tiles of all sequences that precede it in that
    // order -- B^2 / 32 comparisons per block, a few hundred instructions for a batch of 32.
    const int chunks = (p.B + 31) >> 5;
    int lk[4], nt[4], start[4];
    #pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int bb = lane + 32 * u;
      lk[u] = -1; nt[u] = 0; start[u] = 0;
      if (u < chunks && bb < p.B) {
        lk[u] = p.cu_k[bb + 1] - p.cu_k[bb];
        nt[u] = (p.cu_q[bb + 1] - p.cu_q[bb] + TILE_M - 1) / TILE_M;
      }
    }
    #pragma unroll
    for (int u2 = 0; u2 < 4; ++u2) {
      if (u2 < chunks) {
        for (int src = 0; src < 32; ++src) {
          const int olk = __shfl_sync(0xffffffffu, lk[u2], src);
          const int ont = __shfl_sync(0xffffffffu, nt[u2], src);
          const int ob = src + 32 * u2;
          #pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int bb = lane + 32 * u;
            const bool precedes = olk > lk[u] || (olk == lk[u] && ob < bb);
            start[u] += precedes ? ont : 0;
          }
        }
      }
    }
    #pragma unroll
    for (int u = 0; u < 4; ++u) {
      const bool mine = u < chunks && nt[u] > 0 && blk >= start[u] && blk < start[u] + nt[u];
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (m && found_b < 0) {
        const int src = __ffs(m) - 1;
        found_b = src + 32 * u;
        tile_in_seq = blk - __shfl_sync(0xffffffffu, start[u], src);
      }
    }
  } else {
  // Larger batches: the sequences are taken in four classes by key count (quarters of
  // max_seqlen_k = p.N, the caller's upper bound; 0 or a too small bound just puts everything
  // into the first class), each class in index order.
  const int t1 = (int)(((long long)p.N * 3) >> 2), t2 = p.N >> 1, t3 = p.N >> 2;
  for (int cls = 0; cls < 4 && found_b < 0; ++cls) {
    for (int b0 = 0; b0 < p.B && found_b < 0; b0 += 32) {
      const int bb = b0 + lane;
      int nt = 0;
      if (bb < p.B) {
        const int lk = p.cu_k[bb + 1] - p.cu_k[bb];
        const int c = lk > t1 ? 0 : (lk > t2 ? 1 : (lk > t3 ? 2 : 3));
        if (c == cls) nt = (p.cu_q[bb + 1] - p.cu_q[bb] + TILE_M - 1) / TILE_M;
      }
      int incl = nt;
      #pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      const int excl = acc + incl - nt;
      const bool mine = blk >= excl && blk < excl + nt;
      const unsigned m = __ballot_sync(0xffffffffu, mine);
      if (m) {
        const int src = __ffs(m) - 1;
        found_b = b0 + src;
        tile_in_seq = blk - __shfl_sync(0xffffffffu, excl, src);
      }
      acc += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  }
  TileWork w;
  w.b = -1; w.q_row0 = 0; w.rows_in_tile = 0; w.k_row0 = 0; w.len_k = 0; w.qpos0 = 0;
  if (found_b >= 0) {
    // (lengths cut at the tensors' row counts: a cu_seqlens that runs past a tensor must not turn into
    // an access past it)
    const int q0 = min(p.cu_q[found_b], p.total_q), q1 = min(p.cu_q[found_b + 1], p.total_q);
    const int k0 = min(p.cu_k[found_b], p.total_k), k1 = min(p.cu_k[found_b + 1], p.total_k);
    if ((q1 - q0) - tile_in_seq * TILE_M <= 0) return w;
    w.b = 0;
    w.q_row0 = q0 + tile_in_seq * TILE_M;
    w.rows_in_tile = min(TILE_M, (q1 - q0) - tile_in_seq * TILE_M);
    w.k_row0 = k0;
    w.len_k = k1 - k0;
    w.qpos0 = (k1 - k0) - (q1 - q0) + tile_in_seq * TILE_M;
  }
  return w;
}

template <int TILE_M>
__device__ __forceinline__ TileWork dense_tile(const AttnParams& p, int blk_x, int blk_z) {
  TileWork w;
  const int n_tiles = (p.M + TILE_M - 1) / TILE_M;
  const int t = n_tiles - 1 - blk_x;          // causal: longest rows first
  w.b = blk_z;
  w.q_row0 = t * TILE_M;
  w.rows_in_tile = min(TILE_M, p.M - w.q_row0);
  w.k_row0 = 0;
  w.len_k = p.N;
  w.qpos0 = p.q_pos_offset + w.q_row0;
  return w;
}
// Sequence and tile of block `blk` in the concatenated per-sequence tile lists of `cu`
// (ceil(len / tile) tiles each).  Called by one full warp; result valid in every lane.
__device__ __forceinline__ bool find_seq_tile(const int32_t* cu, int B, int tile, int blk, int& seq, int& tile_in_seq) {
  const int lane = threadIdx.x & 31;
  int acc = 0;
  for (int b0 = 0; b0 < B; b0 += 32) {
    const int bb = b0 + lane;
    int nt = 0;
    if (bb < B) nt = (cu[bb + 1] - cu[bb] + tile - 1) / tile;
    int incl = nt;
    #pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    const int excl = acc + incl - nt;
    const bool mine = blk >= excl && blk < excl + nt;
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (m) {
      const int src = __ffs(m) - 1;
      seq = b0 + src;
      tile_in_seq = blk - __shfl_sync(0xffffffffu, excl, src);
      return true;
    }
    acc += __shfl_sync(0xffffffffu, incl, 31);
  }
  return false;
}

// lse (natural log) -> log2 domain; rows that saw no key (-inf) or lie outside the tensor
// get +inf, so that their probabilities come out as exactly 0
__device__ __forceinline__ float lse_to_log2(float lse, bool valid) {
  return (valid && lse > -INFINITY) ? lse * kLog2e : INFINITY;
}

#endif

bool sm100_supports(const t5b_attn_args& a);
int sm100_attention_fwd(const t5b_attn_args& a, const BucketSpec& spec, cudaStream_t stream);
// two-tile kernel (head dim 64, more than 128 query rows): chosen inside sm100_attention_fwd / sm100_tail_plan
bool sm100w_prefers(const t5b_attn_args& a);
TailPlan sm100w_tail_plan(const t5b_attn_args& a);
int sm100w_attention_fwd(const t5b_attn_args& a, const BucketSpec& spec, cudaStream_t stream);
int simt_attention_fwd(const t5b_attn_args& a, const BucketSpec& spec, cudaStream_t stream);
bool sm100_bwd_supports(const t5b_attn_bwd_args& g);
int sm100_attention_bwd(const t5b_attn_bwd_args& g, const BucketSpec& spec, cudaStream_t stream);
int64_t sm100_bwd_workspace_bytes(const t5b_attn_bwd_args& g);
int simt_attention_bwd(const t5b_attn_bwd_args& g, const BucketSpec& spec, cudaStream_t stream);

}  // namespace t5b
