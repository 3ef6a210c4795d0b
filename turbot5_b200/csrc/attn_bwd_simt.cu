// CUDA-core backward of the fused-bias attention for what the tensor-core backward does not
// take: float32 tensors (all arithmetic in float32) and 16-bit rows that are not
// 16-byte aligned.  Same three steps and the same ownership as attn_bwd_sm100.cu (delta; one
// block per 32 query rows for dQ and the bias-table gradient; one block per 32 keys for dK and
// dV; nothing but the small table gradient is accumulated with atomics); same semantics as
// flash_attn_v2_bwd_bias (src/turbot5/ops/fused_bias_attention.py:62-147).  No throughput target.
#include "t5b_common.cuh"
#include "attn_params.cuh"

namespace t5b {
namespace simtb {

constexpr int TM = 32;              // rows per block (query rows | keys)
constexpr int THREADS = 128;        // four threads per row
constexpr int TILE_FLOATS = 4096;   // each streamed tile: 16 KB of float32
constexpr int MAX_BUCKETS = 2 * kMaxBucketsPerSide;

struct Extra {
  const void* dout;
  int64_t do_stride_b, do_stride_h, do_stride_m;
  void* dq; void* dk; void* dv;
  float* dtable;
  float* delta;
  float sm_scale;
};

template <typename T>
__global__ void delta_kernel(const AttnParams p, const Extra e, long long n_rows) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long n_warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long i = warp0; i < n_rows; i += n_warps) {
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
    const T* o = reinterpret_cast<const T*>(p.out) + o_off;
    const T* d = reinterpret_cast<const T*>(e.dout) + do_off;
    float s = 0.f;
    for (int c = lane; c < p.D; c += 32) s = fmaf(to_float(o[c]), to_float(d[c]), s);
    #pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (lane == 0) e.delta[i] = s;
  }
}

// thread `part` of a row holds float4 groups part, part+4, ... of a D-vector
template <typename T, int D>
__device__ __forceinline__ void load_row(float (&dst)[D / 4], const T* src, int part, bool ok) {
  #pragma unroll
  for (int g = 0; g < D / 16; ++g)
    #pragma unroll
    for (int c = 0; c < 4; ++c) dst[g * 4 + c] = ok ? to_float<T>(src[(g * 4 + part) * 4 + c]) : 0.f;
}
template <typename T, int D>
__device__ __forceinline__ void store_row(T* dst, const float (&src)[D / 4], int part, float scale) {
  #pragma unroll
  for (int g = 0; g < D / 16; ++g)
    #pragma unroll
    for (int c = 0; c < 4; ++c) dst[(g * 4 + part) * 4 + c] = from_float<T>(src[g * 4 + c] * scale);
}
template <int D>
__device__ __forceinline__ float dot_part(const float (&a)[D / 4], const float* row, int part) {
  const float4* r4 = reinterpret_cast<const float4*>(row);
  float acc = 0.f;
  #pragma unroll
  for (int g = 0; g < D / 16; ++g) {
    const float4 x = r4[g * 4 + part];
    acc = fmaf(a[g * 4 + 0], x.x, acc); acc = fmaf(a[g * 4 + 1], x.y, acc);
    acc = fmaf(a[g * 4 + 2], x.z, acc); acc = fmaf(a[g * 4 + 3], x.w, acc);
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  return acc;
}
template <int D>
__device__ __forceinline__ void axpy_part(float (&acc)[D / 4], float a, const float* row, int part) {
  const float4* r4 = reinterpret_cast<const float4*>(row);
  #pragma unroll
  for (int g = 0; g < D / 16; ++g) {
    const float4 x = r4[g * 4 + part];
    acc[g * 4 + 0] = fmaf(a, x.x, acc[g * 4 + 0]); acc[g * 4 + 1] = fmaf(a, x.y, acc[g * 4 + 1]);
    acc[g * 4 + 2] = fmaf(a, x.z, acc[g * 4 + 2]); acc[g * 4 + 3] = fmaf(a, x.w, acc[g * 4 + 3]);
  }
}

// Stage rows [row0, row0 + n) of a (rows, D) strided matrix as float32, zero beyond `limit`.
template <typename T, int D>
__device__ __forceinline__ void stage_tile(float* dst, const T* base, int64_t row_stride, int64_t row0, int n,
                                           int64_t limit) {
  for (int i = threadIdx.x; i < n * D; i += THREADS) {
    const int r = i / D, d = i % D;
    dst[i] = (row0 + r < limit) ? to_float<T>(base[(row0 + r) * row_stride + d]) : 0.f;
  }
}

// ---------------------------------------------------------------- dQ and the table gradient
template <typename T, int D>
__global__ void __launch_bounds__(THREADS)
dq_kernel(const __grid_constant__ AttnParams p, const __grid_constant__ Extra e, const __grid_constant__ BucketSpec spec) {
  constexpr int TN = TILE_FLOATS / D;
  extern __shared__ float smem_f[];
  float* sK = smem_f;
  float* sV = smem_f + TILE_FLOATS;
  float* hist = smem_f + 2 * TILE_FLOATS;          // [MAX_BUCKETS]
  float* lut = hist + MAX_BUCKETS;                 // [2 md + 1]
  __shared__ TileWork shared_work;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.y;
  TileWork w;
  if (p.cu_q == nullptr) {
    w = dense_tile<TM>(p, (int)blockIdx.x, (int)blockIdx.z);
  } else {
    if (warp == 0) {
      TileWork f = find_varlen_tile<TM>(p, (int)blockIdx.x);
      if (lane == 0) shared_work = f;
    }
    __syncthreads();
    w = shared_work;
    if (w.b < 0) return;
  }
  const int md = spec.max_distance;
  const bool has_bias = p.table != nullptr;
  int16_t* lutb = reinterpret_cast<int16_t*>(lut + 2 * md + 1);
  if (has_bias) {
    for (int i = tid; i < 2 * md + 1; i += THREADS) {
      const int bucket = bucket_of_delta(spec, i - md);
      lut[i] = load_table(p.table, p.table_dtype, (int64_t)bucket * p.table_stride0 + h) * kLog2e;
      lutb[i] = (int16_t)bucket;
    }
    for (int i = tid; i < MAX_BUCKETS; i += THREADS) hist[i] = 0.f;
  }
  const int r = tid >> 2, part = tid & 3;
  const bool row_ok = r < w.rows_in_tile;
  const int qpos = w.qpos0 + r;
  const int64_t row = (int64_t)w.q_row0 + r;
  const int64_t stat = p.cu_q == nullptr ? ((int64_t)blockIdx.z * p.H + h) * p.M + row : row * p.H + h;
  float q[D / 4], go[D / 4], dq[D / 4];
  load_row<T, D>(q, (const T*)p.q + (int64_t)w.b * p.q_stride_b + (int64_t)h * p.q_stride_h + row * p.q_stride_m, part, row_ok);
  load_row<T, D>(go, (const T*)e.dout + (int64_t)w.b * e.do_stride_b + (int64_t)h * e.do_stride_h + row * e.do_stride_m, part, row_ok);
  #pragma unroll
  for (int i = 0; i < D / 4; ++i) dq[i] = 0.f;
  const float lse2 = lse_to_log2(row_ok ? p.lse[stat] : 0.f, row_ok);
  const float delta_r = row_ok ? e.delta[stat] : 0.f;

  int kv_end = w.len_k;
  if (p.causal) kv_end = min(w.len_k, w.qpos0 + w.rows_in_tile);
  const int n_valid = p.causal ? min(w.len_k, qpos + 1) : w.len_k;
  const T* kbase = (const T*)p.k + (int64_t)w.b * p.k_stride_b + (int64_t)h * p.k_stride_h;
  const T* vbase = (const T*)p.v + (int64_t)w.b * p.v_stride_b + (int64_t)h * p.v_stride_h;
  for (int n0 = 0; n0 < kv_end; n0 += TN) {
    __syncthreads();
    stage_tile<T, D>(sK, kbase, p.k_stride_n, (int64_t)w.k_row0 + n0, TN, (int64_t)w.k_row0 + w.len_k);
    stage_tile<T, D>(sV, vbase, p.v_stride_n, (int64_t)w.k_row0 + n0, TN, (int64_t)w.k_row0 + w.len_k);
    __syncthreads();
    const int tile_n = min(TN, kv_end - n0);
    for (int kk = 0; kk < tile_n; ++kk) {
      const int n = n0 + kk;
      float x = dot_part<D>(q, sK + kk * D, part) * p.scale_log2;
      const float dp = dot_part<D>(go, sV + kk * D, part);
      const int li = min(max(n - qpos + md, 0), 2 * md);
      if (has_bias) x += lut[li];
      const float pr = (n < n_valid) ? exp2f(x - lse2) : 0.f;
      const float ds = pr * (dp - delta_r);
      axpy_part<D>(dq, ds, sK + kk * D, part);
      if (has_bias && part == 0 && ds != 0.f) atomicAdd(&hist[lutb[li]], ds);
    }
  }
  if (row_ok)
    store_row<T, D>((T*)e.dq + (int64_t)w.b * p.q_stride_b + (int64_t)h * p.q_stride_h + row * p.q_stride_m, dq, part, e.sm_scale);
  __syncthreads();
  if (has_bias && e.dtable != nullptr) {
    const int nb = spec.bidirectional ? 2 * spec.n_side : spec.n_side;
    for (int i = tid; i < nb; i += THREADS) {
      const float g = hist[i];
      if (g != 0.f) atomicAdd(&e.dtable[(int64_t)i * p.H + h], g);
    }
  }
}

// ---------------------------------------------------------------- dK and dV
template <typename T, int D>
__global__ void __launch_bounds__(THREADS)
dkv_kernel(const __grid_constant__ AttnParams p, const __grid_constant__ Extra e, const __grid_constant__ BucketSpec spec) {
  constexpr int TN = TILE_FLOATS / D;      // queries per streamed tile
  extern __shared__ float smem_f[];
  float* sQ = smem_f;
  float* sG = smem_f + TILE_FLOATS;
  float* sL = smem_f + 2 * TILE_FLOATS;    // [TN] lse (log2 domain)
  float* sD = sL + 256;                    // [TN] delta   (TN <= 256)
  float* lut = sD + 256;
  __shared__ int shared_seq[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int h = blockIdx.y;
  int b = 0, key0, k_row0 = 0, len_k, q_row0 = 0, len_q, q_off;
  if (p.cu_k == nullptr) {
    b = blockIdx.z;
    key0 = (int)blockIdx.x * TM;
    len_k = p.N; len_q = p.M; q_off = p.q_pos_offset;
  } else {
    if (warp == 0) {
      int seq = -1, t = 0;
      const bool found = find_seq_tile(p.cu_k, p.B, TM, (int)blockIdx.x, seq, t);
      if (lane == 0) { shared_seq[0] = found ? seq : -1; shared_seq[1] = t; }
    }
    __syncthreads();
    const int seq = shared_seq[0];
    if (seq < 0) return;
    key0 = shared_seq[1] * TM;
    k_row0 = min(p.cu_k[seq], p.total_k); len_k = min(p.cu_k[seq + 1], p.total_k) - k_row0;
    q_row0 = min(p.cu_q[seq], p.total_q); len_q = min(p.cu_q[seq + 1], p.total_q) - q_row0;
    q_off = len_k - len_q;
  }
  const int md = spec.max_distance;
  const bool has_bias = p.table != nullptr;
  if (has_bias) {
    for (int i = tid; i < 2 * md + 1; i += THREADS) {
      const int bucket = bucket_of_delta(spec, i - md);
      lut[i] = load_table(p.table, p.table_dtype, (int64_t)bucket * p.table_stride0 + h) * kLog2e;
    }
  }
  const int r = tid >> 2, part = tid & 3;
  const int key = key0 + r;
  const bool key_ok = key < len_k;
  const int64_t krow = (int64_t)k_row0 + key;
  float kx[D / 4], vx[D / 4], dk[D / 4], dv[D / 4];
  load_row<T, D>(kx, (const T*)p.k + (int64_t)b * p.k_stride_b + (int64_t)h * p.k_stride_h + krow * p.k_stride_n, part, key_ok);
  load_row<T, D>(vx, (const T*)p.v + (int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h + krow * p.v_stride_n, part, key_ok);
  #pragma unroll
  for (int i = 0; i < D / 4; ++i) { dk[i] = 0.f; dv[i] = 0.f; }

  int m_first = 0;
  if (p.causal) m_first = max(0, key0 - q_off);      // earlier queries see no key of this tile
  const T* qbase = (const T*)p.q + (int64_t)b * p.q_stride_b + (int64_t)h * p.q_stride_h;
  const T* gbase = (const T*)e.dout + (int64_t)b * e.do_stride_b + (int64_t)h * e.do_stride_h;
  for (int m0 = m_first; m0 < len_q; m0 += TN) {
    __syncthreads();
    stage_tile<T, D>(sQ, qbase, p.q_stride_m, (int64_t)q_row0 + m0, TN, (int64_t)q_row0 + len_q);
    stage_tile<T, D>(sG, gbase, e.do_stride_m, (int64_t)q_row0 + m0, TN, (int64_t)q_row0 + len_q);
    for (int i = tid; i < TN; i += THREADS) {
      const int m = m0 + i;
      const bool valid = m < len_q;
      const int64_t idx = p.cu_q == nullptr ? ((int64_t)b * p.H + h) * p.M + m : ((int64_t)q_row0 + m) * p.H + h;
      sL[i] = lse_to_log2(valid ? p.lse[idx] : 0.f, valid);
      sD[i] = valid ? e.delta[idx] : 0.f;
    }
    __syncthreads();
    const int tile_m = min(TN, len_q - m0);
    for (int mm = 0; mm < tile_m; ++mm) {
      const int qpos = q_off + m0 + mm;
      float x = dot_part<D>(kx, sQ + mm * D, part) * p.scale_log2;
      const float dp = dot_part<D>(vx, sG + mm * D, part);
      if (has_bias) x += lut[min(max(key - qpos + md, 0), 2 * md)];
      const bool visible = key_ok && !(p.causal && key > qpos);
      const float pr = visible ? exp2f(x - sL[mm]) : 0.f;
      const float ds = pr * (dp - sD[mm]);
      axpy_part<D>(dv, pr, sG + mm * D, part);
      axpy_part<D>(dk, ds, sQ + mm * D, part);
    }
  }
  if (key_ok) {
    store_row<T, D>((T*)e.dv + (int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h + krow * p.v_stride_n, dv, part, 1.f);
    store_row<T, D>((T*)e.dk + (int64_t)b * p.k_stride_b + (int64_t)h * p.k_stride_h + krow * p.k_stride_n, dk, part, e.sm_scale);
  }
}

template <typename T, int D>
static int launch_d(const t5b_attn_args& a, const AttnParams& p, const Extra& e, const BucketSpec& spec, cudaStream_t st) {
  const bool varlen = a.cu_seqlens_q != nullptr;
  const int lut_n = a.table ? 2 * spec.max_distance + 1 : 0;
  const size_t smem_q = (2 * TILE_FLOATS + MAX_BUCKETS + lut_n) * sizeof(float) + (size_t)lut_n * 2 + 16;
  const size_t smem_k = (2 * TILE_FLOATS + 512 + lut_n) * sizeof(float);
  auto kq = dq_kernel<T, D>;
  auto kk = dkv_kernel<T, D>;
  if (cudaFuncSetAttribute(kq, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q) != cudaSuccess ||
      cudaFuncSetAttribute(kk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_k) != cudaSuccess) {
    cudaGetLastError();
    return T5B_ERR_LAUNCH;
  }
  dim3 gq, gk;
  if (varlen) {
    gq = dim3((unsigned)((long long)a.total_q / TM + a.B), (unsigned)a.H, 1);
    gk = dim3((unsigned)((long long)a.total_k / TM + a.B), (unsigned)a.H, 1);
  } else {
    gq = dim3((unsigned)((a.M + TM - 1) / TM), (unsigned)a.H, (unsigned)a.B);
    gk = dim3((unsigned)((a.N + TM - 1) / TM), (unsigned)a.H, (unsigned)a.B);
  }
  if (gq.y > 65535 || gq.z > 65535) return T5B_ERR_SHAPE;
  if (gq.x > 0) {
    kq<<<gq, THREADS, smem_q, st>>>(p, e, spec);
    if (cudaGetLastError() != cudaSuccess) return T5B_ERR_LAUNCH;
  }
  if (gk.x > 0) {
    kk<<<gk, THREADS, smem_k, st>>>(p, e, spec);
    if (cudaGetLastError() != cudaSuccess) return T5B_ERR_LAUNCH;
  }
  return T5B_OK;
}

template <typename T>
static int launch_t(const t5b_attn_args& a, const AttnParams& p, const Extra& e, const BucketSpec& spec, cudaStream_t st) {
  const long long n_rows = (a.cu_seqlens_q ? (long long)a.total_q : (long long)a.B * a.M) * a.H;
  long long blocks = (n_rows + 7) / 8;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (blocks > 0) {
    delta_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(p, e, n_rows);
    if (cudaGetLastError() != cudaSuccess) return T5B_ERR_LAUNCH;
  }
  switch (a.D) {
    case 16: return launch_d<T, 16>(a, p, e, spec, st);
    case 32: return launch_d<T, 32>(a, p, e, spec, st);
    case 64: return launch_d<T, 64>(a, p, e, spec, st);
    case 128: return launch_d<T, 128>(a, p, e, spec, st);
  }
  return T5B_ERR_HEAD_DIM;
}

}  // namespace simtb

int simt_attention_bwd(const t5b_attn_bwd_args& g, const BucketSpec& spec, cudaStream_t stream) {
  using namespace simtb;
  const t5b_attn_args& a = g.fwd;
  if (a.table && spec.max_distance > 2048) return T5B_ERR_UNSUPPORTED;
  AttnParams p = make_attn_params(a);
  Extra e;
  e.dout = g.dout;
  e.do_stride_b = g.do_stride_b; e.do_stride_h = g.do_stride_h; e.do_stride_m = g.do_stride_m;
  e.dq = g.dq; e.dk = g.dk; e.dv = g.dv;
  e.dtable = g.dtable; e.delta = g.delta; e.sm_scale = a.sm_scale;
  switch (a.dtype) {
    case T5B_F32: return launch_t<float>(a, p, e, spec, stream);
    case T5B_F16: return launch_t<__half>(a, p, e, spec, stream);
    case T5B_BF16: return launch_t<__nv_bfloat16>(a, p, e, spec, stream);
  }
  return T5B_ERR_DTYPE;
}

}  // namespace t5b
