// CUDA-core forward kernel for the cases the tcgen05 kernel does not take:
// float32 inputs (all arithmetic in float32, for the 1e-4 parity bound) at head
// dims 16/32/64/128, and rows that are not 16-byte aligned.  Same semantics, same
// bias lookup, same packed-sequence scheduling; no throughput target.
//
// A block owns 32 query rows; four threads share a row, each holding a quarter
// of q and of the output accumulator in registers.  K/V tiles are staged in
// shared memory as float32.
#include "t5b_common.cuh"
#include "attn_params.cuh"

namespace t5b {
namespace simt {

constexpr int TM = 32;          // query rows per block
constexpr int THREADS = 128;
constexpr int TILE_FLOATS = 4096;   // K tile and V tile: 16 KB each
constexpr int KG = 8;           // keys handled per inner step

template <typename T, int D>
__global__ void __launch_bounds__(THREADS)
attn_fwd_simt_kernel(const __grid_constant__ AttnParams p, const __grid_constant__ BucketSpec spec) {
  constexpr int TN = TILE_FLOATS / D;     // keys per tile
  constexpr int DP = D / 4;               // floats per thread
  constexpr int NV = DP / 4;              // float4 per thread
  extern __shared__ float smem_f[];
  float* sK = smem_f;
  float* sV = smem_f + TILE_FLOATS;
  float* lut = smem_f + 2 * TILE_FLOATS;
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
  if (has_bias) {
    for (int i = tid; i < 2 * md + 1; i += THREADS) {
      const int bucket = bucket_of_delta(spec, i - md);
      lut[i] = load_table(p.table, p.table_dtype, (int64_t)bucket * p.table_stride0 + h) * kLog2e;
    }
  }

  const int r = tid >> 2, part = tid & 3;
  const bool row_ok = r < w.rows_in_tile;
  const int qpos = w.qpos0 + r;
  const T* qptr = (const T*)p.q + (int64_t)w.b * p.q_stride_b + (int64_t)h * p.q_stride_h +
                  (int64_t)(w.q_row0 + r) * p.q_stride_m;
  // thread `part` holds float4 groups part, part+4, ... of the row
  float q[DP], o[DP];
  #pragma unroll
  for (int g = 0; g < NV; ++g)
    #pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int d = (g * 4 + part) * 4 + e;
      q[g * 4 + e] = row_ok ? to_float<T>(qptr[d]) * p.scale_log2 : 0.f;
      o[g * 4 + e] = 0.f;
    }
  float m_run = -INFINITY, l_run = 0.f;

  int kv_end = w.len_k;
  if (p.causal) kv_end = min(w.len_k, w.qpos0 + w.rows_in_tile);
  const int n_valid = p.causal ? min(w.len_k, qpos + 1) : w.len_k;
  const T* kbase = (const T*)p.k + (int64_t)w.b * p.k_stride_b + (int64_t)h * p.k_stride_h;
  const T* vbase = (const T*)p.v + (int64_t)w.b * p.v_stride_b + (int64_t)h * p.v_stride_h;

  for (int n0 = 0; n0 < kv_end; n0 += TN) {
    __syncthreads();
    for (int i = tid; i < TN * D; i += THREADS) {
      const int n = i / D, d = i % D;
      float kv = 0.f, vv = 0.f;
      if (n0 + n < w.len_k) {
        kv = to_float<T>(kbase[(int64_t)(w.k_row0 + n0 + n) * p.k_stride_n + d]);
        vv = to_float<T>(vbase[(int64_t)(w.k_row0 + n0 + n) * p.v_stride_n + d]);
      }
      sK[i] = kv;
      sV[i] = vv;
    }
    __syncthreads();
    const int tile_n = min(TN, kv_end - n0);
    for (int g0 = 0; g0 < tile_n; g0 += KG) {
      float s[KG];
      #pragma unroll
      for (int kk = 0; kk < KG; ++kk) {
        const float4* kr = reinterpret_cast<const float4*>(sK + (g0 + kk) * D);
        float acc = 0.f;
        #pragma unroll
        for (int g = 0; g < NV; ++g) {
          const float4 kv = kr[g * 4 + part];
          acc = fmaf(q[g * 4 + 0], kv.x, acc);
          acc = fmaf(q[g * 4 + 1], kv.y, acc);
          acc = fmaf(q[g * 4 + 2], kv.z, acc);
          acc = fmaf(q[g * 4 + 3], kv.w, acc);
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        const int n = n0 + g0 + kk;
        if (has_bias) acc += lut[min(max(n - qpos + md, 0), 2 * md)];
        if (n >= n_valid || g0 + kk >= tile_n) acc = -INFINITY;
        s[kk] = acc;
      }
      float mx = s[0];
      #pragma unroll
      for (int kk = 1; kk < KG; ++kk) mx = fmaxf(mx, s[kk]);
      const float m_new = fmaxf(m_run, mx);
      if (m_new == -INFINITY) continue;      // nothing visible yet for this row
      const float alpha = exp2f(m_run - m_new);
      l_run *= alpha;
      #pragma unroll
      for (int e = 0; e < DP; ++e) o[e] *= alpha;
      m_run = m_new;
      #pragma unroll
      for (int kk = 0; kk < KG; ++kk) {
        const float pr = exp2f(s[kk] - m_new);
        l_run += pr;
        const float4* vr = reinterpret_cast<const float4*>(sV + (g0 + kk) * D);
        #pragma unroll
        for (int g = 0; g < NV; ++g) {
          const float4 vv = vr[g * 4 + part];
          o[g * 4 + 0] = fmaf(pr, vv.x, o[g * 4 + 0]);
          o[g * 4 + 1] = fmaf(pr, vv.y, o[g * 4 + 1]);
          o[g * 4 + 2] = fmaf(pr, vv.z, o[g * 4 + 2]);
          o[g * 4 + 3] = fmaf(pr, vv.w, o[g * 4 + 3]);
        }
      }
    }
  }

  if (row_ok) {
    const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
    T* optr = (T*)p.out + (int64_t)w.b * p.o_stride_b + (int64_t)h * p.o_stride_h +
              (int64_t)(w.q_row0 + r) * p.o_stride_m;
    #pragma unroll
    for (int g = 0; g < NV; ++g)
      #pragma unroll
      for (int e = 0; e < 4; ++e)
        optr[(g * 4 + part) * 4 + e] = from_float<T>(o[g * 4 + e] * inv_l);
    if (p.lse != nullptr && part == 0) {
      const float lse = l_run > 0.f ? (m_run + log2f(l_run)) * kLn2 : -INFINITY;
      const int64_t row = (int64_t)w.q_row0 + r;
      if (p.cu_q == nullptr) p.lse[((int64_t)blockIdx.z * p.H + h) * p.M + row] = lse;
      else p.lse[row * p.H + h] = lse;
    }
  }
}

template <typename T>
static int launch_for_type(const t5b_attn_args& a, const AttnParams& p, const BucketSpec& spec,
                           dim3 grid, size_t smem, cudaStream_t stream) {
  auto go = [&](auto kern) -> int {
    if (smem > 48 * 1024) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return T5B_ERR_LAUNCH;
      }
    }
    kern<<<grid, THREADS, smem, stream>>>(p, spec);
    return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
  };
  switch (a.D) {
    case 16: return go(attn_fwd_simt_kernel<T, 16>);
    case 32: return go(attn_fwd_simt_kernel<T, 32>);
    case 64: return go(attn_fwd_simt_kernel<T, 64>);
    case 128: return go(attn_fwd_simt_kernel<T, 128>);
  }
  return T5B_ERR_HEAD_DIM;
}

}  // namespace simt

int simt_attention_fwd(const t5b_attn_args& a, const BucketSpec& spec, cudaStream_t stream) {
  using namespace simt;
  if (a.table && spec.max_distance > 2048) return T5B_ERR_UNSUPPORTED;
  const bool varlen = a.cu_seqlens_q != nullptr;
  AttnParams p = make_attn_params(a);
  dim3 grid;
  if (varlen) grid = dim3((unsigned)((long long)a.total_q / TM + a.B), (unsigned)a.H, 1);
  else grid = dim3((unsigned)((a.M + TM - 1) / TM), (unsigned)a.H, (unsigned)a.B);
  if (grid.y > 65535 || grid.z > 65535) return T5B_ERR_SHAPE;
  const size_t smem = (2 * TILE_FLOATS + (a.table ? 2 * spec.max_distance + 1 : 0)) * sizeof(float);
  switch (a.dtype) {
    case T5B_F32: return launch_for_type<float>(a, p, spec, grid, smem, stream);
    case T5B_F16: return launch_for_type<__half>(a, p, spec, grid, smem, stream);
    case T5B_BF16: return launch_for_type<__nv_bfloat16>(a, p, spec, grid, smem, stream);
  }
  return T5B_ERR_DTYPE;
}

}  // namespace t5b
