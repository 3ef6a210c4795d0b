// Split-KV flash decoding: a handful of query rows per (batch, head) against a
// long key/value cache.  The op is a batch of matrix-vector products, bound by
// HBM bandwidth (about one flop per byte), so it runs on the CUDA cores with
// 16-byte streaming loads and no tensor cores.
//
//   grid = (splits, H, B); a block streams its slice of the keys; a group of
//   D*sizeof(T)/16 lanes owns one key (one 16-byte piece of the row per lane),
//   so a warp load covers whole rows back to back.  Each lane group keeps its own
//   online-softmax state; groups, warps and finally splits are merged with the
//   usual (max, sum, weighted accumulator) rule.  The last block of a (batch,
//   head) to finish merges the splits (no second launch).
//
// Semantics: the cached decode step of T5Attention.forward
// (src/turbot5/model/attentions.py:198,229-234) and the split/merge rule of
// src/turbot5/ops/flash_decoding.py:47-55; bias from the [buckets, H] table with
// delta = n - (kv_len - M + m), unidirectional when causal.
#include "t5b_common.cuh"

namespace t5b {
namespace decode {

constexpr int WARPS = 8;
constexpr int THREADS = WARPS * 32;
constexpr int UNROLL = 4;

struct Params {
  const void* q; const void* k; const void* v; void* out;
  const void* table; const int32_t* seqlens_k;
  int32_t* counters; float* part_ml; float* part_o;
  int64_t q_stride_b, q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_h, k_stride_n;
  int64_t v_stride_b, v_stride_h, v_stride_n;
  int64_t o_stride_b, o_stride_h, o_stride_m;
  int64_t table_stride0;
  int32_t table_dtype;
  int32_t B, H, M, N;
  int32_t causal, q_pos_offset, splits, m0;   // m0: first query row handled by this launch
  float scale_log2;
};

template <typename T> struct Vec16;
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__half> { static constexpr int N = 8; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

template <typename T> __device__ __forceinline__ void unpack16(const uint4& u, float* f);
template <> __device__ __forceinline__ void unpack16<float>(const uint4& u, float* f) {
  f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
  f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
}
template <> __device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  #pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void unpack16<__half>(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  #pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    f[2 * i] = t.x; f[2 * i + 1] = t.y;
  }
}

// MQ query rows per block (1 for plain decoding, 4 for short multi-token steps)
template <typename T, int D, int MQ>
__global__ void __launch_bounds__(THREADS)
decode_kernel(const __grid_constant__ Params p, const __grid_constant__ BucketSpec spec) {
  constexpr int VEC = Vec16<T>::N;
  constexpr int LPK = D / VEC;            // lanes per key
  constexpr int KPW = 32 / LPK;           // keys per warp load
  constexpr int KPI = KPW * UNROLL;       // keys per warp iteration
  static_assert(LPK >= 1 && LPK <= 32, "head dim / element size not supported");

  extern __shared__ float lut[];
  __shared__ float sm_m[WARPS][MQ], sm_l[WARPS][MQ];
  __shared__ float sm_o[WARPS][MQ][D];
  __shared__ int is_last;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int grp = lane / LPK, gl = lane % LPK;
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int kv_len = p.seqlens_k ? min(p.seqlens_k[b], p.N) : p.N;
  const int qoff = p.q_pos_offset >= 0 ? p.q_pos_offset : kv_len - p.M;
  const int md = spec.max_distance;
  const bool has_bias = p.table != nullptr;
  if (has_bias) {
    for (int i = tid; i < 2 * md + 1; i += THREADS) {
      const int bucket = bucket_of_delta(spec, i - md);
      lut[i] = load_table(p.table, p.table_dtype, (int64_t)bucket * p.table_stride0 + h) * kLog2e;
    }
    __syncthreads();
  }

  // slice of keys for this split (multiples of 128 so warps stay aligned)
  int chunk = (kv_len + p.splits - 1) / p.splits;
  chunk = (chunk + 127) / 128 * 128;
  const int n_begin = min(split * chunk, kv_len);
  const int n_end = min(n_begin + chunk, kv_len);

  // query slices (pre-scaled into the log2 domain)
  float q[MQ][VEC];
  #pragma unroll
  for (int m = 0; m < MQ; ++m) {
    const int row = p.m0 + m;
    #pragma unroll
    for (int e = 0; e < VEC; ++e) q[m][e] = 0.f;
    if (row < p.M) {
      const T* qp = (const T*)p.q + (int64_t)b * p.q_stride_b + (int64_t)h * p.q_stride_h +
                    (int64_t)row * p.q_stride_m + gl * VEC;
      #pragma unroll
      for (int e = 0; e < VEC; ++e) q[m][e] = to_float<T>(qp[e]) * p.scale_log2;
    }
  }
  float acc[MQ][VEC], m_run[MQ], l_run[MQ];
  #pragma unroll
  for (int m = 0; m < MQ; ++m) {
    m_run[m] = -INFINITY; l_run[m] = 0.f;
    #pragma unroll
    for (int e = 0; e < VEC; ++e) acc[m][e] = 0.f;
  }

  const char* kbase = (const char*)p.k + sizeof(T) * ((int64_t)b * p.k_stride_b + (int64_t)h * p.k_stride_h + gl * VEC);
  const char* vbase = (const char*)p.v + sizeof(T) * ((int64_t)b * p.v_stride_b + (int64_t)h * p.v_stride_h + gl * VEC);
  const int64_t kstep = (int64_t)sizeof(T) * p.k_stride_n, vstep = (int64_t)sizeof(T) * p.v_stride_n;

  for (int it = n_begin + warp * KPI; it < n_end; it += WARPS * KPI) {
    uint4 kr[UNROLL], vr[UNROLL];
    #pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int n = it + u * KPW + grp;
      kr[u] = make_uint4(0, 0, 0, 0); vr[u] = make_uint4(0, 0, 0, 0);
      if (n < n_end) {
        kr[u] = ld_stream(kbase + n * kstep);
        vr[u] = ld_stream(vbase + n * vstep);
      }
    }
    float s[MQ][UNROLL];
    #pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float kf[VEC];
      unpack16<T>(kr[u], kf);
      const int n = it + u * KPW + grp;
      #pragma unroll
      for (int m = 0; m < MQ; ++m) {
        float d = 0.f;
        #pragma unroll
        for (int e = 0; e < VEC; ++e) d = fmaf(q[m][e], kf[e], d);
        #pragma unroll
        for (int o = 1; o < LPK; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        const int qpos = qoff + p.m0 + m;
        if (has_bias) d += lut[min(max(n - qpos + md, 0), 2 * md)];
        const bool visible = n < n_end && (!p.causal || n <= qpos);
        s[m][u] = visible ? d : -INFINITY;
      }
    }
    #pragma unroll
    for (int m = 0; m < MQ; ++m) {
      float mx = s[m][0];
      #pragma unroll
      for (int u = 1; u < UNROLL; ++u) mx = fmaxf(mx, s[m][u]);
      const float m_new = fmaxf(m_run[m], mx);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = fast_exp2(m_run[m] - m_safe);
      m_run[m] = m_new;
      l_run[m] *= alpha;
      #pragma unroll
      for (int e = 0; e < VEC; ++e) acc[m][e] *= alpha;
      #pragma unroll
      for (int u = 0; u < UNROLL; ++u) s[m][u] = fast_exp2(s[m][u] - m_safe);
    }
    #pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float vf[VEC];
      unpack16<T>(vr[u], vf);
      #pragma unroll
      for (int m = 0; m < MQ; ++m) {
        l_run[m] += s[m][u];
        #pragma unroll
        for (int e = 0; e < VEC; ++e) acc[m][e] = fmaf(s[m][u], vf[e], acc[m][e]);
      }
    }
  }

  // ---- merge lane groups inside the warp
  #pragma unroll
  for (int m = 0; m < MQ; ++m) {
    #pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m_run[m], o);
      const float l_o = __shfl_xor_sync(0xffffffffu, l_run[m], o);
      const float m_new = fmaxf(m_run[m], m_o);
      const float m_safe = m_new == -INFINITY ? 0.f : m_new;
      const float a = fast_exp2(m_run[m] - m_safe), bsc = fast_exp2(m_o - m_safe);
      l_run[m] = l_run[m] * a + l_o * bsc;
      #pragma unroll
      for (int e = 0; e < VEC; ++e) {
        const float o_o = __shfl_xor_sync(0xffffffffu, acc[m][e], o);
        acc[m][e] = acc[m][e] * a + o_o * bsc;
      }
      m_run[m] = m_new;
    }
    if (grp == 0) {
      #pragma unroll
      for (int e = 0; e < VEC; ++e) sm_o[warp][m][gl * VEC + e] = acc[m][e];
      if (gl == 0) { sm_m[warp][m] = m_run[m]; sm_l[warp][m] = l_run[m]; }
    }
  }
  __syncthreads();

  // ---- merge warps: thread (m, d) over MQ*D outputs
  const int64_t bh = (int64_t)b * p.H + h;
  for (int idx = tid; idx < MQ * D; idx += THREADS) {
    const int m = idx / D, d = idx % D;
    const int row = p.m0 + m;
    float mm = -INFINITY;
    #pragma unroll
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, sm_m[w][m]);
    const float m_safe = mm == -INFINITY ? 0.f : mm;
    float l = 0.f, o = 0.f;
    #pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float sc = fast_exp2(sm_m[w][m] - m_safe);
      l += sm_l[w][m] * sc;
      o += sm_o[w][m][d] * sc;
    }
    if (row < p.M) {
      if (p.splits == 1) {
        T* op = (T*)p.out + (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + (int64_t)row * p.o_stride_m;
        op[d] = from_float<T>(l > 0.f ? o / l : 0.f);
      } else {
        const int64_t slot = (bh * p.splits + split) * p.M + row;
        p.part_o[slot * D + d] = o;
        if (d == 0) { p.part_ml[2 * slot] = mm; p.part_ml[2 * slot + 1] = l; }
      }
    }
  }
  if (p.splits == 1) return;

  // ---- the last block of this (batch, head) merges the splits
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int done = atomicAdd(&p.counters[bh], 1);
    is_last = (done == p.splits - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = tid; idx < MQ * D; idx += THREADS) {
    const int m = idx / D, d = idx % D;
    const int row = p.m0 + m;
    if (row >= p.M) continue;
    float mm = -INFINITY;
    for (int s2 = 0; s2 < p.splits; ++s2)
      mm = fmaxf(mm, __ldcg(&p.part_ml[2 * ((bh * p.splits + s2) * p.M + row)]));
    const float m_safe = mm == -INFINITY ? 0.f : mm;
    float l = 0.f, o = 0.f;
    for (int s2 = 0; s2 < p.splits; ++s2) {
      const int64_t slot = (bh * p.splits + s2) * p.M + row;
      const float sc = fast_exp2(__ldcg(&p.part_ml[2 * slot]) - m_safe);
      l += __ldcg(&p.part_ml[2 * slot + 1]) * sc;
      o += __ldcg(&p.part_o[slot * D + d]) * sc;
    }
    T* op = (T*)p.out + (int64_t)b * p.o_stride_b + (int64_t)h * p.o_stride_h + (int64_t)row * p.o_stride_m;
    op[d] = from_float<T>(l > 0.f ? o / l : 0.f);
  }
  __syncthreads();
  // all row-chunks (launches with different m0) share the counter: reset it only
  // after this launch's merge so the buffer is ready for the next call
  if (tid == 0) p.counters[bh] = 0;
}

template <typename T, int D>
static int launch_rows(Params p, const BucketSpec& spec, size_t smem, cudaStream_t stream) {
  dim3 grid((unsigned)p.splits, (unsigned)p.H, (unsigned)p.B);
  if (p.M == 1) {
    p.m0 = 0;
    decode_kernel<T, D, 1><<<grid, THREADS, smem, stream>>>(p, spec);
  } else {
    for (int m0 = 0; m0 < p.M; m0 += 4) {
      p.m0 = m0;
      decode_kernel<T, D, 4><<<grid, THREADS, smem, stream>>>(p, spec);
    }
  }
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

template <typename T>
static int launch_type(const Params& p, int D, const BucketSpec& spec, size_t smem, cudaStream_t stream) {
  switch (D) {
    case 16: return launch_rows<T, 16>(p, spec, smem, stream);
    case 32: return launch_rows<T, 32>(p, spec, smem, stream);
    case 64: return launch_rows<T, 64>(p, spec, smem, stream);
    case 128: return launch_rows<T, 128>(p, spec, smem, stream);
  }
  return T5B_ERR_HEAD_DIM;
}

static int64_t align256(int64_t x) { return (x + 255) / 256 * 256; }

}  // namespace decode
}  // namespace t5b

using namespace t5b;

extern "C" int t5b_decode_num_splits(int B, int H, int N) {
  if (B <= 0 || H <= 0 || N <= 0) return 1;
  // aim for ~8 waves of blocks (148 SMs x ~6 resident blocks) so the tail is small,
  // but keep at least 512 keys per split
  const long long bh = (long long)B * H;
  long long want = (8LL * 148 * 6 + bh - 1) / bh;
  long long cap = (N + 511) / 512;
  long long s = want < cap ? want : cap;
  if (s < 1) s = 1;
  if (s > 64) s = 64;
  return (int)s;
}

extern "C" int64_t t5b_decode_workspace_bytes(int B, int H, int M, int D, int num_splits) {
  if (B <= 0 || H <= 0 || M <= 0 || D <= 0 || num_splits <= 0) return 0;
  const int64_t bh = (int64_t)B * H;
  return decode::align256(bh * 4) + decode::align256(bh * num_splits * M * 2 * 4) +
         decode::align256(bh * num_splits * M * (int64_t)D * 4);
}

// Argument checks shared by both entry points; on T5B_OK `*splits` holds the split count and
// `*empty` says that there is nothing to launch.
static int decode_validate(const t5b_decode_args* a, BucketSpec* spec, int* splits, bool* empty) {
  *empty = false;
  if (!a || !a->q || !a->k || !a->v || !a->out) return T5B_ERR_ARG;
  if (a->B < 0 || a->H < 0 || a->M < 0 || a->N < 0) return T5B_ERR_SHAPE;
  if (a->D != 16 && a->D != 32 && a->D != 64 && a->D != 128) return T5B_ERR_HEAD_DIM;
  if (a->dtype != T5B_F32 && a->dtype != T5B_F16 && a->dtype != T5B_BF16) return T5B_ERR_DTYPE;
  if (a->B == 0 || a->H == 0 || a->M == 0) { *empty = true; return T5B_OK; }
  if (a->H > 65535 || a->B > 65535) return T5B_ERR_SHAPE;
  const int es = dtype_bytes(a->dtype);
  auto al16 = [](const void* p) { return ((uintptr_t)p & 15) == 0; };
  if (!al16(a->k) || !al16(a->v)) return T5B_ERR_ALIGN;
  const int64_t strides[] = {a->k_stride_b, a->k_stride_h, a->k_stride_n,
                             a->v_stride_b, a->v_stride_h, a->v_stride_n};
  for (int64_t s : strides) if ((s * es) % 16 != 0) return T5B_ERR_ALIGN;
  spec->n_side = 2; spec->bidirectional = 0; spec->max_distance = 1; spec->n_first = 0;
  if (a->table) {
    if (a->table_dtype != T5B_F32 && a->table_dtype != T5B_F16 && a->table_dtype != T5B_BF16) return T5B_ERR_DTYPE;
    int st = make_bucket_spec(a->num_buckets, a->max_distance, a->causal ? 0 : 1, spec);
    if (st != T5B_OK) return st;
    if (spec->max_distance > 2048) return T5B_ERR_UNSUPPORTED;
  }
  int n = a->num_splits > 0 ? a->num_splits : t5b_decode_num_splits(a->B, a->H, a->N);
  if (n > 256) return T5B_ERR_ARG;
  if (a->N == 0) n = 1;
  *splits = n;
  return T5B_OK;
}

extern "C" int t5b_decode_fwd(const t5b_decode_args* a, void* stream) {
  BucketSpec spec;
  int splits = 1;
  bool empty = false;
  const int vst = decode_validate(a, &spec, &splits, &empty);
  if (vst != T5B_OK || empty) return vst;

  decode::Params p;
  p.q = a->q; p.k = a->k; p.v = a->v; p.out = a->out; p.table = a->table; p.seqlens_k = a->seqlens_k;
  p.counters = nullptr; p.part_ml = nullptr; p.part_o = nullptr;
  if (splits > 1) {
    const int64_t need = t5b_decode_workspace_bytes(a->B, a->H, a->M, a->D, splits);
    if (!a->workspace || a->workspace_bytes < need || ((uintptr_t)a->workspace & 255) != 0) return T5B_ERR_WORKSPACE;
    const int64_t bh = (int64_t)a->B * a->H;
    char* w = (char*)a->workspace;
    p.counters = (int32_t*)w;
    w += decode::align256(bh * 4);
    p.part_ml = (float*)w;
    w += decode::align256(bh * splits * a->M * 2 * 4);
    p.part_o = (float*)w;
  }
  p.q_stride_b = a->q_stride_b; p.q_stride_h = a->q_stride_h; p.q_stride_m = a->q_stride_m;
  p.k_stride_b = a->k_stride_b; p.k_stride_h = a->k_stride_h; p.k_stride_n = a->k_stride_n;
  p.v_stride_b = a->v_stride_b; p.v_stride_h = a->v_stride_h; p.v_stride_n = a->v_stride_n;
  p.o_stride_b = a->o_stride_b; p.o_stride_h = a->o_stride_h; p.o_stride_m = a->o_stride_m;
  p.table_stride0 = a->table_stride0; p.table_dtype = a->table_dtype;
  p.B = a->B; p.H = a->H; p.M = a->M; p.N = a->N;
  p.causal = a->causal; p.q_pos_offset = a->q_pos_offset; p.splits = splits; p.m0 = 0;
  p.scale_log2 = a->sm_scale * kLog2e;
  const size_t smem = a->table ? (size_t)(2 * spec.max_distance + 1) * 4 : 0;
  cudaStream_t st = (cudaStream_t)stream;
  switch (a->dtype) {
    case T5B_F32: return decode::launch_type<float>(p, a->D, spec, smem, st);
    case T5B_F16: return decode::launch_type<__half>(p, a->D, spec, smem, st);
    case T5B_BF16: return decode::launch_type<__nv_bfloat16>(p, a->D, spec, smem, st);
  }
  return T5B_ERR_DTYPE;
}

// ---------------------------------------------------------------------------
// Decoding without any allocation by the caller or by this library.
//
// Some hosts of this kernel cannot call cudaMalloc (or torch's allocator) at the
// point where they decode: serving loops with a frozen memory budget, latency-
// critical threads where an allocation could block, or plain C callers that were
// handed only the input and output buffers.  For them the split-KV scratch lives in a
// fixed array inside the library image; every GPU that loads the library holds
// these bytes until the process exits.
//
// The array's name is a host-side handle, not a device address, so its address
// is obtained with cudaGetSymbolAddress once per device (with that device
// current) on the first call made on that device; make that first call before
// starting any stream capture.  All calls share the one array: the split counters
// at its front are cleared on the stream before every launch, and two calls
// whose kernels overlap on the GPU (different streams) would race on it.  The
// looked-up address is kept for the life of the process: after cudaDeviceReset
// it is stale, and this entry point must not be used again in that process.
constexpr long long kStaticScratchBytes = 4ll << 20;   // 4 MiB
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

#include <mutex>

static void* static_scratch_address(int* status) {
  static std::mutex mu;
  static void* cached[64] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { *status = T5B_ERR_LAUNCH; return nullptr; }
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
      cudaGetLastError();
      *status = T5B_ERR_LAUNCH;
      return nullptr;
    }
    cached[dev] = ptr;
  }
  *status = T5B_OK;
  return cached[dev];
}

extern "C" int64_t t5b_decode_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int t5b_decode_fwd_static_scratch(const t5b_decode_args* a, void* stream) {
  // every argument check comes first: a refused call leaves the shared array untouched
  BucketSpec spec;
  int splits = 1;
  bool empty = false;
  const int vst = decode_validate(a, &spec, &splits, &empty);
  if (vst != T5B_OK || empty) return vst;
  t5b_decode_args b = *a;
  b.num_splits = splits;
  b.workspace = nullptr;
  b.workspace_bytes = 0;
  if (splits > 1) {
    const int64_t need = t5b_decode_workspace_bytes(a->B, a->H, a->M, a->D, splits);
    if (need > kStaticScratchBytes) return T5B_ERR_WORKSPACE;   // beyond the built-in scratch: use t5b_decode_fwd
    int st = T5B_OK;
    void* ptr = static_scratch_address(&st);
    if (st != T5B_OK) return st;
    // the array keeps whatever the previous call left: the counters must start at zero
    const int64_t counter_bytes = decode::align256((int64_t)a->B * a->H * 4);
    if (cudaMemsetAsync(ptr, 0, (size_t)counter_bytes, (cudaStream_t)stream) != cudaSuccess) {
      cudaGetLastError();
      return T5B_ERR_LAUNCH;
    }
    b.workspace = ptr;
    b.workspace_bytes = kStaticScratchBytes;
  }
  return t5b_decode_fwd(&b, stream);
}
