// Token-wise kernels around the attention path of a T5 block, each one pass over HBM:
//
//   add_rmsnorm   hidden' = hidden + branch (rounded to the hidden type, as the residual add of
//                 T5LayerSelfAttention / T5LayerFF does, src/turbot5/model/modeling.py:124-128,
//                 142-164), normed = T5 RMSNorm(hidden') with the rounding points of
//                 T5LayerNorm._forward (src/turbot5/model/modules.py:52-60).  Replaces an add, a
//                 norm and a cast launch per sub-layer: reads two rows, writes two rows.
//   gated_gelu    out = gelu_tanh(x[:, :F]) * x[:, F:] over the output of ONE matrix product with
//                 the concatenated wi_0 | wi_1 weights (T5DenseGatedActDense,
//                 src/turbot5/model/modeling.py:83-100; the reference's own fused attempt is
//                 src/turbot5/ops/gated_mlp.py:83-225).  The activation is rounded to the element
//                 type before the product, as two separate torch ops would.
//   merge         out = sum_i w_i * part_i, w_i = exp(lse_i - max lse) / sum: combines attention
//                 results computed over disjoint key ranges (float32 partial outputs and their
//                 log-sum-exp) into the result over all keys -- the rule of the split-KV merge
//                 (src/turbot5/ops/flash_decoding.py:47-55) applied to normalised partials.
//
// All three are bound by HBM bandwidth; 16-byte accesses, grids sized from the SM count.
#include "t5b_common.cuh"

#include <atomic>

namespace t5b {
namespace fused {

__device__ __forceinline__ uint4 ld16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void st16(void* p, const uint4& v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

static int sm_count() {
  static std::atomic<int> sms[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 148; }
  int n = sms[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); return 148; }
    sms[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// Blocks of `threads` threads of kernel `fn` that the current GPU holds at once; the answer depends
// on the registers the compiler gave the kernel and is kept in `per_sm`, a static of the call site
// (one per kernel instantiation).
template <typename Fn>
static int64_t resident_blocks(Fn fn, int threads, std::atomic<int>& per_sm) {
  int n = per_sm.load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, threads, 0) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 1; }
    per_sm.store(n, std::memory_order_relaxed);
  }
  return (int64_t)n * sm_count();
}

// Grid for a grid-stride kernel with `work` block-sized pieces when the GPU holds `cap` blocks at
// once: every block makes the same number of rounds (no thin last round).
static int64_t balanced_blocks(int64_t work, int64_t cap) {
  if (work < 1) return 1;
  if (work <= cap) return work;
  const int64_t rounds = (work + cap - 1) / cap;
  return (work + rounds - 1) / rounds;
}

// ---------------------------------------------------------------- residual add + RMSNorm
// A warp owns a row at a time (grid stride) and keeps the summed row in registers between the
// sum of squares and the scaling.  T: 16-bit element type of hidden, branch and both outputs;
// TW: type of the weight.  VPL 16-byte vectors per lane.
template <typename T, typename TW, int VPL>
__global__ void __launch_bounds__(256)
add_rmsnorm_kernel(const T* __restrict__ hidden, const T* __restrict__ branch, const TW* __restrict__ w,
                   T* __restrict__ hidden_out, T* __restrict__ normed, int64_t rows, int d,
                   int64_t hs, int64_t bs, int64_t hos, int64_t ns, float eps, int w_aligned) {
  const int lane = threadIdx.x & 31;
  const int nvec = d / 8;
  const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const float inv_d = 1.f / (float)d;
  // this lane's weights, read once (vector loads when the weight is aligned for them) and kept for every row
  struct alignas(8 * sizeof(TW)) WVec { TW v[8]; };
  WVec wv[VPL];
  #pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + i * 32;
    if (v < nvec && w_aligned) wv[i] = *reinterpret_cast<const WVec*>(w + v * 8);
    else {
      #pragma unroll
      for (int k = 0; k < 8; ++k) wv[i].v[k] = v < nvec ? w[v * 8 + k] : from_float<TW>(0.f);
    }
  }
  for (int64_t row = warp_id; row < rows; row += n_warps) {
    uint4 a[VPL], b[VPL];
    #pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + i * 32;
      a[i] = make_uint4(0, 0, 0, 0);
      b[i] = make_uint4(0, 0, 0, 0);
      if (v < nvec) {
        a[i] = ld16(hidden + row * hs + v * 8);
        b[i] = ld16(branch + row * bs + v * 8);
      }
    }
    float ss = 0.f;
    #pragma unroll
    for (int i = 0; i < VPL; ++i) {
      T* ea = reinterpret_cast<T*>(&a[i]);
      const T* eb = reinterpret_cast<const T*>(&b[i]);
      #pragma unroll
      for (int k = 0; k < 8; ++k) {
        ea[k] = from_float<T>(to_float<T>(ea[k]) + to_float<T>(eb[k]));   // the residual stream, rounded
        const float f = to_float<T>(ea[k]);
        ss = fmaf(f, f, ss);
      }
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss * inv_d + eps);
    #pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        st16(hidden_out + row * hos + v * 8, a[i]);
        const T* ea = reinterpret_cast<const T*>(&a[i]);
        uint4 o4;
        T* eo = reinterpret_cast<T*>(&o4);
        #pragma unroll
        for (int k = 0; k < 8; ++k) {
          float xn = to_float<T>(ea[k]) * rstd;
          if (sizeof(TW) == 2) xn = to_float<TW>(from_float<TW>(xn));   // first rounding, to the weight's type
          eo[k] = from_float<T>(to_float<TW>(wv[i].v[k]) * xn);
        }
        st16(normed + row * ns + v * 8, o4);
      }
    }
  }
}

template <typename T, typename TW>
static int launch_add_rmsnorm(const void* hidden, const void* branch, const void* w, void* hidden_out, void* normed,
                              int64_t rows, int d, int64_t hs, int64_t bs, int64_t hos, int64_t ns, float eps,
                              cudaStream_t stream) {
  const int vpl = (d / 8 + 31) / 32;
  // 8 warps per block, a row per warp; as many blocks as the GPU holds at once, then grid-stride
#define T5B_AR_LAUNCH(V) do { \
    auto kern = add_rmsnorm_kernel<T, TW, V>; \
    static std::atomic<int> per_sm{0}; \
    const int64_t blocks = balanced_blocks((rows + 7) / 8, resident_blocks(kern, 256, per_sm)); \
    kern<<<(unsigned)blocks, 256, 0, stream>>>((const T*)hidden, (const T*)branch, (const TW*)w, (T*)hidden_out, \
                                               (T*)normed, rows, d, hs, bs, hos, ns, eps, \
                                               ((uintptr_t)w % (8 * sizeof(TW))) == 0 ? 1 : 0); } while (0)
  if (vpl <= 1) T5B_AR_LAUNCH(1);
  else if (vpl == 2) T5B_AR_LAUNCH(2);
  else if (vpl == 3) T5B_AR_LAUNCH(3);
  else if (vpl == 4) T5B_AR_LAUNCH(4);
  else if (vpl <= 6) T5B_AR_LAUNCH(6);
  else T5B_AR_LAUNCH(8);
#undef T5B_AR_LAUNCH
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

// ---------------------------------------------------------------- gated GELU
// gelu_tanh(a) = a * sigmoid(2u), u = sqrt(2/pi) * (a + 0.044715 a^3): one ex2 and one reciprocal,
// no cancellation for negative a.
__device__ __forceinline__ float gelu_tanh(float a) {
  const float u2 = 1.5957691216057308f * a * fmaf(0.044715f * a, a, 1.f);      // 2u
  return a * __frcp_rn(1.f + fast_exp2(-u2 * kLog2e));
}

// A warp walks whole rows (grid stride), its lanes the 16-byte vectors of a row, two vectors of each
// half in flight per lane.
template <typename T>
__global__ void __launch_bounds__(256)
gated_gelu_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t rows, int f, int64_t xs, int64_t os) {
  const int lane = threadIdx.x & 31;
  const int nvec = f / 8;
  const int64_t warp_id = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t row = warp_id; row < rows; row += n_warps) {
    const T* xr = x + row * xs;
    T* orow = out + row * os;
    for (int v0 = lane; v0 < nvec; v0 += 64) {
      const int v1 = v0 + 32;
      const bool two = v1 < nvec;
      const uint4 a0 = ld16(xr + v0 * 8), b0 = ld16(xr + f + v0 * 8);
      uint4 a1 = make_uint4(0, 0, 0, 0), b1 = make_uint4(0, 0, 0, 0);
      if (two) { a1 = ld16(xr + v1 * 8); b1 = ld16(xr + f + v1 * 8); }
      uint4 o0, o1;
      const T* ea = reinterpret_cast<const T*>(&a0);
      const T* eb = reinterpret_cast<const T*>(&b0);
      T* eo = reinterpret_cast<T*>(&o0);
      #pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float g = to_float<T>(from_float<T>(gelu_tanh(to_float<T>(ea[k]))));   // the activation, rounded
        eo[k] = from_float<T>(g * to_float<T>(eb[k]));
      }
      st16(orow + v0 * 8, o0);
      if (two) {
        ea = reinterpret_cast<const T*>(&a1);
        eb = reinterpret_cast<const T*>(&b1);
        eo = reinterpret_cast<T*>(&o1);
        #pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float g = to_float<T>(from_float<T>(gelu_tanh(to_float<T>(ea[k]))));
          eo[k] = from_float<T>(g * to_float<T>(eb[k]));
        }
        st16(orow + v1 * 8, o1);
      }
    }
  }
}

// ---------------------------------------------------------------- merge of attention partials
constexpr int kMaxParts = T5B_MERGE_MAX_PARTS;

struct MergeParams {
  const float* po[kMaxParts];
  const float* pl[kMaxParts];
  void* out;
  float* lse_out;
  int64_t po_stride_b, po_stride_h, po_stride_m;
  int64_t o_stride_b, o_stride_h, o_stride_m;
  int32_t n_parts, B, H, M, D;
};

// One thread per (row, 4 dims); blockIdx.y = batch * H + head, blockIdx.x walks the rows in pieces
// of 256 / (D / 4) (D / 4 is a power of two).
template <typename TO>
__global__ void __launch_bounds__(256)
merge_kernel(const __grid_constant__ MergeParams p, int vec_shift) {
  const int vec = 1 << vec_shift;
  const int c = threadIdx.x & (vec - 1);
  const int rows_per_block = 256 >> vec_shift;
  const int bh = blockIdx.y;
  const int h = bh % p.H;
  const int64_t b = bh / p.H;
  for (int m = blockIdx.x * rows_per_block + (threadIdx.x >> vec_shift); m < p.M; m += gridDim.x * rows_per_block) {
    const int64_t r = (int64_t)bh * p.M + m;
    // every load of the row is issued before the first value is used: the partial rows do not
    // wait for the log-sum-exps (a partial that saw no keys holds zeros, and is skipped below)
    const int64_t off = b * p.po_stride_b + h * p.po_stride_h + (int64_t)m * p.po_stride_m + c * 4;
    float lse[kMaxParts];
    float4 v[kMaxParts];
    #pragma unroll
    for (int s = 0; s < kMaxParts; ++s) {
      lse[s] = -INFINITY;
      v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s < p.n_parts) {
        lse[s] = __ldg(p.pl[s] + r);
        v[s] = __ldcs(reinterpret_cast<const float4*>(p.po[s] + off));
      }
    }
    float mx = -INFINITY;
    #pragma unroll
    for (int s = 0; s < kMaxParts; ++s) mx = fmaxf(mx, lse[s]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    if (mx > -INFINITY) {
      #pragma unroll
      for (int s = 0; s < kMaxParts; ++s) {
        if (lse[s] > -INFINITY) {
          const float wgt = __expf(lse[s] - mx);
          acc.x = fmaf(wgt, v[s].x, acc.x); acc.y = fmaf(wgt, v[s].y, acc.y);
          acc.z = fmaf(wgt, v[s].z, acc.z); acc.w = fmaf(wgt, v[s].w, acc.w);
          wsum += wgt;
        }
      }
      const float inv = 1.f / wsum;
      acc.x *= inv; acc.y *= inv; acc.z *= inv; acc.w *= inv;
    }
    TO* o = reinterpret_cast<TO*>(p.out) + b * p.o_stride_b + h * p.o_stride_h + (int64_t)m * p.o_stride_m + c * 4;
    if (sizeof(TO) == 2) {
      uint2 w2;
      TO* e = reinterpret_cast<TO*>(&w2);
      e[0] = from_float<TO>(acc.x); e[1] = from_float<TO>(acc.y); e[2] = from_float<TO>(acc.z); e[3] = from_float<TO>(acc.w);
      *reinterpret_cast<uint2*>(o) = w2;
    } else {
      o[0] = from_float<TO>(acc.x); o[1] = from_float<TO>(acc.y); o[2] = from_float<TO>(acc.z); o[3] = from_float<TO>(acc.w);
    }
    if (p.lse_out != nullptr && c == 0) p.lse_out[r] = mx > -INFINITY ? mx + __logf(wsum) : -INFINITY;
  }
}

}  // namespace fused
}  // namespace t5b

using namespace t5b;

extern "C" int t5b_add_rmsnorm_fwd(const void* hidden, const void* branch, const void* weight, void* hidden_out,
                                   void* normed, int64_t rows, int32_t d, int64_t hidden_stride,
                                   int64_t branch_stride, int64_t hidden_out_stride, int64_t normed_stride,
                                   int32_t dtype, int32_t w_dtype, float eps, void* stream) {
  if (rows < 0 || d <= 0) return T5B_ERR_SHAPE;
  if (rows == 0) return T5B_OK;
  if (!hidden || !branch || !weight || !hidden_out || !normed) return T5B_ERR_ARG;
  if (dtype != T5B_BF16 && dtype != T5B_F16) return T5B_ERR_DTYPE;
  if (w_dtype != dtype && w_dtype != T5B_F32) return T5B_ERR_DTYPE;
  if (d % 8 != 0 || d > 8 * 256) return T5B_ERR_SHAPE;
  const uintptr_t bits = (uintptr_t)hidden | (uintptr_t)branch | (uintptr_t)hidden_out | (uintptr_t)normed;
  if ((bits & 15) != 0 || ((hidden_stride | branch_stride | hidden_out_stride | normed_stride) % 8) != 0) return T5B_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  using namespace t5b::fused;
  if (dtype == T5B_BF16) {
    if (w_dtype == T5B_F32)
      return launch_add_rmsnorm<__nv_bfloat16, float>(hidden, branch, weight, hidden_out, normed, rows, d, hidden_stride,
                                                      branch_stride, hidden_out_stride, normed_stride, eps, st);
    return launch_add_rmsnorm<__nv_bfloat16, __nv_bfloat16>(hidden, branch, weight, hidden_out, normed, rows, d, hidden_stride,
                                                            branch_stride, hidden_out_stride, normed_stride, eps, st);
  }
  if (w_dtype == T5B_F32)
    return launch_add_rmsnorm<__half, float>(hidden, branch, weight, hidden_out, normed, rows, d, hidden_stride,
                                             branch_stride, hidden_out_stride, normed_stride, eps, st);
  return launch_add_rmsnorm<__half, __half>(hidden, branch, weight, hidden_out, normed, rows, d, hidden_stride,
                                            branch_stride, hidden_out_stride, normed_stride, eps, st);
}

extern "C" int t5b_gated_gelu_fwd(const void* x, void* out, int64_t rows, int32_t d_ff, int64_t x_stride,
                                  int64_t out_stride, int32_t dtype, void* stream) {
  if (rows < 0 || d_ff <= 0) return T5B_ERR_SHAPE;
  if (rows == 0) return T5B_OK;
  if (!x || !out) return T5B_ERR_ARG;
  if (dtype != T5B_BF16 && dtype != T5B_F16) return T5B_ERR_DTYPE;
  if (d_ff % 8 != 0) return T5B_ERR_SHAPE;
  if ((((uintptr_t)x | (uintptr_t)out) & 15) != 0 || ((x_stride | out_stride) % 8) != 0) return T5B_ERR_ALIGN;
  cudaStream_t st = (cudaStream_t)stream;
  using namespace t5b::fused;
  if (dtype == T5B_BF16) {
    auto kern = gated_gelu_kernel<__nv_bfloat16>;
    static std::atomic<int> per_sm{0};
    const int64_t blocks = balanced_blocks((rows + 7) / 8, resident_blocks(kern, 256, per_sm));
    kern<<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, rows, d_ff, x_stride, out_stride);
  } else {
    auto kern = gated_gelu_kernel<__half>;
    static std::atomic<int> per_sm{0};
    const int64_t blocks = balanced_blocks((rows + 7) / 8, resident_blocks(kern, 256, per_sm));
    kern<<<(unsigned)blocks, 256, 0, st>>>((const __half*)x, (__half*)out, rows, d_ff, x_stride, out_stride);
  }
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

extern "C" int t5b_attention_merge(const t5b_merge_args* a, void* stream) {
  if (!a) return T5B_ERR_ARG;
  if (a->n_parts < 1 || a->n_parts > T5B_MERGE_MAX_PARTS) return T5B_ERR_ARG;
  if (a->B < 0 || a->H < 0 || a->M < 0) return T5B_ERR_SHAPE;
  if (a->D <= 0 || a->D % 4 != 0) return T5B_ERR_HEAD_DIM;
  if (a->B == 0 || a->H == 0 || a->M == 0) return T5B_OK;
  if (!a->out) return T5B_ERR_ARG;
  if (a->out_dtype != T5B_F32 && a->out_dtype != T5B_F16 && a->out_dtype != T5B_BF16) return T5B_ERR_DTYPE;
  t5b::fused::MergeParams p;
  for (int s = 0; s < T5B_MERGE_MAX_PARTS; ++s) {
    p.po[s] = s < a->n_parts ? a->part_out[s] : nullptr;
    p.pl[s] = s < a->n_parts ? a->part_lse[s] : nullptr;
    if (s < a->n_parts && (!p.po[s] || !p.pl[s])) return T5B_ERR_ARG;
    if (s < a->n_parts && ((uintptr_t)p.po[s] & 15) != 0) return T5B_ERR_ALIGN;
  }
  if (((a->part_stride_b | a->part_stride_h | a->part_stride_m) % 4) != 0) return T5B_ERR_ALIGN;
  p.out = a->out; p.lse_out = a->lse_out;
  p.po_stride_b = a->part_stride_b; p.po_stride_h = a->part_stride_h; p.po_stride_m = a->part_stride_m;
  p.o_stride_b = a->o_stride_b; p.o_stride_h = a->o_stride_h; p.o_stride_m = a->o_stride_m;
  p.n_parts = a->n_parts; p.B = a->B; p.H = a->H; p.M = a->M; p.D = a->D;
  const int vec = a->D / 4;
  if ((vec & (vec - 1)) != 0 || vec > 256) return T5B_ERR_HEAD_DIM;        // D / 4 a power of two
  int vec_shift = 0;
  while ((1 << vec_shift) < vec) ++vec_shift;
  if (((a->o_stride_b | a->o_stride_h | a->o_stride_m) % 4) != 0 || ((uintptr_t)a->out & 7) != 0) return T5B_ERR_ALIGN;
  const int64_t bh = (int64_t)a->B * a->H;
  if (bh > 65535) return T5B_ERR_SHAPE;
  const int rows_per_block = 256 >> vec_shift;
  int64_t gx = ((int64_t)a->M + rows_per_block - 1) / rows_per_block;
  const int64_t per_bh = (8LL * t5b::fused::sm_count() + bh - 1) / bh;     // about eight blocks per SM in all
  if (gx > per_bh) gx = t5b::fused::balanced_blocks(gx, per_bh);
  dim3 grid((unsigned)gx, (unsigned)bh, 1);
  cudaStream_t st = (cudaStream_t)stream;
  if (a->out_dtype == T5B_BF16) t5b::fused::merge_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, vec_shift);
  else if (a->out_dtype == T5B_F16) t5b::fused::merge_kernel<__half><<<grid, 256, 0, st>>>(p, vec_shift);
  else t5b::fused::merge_kernel<float><<<grid, 256, 0, st>>>(p, vec_shift);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}
