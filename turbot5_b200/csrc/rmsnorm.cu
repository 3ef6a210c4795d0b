// T5 RMSNorm forward: y = w * round_w(x * rsqrt(mean(x^2) + eps)), float32
// statistics, no mean subtraction, no bias.  HBM-bound: every element is read
// once and written once; a warp owns two rows at a time and keeps them in registers
// between the reduction and the scaling (rows up to 8 x 512 bytes), 16-byte streaming
// accesses, grid-stride over the rows.
//
// Rounding points follow T5LayerNorm._forward (src/turbot5/model/modules.py:
// 52-60): with a half-precision weight the normalised value is first rounded to
// the weight's type and the product is rounded again; with a float32 weight the
// result stays float32.
#include "t5b_common.cuh"

#include <type_traits>

namespace t5b {
namespace rms {

constexpr int WARPS = 4;

template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename TX, typename TW, typename TY>
__device__ __forceinline__ TY scale_one(float x, float rstd, TW w) {
  float xn = x * rstd;
  if (sizeof(TW) == 2) xn = to_float<TW>(from_float<TW>(xn));   // first rounding, to the weight's type
  return from_float<TY>(to_float<TW>(w) * xn);
}

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_stream16(void* p, const uint4& v) {

  asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Vector path: a warp owns ROWS rows at a time and keeps them in registers (VPL 16-byte
// vectors per lane and row) between the sum of squares and the scaling, so every element is
// read once and written once.  All loads of the ROWS rows are issued before the first
// reduction, and warps walk the rows with a grid stride (no tail wave).
template <typename TX, typename TW, typename TY, int VPL, int ROWS>
__global__ void __launch_bounds__(WARPS * 32)
rmsnorm_vec_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y,
                   float* __restrict__ rstd_out, int64_t rows, int d, int64_t xs, int64_t ys, float eps,
                   int w_aligned) {
  constexpr int VX = VecOf<TX>::N;
  constexpr int OUT16 = (int)(VX * sizeof(TY) / 16);   // 16-byte stores per input vector (1 or 2)
  const int lane = threadIdx.x & 31;
  const int nvec = d / VX;
  const int64_t warp_id = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  const int64_t n_warps = (int64_t)gridDim.x * WARPS;
  const float inv_d = 1.f / (float)d;
  // this lane's weights, read once (one vector load per 16-byte vector of x when the weight is
  // aligned for it: 8 two-byte loads per vector and row cost 5 % of the kernel) and kept for every row
  struct alignas(VX * sizeof(TW)) WVec { TW v[VX]; };
  WVec wv[VPL];
  #pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int v = lane + i * 32;
    if (v < nvec && w_aligned) wv[i] = *reinterpret_cast<const WVec*>(w + v * VX);
    else {
      #pragma unroll
      for (int k = 0; k < VX; ++k) wv[i].v[k] = v < nvec ? w[v * VX + k] : from_float<TW>(0.f);
    }
  }
  for (int64_t row0 = warp_id * ROWS; row0 < rows; row0 += n_warps * ROWS) {
    uint4 cache[ROWS][VPL];
    #pragma unroll
    for (int r = 0; r < ROWS; ++r)
      #pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int v = lane + i * 32;
        cache[r][i] = make_uint4(0, 0, 0, 0);
        if (row0 + r < rows && v < nvec) cache[r][i] = ld_stream16(x + (row0 + r) * xs + v * VX);
      }
    #pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (row0 + r >= rows) break;
      float ss = 0.f;
      #pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const TX* e = reinterpret_cast<const TX*>(&cache[r][i]);
        #pragma unroll
        for (int k = 0; k < VX; ++k) { const float f = to_float<TX>(e[k]); ss = fmaf(f, f, ss); }
      }
      #pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float rstd = rsqrtf(ss * inv_d + eps);
      if (rstd_out && lane == 0) rstd_out[row0 + r] = rstd;
      TY* yr = y + (row0 + r) * ys;
      #pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int v = lane + i * 32;
        if (v < nvec) {
          const TX* e = reinterpret_cast<const TX*>(&cache[r][i]);
          TY outv[VX];
          #pragma unroll
          for (int k = 0; k < VX; ++k) outv[k] = scale_one<TX, TW, TY>(to_float<TX>(e[k]), rstd, wv[i].v[k]);
          const uint4* src = reinterpret_cast<const uint4*>(outv);
          #pragma unroll
          for (int k = 0; k < OUT16; ++k) st_stream16(yr + v * VX + k * (16 / (int)sizeof(TY)), src[k]);
        }
      }
    }
  }
}

// Generic path: any d, any alignment; the row is read twice (the second read hits L1/L2).
template <typename TX, typename TW, typename TY>
__global__ void __launch_bounds__(WARPS * 32)
rmsnorm_generic_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y,
                       float* __restrict__ rstd_out, int64_t rows, int d, int64_t xs, int64_t ys, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const TX* xr = x + row * xs;
  TY* yr = y + row * ys;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) { const float f = to_float<TX>(xr[i]); ss = fmaf(f, f, ss); }
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float rstd = rsqrtf(ss / (float)d + eps);
  if (rstd_out && lane == 0) rstd_out[row] = rstd;
  for (int i = lane; i < d; i += 32) yr[i] = scale_one<TX, TW, TY>(to_float<TX>(xr[i]), rstd, w[i]);
}

template <typename TX, typename TW, typename TY>
static int launch(const void* x, const void* w, void* y, float* rstd, int64_t rows, int d,
                  int64_t xs, int64_t ys, float eps, cudaStream_t stream) {
  constexpr int VX = VecOf<TX>::N;
  const bool vec = d % VX == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
                   (xs * sizeof(TX)) % 16 == 0 && (ys * sizeof(TY)) % 16 == 0 &&
                   (VX * sizeof(TY)) % 16 == 0 && d / VX <= 32 * 8;
  const TX* xp = (const TX*)x; const TW* wp = (const TW*)w; TY* yp = (TY*)y;
  if (vec) {
    const int vpl = (d / VX + 31) / 32;
    constexpr int ROWS = 2;
    const int w_aligned = ((uintptr_t)w % (VX * sizeof(TW))) == 0 ? 1 : 0;
    // One block per WARPS * ROWS rows, no cap: measured at 100 000 x 768 bf16 (rows of 1.5 KB), 58.2 us
    // against 62.3 us for a grid capped at what the GPU holds at once and walked with a grid stride
    // (every block the same number of rounds), and 59.6-71.9 us for blocks of 8 or 16 warps.  The
    // kernel keeps its grid-stride loop for row counts beyond the grid limit.
#define T5B_RMS_LAUNCH(V) do { \
      auto kern = rmsnorm_vec_kernel<TX, TW, TY, V, ROWS>; \
      int64_t blocks = (rows + WARPS * ROWS - 1) / (WARPS * ROWS); \
      if (blocks > 0x7fffffffLL) blocks = 0x7fffffffLL; \
      kern<<<(unsigned)blocks, WARPS * 32, 0, stream>>>(xp, wp, yp, rstd, rows, d, xs, ys, eps, w_aligned); } while (0)
    if (vpl <= 1) T5B_RMS_LAUNCH(1);
    else if (vpl == 2) T5B_RMS_LAUNCH(2);
    else if (vpl == 3) T5B_RMS_LAUNCH(3);
    else if (vpl == 4) T5B_RMS_LAUNCH(4);
    else if (vpl <= 6) T5B_RMS_LAUNCH(6);
    else T5B_RMS_LAUNCH(8);
#undef T5B_RMS_LAUNCH
  } else {
    const int64_t blocks = (rows + WARPS - 1) / WARPS;
    if (blocks > 0x7fffffffLL) return T5B_ERR_SHAPE;
    rmsnorm_generic_kernel<TX, TW, TY><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(xp, wp, yp, rstd, rows, d, xs, ys, eps);
  }
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

}  // namespace rms
}  // namespace t5b

using namespace t5b;

namespace t5b {
namespace rms {

// Backward of y = w * round_w(x * rstd), rstd = rsqrt(mean(x^2) + eps)
// (rms_layer_norm_bwd_dx_fused + the weight-gradient reduction, src/turbot5/ops/rms_norm.py:53-124):
//   g = w * dy;  dx = rstd * g - x * rstd^3 * mean(g * x);  dw += dy * round_w(x * rstd).
// A warp owns a row (grid-stride); the row is read twice, the second time from L1/L2.  The
// weight gradient is summed per block in shared memory (lanes hit consecutive words) and
// added to the float32 result with one atomic per column and block.
template <typename TX, typename TW, typename TDY>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const TDY* __restrict__ dy,
                   TX* __restrict__ dx, float* __restrict__ dw, int64_t rows, int d,
                   int64_t x_stride, int64_t dy_stride, int64_t dx_stride, float eps) {
  extern __shared__ float s_dw[];
  for (int c = threadIdx.x; c < d; c += blockDim.x) s_dw[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const float inv_d = 1.f / (float)d;
  for (int64_t r = warp0; r < rows; r += n_warps) {
    const TX* xr = x + r * x_stride;
    const TDY* gr = dy + r * dy_stride;
    TX* dxr = dx + r * dx_stride;
    float ss = 0.f, sg = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float xv = to_float(xr[c]);
      ss = fmaf(xv, xv, ss);
      sg = fmaf(to_float(w[c]) * to_float(gr[c]), xv, sg);
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
      sg += __shfl_xor_sync(0xffffffffu, sg, o);
    }
    const float rstd = rsqrtf(ss * inv_d + eps);
    const float k = rstd * rstd * rstd * sg * inv_d;
    for (int c = lane; c < d; c += 32) {
      const float xv = to_float(xr[c]);
      const float gv = to_float(gr[c]);
      dxr[c] = from_float<TX>(rstd * to_float(w[c]) * gv - xv * k);
      const float xhat = to_float(from_float<TW>(xv * rstd));     // as the forward rounds it
      atomicAdd(&s_dw[c], gv * xhat);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    const float g = s_dw[c];
    if (g != 0.f) atomicAdd(&dw[c], g);
  }
}

// d = 256 * NT, 16-bit x and dy, 16-byte aligned rows: a lane owns 8 consecutive columns of every
// 256-column group, reads them with one 16-byte load, keeps the row in registers between the two
// reductions and the outputs, and carries its share of the weight gradient in registers over all
// the rows of its warp (one shared-memory add per column and warp at the end).
template <typename TX, typename TW, int NT>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_vec_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const TX* __restrict__ dy,
                       TX* __restrict__ dx, float* __restrict__ dw, int64_t rows,
                       int64_t x_stride, int64_t dy_stride, int64_t dx_stride, float eps) {
  constexpr int D = 256 * NT;
  __shared__ float s_dw[D];
  for (int c = threadIdx.x; c < D; c += blockDim.x) s_dw[c] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t n_warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  float wv[NT][8], acc[NT][8];
  #pragma unroll
  for (int t = 0; t < NT; ++t)
    #pragma unroll
    for (int k = 0; k < 8; ++k) { wv[t][k] = to_float(w[t * 256 + lane * 8 + k]); acc[t][k] = 0.f; }
  for (int64_t r = warp0; r < rows; r += n_warps) {
    float xv[NT][8], gv[NT][8];
    float ss = 0.f, sg = 0.f;
    #pragma unroll
    for (int t = 0; t < NT; ++t) {
      const uint4 xa = ld_stream16(x + r * x_stride + t * 256 + lane * 8);
      const uint4 ga = ld_stream16(dy + r * dy_stride + t * 256 + lane * 8);
      const TX* xe = reinterpret_cast<const TX*>(&xa);
      const TX* ge = reinterpret_cast<const TX*>(&ga);
      #pragma unroll
      for (int k = 0; k < 8; ++k) {
        xv[t][k] = to_float(xe[k]);
        gv[t][k] = to_float(ge[k]);
        ss = fmaf(xv[t][k], xv[t][k], ss);
        sg = fmaf(wv[t][k] * gv[t][k], xv[t][k], sg);
      }
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
      sg += __shfl_xor_sync(0xffffffffu, sg, o);
    }
    const float rstd = rsqrtf(ss * (1.f / D) + eps);
    const float kk = rstd * rstd * rstd * sg * (1.f / D);
    #pragma unroll
    for (int t = 0; t < NT; ++t) {
      uint4 oa;
      TX* oe = reinterpret_cast<TX*>(&oa);
      #pragma unroll
      for (int k = 0; k < 8; ++k) {
        oe[k] = from_float<TX>(rstd * wv[t][k] * gv[t][k] - xv[t][k] * kk);
        const float xhat = to_float(from_float<TW>(xv[t][k] * rstd));
        acc[t][k] = fmaf(gv[t][k], xhat, acc[t][k]);
      }
      *reinterpret_cast<uint4*>(dx + r * dx_stride + t * 256 + lane * 8) = oa;
    }
  }
  #pragma unroll
  for (int t = 0; t < NT; ++t)
    #pragma unroll
    for (int k = 0; k < 8; ++k) atomicAdd(&s_dw[t * 256 + lane * 8 + k], acc[t][k]);
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    const float g = s_dw[c];
    if (g != 0.f) atomicAdd(&dw[c], g);
  }
}

template <typename TX, typename TW, typename TDY>
int launch_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw, int64_t rows, int d,
               int64_t xs, int64_t dys, int64_t dxs, float eps, cudaStream_t st) {
  if constexpr (sizeof(TX) == 2 && std::is_same<TX, TDY>::value) {
    const bool aligned = ((uintptr_t)x % 16 == 0) && ((uintptr_t)dy % 16 == 0) && ((uintptr_t)dx % 16 == 0) &&
                         xs % 8 == 0 && dys % 8 == 0 && dxs % 8 == 0;
    if (aligned && (d == 512 || d == 768 || d == 1024)) {
      int64_t nblk = (rows + 7) / 8;
      if (nblk > 148 * 4) nblk = 148 * 4;
#define T5B_RMSB_VEC(NT)                                                                            \
      rmsnorm_bwd_vec_kernel<TX, TW, NT><<<(unsigned)nblk, 256, 0, st>>>(                               \
          (const TX*)x, (const TW*)w, (const TX*)dy, (TX*)dx, dw, rows, xs, dys, dxs, eps)
      if (d == 512) T5B_RMSB_VEC(2); else if (d == 768) T5B_RMSB_VEC(3); else T5B_RMSB_VEC(4);
#undef T5B_RMSB_VEC
      return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
    }
  }
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return T5B_ERR_SHAPE;
  auto kern = rmsnorm_bwd_kernel<TX, TW, TDY>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    cudaGetLastError();
    return T5B_ERR_LAUNCH;
  }
  int64_t blocks = (rows + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  kern<<<(unsigned)blocks, 256, smem, st>>>((const TX*)x, (const TW*)w, (const TDY*)dy, (TX*)dx, dw, rows, d,
                                            xs, dys, dxs, eps);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

}  // namespace rms
}  // namespace t5b

extern "C" int t5b_rmsnorm_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw,
                               int64_t rows, int32_t d, int64_t x_row_stride, int64_t dy_row_stride,
                               int64_t dx_row_stride, int32_t x_dtype, int32_t w_dtype, float eps, void* stream) {
  using namespace t5b;
  if (!x || !w || !dy || !dx || !dw) return T5B_ERR_ARG;
  if (rows < 0 || d <= 0) return T5B_ERR_SHAPE;
  if (rows == 0) return T5B_OK;
  cudaStream_t st = (cudaStream_t)stream;
  // dy has the type of the forward's output: w's type when w is 16-bit, float32 otherwise
#define T5B_RMSB(TXE, TX, TWE, TW, TDY)                                                       \
  if (x_dtype == TXE && w_dtype == TWE)                                                      \
    return rms::launch_bwd<TX, TW, TDY>(x, w, dy, dx, dw, rows, d, x_row_stride, dy_row_stride, dx_row_stride, eps, st);
  T5B_RMSB(T5B_BF16, __nv_bfloat16, T5B_BF16, __nv_bfloat16, __nv_bfloat16)
  T5B_RMSB(T5B_BF16, __nv_bfloat16, T5B_F32, float, float)
  T5B_RMSB(T5B_F16, __half, T5B_F16, __half, __half)
  T5B_RMSB(T5B_F16, __half, T5B_F32, float, float)
  T5B_RMSB(T5B_F32, float, T5B_F32, float, float)
  T5B_RMSB(T5B_F32, float, T5B_BF16, __nv_bfloat16, __nv_bfloat16)
  T5B_RMSB(T5B_F32, float, T5B_F16, __half, __half)
#undef T5B_RMSB
  return T5B_ERR_DTYPE;
}

extern "C" int t5b_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t rows,
                               int32_t d, int64_t x_row_stride, int64_t y_row_stride,
                               int32_t x_dtype, int32_t w_dtype, float eps, void* stream) {
  if (!x || !w || !y) return T5B_ERR_ARG;
  if (rows < 0 || d <= 0) return T5B_ERR_SHAPE;
  if (rows == 0) return T5B_OK;
  cudaStream_t st = (cudaStream_t)stream;
#define T5B_RMS(TXE, TX, TWE, TW, TY)                                                        \
  if (x_dtype == TXE && w_dtype == TWE)                                                      \
    return rms::launch<TX, TW, TY>(x, w, y, rstd, rows, d, x_row_stride, y_row_stride, eps, st);
  T5B_RMS(T5B_BF16, __nv_bfloat16, T5B_BF16, __nv_bfloat16, __nv_bfloat16)
  T5B_RMS(T5B_BF16, __nv_bfloat16, T5B_F32, float, float)
  T5B_RMS(T5B_F16, __half, T5B_F16, __half, __half)
  T5B_RMS(T5B_F16, __half, T5B_F32, float, float)
  T5B_RMS(T5B_F32, float, T5B_F32, float, float)
  T5B_RMS(T5B_F32, float, T5B_BF16, __nv_bfloat16, __nv_bfloat16)
  T5B_RMS(T5B_F32, float, T5B_F16, __half, __half)
#undef T5B_RMS
  return T5B_ERR_DTYPE;
}
