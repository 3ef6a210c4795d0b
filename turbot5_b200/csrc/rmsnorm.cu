// T5 RMSNorm forward: y = w * round_w(x * rsqrt(mean(x^2) + eps)), float32
// statistics, no mean subtraction, no bias.  HBM-bound: every element is read
// once and written once; a warp owns a row and keeps it in registers between
// the reduction and the scaling (rows up to 8 x 512 bytes), 16-byte accesses.
//
// Rounding points follow T5LayerNorm._forward (src/turbot5/model/modules.py:
// 52-60): with a half-precision weight the normalised value is first rounded to
// the weight's type and the product is rounded again; with a float32 weight the
// result stays float32.
#include "t5b_common.cuh"

namespace t5b {
namespace rms {

constexpr int WARPS = 4;
constexpr int MAXV = 8;   // 16-byte vectors cached per lane

template <typename T> struct VecOf { static constexpr int N = 16 / sizeof(T); };

template <typename TX, typename TW, typename TY>
__device__ __forceinline__ TY scale_one(float x, float rstd, TW w) {
  float xn = x * rstd;
  if (sizeof(TW) == 2) xn = to_float<TW>(from_float<TW>(xn));   // first rounding, to the weight's type
  return from_float<TY>(to_float<TW>(w) * xn);
}

template <typename TX, typename TW, typename TY, bool VECTOR>
__global__ void __launch_bounds__(WARPS * 32)
rmsnorm_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TY* __restrict__ y,
               float* __restrict__ rstd_out, int64_t rows, int d, int64_t xs, int64_t ys, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const TX* xr = x + row * xs;
  TY* yr = y + row * ys;
  float ss = 0.f;
  if (VECTOR) {
    constexpr int VX = VecOf<TX>::N;
    const int nvec = d / VX;
    uint4 cache[MAXV];
    #pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) {
        cache[i] = *reinterpret_cast<const uint4*>(xr + v * VX);
        const TX* e = reinterpret_cast<const TX*>(&cache[i]);
        #pragma unroll
        for (int k = 0; k < VX; ++k) { const float f = to_float<TX>(e[k]); ss = fmaf(f, f, ss); }
      }
    }
    for (int v = lane + MAXV * 32; v < nvec; v += 32) {
      const uint4 u = *reinterpret_cast<const uint4*>(xr + v * VX);
      const TX* e = reinterpret_cast<const TX*>(&u);
      #pragma unroll
      for (int k = 0; k < VX; ++k) { const float f = to_float<TX>(e[k]); ss = fmaf(f, f, ss); }
    }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / (float)d + eps);
    if (rstd_out && lane == 0) rstd_out[row] = rstd;
    auto emit = [&](const uint4& u, int v) {
      const TX* e = reinterpret_cast<const TX*>(&u);
      TY outv[VX];
      #pragma unroll
      for (int k = 0; k < VX; ++k) outv[k] = scale_one<TX, TW, TY>(to_float<TX>(e[k]), rstd, w[v * VX + k]);
      constexpr int OUT16 = (int)(VX * sizeof(TY) / 16);
      const uint4* src = reinterpret_cast<const uint4*>(outv);
      uint4* dst = reinterpret_cast<uint4*>(yr + v * VX);
      #pragma unroll
      for (int k = 0; k < OUT16; ++k) dst[k] = src[k];
      if (OUT16 == 0) {   // 8-byte case cannot happen for the supported type pairs
        #pragma unroll
        for (int k = 0; k < VX; ++k) yr[v * VX + k] = outv[k];
      }
    };
    #pragma unroll
    for (int i = 0; i < MAXV; ++i) {
      const int v = lane + i * 32;
      if (v < nvec) emit(cache[i], v);
    }
    for (int v = lane + MAXV * 32; v < nvec; v += 32)
      emit(*reinterpret_cast<const uint4*>(xr + v * VX), v);
  } else {
    for (int i = lane; i < d; i += 32) { const float f = to_float<TX>(xr[i]); ss = fmaf(f, f, ss); }
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = rsqrtf(ss / (float)d + eps);
    if (rstd_out && lane == 0) rstd_out[row] = rstd;
    for (int i = lane; i < d; i += 32) yr[i] = scale_one<TX, TW, TY>(to_float<TX>(xr[i]), rstd, w[i]);
  }
}

template <typename TX, typename TW, typename TY>
static int launch(const void* x, const void* w, void* y, float* rstd, int64_t rows, int d,
                  int64_t xs, int64_t ys, float eps, cudaStream_t stream) {
  constexpr int VX = VecOf<TX>::N;
  const bool vec = d % VX == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0 &&
                   (xs * sizeof(TX)) % 16 == 0 && (ys * sizeof(TY)) % 16 == 0 &&
                   (VX * sizeof(TY)) % 16 == 0;
  const int64_t blocks = (rows + WARPS - 1) / WARPS;
  if (blocks > 0x7fffffffLL) return T5B_ERR_SHAPE;
  if (vec)
    rmsnorm_kernel<TX, TW, TY, true><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
        (const TX*)x, (const TW*)w, (TY*)y, rstd, rows, d, xs, ys, eps);
  else
    rmsnorm_kernel<TX, TW, TY, false><<<(unsigned)blocks, WARPS * 32, 0, stream>>>(
        (const TX*)x, (const TW*)w, (TY*)y, rstd, rows, d, xs, ys, eps);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

}  // namespace rms
}  // namespace t5b

using namespace t5b;

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
