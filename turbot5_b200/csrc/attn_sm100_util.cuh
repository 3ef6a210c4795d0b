// Pieces shared by the tensor-core attention kernels (forward and backward): the TMA
// descriptor builder and the 16-bit pair packing.
#pragma once

#include "t5b_common.cuh"

#include <cuda.h>

namespace t5b {
namespace sm100 {

template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (kBf16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}

// 2^-k for a non-negative whole number k held in a float (0 once it leaves the normal range).
__device__ __forceinline__ float pow2_neg(float k) {
  return k >= 127.f ? 0.f : __int_as_float((127 - (int)k) << 23);
}

// Both halves of a packed pair times a power of two (exact unless the result leaves the
// normal range, where it no longer matters).
template <bool kBf16>
__device__ __forceinline__ uint32_t scale_packed(uint32_t v, float beta) {
  float lo, hi;
  if (kBf16) {
    lo = __uint_as_float(v << 16);
    hi = __uint_as_float(v & 0xffff0000u);
  } else {
    const __half2 h = *reinterpret_cast<const __half2*>(&v);
    lo = __low2float(h);
    hi = __high2float(h);
  }
  return pack2<kBf16>(lo * beta, hi * beta);
}


// ---- packed 2 x fp32 values held in one 64-bit register pair
__device__ __forceinline__ uint64_t pk2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpk2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// Exponentials on the FMA pipe.  The exponential unit retires 16 ex2 per clock per SM, and at head
// dim 64 that is the scarcest resource of this kernel; the FMA pipe has room.  A compile-time share
// of each thread's column pairs (kPoly of every 8) is therefore computed as
//   2^(s*mul + add) = 2^n * g * 2^f,  n = rint(add) + rint(s*mul),  f = s*mul - rint(s*mul) in [-1/2, 1/2],
//   g = 2^(add - rint(add))  (one ex2 per thread and tile, folded into the coefficients),
// with n found by adding 1.5 * 2^23 (the sum's low mantissa bits then hold n), a cubic for 2^f
// (relative error 7.5e-5: P is rounded to 8 or 11 bits afterwards) and n added to the exponent field
// by one integer add.  s is clamped from below so that the exponent field stays positive.
constexpr float kExpMagic = 12582912.f;      // 1.5 * 2^23
constexpr float kExpC0 = 0x1.fff694p-1f, kExpC1 = 0x1.62f31ap-1f, kExpC2 = 0x1.f0ddf6p-3f, kExpC3 = 0x1.c3f6fp-5f;
// pair i (of the 16 pairs of a 32-column chunk) goes to the FMA pipe when this is true: k of every 8, evenly spread
__host__ __device__ constexpr bool poly_pair(int i, int k) { return ((i % 8 + 1) * k / 8) != ((i % 8) * k / 8); }

struct PolyExp {
  uint64_t mul, m1, c0, c1, c2, c3;
  float lo;
  // mul > 0
  __device__ __forceinline__ void setup(float e_mul, float inv_mul, float e_add) {
    const float a_int = rintf(e_add);
    const float g = fast_exp2(e_add - a_int);
    mul = pk2(e_mul, e_mul);
    m1 = pk2(kExpMagic + a_int, kExpMagic + a_int);
    c0 = pk2(g * kExpC0, g * kExpC0);
    c1 = pk2(g * kExpC1, g * kExpC1);
    c2 = pk2(g * kExpC2, g * kExpC2);
    c3 = pk2(g * kExpC3, g * kExpC3);
    lo = (-123.f - a_int) * inv_mul;
  }
  __device__ __forceinline__ void eval(float s0, float s1, float& p0, float& p1) const {
    const uint64_t s = pk2(fmaxf(s0, lo), fmaxf(s1, lo));
    const uint64_t t = ffma2(s, mul, m1);                     // magic + n
    const uint64_t nk = ffma2(t, pk2(-1.f, -1.f), m1);        // -rint(s*mul), exact
    const uint64_t f = ffma2(s, mul, nk);
    uint64_t q = ffma2(f, c3, c2);
    q = ffma2(q, f, c1);
    q = ffma2(q, f, c0);
    float t0, t1, q0, q1;
    unpk2(t, t0, t1);
    unpk2(q, q0, q1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
  }
};

// kBf16: element type of Q/K/V/out (P uses the same type: tcgen05.mma kind::f16
// takes A and B of one format; mixing fp16 P with bf16 V is an illegal instruction).
// O and the row sum are rescaled only when a row maximum grows by more than this many powers
// of two over the value the exponentials are taken against.  Until then P may exceed 1: bf16
// has the exponent range of fp32, so P <= 2^40 (and O, l <= 2^40 x keys x |v|) is harmless and
// rounding stays relative; fp16 P must stay below 65504, hence 2^10.
template <bool kBf16> constexpr float kRescaleThreshold = kBf16 ? 40.f : 10.f;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess) return nullptr;
    if (qres != cudaDriverEntryPointSuccess) return nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

// (D, rows, H, B) view with element strides; box = one [box_rows][64 dims] sub-tile.  With
// D < 64 the box reaches past the tensor's inner extent and those columns arrive as zeros.
inline int make_tmap(CUtensorMap* map, const void* ptr, bool bf16, int HD, int box_rows, int64_t rows, int H, int B,
                     int64_t stride_row, int64_t stride_h, int64_t stride_b) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return T5B_ERR_DRIVER;
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)rows, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)stride_row * 2, (cuuint64_t)stride_h * 2,
                           (cuuint64_t)(B > 1 ? stride_b : (int64_t)HD) * 2};
  // unit dims may carry any stride in the caller's tensor; give them a legal one
  if (H == 1) strides[1] = (cuuint64_t)HD * 2;
  if (rows == 1) strides[0] = (cuuint64_t)HD * 2;
  cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? T5B_OK : T5B_ERR_DRIVER;
}

}  // namespace sm100
}  // namespace t5b
