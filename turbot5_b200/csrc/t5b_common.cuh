// Shared device/host helpers: element types, bucket thresholds, and thin
// wrappers over the sm_100a PTX used by the kernels (mbarrier, TMA, tcgen05).
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/turbot5_b200.h"

namespace t5b {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr int kMaxBucketsPerSide = 256;

// Step function distance -> bucket, as thresholds: bucket(d) = #{i : first[i] <= d}
// with first[] non-decreasing.  Built on the host (bucket.cu) from the same
// float32 formula as the reference, passed to kernels by value.
struct BucketSpec {
  int32_t n_side;         // buckets per side (num_buckets/2 bidirectional, num_buckets otherwise)
  int32_t bidirectional;  // 1: keys after the query use buckets [n_side, 2*n_side)
  int32_t max_distance;   // the step function is constant for d >= max_distance
  int32_t n_first;        // number of thresholds (= n_side - 1)
  int16_t first[kMaxBucketsPerSide];  // first[i] = smallest distance whose bucket is >= i+1
};

int make_bucket_spec(int num_buckets, int max_distance, int bidirectional, BucketSpec* spec);
int host_bucket_of_delta(const BucketSpec& spec, long long delta);

__device__ __forceinline__ int bucket_of_delta(const BucketSpec& s, int delta) {
  int d = s.bidirectional ? (delta < 0 ? -delta : delta) : (delta < 0 ? -delta : 0);
  d = min(d, s.max_distance);
  // upper_bound over the thresholds
  int lo = 0, hi = s.n_first;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if ((int)s.first[mid] <= d) lo = mid + 1; else hi = mid;
  }
  return lo + ((s.bidirectional && delta > 0) ? s.n_side : 0);
}

// The same bucket, found by counting the thresholds that do not exceed |delta|: every lane reads
// the same threshold in the same iteration (one broadcast read of the kernel parameters), where
// the binary search reads a different one per lane and is serialised.  For building a table of
// consecutive deltas with a whole block.
__device__ __forceinline__ int bucket_of_delta_counted(const BucketSpec& s, int delta) {
  int d = s.bidirectional ? (delta < 0 ? -delta : delta) : (delta < 0 ? -delta : 0);
  d = min(d, s.max_distance);
  int n = 0;
  for (int k = 0; k < s.n_first; ++k) n += ((int)s.first[k] <= d) ? 1 : 0;
  return n + ((s.bidirectional && delta > 0) ? s.n_side : 0);
}

template <typename T> __device__ __forceinline__ float to_float(T x);
template <> __device__ __forceinline__ float to_float<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_float<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_float<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float load_table(const void* table, int dtype, int64_t idx) {
  if (dtype == T5B_F32) return ((const float*)table)[idx];
  if (dtype == T5B_F16) return __half2float(((const __half*)table)[idx]);
  return __bfloat162float(((const __nv_bfloat16*)table)[idx]);
}

__host__ __device__ __forceinline__ int dtype_bytes(int dtype) { return dtype == T5B_F32 ? 4 : 2; }

// ----------------------------------------------------------------------------
// PTX wrappers (sm_100a)
// ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Same, but the hardware may keep the thread suspended for up to `hint_ns` before it
// reports "not yet" (it still wakes as soon as the phase completes): far fewer polling
// instructions competing with the working warps for issue slots.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

#ifndef T5B_WAIT_LIMIT_CYCLES
#define T5B_WAIT_LIMIT_CYCLES 2000000000LL      // about a second
#endif
// Bounded wait: polls the barrier; gives up after `limit_cycles` SM cycles or as
// soon as another thread of the block has raised *abort_flag (shared memory).
// Returns false when it gave up.  Nothing in this library waits without a bound.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag,
                                                  long long limit_cycles = T5B_WAIT_LIMIT_CYCLES) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait_hint(bar, parity, 20000u)) return true;   // sleeps up to 20 us per attempt
    if (*abort_flag != 0) return false;
    if (clock64() - t0 > limit_cycles) { *abort_flag = 1; return false; }
  }
}

// The same for a whole converged warp: every lane gets the same answer, so a warp that gives up
// leaves its loop together (a later __syncwarp or warp vote must never wait for lanes that
// already left).
__device__ __forceinline__ bool mbar_wait_bounded_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const bool done = mbar_wait_bounded(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, done);
}

// The same with one probe and one vote in the common case (the phase is already complete): the
// vote makes the branch uniform, so no divergence bookkeeping surrounds the probe.
__device__ __forceinline__ bool mbar_wait_warp_fast(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  return mbar_wait_bounded_warp(bar, parity, abort_flag);
}

// 4-D tiled TMA load, global -> shared, completion on an mbarrier (no multicast).
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const void* tmap, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst_smem), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// ---- tensor memory -----------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every tcgen05 operation issued so far by this
// thread has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread t of the warp gets lane (base+t), reg i = column i.
__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 3-input maximum and packed 2 x fp32 arithmetic (one issue slot for two elements).
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// (d0, d1) = (a0, a1) * (b, b) + (c, c)
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// (d0, d1) = (a0, a1) * (b, b) + (c0, c1)
__device__ __forceinline__ void fma2v(float& d0, float& d1, float a0, float a1, float b, float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %6};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c0), "f"(c1));
}
// (d0, d1) = (a0, a1) * (b0, b1)
__device__ __forceinline__ void mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// (acc0, acc1) += (x0, x1)
__device__ __forceinline__ void add2(float& acc0, float& acc1, float x0, float x1) {
  asm("{\n\t.reg .b64 ra, rx;\n\t"
      "mov.b64 ra, {%0, %1};\n\tmov.b64 rx, {%2, %3};\n\t"
      "add.rn.f32x2 ra, ra, rx;\n\tmov.b64 {%0, %1}, ra;\n\t}"
      : "+f"(acc0), "+f"(acc1) : "f"(x0), "f"(x1));
}

// Shared-memory matrix descriptor for tcgen05.mma (128-byte swizzle, version 1).
// start address, leading/stride byte offsets are encoded >> 4.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                         uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)2 << 61;   // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, A and B each fp16 or bf16.
__host__ __device__ constexpr uint32_t make_idesc_f16(bool a_bf16, bool b_bf16, int m, int n,
                                                      bool a_mn_major, bool b_mn_major) {
  return (1u << 4)                         // D format: f32
         | ((a_bf16 ? 1u : 0u) << 7)       // A format: 0 = f16, 1 = bf16
         | ((b_bf16 ? 1u : 0u) << 10)      // B format
         | ((a_mn_major ? 1u : 0u) << 15)
         | ((b_mn_major ? 1u : 0u) << 16)
         | ((uint32_t)(n >> 3) << 17)
         | ((uint32_t)(m >> 4) << 24);
}

}  // namespace t5b
