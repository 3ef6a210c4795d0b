// Unpad / pad glue for packed sequences, without host synchronisation.
//
// The reference turns a 0/1 (B, L) mask into token indices with torch.nonzero and
// reads the longest length back to the host (src/turbot5/model/padding.py:79-88),
// gathers the kept rows (index_first_axis, :46-76) and scatters results into a
// zero tensor (pad_input, :30-44).  Here the plan (lengths, cumulative lengths,
// destination row of every token) is computed on the device and the packed
// buffers are sized for the worst case, so nothing is read back.
#include "t5b_common.cuh"

namespace t5b {
namespace pad {

__device__ __forceinline__ bool mask_at(const void* mask, int eb, int64_t i) {
  switch (eb) {
    case 1: return ((const uint8_t*)mask)[i] != 0;
    case 2: return ((const uint16_t*)mask)[i] != 0;
    case 4: return ((const uint32_t*)mask)[i] != 0;
    default: return ((const uint64_t*)mask)[i] != 0;
  }
}

__device__ __forceinline__ int block_sum(int v, int* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  #pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  int t = 0;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += scratch[i];
  return t;
}

// one block per batch row: number of kept tokens
__global__ void count_kernel(const void* mask, int eb, int L, int32_t* seqlens) {
  __shared__ int scratch[32];
  const int b = blockIdx.x;
  int c = 0;
  for (int i = threadIdx.x; i < L; i += blockDim.x) c += mask_at(mask, eb, (int64_t)b * L + i) ? 1 : 0;
  const int total = block_sum(c, scratch);
  if (threadIdx.x == 0) seqlens[b] = total;
}

// one block per batch row: cumulative lengths and destination rows.  Kept token ->
// its packed row (>= 0).  Dropped token -> -2 - r, where r is a distinct row of the
// unused tail of the worst-case-sized packed buffer: the gather zero-fills that row,
// so the whole packed buffer is defined (a tile that runs past the last sequence
// must never multiply a zero probability with uninitialised memory).
__global__ void plan_kernel(const void* mask, int eb, int B, int L, const int32_t* seqlens,
                            int32_t* cu, int32_t* dest) {
  __shared__ int scratch[32];
  __shared__ int warp_base[32];
  const int b = blockIdx.x;
  int before = 0, all = 0;
  for (int i = threadIdx.x; i < B; i += blockDim.x) {
    const int n = seqlens[i];
    all += n;
    if (i < b) before += n;
  }
  before = block_sum(before, scratch);
  all = block_sum(all, scratch);
  if (threadIdx.x == 0) {
    cu[b] = before;
    if (b == B - 1) cu[B] = before + seqlens[b];
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  int run = before;
  for (int i0 = 0; i0 < L; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    const bool keep = i < L && mask_at(mask, eb, (int64_t)b * L + i);
    const unsigned bal = __ballot_sync(0xffffffffu, keep);
    __syncthreads();
    if (lane == 0) warp_base[warp] = __popc(bal);
    __syncthreads();
    int base = run, total = 0;
    for (int w2 = 0; w2 < nwarp; ++w2) {
      if (w2 < warp) base += warp_base[w2];
      total += warp_base[w2];
    }
    if (i < L) {
      const int kept_before = base + __popc(bal & ((1u << lane) - 1));   // kept tokens before this one, all rows
      const int flat = b * L + i;
      dest[(int64_t)flat] = keep ? kept_before : -2 - (all + (flat - kept_before));
    }
    run += total;
  }
}

__global__ void gather_kernel(const uint4* __restrict__ padded, int64_t ps16, uint4* __restrict__ packed,
                              int64_t ks16, const int32_t* __restrict__ dest, int64_t n_rows, int v16) {
  const int64_t total = n_rows * v16;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / v16; const int c = (int)(i % v16);
    const int d = dest[r];
    if (d >= 0) packed[(int64_t)d * ks16 + c] = padded[r * ps16 + c];
    else packed[(int64_t)(-2 - d) * ks16 + c] = make_uint4(0, 0, 0, 0);
  }
}

__global__ void scatter_kernel(const uint4* __restrict__ packed, int64_t ks16, uint4* __restrict__ padded,
                               int64_t ps16, const int32_t* __restrict__ dest, int64_t n_rows, int v16) {
  const int64_t total = n_rows * v16;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / v16; const int c = (int)(i % v16);
    const int d = dest[r];
    padded[r * ps16 + c] = d >= 0 ? packed[(int64_t)d * ks16 + c] : make_uint4(0, 0, 0, 0);
  }
}

static unsigned grid_for(int64_t work) {
  int64_t b = (work + 255) / 256;
  const int64_t cap = 148 * 16;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace pad
}  // namespace t5b

using namespace t5b;

extern "C" int t5b_unpad_plan(const void* mask, int32_t eb, int32_t B, int32_t L, int32_t* seqlens,
                              int32_t* cu_seqlens, int32_t* dest, void* stream) {
  if (!mask || !seqlens || !cu_seqlens || !dest) return T5B_ERR_ARG;
  if (eb != 1 && eb != 2 && eb != 4 && eb != 8) return T5B_ERR_DTYPE;
  if (B < 0 || L < 0) return T5B_ERR_SHAPE;
  if (B == 0) return T5B_OK;
  cudaStream_t st = (cudaStream_t)stream;
  pad::count_kernel<<<B, 256, 0, st>>>(mask, eb, L, seqlens);
  pad::plan_kernel<<<B, 256, 0, st>>>(mask, eb, B, L, seqlens, cu_seqlens, dest);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

static int check_rows(const void* a, const void* b, int64_t sa, int64_t sb, int32_t row_bytes) {
  if (!a || !b) return T5B_ERR_ARG;
  if (row_bytes <= 0 || row_bytes % 16 || sa % 16 || sb % 16 || ((uintptr_t)a & 15) || ((uintptr_t)b & 15))
    return T5B_ERR_ALIGN;
  return T5B_OK;
}

extern "C" int t5b_gather_rows(const void* padded, int64_t ps, void* packed, int64_t ks,
                               const int32_t* dest, int64_t n_rows, int32_t row_bytes, void* stream) {
  int st = check_rows(padded, packed, ps, ks, row_bytes);
  if (st != T5B_OK) return st;
  if (!dest) return T5B_ERR_ARG;
  if (n_rows <= 0) return n_rows == 0 ? T5B_OK : T5B_ERR_SHAPE;
  const int v16 = row_bytes / 16;
  pad::gather_kernel<<<pad::grid_for(n_rows * v16), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)padded, ps / 16, (uint4*)packed, ks / 16, dest, n_rows, v16);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

extern "C" int t5b_scatter_rows(const void* packed, int64_t ks, void* padded, int64_t ps,
                                const int32_t* dest, int64_t n_rows, int32_t row_bytes, void* stream) {
  int st = check_rows(packed, padded, ks, ps, row_bytes);
  if (st != T5B_OK) return st;
  if (!dest) return T5B_ERR_ARG;
  if (n_rows <= 0) return n_rows == 0 ? T5B_OK : T5B_ERR_SHAPE;
  const int v16 = row_bytes / 16;
  pad::scatter_kernel<<<pad::grid_for(n_rows * v16), 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)packed, ks / 16, (uint4*)padded, ps / 16, dest, n_rows, v16);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}
