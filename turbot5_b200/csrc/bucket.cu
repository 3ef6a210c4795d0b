// Relative-position buckets: the host-side table (the float32 formula of the
// reference, evaluated once per distance) and the device check kernel.
//
// Reference: T5Attention._relative_position_bucket,
// src/turbot5/model/attentions.py:78-124.  The logarithmic part is
//   max_exact + trunc( log(float(d) / max_exact) / log(max_distance / max_exact)
//                      * (n_side - max_exact) )
// with float32 tensor arithmetic and a double-precision scalar divisor that is
// rounded to float32 when it meets the float32 tensor.
#include <math.h>

#include "t5b_common.cuh"

namespace t5b {

static int bucket_of_distance_host(int d, int n_side, int max_distance) {
  const int max_exact = n_side / 2;
  if (d < max_exact) return d;
  volatile float ratio = (float)d / (float)max_exact;
  volatile float lg = logf(ratio);
  volatile float denom = (float)log((double)max_distance / (double)max_exact);
  volatile float q = lg / denom;
  volatile float t = q * (float)(n_side - max_exact);
  long long v = (long long)max_exact + (long long)t;   // truncation toward zero
  if (v > n_side - 1) v = n_side - 1;
  return (int)v;
}

int make_bucket_spec(int num_buckets, int max_distance, int bidirectional, BucketSpec* spec) {
  if (num_buckets < 2 || max_distance < 1 || max_distance > 32000) return T5B_ERR_ARG;
  int n_side = bidirectional ? num_buckets / 2 : num_buckets;
  if (n_side < 2 || n_side > kMaxBucketsPerSide) return T5B_ERR_ARG;
  if (max_distance <= n_side / 2) return T5B_ERR_ARG;   // log of a ratio <= 1: undefined in the reference too
  spec->n_side = n_side;
  spec->bidirectional = bidirectional ? 1 : 0;
  spec->max_distance = max_distance;
  spec->n_first = n_side - 1;
  // first[i] = smallest distance with bucket >= i+1 (max_distance+1 if never reached)
  int d = 0;
  for (int i = 0; i < n_side - 1; ++i) {
    while (d <= max_distance && bucket_of_distance_host(d, n_side, max_distance) < i + 1) ++d;
    spec->first[i] = (int16_t)d;   // d == max_distance+1 means "never"
  }
  for (int i = n_side - 1; i < kMaxBucketsPerSide; ++i) spec->first[i] = 32767;
  return T5B_OK;
}

int host_bucket_of_delta(const BucketSpec& s, long long delta) {
  long long d = s.bidirectional ? (delta < 0 ? -delta : delta) : (delta < 0 ? -delta : 0);
  if (d > s.max_distance) d = s.max_distance;
  int b = 0;
  while (b < s.n_first && (long long)s.first[b] <= d) ++b;
  return b + ((s.bidirectional && delta > 0) ? s.n_side : 0);
}

__global__ void bucket_indices_kernel(int32_t* __restrict__ out, int M, int N, int q_pos_offset,
                                      const __grid_constant__ BucketSpec spec) {
  const long long total = (long long)M * N;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int m = (int)(i / N), n = (int)(i % N);
    out[i] = bucket_of_delta(spec, n - (q_pos_offset + m));
  }
}

}  // namespace t5b

extern "C" int t5b_bucket_table_host(int num_buckets, int max_distance, int bidirectional,
                                     int lo, int hi, int32_t* out) {
  if (!out || hi < lo) return T5B_ERR_ARG;
  t5b::BucketSpec spec;
  int st = t5b::make_bucket_spec(num_buckets, max_distance, bidirectional, &spec);
  if (st != T5B_OK) return st;
  for (long long d = lo; d <= hi; ++d) out[d - lo] = t5b::host_bucket_of_delta(spec, d);
  return T5B_OK;
}

extern "C" int t5b_bucket_indices(int32_t* out_dev, int M, int N, int q_pos_offset,
                                  int bidirectional, int num_buckets, int max_distance,
                                  void* stream) {
  if (!out_dev) return T5B_ERR_ARG;
  if (M < 0 || N < 0) return T5B_ERR_SHAPE;
  if (M == 0 || N == 0) return T5B_OK;
  t5b::BucketSpec spec;
  int st = t5b::make_bucket_spec(num_buckets, max_distance, bidirectional, &spec);
  if (st != T5B_OK) return st;
  long long total = (long long)M * N;
  int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  t5b::bucket_indices_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(out_dev, M, N, q_pos_offset, spec);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}
