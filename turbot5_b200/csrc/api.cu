// C-ABI entry point of the attention forward: validation and kernel choice.
#include "t5b_common.cuh"
#include "attn_params.cuh"

using namespace t5b;

extern "C" const char* t5b_status_string(int s) {
  switch (s) {
    case T5B_OK: return "ok";
    case T5B_ERR_DTYPE: return "unsupported element type";
    case T5B_ERR_SHAPE: return "bad shape";
    case T5B_ERR_ALIGN: return "pointer or stride not aligned";
    case T5B_ERR_HEAD_DIM: return "head dim must be 16, 32, 64 or 128";
    case T5B_ERR_ARG: return "bad argument";
    case T5B_ERR_LAUNCH: return "kernel launch failed";
    case T5B_ERR_DEVICE_TIMEOUT: return "a device-side wait ran out";
    case T5B_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case T5B_ERR_DRIVER: return "tensor-map encode unavailable or failed";
    case T5B_ERR_UNSUPPORTED: return "no kernel for this request";
  }
  return "unknown status";
}

extern "C" int t5b_abi_version(void) { return 1; }

extern "C" int t5b_attention_fwd(const t5b_attn_args* a, void* stream) {
  if (!a) return T5B_ERR_ARG;
  if (a->dtype != T5B_F32 && a->dtype != T5B_F16 && a->dtype != T5B_BF16) return T5B_ERR_DTYPE;
  if (a->D != 16 && a->D != 32 && a->D != 64 && a->D != 128) return T5B_ERR_HEAD_DIM;
  if (a->B < 0 || a->H < 0 || a->M < 0 || a->N < 0) return T5B_ERR_SHAPE;
  const bool varlen = a->cu_seqlens_q != nullptr || a->cu_seqlens_k != nullptr;
  if (varlen) {
    if (!a->cu_seqlens_q || !a->cu_seqlens_k) return T5B_ERR_ARG;
    if (a->total_q < 0 || a->total_k < 0) return T5B_ERR_SHAPE;
    if (a->B == 0 || a->H == 0 || a->total_q == 0) return T5B_OK;
  } else {
    if (a->B == 0 || a->H == 0 || a->M == 0) return T5B_OK;
  }
  if (!a->q || !a->out) return T5B_ERR_ARG;
  if ((!a->k || !a->v) && (varlen ? a->total_k : a->N) > 0) return T5B_ERR_ARG;
  if (a->kernel < T5B_KERNEL_AUTO || a->kernel > T5B_KERNEL_TCGEN05_2TILE) return T5B_ERR_ARG;

  BucketSpec spec;
  spec.n_side = 2; spec.bidirectional = 0; spec.max_distance = 1; spec.n_first = 0;
  if (a->table) {
    if (a->table_dtype != T5B_F32 && a->table_dtype != T5B_F16 && a->table_dtype != T5B_BF16) return T5B_ERR_DTYPE;
    const int st = make_bucket_spec(a->num_buckets, a->max_distance, a->causal ? 0 : 1, &spec);
    if (st != T5B_OK) return st;
  }
  cudaStream_t st = (cudaStream_t)stream;
  const bool tc_ok = sm100_supports(*a) && (varlen ? a->total_k : a->N) > 0;
  if (a->kernel != T5B_KERNEL_AUTO && a->kernel != T5B_KERNEL_SIMT && !tc_ok) return T5B_ERR_UNSUPPORTED;
  if (a->local_block != 0 && (!tc_ok || a->kernel == T5B_KERNEL_SIMT)) return T5B_ERR_UNSUPPORTED;
  if (a->out_f32 != 0 && (!tc_ok || a->kernel == T5B_KERNEL_SIMT)) return T5B_ERR_UNSUPPORTED;
  if (a->window != 0 && (!tc_ok || a->kernel == T5B_KERNEL_SIMT)) return T5B_ERR_UNSUPPORTED;
  if (a->kernel != T5B_KERNEL_SIMT && tc_ok) return sm100_attention_fwd(*a, spec, st);
  return simt_attention_fwd(*a, spec, st);
}

extern "C" int t5b_attention_bwd(const t5b_attn_bwd_args* g, void* stream) {
  if (!g) return T5B_ERR_ARG;
  const t5b_attn_args* a = &g->fwd;
  if (a->dtype != T5B_F32 && a->dtype != T5B_F16 && a->dtype != T5B_BF16) return T5B_ERR_DTYPE;
  if (a->D != 16 && a->D != 32 && a->D != 64 && a->D != 128) return T5B_ERR_HEAD_DIM;
  if (a->B < 0 || a->H < 0 || a->M < 0 || a->N < 0) return T5B_ERR_SHAPE;
  const bool varlen = a->cu_seqlens_q != nullptr || a->cu_seqlens_k != nullptr;
  if (varlen) {
    if (!a->cu_seqlens_q || !a->cu_seqlens_k) return T5B_ERR_ARG;
    if (a->total_q < 0 || a->total_k < 0) return T5B_ERR_SHAPE;
    if (a->B == 0 || a->H == 0 || (a->total_q == 0 && a->total_k == 0)) return T5B_OK;
  } else {
    if (a->B == 0 || a->H == 0 || (a->M == 0 && a->N == 0)) return T5B_OK;
  }
  if (!a->q || !a->k || !a->v || !a->out || !a->lse) return T5B_ERR_ARG;
  if (!g->dout || !g->dq || !g->dk || !g->dv || !g->delta) return T5B_ERR_ARG;
  if (a->local_block != 0 && (!sm100_bwd_supports(*g) || a->kernel == T5B_KERNEL_SIMT)) return T5B_ERR_UNSUPPORTED;
  if (a->out_f32 != 0) return T5B_ERR_UNSUPPORTED;                        // a forward-only mode
  if (a->window != 0 && (a->window < 0 || a->causal || a->local_block != 0 || !sm100_bwd_supports(*g) ||
                         a->kernel == T5B_KERNEL_SIMT)) return T5B_ERR_UNSUPPORTED;
  if (a->table && !g->dtable) return T5B_ERR_ARG;
  if ((varlen ? a->total_k : a->N) == 0 || (varlen ? a->total_q : a->M) == 0) return T5B_ERR_UNSUPPORTED;
  BucketSpec spec;
  spec.n_side = 2; spec.bidirectional = 0; spec.max_distance = 1; spec.n_first = 0;
  if (a->table) {
    if (a->table_dtype != T5B_F32 && a->table_dtype != T5B_F16 && a->table_dtype != T5B_BF16) return T5B_ERR_DTYPE;
    const int st = make_bucket_spec(a->num_buckets, a->max_distance, a->causal ? 0 : 1, &spec);
    if (st != T5B_OK) return st;
  }
  if (a->kernel != T5B_KERNEL_AUTO && a->kernel != T5B_KERNEL_SIMT && !sm100_bwd_supports(*g)) return T5B_ERR_UNSUPPORTED;
  if (a->kernel != T5B_KERNEL_SIMT && sm100_bwd_supports(*g)) return sm100_attention_bwd(*g, spec, (cudaStream_t)stream);
  return simt_attention_bwd(*g, spec, (cudaStream_t)stream);
}

extern "C" int64_t t5b_attention_bwd_workspace_bytes(const t5b_attn_bwd_args* g) {
  if (!g) return 0;
  const t5b_attn_args* a = &g->fwd;
  if (a->B <= 0 || a->H <= 0 || a->M <= 0 || a->N <= 0 || a->kernel == T5B_KERNEL_SIMT) return 0;
  return sm100_bwd_workspace_bytes(*g);
}

extern "C" int64_t t5b_attention_workspace_bytes(const t5b_attn_args* a) {
  if (!a || a->B <= 0 || a->H <= 0 || a->M <= 0 || a->N <= 0) return 0;
  if (a->kernel == T5B_KERNEL_SIMT || !sm100_supports(*a)) return 0;
  const TailPlan plan = sm100_tail_plan(*a);
  return plan.parts > 1 ? plan.bytes() : 0;
}

// ---------------------------------------------------------------------------
// Device-side waits that run out: reading the status word, and a self-test of the mechanism.
//
// Every wait in the tensor-core kernels is bounded (mbar_wait_bounded): when it runs out the
// thread raises its block's abort flag, stores a non-zero code in the caller's device_status
// word, and the block still frees its tensor memory and returns.  t5b_check_status is how a C
// caller reads that word; t5b_selftest_bounded_wait makes a wait run out on purpose -- a barrier
// nobody arrives at, with a short limit -- so that the path is exercised without any fault.
namespace {

__global__ void bounded_wait_selftest_kernel(int32_t* status, long long limit_cycles) {
  __shared__ unsigned long long bar_word;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_word);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar, 1);            // one arrival expected; none will come
    fence_barrier_init();
  }
  __syncthreads();
  volatile int* flag = &abort_flag;
  int fail = 0;
  if (threadIdx.x == 0) {
    // a single waiting thread, as the issuing threads of the attention kernels wait
    if (!mbar_wait_bounded(bar, 0, flag, limit_cycles)) fail = 1;
  } else if (threadIdx.x >= 32) {
    // a whole warp, as the softmax warps wait: it leaves together once the flag is up
    if (!mbar_wait_bounded_warp(bar, 0, flag)) fail = 2;
  }
  if (fail != 0 && status != nullptr) atomicCAS(status, 0, 9000 + fail);
  __syncthreads();                // every thread gets here: nothing is left waiting
}

}  // namespace

extern "C" int t5b_selftest_bounded_wait(int32_t* device_status, int64_t limit_cycles, void* stream) {
  if (!device_status) return T5B_ERR_ARG;
  if (limit_cycles <= 0 || limit_cycles > 2000000000LL) return T5B_ERR_ARG;     // at most about a second
  bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(device_status, (long long)limit_cycles);
  return cudaGetLastError() == cudaSuccess ? T5B_OK : T5B_ERR_LAUNCH;
}

extern "C" int t5b_check_status(int32_t* device_status, int32_t* code_out, void* stream) {
  if (!device_status) return T5B_ERR_ARG;
  int32_t code = 0;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemcpyAsync(&code, device_status, sizeof(code), cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess) {
    cudaGetLastError();
    return T5B_ERR_LAUNCH;
  }
  if (code_out) *code_out = code;
  if (code == 0) return T5B_OK;
  if (cudaMemsetAsync(device_status, 0, sizeof(code), st) != cudaSuccess) { cudaGetLastError(); return T5B_ERR_LAUNCH; }
  return T5B_ERR_DEVICE_TIMEOUT;
}
