/*
 * turbot5_b200 -- C ABI of the B200 (sm_100a) T5 fused-relative-bias attention path.
 *
 * Every entry point takes plain pointers, sizes and element strides, launches on
 * the CUDA stream it is given (a cudaStream_t passed as void*; NULL = the legacy
 * default stream), allocates nothing, never synchronises, and returns a
 * t5b_status (0 = ok).  Device pointers must belong to the current CUDA device.
 *
 * Each declaration names the interface of the TurboT5 reference it stands in
 * for (path inside the reference project : line).
 */
#ifndef TURBOT5_B200_H_
#define TURBOT5_B200_H_

#include <stdint.h>

#if defined(__GNUC__)
#define T5B_API __attribute__((visibility("default")))
#else
#define T5B_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  T5B_OK = 0,
  T5B_ERR_DTYPE = 1,          /* unknown / unsupported element type                      */
  T5B_ERR_SHAPE = 2,          /* negative or inconsistent sizes                          */
  T5B_ERR_ALIGN = 3,          /* pointer or stride not aligned as the kernel needs       */
  T5B_ERR_HEAD_DIM = 4,       /* head dim not in {16, 32, 64, 128}                       */
  T5B_ERR_ARG = 5,            /* null pointer, bad flag, bad bucket settings             */
  T5B_ERR_LAUNCH = 6,         /* the CUDA runtime refused the launch                     */
  T5B_ERR_DEVICE_TIMEOUT = 7, /* t5b_check_status: a kernel's bounded wait ran out        */
  T5B_ERR_WORKSPACE = 8,      /* scratch buffer missing or too small                     */
  T5B_ERR_DRIVER = 9,         /* tensor-map encode entry point unavailable / failed      */
  T5B_ERR_UNSUPPORTED = 10    /* valid request the library has no kernel for             */
} t5b_status;

typedef enum { T5B_F32 = 0, T5B_F16 = 1, T5B_BF16 = 2 } t5b_dtype;

/* Which kernel family a forward call should use.  AUTO picks the tcgen05/TMA
 * kernel whenever dtype/shape/alignment allow (bf16 or fp16, 16-byte aligned pointers and
 * strides; head dims 16 and 32 run as head dim 64 with the missing columns read as zeros and
 * only the real ones written) and the CUDA-core kernel otherwise.
 * TCGEN05_POLYEXP is the tcgen05 kernel with EVERY exponential of an unmasked tile
 * evaluated by its FMA-pipe polynomial (the default kernel sends a compile-time share of
 * them that way, none as shipped: it measured no faster); it exists so that tests can pin that
 * code path on its own.
 * The tcgen05 family has a second forward kernel at head dim 64 that gives a block two
 * 128-row query tiles and one thread per row; TCGEN05_2TILE selects it where it applies
 * (full attention, more than 128 query rows; the default kernel otherwise).  It is slower
 * than the default on B200 today and is kept selectable for measurement. */
typedef enum {
  T5B_KERNEL_AUTO = 0, T5B_KERNEL_TCGEN05 = 1, T5B_KERNEL_SIMT = 2, T5B_KERNEL_TCGEN05_POLYEXP = 3,
  T5B_KERNEL_TCGEN05_2TILE = 4
} t5b_kernel;

T5B_API const char* t5b_status_string(int status);
T5B_API int t5b_abi_version(void);

/* ---- device-side waits that ran out ----------------------------------------------
 * No counterpart in the reference (its Triton kernels have no waits of their own).  Every wait
 * inside the tensor-core kernels is bounded; one that runs out stores a non-zero code in the
 * int32 device word the call was given (device_status) and the kernel returns.
 * t5b_check_status is the one entry point that SYNCHRONISES: it waits for `stream`, reads the
 * word, and returns T5B_OK if it is zero, else T5B_ERR_DEVICE_TIMEOUT after storing the code in
 * *code_out (optional) and clearing the word.
 * t5b_selftest_bounded_wait launches a one-block kernel whose threads wait, with a limit of
 * limit_cycles SM cycles (1 .. 2e9), on a barrier that nobody arrives at, so that the give-up
 * path can be exercised on purpose: afterwards the word holds 9001 and the GPU is as usable
 * as before. */
T5B_API int t5b_check_status(int32_t* device_status, int32_t* code_out, void* stream);
T5B_API int t5b_selftest_bounded_wait(int32_t* device_status, int64_t limit_cycles, void* stream);

/* ---- relative-position buckets ------------------------------------------------
 * Stands in for T5Attention._relative_position_bucket
 * (src/turbot5/model/attentions.py:78-124).  Writes bucket(delta) for every
 * delta in [lo, hi] (delta = key position - query position) to out[hi-lo+1]
 * on the HOST.  This is the table the kernels are driven by. */
T5B_API int t5b_bucket_table_host(int num_buckets, int max_distance, int bidirectional,
                          int lo, int hi, int32_t* out);

/* Device check of the same mapping: out[m*N + n] = bucket(n - (q_pos_offset + m)),
 * computed by the device-side lookup the attention kernels use.  Replaces the
 * L x L bucket grid of T5Attention.compute_bias (attentions.py:126-137). */
T5B_API int t5b_bucket_indices(int32_t* out_dev, int M, int N, int q_pos_offset, int bidirectional,
                       int num_buckets, int max_distance, void* stream);

/* ---- fused-bias flash attention, forward --------------------------------------
 * Stands in for flash_attention_with_fusing_bias -> FlashAttentionBias.forward ->
 * flash_attn_v2_fwd_bias (src/turbot5/ops/fused_bias_attention.py:876, 822-849,
 * 23-59) and, with cu_seqlens set, for flash_attention_with_fusing_bias_varlen
 * (src/turbot5/ops/varlen_fused_bias_attn.py:870, 802-837, 37-80).
 *
 *   out = softmax(sm_scale * Q K^T + table[bucket(delta), h] (+ causal mask)) V
 *   delta = n - (q_pos_offset + m);  causal keeps delta <= 0 and selects
 *   unidirectional buckets, exactly as `causal` does in the reference.
 *
 * Dense:  q (B,H,M,D), k/v (B,H,N,D), out (B,H,M,D); strides in ELEMENTS for the
 *         batch, head and row dims; the last dim must have stride 1.
 * Varlen: cu_seqlens_q/k are int32[B+1] device arrays; q (total_q,H,D),
 *         k/v (total_k,H,D); stride_b is ignored, M/N are max_seqlen_q/k (upper
 *         bounds, used only for sizing the grid); positions are relative to each
 *         sequence and q_pos_offset is len_k - len_q per sequence.
 * table:  [num_buckets, H] in table_dtype with element stride table_stride0
 *         between buckets (stride 1 between heads); NULL = no bias.
 * lse:    optional float32 (B,H,M) dense / (total_q,H) varlen, natural log.
 * device_status: optional int32 device word; a kernel whose bounded wait ran out
 *         stores a non-zero code there instead of hanging.
 */
typedef struct {
  const void* q; const void* k; const void* v; void* out;
  float* lse;
  const void* table;
  const int32_t* cu_seqlens_q; const int32_t* cu_seqlens_k;
  int32_t* device_status;
  int64_t q_stride_b, q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_h, k_stride_n;
  int64_t v_stride_b, v_stride_h, v_stride_n;
  int64_t o_stride_b, o_stride_h, o_stride_m;
  int64_t table_stride0;
  int32_t dtype;          /* t5b_dtype of q, k, v, out */
  int32_t table_dtype;    /* t5b_dtype of table        */
  int32_t B, H, M, N, D;
  int32_t total_q, total_k;   /* varlen only: rows of q / of k and v; a cu_seqlens entry beyond them is cut there
                               * (the kernels never touch a row past a tensor) */
  int32_t causal;
  int32_t num_buckets, max_distance;
  int32_t q_pos_offset;       /* dense only; the reference's P_SEQ = N - M for cached decoding */
  int32_t kernel;             /* t5b_kernel */
  float sm_scale;
  /* Optional scratch (may be NULL): lets the tensor-core kernel split the key range of the
   * query tiles of the last, partially filled wave of blocks over several blocks and merge
   * the partial results in the same launch.  Size from t5b_attention_workspace_bytes();
   * 256-byte aligned; must be zero before its first use (the kernel leaves its counters at
   * zero); one buffer per stream in flight. */
  void* workspace;
  int64_t workspace_bytes;
  /* > 0: block-local attention as T5LocalAttention computes it
   * (src/turbot5/model/attentions.py:523-650): the queries of block i of `local_block` rows see
   * the keys of blocks i-1, i and i+1; a sequence shorter than local_block is one block; keys
   * before the first or after the last token are the reference's zero padding blocks and take
   * part unmasked.  Dense self-attention (M == N, q_pos_offset 0), not causal, tensor-core
   * kernels only, forward and backward (bf16/fp16, head dim 64/128; local_block a multiple of
   * 128 unless the sequence fits in one block), T5B_ERR_UNSUPPORTED otherwise.  0: off. */
  int32_t local_block;
  /* != 0: `out` is float32 (same element strides) although q/k/v are bf16/fp16: a partial result
   * over a slice of the keys that t5b_attention_merge combines with others before the one rounding
   * to the element type.  Tensor-core forward kernels only (T5B_ERR_UNSUPPORTED otherwise); pass
   * lse as well, the merge needs it. */
  int32_t out_f32;
  /* > 0: sliding window -- query at position p sees the keys n with |n - p| < window (and below the
   * sequence's length).  This is what T5LocalAttention computes when it is given its padding mask
   * (src/turbot5/model/utils.py:149-155,174-188: the 3-block mask ANDed with |n - m| < block_len):
   * pack the valid tokens (cu_seqlens) and pass window = block_len.  Dense or packed, not causal,
   * not combined with local_block; the tensor-core kernels only, forward (one-tile kernel) and
   * backward (T5B_ERR_UNSUPPORTED otherwise).  0: off. */
  int32_t window;
} t5b_attn_args;

T5B_API int t5b_attention_fwd(const t5b_attn_args* args, void* stream);
/* Bytes of scratch that would let t5b_attention_fwd balance its last wave on the current
 * device for these arguments (0 if splitting would not help or does not apply). */
T5B_API int64_t t5b_attention_workspace_bytes(const t5b_attn_args* args);

/* ------------------------------------------------------------------------ *
 * Backward of the fused-bias attention: replaces FlashAttentionBias.backward ->
 * flash_attn_v2_bwd_bias (src/turbot5/ops/fused_bias_attention.py:852-873, 62-147:
 * _bwd_preprocess :398-437, _bwd_kv_bias_kernel :440-632, _bwd_q_kernel_with_bias_calculation
 * :635-820) and the varlen counterpart (src/turbot5/ops/varlen_fused_bias_attn.py).
 *
 *   fwd     the forward call whose gradient is taken: same pointers, strides, sizes and
 *           flags; fwd.out and fwd.lse hold its results (lse is required here).
 *   dout    gradient of out, dtype of out, element strides do_stride_*, last dim contiguous.
 *   dq, dk, dv   written; dtype and strides of q, k, v.
 *   dtable  float32 [num_buckets, H], contiguous; the gradient of the bias table is ADDED to
 *           it (the caller zeroes it); NULL when fwd.table is NULL.
 *   delta   float32 scratch of the shape of lse.
 * bf16/fp16 with 16-byte aligned rows run on the tensor-core kernels (head dims 16 and 32 as head
 * dim 64, zero-filled); everything else the forward accepts (float32, other alignments) on CUDA-core kernels; fwd.kernel
 * selects as in the forward.  M > 0 and N > 0 (T5B_ERR_UNSUPPORTED otherwise: the gradients are
 * zero and the caller writes them).
 */
typedef struct {
  t5b_attn_args fwd;
  const void* dout;
  int64_t do_stride_b, do_stride_h, do_stride_m;
  void* dq; void* dk; void* dv;
  float* dtable;
  float* delta;
  /* Optional scratch (may be NULL), t5b_attention_bwd_workspace_bytes() bytes, 256-byte aligned,
   * ALL ZERO before its first use (the kernels leave it all zero): lets the tensor-core kernels
   * split the tiles of a partially filled last wave of blocks and add the partial gradients up
   * in float32.  One buffer per stream in flight. */
  void* workspace;
  int64_t workspace_bytes;
} t5b_attn_bwd_args;

T5B_API int t5b_attention_bwd(const t5b_attn_bwd_args* args, void* stream);
T5B_API int64_t t5b_attention_bwd_workspace_bytes(const t5b_attn_bwd_args* args);

/* ---- split-KV flash decoding ---------------------------------------------------
 * Stands in for the split/merge semantics of flash_attn_v2_fwd
 * (src/turbot5/ops/flash_decoding.py:6-55; never wired into the reference's
 * modules) and for the cached decode step of T5Attention.forward
 * (src/turbot5/model/attentions.py:198,229-234): q (B,H,M,D) with small M against
 * the first kv_len keys of k/v (B,H,capacity,D).  kv_len is either the scalar N
 * or, when seqlens_k != NULL, int32[B] on the device.  delta = n - (kv_len - M + m)
 * unless q_pos_offset >= 0 is given explicitly (cross attention passes table=NULL).
 * Splits are merged inside the same launch by the last block to finish; the
 * scratch buffer must hold t5b_decode_workspace_bytes(...) bytes and its first
 * B*H int32 counters must be zero before the first call (the kernel leaves them
 * zero again). */
typedef struct {
  const void* q; const void* k; const void* v; void* out;
  const void* table;
  const int32_t* seqlens_k;
  void* workspace; int64_t workspace_bytes;
  int64_t q_stride_b, q_stride_h, q_stride_m;
  int64_t k_stride_b, k_stride_h, k_stride_n;
  int64_t v_stride_b, v_stride_h, v_stride_n;
  int64_t o_stride_b, o_stride_h, o_stride_m;
  int64_t table_stride0;
  int32_t dtype, table_dtype;
  int32_t B, H, M, N, D;
  int32_t causal;              /* unidirectional buckets + causal mask */
  int32_t num_buckets, max_distance;
  int32_t q_pos_offset;        /* < 0: kv_len - M */
  int32_t num_splits;          /* 0 = choose */
  float sm_scale;
} t5b_decode_args;

T5B_API int64_t t5b_decode_workspace_bytes(int B, int H, int M, int D, int num_splits);
T5B_API int t5b_decode_num_splits(int B, int H, int N);
T5B_API int t5b_decode_fwd(const t5b_decode_args* args, void* stream);

/* Same decoding step for callers that cannot allocate device memory where they
 * decode (a serving loop under a frozen memory budget, a latency-critical thread
 * where an allocation could block, or C code that owns nothing but the input and
 * output buffers).  No counterpart in the
 * reference.  args->workspace and args->workspace_bytes are ignored: the split
 * scratch is a fixed 4 MiB array inside the library (held by every GPU that loads
 * it, until the process exits; t5b_decode_static_scratch_bytes() returns the
 * size).  Problems whose scratch need (t5b_decode_workspace_bytes) exceeds it are
 * refused with T5B_ERR_WORKSPACE.  The call allocates nothing and frees nothing.
 * The first call on each device looks up the array's device address; make it
 * before any stream capture begins.  All calls share the array: the counters are
 * cleared on `stream` before each launch, and calls whose kernels overlap on the
 * GPU (issued on different streams) race on it -- issue them on one stream.  Arguments are
 * checked before anything is queued: a refused call leaves the array untouched.  The address
 * looked up on the first call is kept for the life of the process; do not call this entry point
 * again after a cudaDeviceReset. */
T5B_API int64_t t5b_decode_static_scratch_bytes(void);
T5B_API int t5b_decode_fwd_static_scratch(const t5b_decode_args* args, void* stream);

/* ---- T5 RMSNorm, forward -------------------------------------------------------
 * Stands in for T5LayerNorm._forward (src/turbot5/model/modules.py:52-60) and
 * RMSLayerNorm.forward / rms_layer_norm_fwd_fused (src/turbot5/ops/rms_norm.py:
 * 129-152, 5-51).  y = w * round_w(x * rsqrt(mean(x^2) + eps)): float32 variance,
 * no mean subtraction; when w is fp16/bf16 the normalised value is rounded to w's
 * type before the multiply and y has w's type, otherwise y is float32.
 * rstd (optional, float32[rows]) receives rsqrt(mean(x^2)+eps). */
T5B_API int t5b_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd,
                    int64_t rows, int32_t d, int64_t x_row_stride, int64_t y_row_stride,
                    int32_t x_dtype, int32_t w_dtype, float eps, void* stream);

/* ---- T5 RMSNorm, backward ------------------------------------------------------
 * Stands in for RMSLayerNorm.backward -> rms_layer_norm_bwd_dx_fused and the weight-gradient
 * reduction (src/turbot5/ops/rms_norm.py:53-124, 154-185) and for autograd through
 * T5LayerNorm._forward (src/turbot5/model/modules.py:52-60).  dy has the type of the
 * forward's output (w's type when w is fp16/bf16, float32 otherwise); dx has x's type; the
 * weight gradient is ADDED to dw, float32[d] (the caller zeroes it). */
T5B_API int t5b_rmsnorm_bwd(const void* x, const void* w, const void* dy, void* dx, float* dw,
                            int64_t rows, int32_t d, int64_t x_row_stride, int64_t dy_row_stride,
                            int64_t dx_row_stride, int32_t x_dtype, int32_t w_dtype, float eps,
                            void* stream);

/* ---- merge of attention results over disjoint key ranges ---------------------------
 * out = sum_i w_i * part_out[i],  w_i = exp(part_lse[i] - max_j part_lse[j]) / sum: each part is
 * a forward call over its own slice of the keys (out_f32 set, lse requested, q_pos_offset shifted
 * by the slice's first key), and the merged result equals the call over all keys.  The rule is
 * the split merge of src/turbot5/ops/flash_decoding.py:47-55; the reference has no caller for
 * it on full attention -- here the sequence-parallel encoder uses it to start on the keys a GPU
 * already holds while the other GPUs' keys are still arriving.  part_out[i]: float32 (B,H,M,D),
 * all parts with the same element strides part_stride_*; part_lse[i]: float32 (B,H,M) contiguous,
 * natural log, -inf for a row that saw no key in that part; out: out_dtype, strides o_stride_*;
 * lse_out: optional merged log-sum-exp. */
#define T5B_MERGE_MAX_PARTS 8
typedef struct {
  const float* part_out[T5B_MERGE_MAX_PARTS];
  const float* part_lse[T5B_MERGE_MAX_PARTS];
  void* out;
  float* lse_out;
  int64_t part_stride_b, part_stride_h, part_stride_m;
  int64_t o_stride_b, o_stride_h, o_stride_m;
  int32_t n_parts;
  int32_t out_dtype;      /* t5b_dtype of out */
  int32_t B, H, M, D;
} t5b_merge_args;

T5B_API int t5b_attention_merge(const t5b_merge_args* args, void* stream);

/* ---- residual add + T5 RMSNorm in one pass ---------------------------------------
 * hidden_out = hidden + branch (rounded to the element type, as the residual adds of
 * T5LayerSelfAttention / T5LayerFF do, src/turbot5/model/modeling.py:124-128, 142-164);
 * normed = T5 RMSNorm(hidden_out) with the rounding points of t5b_rmsnorm_fwd
 * (src/turbot5/model/modules.py:52-60).  hidden_out may alias hidden.  bf16/fp16 rows of
 * d elements (d % 8 == 0, d <= 2048), 16-byte aligned, row strides in elements; the weight
 * has the element type or is float32 (normed keeps the element type either way). */
T5B_API int t5b_add_rmsnorm_fwd(const void* hidden, const void* branch, const void* weight, void* hidden_out,
                                void* normed, int64_t rows, int32_t d, int64_t hidden_stride,
                                int64_t branch_stride, int64_t hidden_out_stride, int64_t normed_stride,
                                int32_t dtype, int32_t w_dtype, float eps, void* stream);

/* ---- gated GELU over one concatenated projection -------------------------------------
 * out[r, c] = round(gelu_tanh(x[r, c])) * x[r, d_ff + c] for x = hidden @ [wi_0; wi_1]^T, the
 * middle of T5DenseGatedActDense (src/turbot5/model/modeling.py:83-100; the reference's own
 * fused version is src/turbot5/ops/gated_mlp.py:83-225).  bf16/fp16, d_ff % 8 == 0, 16-byte
 * aligned rows, row strides in elements. */
T5B_API int t5b_gated_gelu_fwd(const void* x, void* out, int64_t rows, int32_t d_ff, int64_t x_stride,
                               int64_t out_stride, int32_t dtype, void* stream);

/* ---- unpad / pad glue -----------------------------------------------------------
 * Stand in for _get_unpad_data, index_first_axis and pad_input
 * (src/turbot5/model/padding.py:79-88, 46-76, 30-44) without the host
 * synchronisation of the reference (.item() at padding.py:82).
 *
 * t5b_unpad_plan: mask (B, L) of mask_dtype_bytes-wide integers (1/2/4/8; non-zero
 *   = keep) -> seqlens int32[B], cu_seqlens int32[B+1], dest int32[B*L]: the row of
 *   each kept token in the packed layout (>= 0); a dropped token gets -2 - r with r
 *   a distinct row of the unused tail [total_kept, B*L) of the packed buffer.
 * t5b_gather_rows: packed[dest[i], :] = padded[i, :] for kept tokens, and the tail
 *   row of every dropped token is zero-filled, so all B*L packed rows are defined.
 * t5b_scatter_rows: padded[i, :] = dest[i] >= 0 ? packed[dest[i], :] : 0.
 * Rows are row_bytes long (multiple of 16), row strides in bytes. */
T5B_API int t5b_unpad_plan(const void* mask, int32_t mask_elem_bytes, int32_t B, int32_t L,
                   int32_t* seqlens, int32_t* cu_seqlens, int32_t* dest, void* stream);
T5B_API int t5b_gather_rows(const void* padded, int64_t padded_row_stride_bytes, void* packed,
                    int64_t packed_row_stride_bytes, const int32_t* dest, int64_t n_rows,
                    int32_t row_bytes, void* stream);
T5B_API int t5b_scatter_rows(const void* packed, int64_t packed_row_stride_bytes, void* padded,
                     int64_t padded_row_stride_bytes, const int32_t* dest, int64_t n_rows,
                     int32_t row_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TURBOT5_B200_H_ */
