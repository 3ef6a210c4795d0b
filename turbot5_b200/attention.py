"""Fused relative-position-bias attention: the functional surface.

Same names, argument meaning and error behaviour as the TurboT5 operators they
replace:

* `flash_attention_with_fusing_bias`         src/turbot5/ops/fused_bias_attention.py:876
* `flash_attention_with_fusing_bias_varlen`  src/turbot5/ops/varlen_fused_bias_attn.py:870

plus the split-KV decoding operator the reference only sketches
(src/turbot5/ops/flash_decoding.py) and a bucket-index check.  Both attention
operators are differentiable (q, k, v and the bias table) through
`torch.autograd.Function`s that mirror `FlashAttentionBias`
(src/turbot5/ops/fused_bias_attention.py:822-873).
"""
import math
from typing import Optional

import torch

from . import _native as nat

_status_words = {}
_workspaces = {}


def device_status(device) -> torch.Tensor:
    """Per-device int32 word the kernels write to when a bounded wait runs out."""
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _status_words[key]


def check_device_status(device="cuda") -> None:
    """Synchronising check of the status word through the library's `t5b_check_status`: raises
    if a kernel's bounded wait ran out since the last check (and clears the word)."""
    word = device_status(device)
    code = nat.C.c_int32(0)
    with torch.cuda.device(word.device):
        st = nat.lib().t5b_check_status(word.data_ptr(), nat.C.byref(code), nat.stream_ptr(word.device))
    if st == nat.ERR_DEVICE_TIMEOUT:
        raise RuntimeError(f"turbot5_b200 kernel gave up waiting on the device (code {code.value})")
    nat.check(st, "check_device_status")


def _check_qkv(q, k, v):
    Dq, Dk, Dv = q.shape[-1], k.shape[-1], v.shape[-1]
    assert Dq == Dk == Dv
    assert Dk in {16, 32, 64, 128}
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("q, k and v must share a dtype")
    nat.require_cuda(q, k, v)


def _table_args(bias, H):
    if bias is None:
        return None, nat.F32, 0
    nat.require_cuda(bias)
    if bias.dim() != 2 or bias.shape[1] != H:
        raise ValueError(f"bias table must be [NUM_BUCKETS, {H}], got {tuple(bias.shape)}")
    if bias.stride(1) != 1:
        bias = bias.contiguous()
    return bias, nat.dtype_code(bias.dtype), bias.stride(0)


def _unit_stride_last(t):
    return t if t.stride(-1) == 1 else t.contiguous()


def flash_attention_with_fusing_bias(q, k, v, bias, causal=False, sm_scale=None,
                                     NUM_BUCKETS=32, MAX_DISTANCE=128, *, q_pos_offset=None,
                                     return_lse=False, kernel="auto", balance_last_wave=True, local_block=None,
                                     window=None):
    """See `_dense_forward`; differentiable in q, k, v and the bias table.  `local_block` turns the
    call into block-local attention (T5LocalAttention: the keys of the three neighbouring blocks);
    `window` into a sliding window |n - query position| < window (tensor-core kernels only:
    bf16/fp16, not causal)."""
    local_block = int(local_block or 0)
    window = int(window or 0)
    if local_block or window:
        balance_last_wave = False
    if local_block:
        q_pos_offset = 0
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, bias)):
        out, lse = _DenseAttention.apply(q, k, v, bias, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE, q_pos_offset,
                                         kernel, balance_last_wave, local_block, window)
        return (out, lse) if return_lse else out
    return _dense_forward(q, k, v, bias, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE, q_pos_offset=q_pos_offset,
                          return_lse=return_lse, kernel=kernel, balance_last_wave=balance_last_wave,
                          local_block=local_block, window=window)


def _dense_forward(q, k, v, bias, causal=False, sm_scale=None, NUM_BUCKETS=32, MAX_DISTANCE=128, *,
                   q_pos_offset=None, return_lse=False, kernel="auto", balance_last_wave=True, _keep=None,
                   local_block=0, out_f32=False, window=0):
    """softmax(sm_scale * Q K^T + T5 bias(n - m) [+ causal mask]) V without an L x L tensor.

    q (B,H,M,D), k/v (B,H,N,D), any batch/head/row strides (last dim contiguous);
    bias is the [NUM_BUCKETS, H] relative-attention table or None.  `causal`
    selects the mask and unidirectional buckets together, as in the reference.
    `sm_scale=None` means 1/sqrt(D); T5 modules pass 1.0.  The query at row m sits
    at key position `q_pos_offset + m` (default N - M, the cached-decoding
    alignment of the reference's `basic` path; sequence parallel callers pass
    their shard offset).  Returns a tensor with q's shape, dtype and strides.
    `balance_last_wave` lets the kernel split the key range of the query tiles of a partially
    filled last wave of blocks (scratch comes from a per-stream cache).
    """
    _check_qkv(q, k, v)
    B, H, M, D = q.shape
    N = k.shape[2]
    if k.shape[:2] != (B, H) or v.shape != k.shape:
        raise ValueError("k/v must be (B, H, N, D) with q's batch and heads")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    q, k, v = _unit_stride_last(q), _unit_stride_last(k), _unit_stride_last(v)
    table, tdt, ts0 = _table_args(bias, H)
    out_dtype = torch.float32 if out_f32 else q.dtype
    if q.stride(3) == 1 and q.stride(1) == D and q.stride(2) >= H * D:
        # q is a (B,H,M,D) view of token-major rows (a projection output, possibly one slice of a stacked
        # q|k|v projection): the result is laid out (B,M,H,D) so that merging the heads afterwards is free
        out = torch.empty((B, M, H, D), dtype=out_dtype, device=q.device).transpose(1, 2)
    else:
        out = torch.empty_like(q, dtype=out_dtype)
        if out.stride(-1) != 1:
            out = torch.empty(q.shape, dtype=out_dtype, device=q.device)
    lse = torch.empty((B, H, M), dtype=torch.float32, device=q.device) if return_lse else None
    a = nat.AttnArgs()
    a.out_f32 = int(bool(out_f32))
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.lse, a.table = nat.ptr(lse), nat.ptr(table)
    a.cu_seqlens_q = a.cu_seqlens_k = None
    a.device_status = device_status(q.device).data_ptr()
    a.q_stride_b, a.q_stride_h, a.q_stride_m = q.stride(0), q.stride(1), q.stride(2)
    a.k_stride_b, a.k_stride_h, a.k_stride_n = k.stride(0), k.stride(1), k.stride(2)
    a.v_stride_b, a.v_stride_h, a.v_stride_n = v.stride(0), v.stride(1), v.stride(2)
    a.o_stride_b, a.o_stride_h, a.o_stride_m = out.stride(0), out.stride(1), out.stride(2)
    a.table_stride0 = ts0
    a.dtype, a.table_dtype = nat.dtype_code(q.dtype), tdt
    a.B, a.H, a.M, a.N, a.D = B, H, M, N, D
    a.total_q = a.total_k = 0
    a.causal = int(bool(causal))
    a.num_buckets, a.max_distance = int(NUM_BUCKETS), int(MAX_DISTANCE)
    a.q_pos_offset = (N - M) if q_pos_offset is None else int(q_pos_offset)
    a.kernel = nat.KERNELS[kernel]
    a.sm_scale = float(sm_scale)
    a.workspace, a.workspace_bytes = None, 0
    a.local_block = int(local_block)
    a.window = int(window)
    with torch.cuda.device(q.device):
        if balance_last_wave:
            need = nat.lib().t5b_attention_workspace_bytes(a)
            if need > 0:
                ws = _scratch(q.device, "attn", need)
                a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        st = nat.lib().t5b_attention_fwd(a, nat.stream_ptr(q.device))
        if st == nat.ERR_UNSUPPORTED and (out_f32 or window):
            raise NotImplementedError("float32 partial outputs and sliding windows need the tensor-core forward "
                                      "kernel (bf16/fp16, 16-byte aligned rows)")
        nat.check(st, "flash_attention_with_fusing_bias")
    if _keep is not None:
        _keep.update(args=a, q=q, k=k, v=v, table=table)
    return (out, lse) if return_lse else out


def flash_attention_partial(q, k, v, bias, causal=False, sm_scale=None, NUM_BUCKETS=32, MAX_DISTANCE=128, *,
                            q_pos_offset=0, kernel="auto"):
    """Attention of q over a SLICE of the keys: returns (out, lse) with `out` in float32, for
    `merge_attention_partials`.  `q_pos_offset` is the position of query row 0 relative to the
    slice's first key (absolute query position minus the slice's first key position; may be
    negative).  Forward only."""
    try:
        return _dense_forward(q, k, v, bias, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE, q_pos_offset=q_pos_offset,
                              return_lse=True, kernel=kernel, out_f32=True)
    except NotImplementedError:
        # shapes the tensor-core kernels do not take: the partial is rounded to the element type first
        out, lse = _dense_forward(q, k, v, bias, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE,
                                  q_pos_offset=q_pos_offset, return_lse=True, kernel=kernel)
        return out.float(), lse


def merge_attention_partials(parts, dtype, return_lse=False):
    """Combine `(out float32 (B,H,M,D), lse float32 (B,H,M))` pairs computed over disjoint key
    slices into the attention over all of them (one rounding to `dtype`).  The result has the
    layout of the first partial."""
    if not 1 <= len(parts) <= nat.MERGE_MAX_PARTS:
        raise ValueError(f"between 1 and {nat.MERGE_MAX_PARTS} partial results can be merged")
    o0 = parts[0][0]
    nat.require_cuda(o0)
    B, H, M, D = o0.shape
    outs, lses = [], []
    for o, l in parts:
        if o.dtype != torch.float32 or l.dtype != torch.float32 or o.shape != o0.shape or l.shape != (B, H, M):
            raise ValueError("partials must be float32 (B,H,M,D) outputs with float32 (B,H,M) log-sum-exps")
        outs.append(o if o.stride() == o0.stride() else o.contiguous() if o0.is_contiguous() else
                    torch.empty_like(o0).copy_(o))
        lses.append(l.contiguous())
    out = torch.empty_like(o0, dtype=dtype)
    lse = torch.empty((B, H, M), dtype=torch.float32, device=o0.device) if return_lse else None
    a = nat.MergeArgs()
    for i, (o, l) in enumerate(zip(outs, lses)):
        a.part_out[i], a.part_lse[i] = o.data_ptr(), l.data_ptr()
    a.out, a.lse_out = out.data_ptr(), nat.ptr(lse)
    a.part_stride_b, a.part_stride_h, a.part_stride_m = o0.stride(0), o0.stride(1), o0.stride(2)
    a.o_stride_b, a.o_stride_h, a.o_stride_m = out.stride(0), out.stride(1), out.stride(2)
    a.n_parts, a.out_dtype = len(parts), nat.dtype_code(dtype)
    a.B, a.H, a.M, a.D = B, H, M, D
    with torch.cuda.device(o0.device):
        nat.check(nat.lib().t5b_attention_merge(a, nat.stream_ptr(o0.device)), "merge_attention_partials")
    return (out, lse) if return_lse else out


def flash_attention_with_fusing_bias_varlen(q, k, v, bias, cu_seqlens_q, cu_seqlens_k,
                                            max_seqlen_q, max_seqlen_k, causal=False, sm_scale=None,
                                            NUM_BUCKETS=32, MAX_DISTANCE=128, *, return_lse=False,
                                            kernel="auto", window=None):
    """See `_varlen_forward`; differentiable in q, k, v and the bias table.  `window`: sliding window
    |n - query position| < window inside every sequence (tensor-core kernels only).

    q, k and v may have more rows than `cu_seqlens[-1]` (buffers sized for the worst case): those rows
    are never attended and the matching output rows are not written, but the rows of k and v must
    hold finite numbers -- the last tile of the last sequence can load them, a masked key has
    probability 0, and 0 x NaN is NaN."""
    window = int(window or 0)
    if torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in (q, k, v, bias)):
        out, lse = _VarlenAttention.apply(q, k, v, bias, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                          causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE, kernel, window)
        return (out, lse) if return_lse else out
    return _varlen_forward(q, k, v, bias, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal, sm_scale,
                           NUM_BUCKETS, MAX_DISTANCE, return_lse=return_lse, kernel=kernel, window=window)


def _varlen_forward(q, k, v, bias, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=False,
                    sm_scale=None, NUM_BUCKETS=32, MAX_DISTANCE=128, *, return_lse=False, kernel="auto", _keep=None,
                    window=0):
    """Packed-sequence variant: q (Tq,H,D), k/v (Tk,H,D), int32 cu_seqlens on the device.

    Positions are relative to each sequence.  Tiles are scheduled on the device
    from cu_seqlens: no host loop, no host read of the lengths.  `max_seqlen_*`
    are accepted for signature compatibility and are not needed.
    """
    _check_qkv(q, k, v)
    Tq, H, D = q.shape
    Tk = k.shape[0]
    if k.shape[1:] != (H, D) or v.shape != k.shape:
        raise ValueError("k/v must be (Tk, H, D) with q's heads")
    nat.require_cuda(cu_seqlens_q, cu_seqlens_k)
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise TypeError("cu_seqlens must be int32")
    if cu_seqlens_q.numel() != cu_seqlens_k.numel() or cu_seqlens_q.numel() < 1:
        raise ValueError("cu_seqlens_q and cu_seqlens_k must both hold batch+1 entries")
    cu_seqlens_q, cu_seqlens_k = cu_seqlens_q.contiguous(), cu_seqlens_k.contiguous()
    nb = cu_seqlens_q.numel() - 1
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    q, k, v = _unit_stride_last(q), _unit_stride_last(k), _unit_stride_last(v)
    table, tdt, ts0 = _table_args(bias, H)
    out = torch.empty_like(q)
    if out.stride(-1) != 1:
        out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.zeros((Tq, H), dtype=torch.float32, device=q.device) if return_lse else None
    a = nat.AttnArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.lse, a.table = nat.ptr(lse), nat.ptr(table)
    a.cu_seqlens_q, a.cu_seqlens_k = cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr()
    a.device_status = device_status(q.device).data_ptr()
    a.q_stride_b, a.q_stride_h, a.q_stride_m = 0, q.stride(1), q.stride(0)
    a.k_stride_b, a.k_stride_h, a.k_stride_n = 0, k.stride(1), k.stride(0)
    a.v_stride_b, a.v_stride_h, a.v_stride_n = 0, v.stride(1), v.stride(0)
    a.o_stride_b, a.o_stride_h, a.o_stride_m = 0, out.stride(1), out.stride(0)
    a.table_stride0 = ts0
    a.dtype, a.table_dtype = nat.dtype_code(q.dtype), tdt
    a.B, a.H, a.M, a.N, a.D = nb, H, int(max_seqlen_q or 0), int(max_seqlen_k or 0), D
    a.total_q, a.total_k = Tq, Tk
    a.causal = int(bool(causal))
    a.num_buckets, a.max_distance = int(NUM_BUCKETS), int(MAX_DISTANCE)
    a.q_pos_offset = 0
    a.kernel = nat.KERNELS[kernel]
    a.sm_scale = float(sm_scale)
    a.workspace, a.workspace_bytes = None, 0
    a.local_block = 0
    a.window = int(window)
    with torch.cuda.device(q.device):
        st = nat.lib().t5b_attention_fwd(a, nat.stream_ptr(q.device))
        if st == nat.ERR_UNSUPPORTED and window:
            raise NotImplementedError("sliding windows need the tensor-core forward kernel (bf16/fp16, head dim 64 "
                                      "or 128, 16-byte aligned rows)")
        nat.check(st, "flash_attention_with_fusing_bias_varlen")
    if _keep is not None:
        _keep.update(args=a, q=q, k=k, v=v, table=table, cu_q=cu_seqlens_q, cu_k=cu_seqlens_k)
    return (out, lse) if return_lse else out


def _attention_backward(keep, out, lse, dout, varlen):
    """dq, dk, dv, dtable for the forward call recorded in `keep` (its argument block and the
    tensors it points to).  Mirrors flash_attn_v2_bwd_bias
    (src/turbot5/ops/fused_bias_attention.py:62-147): delta, then the k/v and q kernels."""
    q, k, v, table = keep["q"], keep["k"], keep["v"], keep["table"]
    row_dim = 0 if varlen else 2
    if dout.dtype != out.dtype:
        dout = dout.to(out.dtype)
    if dout.stride(-1) != 1 or dout.data_ptr() % 16 or any(s % 8 for s in dout.stride()[:-1]):
        dout = dout.contiguous()
    dq = torch.empty_strided(q.shape, q.stride(), dtype=q.dtype, device=q.device)
    dk = torch.empty_strided(k.shape, k.stride(), dtype=k.dtype, device=k.device)
    dv = torch.empty_strided(v.shape, v.stride(), dtype=v.dtype, device=v.device)
    n_keys = k.shape[row_dim]
    if n_keys == 0 or q.shape[row_dim] == 0:
        dtab = None if table is None else torch.zeros_like(table)
        return dq.zero_(), dk.zero_(), dv.zero_(), dtab
    H = q.shape[1]
    g = nat.AttnBwdArgs()
    g.fwd = keep["args"]
    g.fwd.out, g.fwd.lse = out.data_ptr(), lse.data_ptr()
    g.fwd.o_stride_h = out.stride(1)
    g.fwd.o_stride_b, g.fwd.o_stride_m = (0, out.stride(0)) if varlen else (out.stride(0), out.stride(2))
    g.fwd.workspace, g.fwd.workspace_bytes = None, 0
    g.fwd.device_status = device_status(q.device).data_ptr()
    g.dout = dout.data_ptr()
    g.do_stride_h = dout.stride(1)
    g.do_stride_b, g.do_stride_m = (0, dout.stride(0)) if varlen else (dout.stride(0), dout.stride(2))
    g.dq, g.dk, g.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    dtable = None
    if table is not None:
        dtable = torch.zeros((g.fwd.num_buckets, H), dtype=torch.float32, device=q.device)
    delta = torch.empty_like(lse)
    g.dtable, g.delta = nat.ptr(dtable), delta.data_ptr()
    g.workspace, g.workspace_bytes = None, 0
    with torch.cuda.device(q.device):
        need = nat.lib().t5b_attention_bwd_workspace_bytes(g)
        if need > 0:
            ws = _scratch(q.device, "attn_bwd", need)      # all zero at rest (the kernels restore it)
            g.workspace, g.workspace_bytes = ws.data_ptr(), ws.numel()
        st = nat.lib().t5b_attention_bwd(g, nat.stream_ptr(q.device))
    if st == nat.ERR_UNSUPPORTED:
        raise NotImplementedError("no backward kernel for this call (max_distance above 2048, a sliding window or "
                                  "kernel='tcgen05' on a shape the tensor-core backward does not take: bf16/fp16, "
                                  "16-byte aligned rows)")
    nat.check(st, "flash_attention_with_fusing_bias (backward)")
    if dtable is not None:
        dtable = dtable[: table.shape[0]].to(table.dtype)
    return dq, dk, dv, dtable


class _DenseAttention(torch.autograd.Function):
    """Autograd wrapper of the dense operator, as FlashAttentionBias
    (src/turbot5/ops/fused_bias_attention.py:822-873)."""

    @staticmethod
    def forward(ctx, q, k, v, bias, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE, q_pos_offset, kernel, balance,
                local_block=0, window=0):
        keep = {}
        out, lse = _dense_forward(q, k, v, bias, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE,
                                  q_pos_offset=q_pos_offset, return_lse=True, kernel=kernel,
                                  balance_last_wave=balance, _keep=keep, local_block=local_block, window=window)
        ctx.keep = keep
        ctx.save_for_backward(out, lse)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        out, lse = ctx.saved_tensors
        dq, dk, dv, dtable = _attention_backward(ctx.keep, out, lse, dout, varlen=False)
        return dq, dk, dv, dtable, None, None, None, None, None, None, None, None, None


class _VarlenAttention(torch.autograd.Function):
    """Autograd wrapper of the packed-sequence operator
    (src/turbot5/ops/varlen_fused_bias_attn.py: FlashAttentionBias of that file)."""

    @staticmethod
    def forward(ctx, q, k, v, bias, cu_q, cu_k, max_q, max_k, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE, kernel,
                window=0):
        keep = {}
        out, lse = _varlen_forward(q, k, v, bias, cu_q, cu_k, max_q, max_k, causal, sm_scale, NUM_BUCKETS,
                                   MAX_DISTANCE, return_lse=True, kernel=kernel, _keep=keep, window=window)
        ctx.keep = keep
        ctx.save_for_backward(out, lse)
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        out, lse = ctx.saved_tensors
        dq, dk, dv, dtable = _attention_backward(ctx.keep, out, lse, dout, varlen=True)
        return dq, dk, dv, dtable, None, None, None, None, None, None, None, None, None, None


def _scratch(device, kind: str, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch, one buffer per (device, stream, kernel kind).  The counters at
    its front must start at zero; the kernels leave them zero."""
    dev = torch.device(device)
    key = (kind, dev.index if dev.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(dev).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def _decode_workspace(device, nbytes: int) -> torch.Tensor:
    return _scratch(device, "decode", nbytes)


def flash_decoding_with_fusing_bias(q, k, v, bias, causal=False, sm_scale=None, NUM_BUCKETS=32,
                                    MAX_DISTANCE=128, *, kv_len=None, seqlens_k=None,
                                    q_pos_offset=None, num_splits=0, workspace=None):
    """Split-KV decoding step: q (B,H,M,D) with small M against a K/V cache (B,H,cap,D).

    Only the first `kv_len` keys (default: all) -- or `seqlens_k[b]` keys per batch
    row, an int32 device tensor -- are attended.  Query row m sits at key position
    kv_len - M + m unless `q_pos_offset` is given; `causal` gives the decoder
    self-attention mask and unidirectional buckets, cross attention passes
    bias=None, causal=False.  One launch: the last block per (batch, head) merges
    the splits.  Scratch comes from a per-stream cache unless `workspace` is given.
    """
    _check_qkv(q, k, v)
    B, H, M, D = q.shape
    cap = k.shape[2]
    N = cap if kv_len is None else int(kv_len)
    if N > cap or N < 0:
        raise ValueError("kv_len exceeds the cache capacity")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    q, k, v = _unit_stride_last(q), _unit_stride_last(k), _unit_stride_last(v)
    table, tdt, ts0 = _table_args(bias, H)
    out = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    L = nat.lib()
    splits = int(num_splits) if num_splits else L.t5b_decode_num_splits(B, H, N)
    need = L.t5b_decode_workspace_bytes(B, H, M, D, splits) if splits > 1 else 0
    if workspace is None and need:
        workspace = _decode_workspace(q.device, need)
    a = nat.DecodeArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.table = nat.ptr(table)
    if seqlens_k is not None:
        nat.require_cuda(seqlens_k)
        if seqlens_k.dtype != torch.int32 or seqlens_k.numel() != B:
            raise TypeError("seqlens_k must be int32 with one entry per batch row")
        seqlens_k = seqlens_k.contiguous()
    a.seqlens_k = nat.ptr(seqlens_k)
    a.workspace = nat.ptr(workspace)
    a.workspace_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    a.q_stride_b, a.q_stride_h, a.q_stride_m = q.stride(0), q.stride(1), q.stride(2)
    a.k_stride_b, a.k_stride_h, a.k_stride_n = k.stride(0), k.stride(1), k.stride(2)
    a.v_stride_b, a.v_stride_h, a.v_stride_n = v.stride(0), v.stride(1), v.stride(2)
    a.o_stride_b, a.o_stride_h, a.o_stride_m = out.stride(0), out.stride(1), out.stride(2)
    a.table_stride0 = ts0
    a.dtype, a.table_dtype = nat.dtype_code(q.dtype), tdt
    a.B, a.H, a.M, a.N, a.D = B, H, M, N, D
    a.causal = int(bool(causal))
    a.num_buckets, a.max_distance = int(NUM_BUCKETS), int(MAX_DISTANCE)
    a.q_pos_offset = -1 if q_pos_offset is None else int(q_pos_offset)
    a.num_splits = splits
    a.sm_scale = float(sm_scale)
    with torch.cuda.device(q.device):
        nat.check(L.t5b_decode_fwd(a, nat.stream_ptr(q.device)), "flash_decoding_with_fusing_bias")
    return out


def relative_position_bucket_table(num_buckets=32, max_distance=128, bidirectional=True,
                                   lo=None, hi=None) -> torch.Tensor:
    """bucket(delta) for delta in [lo, hi] as an int32 CPU tensor (host table of the library)."""
    lo = -max_distance - 1 if lo is None else int(lo)
    hi = max_distance + 1 if hi is None else int(hi)
    out = torch.empty(hi - lo + 1, dtype=torch.int32)
    nat.check(nat.lib().t5b_bucket_table_host(int(num_buckets), int(max_distance), int(bool(bidirectional)),
                                              lo, hi, out.data_ptr()), "relative_position_bucket_table")
    return out


def relative_position_bucket_grid(M, N, q_pos_offset=0, bidirectional=True, num_buckets=32,
                                  max_distance=128, device="cuda") -> torch.Tensor:
    """(M, N) int32 bucket indices computed by the device lookup the kernels use."""
    out = torch.empty((M, N), dtype=torch.int32, device=device)
    with torch.cuda.device(out.device):
        nat.check(nat.lib().t5b_bucket_indices(out.data_ptr(), M, N, int(q_pos_offset), int(bool(bidirectional)),
                                               int(num_buckets), int(max_distance), nat.stream_ptr(out.device)),
                  "relative_position_bucket_grid")
    return out
