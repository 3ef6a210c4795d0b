"""Module-level drop-ins: `T5LayerNorm`, `T5FlashAttention`, `T5ATTENTION_TYPES`.

Same constructor arguments, parameter names (`q`, `k`, `v`, `o`,
`relative_attention_bias`, `weight`) and return tuples as the TurboT5 modules
(src/turbot5/model/attentions.py:387-521, src/turbot5/model/modules.py:43-67,
registry at src/turbot5/model/modeling.py:54-61), so HF T5 checkpoints load
unchanged and `attention_type='flash'` selects this module.
"""
import torch
from torch import nn

from . import _native as nat
from .attention import (flash_attention_with_fusing_bias, flash_attention_with_fusing_bias_varlen,
                        flash_decoding_with_fusing_bias)
from .padding import get_unpad_plan, pad_rows, unpad_rows


def rms_layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, return_rstd: bool = False):
    """T5 RMSNorm on the device (replaces RMSLayerNorm.apply, src/turbot5/ops/rms_norm.py:129-185);
    differentiable in x and weight."""
    if not return_rstd and torch.is_grad_enabled() and (x.requires_grad or weight.requires_grad):
        return _RMSNormFn.apply(x, weight, eps)
    return _rms_layer_norm_fwd(x, weight, eps, return_rstd)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        ctx.save_for_backward(x, weight)
        ctx.eps = eps
        return _rms_layer_norm_fwd(x, weight, eps)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        d = x.shape[-1]
        x2 = x.reshape(-1, d)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        out_dtype = weight.dtype if weight.dtype in (torch.float16, torch.bfloat16) else torch.float32
        dy2 = dy.reshape(-1, d).to(out_dtype)
        if dy2.stride(-1) != 1:
            dy2 = dy2.contiguous()
        dx = torch.empty((x2.shape[0], d), dtype=x.dtype, device=x.device)
        dw = torch.zeros((d,), dtype=torch.float32, device=x.device)
        w = weight.contiguous()
        with torch.cuda.device(x.device):
            nat.check(nat.lib().t5b_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), dx.data_ptr(),
                                                dw.data_ptr(), x2.shape[0], d, x2.stride(0), dy2.stride(0),
                                                dx.stride(0), nat.dtype_code(x.dtype), nat.dtype_code(w.dtype),
                                                float(ctx.eps), nat.stream_ptr(x.device)), "rms_layer_norm (backward)")
        return dx.view(x.shape), dw.to(weight.dtype), None


def _rms_layer_norm_fwd(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, return_rstd: bool = False):
    nat.require_cuda(x, weight)
    d = x.shape[-1]
    if weight.shape != (d,):
        raise ValueError("weight must have the size of the last dimension")
    x2 = x.reshape(-1, d)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    weight = weight.contiguous()
    out_dtype = weight.dtype if weight.dtype in (torch.float16, torch.bfloat16) else torch.float32
    y = torch.empty((x2.shape[0], d), dtype=out_dtype, device=x.device)
    rstd = torch.empty((x2.shape[0],), dtype=torch.float32, device=x.device) if return_rstd else None
    with torch.cuda.device(x.device):
        nat.check(nat.lib().t5b_rmsnorm_fwd(x2.data_ptr(), weight.data_ptr(), y.data_ptr(), nat.ptr(rstd),
                                            x2.shape[0], d, x2.stride(0), y.stride(0), nat.dtype_code(x.dtype),
                                            nat.dtype_code(weight.dtype), float(eps), nat.stream_ptr(x.device)),
                  "rms_layer_norm")
    y = y.view(*x.shape[:-1], d)
    return (y, rstd) if return_rstd else y


def add_rms_layer_norm(hidden: torch.Tensor, branch: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6,
                       inplace: bool = False):
    """(hidden + branch, T5 RMSNorm(hidden + branch)) in one pass over memory: the residual add that
    closes a sub-layer fused with the norm that opens the next one
    (src/turbot5/model/modeling.py:124-128,142-164 + src/turbot5/model/modules.py:52-60).  bf16/fp16,
    forward only; with `inplace` the sum overwrites `hidden`."""
    nat.require_cuda(hidden, branch, weight)
    d = hidden.shape[-1]
    if branch.shape != hidden.shape or branch.dtype != hidden.dtype or weight.shape != (d,):
        raise ValueError("hidden and branch must match; weight must have the size of the last dimension")
    h2, b2 = hidden.reshape(-1, d), branch.reshape(-1, d)
    if h2.stride(-1) != 1:
        h2 = h2.contiguous()
    if b2.stride(-1) != 1:
        b2 = b2.contiguous()
    same = inplace and h2.data_ptr() == hidden.data_ptr()
    h_out = h2 if same else torch.empty((h2.shape[0], d), dtype=hidden.dtype, device=hidden.device)
    normed = torch.empty((h2.shape[0], d), dtype=hidden.dtype, device=hidden.device)
    weight = weight.contiguous()
    with torch.cuda.device(hidden.device):
        nat.check(nat.lib().t5b_add_rmsnorm_fwd(h2.data_ptr(), b2.data_ptr(), weight.data_ptr(), h_out.data_ptr(),
                                                normed.data_ptr(), h2.shape[0], d, h2.stride(0), b2.stride(0),
                                                h_out.stride(0), normed.stride(0), nat.dtype_code(hidden.dtype),
                                                nat.dtype_code(weight.dtype), float(eps),
                                                nat.stream_ptr(hidden.device)), "add_rms_layer_norm")
    return h_out.view(hidden.shape), normed.view(hidden.shape)


def gated_gelu(x: torch.Tensor) -> torch.Tensor:
    """gelu_tanh(x[..., :F]) * x[..., F:] for the output x of one matrix product with the
    concatenated wi_0 | wi_1 weights (T5DenseGatedActDense, src/turbot5/model/modeling.py:83-100).
    bf16/fp16, forward only."""
    nat.require_cuda(x)
    f2 = x.shape[-1]
    if f2 % 2:
        raise ValueError("the last dimension holds the two projections side by side")
    x2 = x.reshape(-1, f2)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty((x2.shape[0], f2 // 2), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        nat.check(nat.lib().t5b_gated_gelu_fwd(x2.data_ptr(), out.data_ptr(), x2.shape[0], f2 // 2, x2.stride(0),
                                               out.stride(0), nat.dtype_code(x.dtype), nat.stream_ptr(x.device)),
                  "gated_gelu")
    return out.view(*x.shape[:-1], f2 // 2)


class RMSLayerNorm:
    """`RMSLayerNorm.apply(x, weight, eps)` call shape of the reference."""

    @staticmethod
    def apply(x, weight, eps):
        return rms_layer_norm(x, weight, eps)


class T5LayerNorm(nn.Module):
    """T5-style RMS norm: no mean subtraction, no bias (src/turbot5/model/modules.py:43-67).

    `use_triton` is accepted for source compatibility and ignored: the CUDA
    kernel is the only implementation.
    """

    def __init__(self, dim: int, eps: float = 1e-6, use_triton=False):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))
        self.use_triton = use_triton

    def forward(self, x: torch.Tensor):
        return rms_layer_norm(x, self.weight, self.eps)


class T5FlashAttention(nn.Module):
    """Attention module backed by the fused-bias kernels.

    Constructor and forward signature of src/turbot5/model/attentions.py:387-403.
    Differences from the reference module, all in the direction of its `basic`
    semantics: cached decoding uses absolute positions (delta = n - (N - M + m));
    a padding mask never triggers a host synchronisation (the reference calls
    `torch.sum(mask)` and `.item()`, attentions.py:410-416, padding.py:82); decoder
    self- and cross-attention are supported (`cross_attention=True` => no mask,
    no bias unless the layer owns a table).  `layer_head_mask`, dropout and
    `output_attentions` are ignored exactly as in the reference (:483).
    """

    def __init__(self, config, cross_attention=False, has_relative_attention_bias=False):
        super().__init__()
        self.config = config
        self.is_decoder = config.is_decoder
        self.has_relative_attention_bias = has_relative_attention_bias
        self.relative_attention_num_buckets = config.relative_attention_num_buckets
        self.relative_attention_max_distance = config.relative_attention_max_distance
        self.d_model = config.d_model
        self.key_value_proj_dim = config.d_kv
        self.n_heads = config.num_heads
        self.dropout = config.dropout_rate
        self.inner_dim = self.n_heads * self.key_value_proj_dim
        self.q = nn.Linear(self.d_model, self.inner_dim, bias=False)
        self.k = nn.Linear(self.d_model, self.inner_dim, bias=False)
        self.v = nn.Linear(self.d_model, self.inner_dim, bias=False)
        self.o = nn.Linear(self.inner_dim, self.d_model, bias=False)
        if self.has_relative_attention_bias:
            self.relative_attention_bias = nn.Embedding(self.relative_attention_num_buckets, self.n_heads)
        self.pruned_heads = set()
        self.gradient_checkpointing = False
        self.causal = config.is_decoder and not cross_attention
        # decoding steps with at most this many query rows use the split-KV kernel
        self.decode_max_rows = 8

    def forward(self, hidden_states, mask=None, key_value_states=None, position_bias=None,
                past_key_value=None, layer_head_mask=None, query_length=None, use_cache=False,
                output_attentions=False):
        batch_size, seq_length = hidden_states.shape[:2]
        H, D = self.n_heads, self.key_value_proj_dim
        if past_key_value is not None and len(past_key_value) != 2:
            raise ValueError(
                f"past_key_value should have 2 past states: keys and values. Got { len(past_key_value)} past states")

        def shape(states):
            return states.view(batch_size, -1, H, D).transpose(1, 2)

        def unshape(states):
            return states.transpose(1, 2).contiguous().view(batch_size, -1, self.inner_dim)

        def project(hidden, proj, kv_states, past):
            if kv_states is None:
                out = shape(proj(hidden))
                if past is not None:
                    out = torch.cat([past, out], dim=2)
                return out
            if past is None or past.shape[2] != kv_states.shape[1]:
                return shape(proj(kv_states))
            return past

        query_states = shape(self.q(hidden_states))
        key_states = project(hidden_states, self.k, key_value_states,
                             past_key_value[0] if past_key_value is not None else None)
        value_states = project(hidden_states, self.v, key_value_states,
                               past_key_value[1] if past_key_value is not None else None)
        if position_bias is None and self.has_relative_attention_bias:
            position_bias = self.relative_attention_bias.weight
        table = position_bias if (position_bias is not None and position_bias.dim() == 2) else None
        nb, md = self.relative_attention_num_buckets, self.relative_attention_max_distance

        needs_grad = torch.is_grad_enabled() and any(
            t is not None and t.requires_grad for t in (query_states, key_states, value_states, table))
        if mask is None:
            # the split-KV decoding operator has no backward: a short decoder input in training
            # (e.g. a few target tokens against a long encoder memory) takes the dense operator
            if seq_length <= self.decode_max_rows and key_states.shape[2] > seq_length and not needs_grad:
                attn = flash_decoding_with_fusing_bias(query_states, key_states, value_states, table,
                                                       causal=self.causal, sm_scale=1.0,
                                                       NUM_BUCKETS=nb, MAX_DISTANCE=md,
                                                       q_pos_offset=0 if key_value_states is not None else None)
            else:
                attn = flash_attention_with_fusing_bias(query_states, key_states, value_states, table,
                                                        causal=self.causal, sm_scale=1.0,
                                                        NUM_BUCKETS=nb, MAX_DISTANCE=md,
                                                        q_pos_offset=0 if key_value_states is not None else None)
        else:
            # padded batch: pack the kept tokens, run the packed-sequence kernel, scatter back
            if mask.dim() != 2:
                raise ValueError("T5FlashAttention takes the raw 0/1 (batch, key_length) mask")
            plan_k = get_unpad_plan(mask)
            k_p = unpad_rows(key_states.transpose(1, 2), plan_k)
            v_p = unpad_rows(value_states.transpose(1, 2), plan_k)
            # The mask describes the KEYS.  Only in plain self-attention (no encoder memory, no
            # cache) are the queries the same padded tokens; in cross attention the decoder rows
            # are all real even when the decoder happens to be as long as the encoder.
            if key_value_states is None and past_key_value is None:
                plan_q = plan_k
                q_p = unpad_rows(query_states.transpose(1, 2), plan_q)
            else:
                # queries are not padded (cross attention / cached decoding): every row is kept
                plan_q = get_unpad_plan(torch.ones((batch_size, seq_length), dtype=torch.uint8,
                                                   device=hidden_states.device))
                q_p = query_states.transpose(1, 2).reshape(batch_size * seq_length, H, D)
            out_p = flash_attention_with_fusing_bias_varlen(
                q_p, k_p, v_p, table, plan_q.cu_seqlens, plan_k.cu_seqlens, seq_length, key_states.shape[2],
                causal=self.causal, sm_scale=1.0, NUM_BUCKETS=nb, MAX_DISTANCE=md)
            attn = pad_rows(out_p, plan_q).transpose(1, 2)

        attn_output = self.o(unshape(attn))
        present_key_value_state = (key_states, value_states) if (self.is_decoder and use_cache) else None
        outputs = (attn_output,) + (present_key_value_state,) + (position_bias,)
        if output_attentions:
            outputs = outputs + (None,)
        return outputs


class T5LocalFlashAttention(T5FlashAttention):
    """Block-local attention (LongT5-style) on the fused-bias kernel: `T5LocalAttention` of the
    reference (src/turbot5/model/attentions.py:523-650) without its reshapes.

    The reference splits q/k/v into blocks of `config.sliding_window` rows, concatenates each
    block's two neighbours (zero blocks at the ends) and materialises a (block, 3 x block) bias; here
    the same kernel that serves full attention walks only the three blocks of keys a query tile
    can see, the zero blocks come from the TMA's out-of-bounds fill, and the bias is looked up
    per element as always.  Encoder self-attention, no cache; differentiable without a mask.

    With the raw 0/1 (batch, length) padding mask the reference's mask for this module
    (`_get_local_attention_mask`, src/turbot5/model/utils.py:149-155,174-188, added as -1e10 at
    attentions.py:600-603,619-621) makes a pair visible when both tokens are valid and
    |key - query| < block length: a sliding window over the valid keys.  Here the valid tokens are
    packed (no host synchronisation), the packed-sequence kernel runs with that window, and the
    rows of padded queries come back as zeros (differentiable: the packed kernel's backward takes
    the same window).  As in the full-attention module the
    mask is taken to be right-padded (positions are counted inside the packed sequences).
    """

    def __init__(self, config, has_relative_attention_bias=False, **kwargs):
        super().__init__(config, cross_attention=False, has_relative_attention_bias=has_relative_attention_bias)
        self.block_len = config.sliding_window

    def forward(self, hidden_states, mask=None, position_bias=None, layer_head_mask=None, past_key_value=None,
                use_cache=None, output_attentions=False, **kwargs):
        if self.is_decoder:
            raise NotImplementedError("T5LocalFlashAttention covers encoder self-attention only")
        batch_size, seq_length = hidden_states.shape[:2]
        H, D = self.n_heads, self.key_value_proj_dim
        shape = lambda x: x.view(batch_size, -1, H, D).transpose(1, 2)
        q, k, v = shape(self.q(hidden_states)), shape(self.k(hidden_states)), shape(self.v(hidden_states))
        table = None
        if position_bias is not None:
            table = position_bias
        elif self.has_relative_attention_bias:
            table = self.relative_attention_bias.weight
        nb, md = self.relative_attention_num_buckets, self.relative_attention_max_distance
        if mask is None:
            attn = flash_attention_with_fusing_bias(q, k, v, table, causal=False, sm_scale=1.0, NUM_BUCKETS=nb,
                                                    MAX_DISTANCE=md, local_block=self.block_len)
        else:
            if mask.dim() != 2:
                raise ValueError("T5LocalFlashAttention takes the raw 0/1 (batch, length) mask")
            plan = get_unpad_plan(mask)
            q_p, k_p, v_p = (unpad_rows(t.transpose(1, 2), plan) for t in (q, k, v))
            out_p = flash_attention_with_fusing_bias_varlen(q_p, k_p, v_p, table, plan.cu_seqlens, plan.cu_seqlens,
                                                            seq_length, seq_length, causal=False, sm_scale=1.0,
                                                            NUM_BUCKETS=nb, MAX_DISTANCE=md, window=self.block_len)
            attn = pad_rows(out_p, plan).transpose(1, 2)
        out = self.o(attn.transpose(1, 2).contiguous().view(batch_size, -1, self.inner_dim))
        outputs = (out, None, table)
        if output_attentions:
            outputs = outputs + (None,)
        return outputs


T5ATTENTION_TYPES = {
    "flash": T5FlashAttention,
    "local": T5LocalFlashAttention,
}
