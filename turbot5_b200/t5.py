"""A thin T5 encoder / decoder stack around the fused-bias kernels.

Only what is needed to drive the attention path end to end (and to measure
encoder tokens/s): embeddings, pre-norm blocks (RMSNorm -> attention -> residual,
RMSNorm -> feed-forward -> residual), final norm, LM head.  Linear layers are
plain `nn.Linear` (cuBLAS); attention, RMSNorm and decoding go through the
library.  Module and parameter names follow the Hugging Face / TurboT5 layout
(`shared`, `encoder.block.N.layer.0.SelfAttention.q`, `...layer.1.DenseReluDense.wi_0`,
`decoder.block.N.layer.1.EncDecAttention.k`, `lm_head`), so a T5 state dict
loads with `load_state_dict`.

Restates the control flow of `T5Stack` / `T5Block` / `T5LayerSelfAttention` /
`T5LayerCrossAttention` / `T5LayerFF` (src/turbot5/model/modeling.py:63-342,
352-632) and the LM head of `T5ForConditionalGeneration`
(src/turbot5/heads/t5_heads.py:132-260).  Differences: the decoder uses the
flash module too (the reference hard-wires its `basic` attention there,
modeling.py:134-135,170) and generation keeps a preallocated K/V cache that the
split-KV decoding kernel reads in place, instead of `torch.cat` per step
(src/turbot5/model/attentions.py:198).
"""
from dataclasses import dataclass
from typing import List, Optional

import torch
from torch import nn

from .attention import (flash_attention_with_fusing_bias, flash_attention_with_fusing_bias_varlen,
                        flash_decoding_with_fusing_bias)
from .modules import (T5ATTENTION_TYPES, T5FlashAttention, T5LayerNorm, add_rms_layer_norm, gated_gelu,
                      rms_layer_norm)


@dataclass
class T5StackConfig:
    vocab_size: int = 32128
    d_model: int = 768
    d_kv: int = 64
    d_ff: int = 2048
    num_layers: int = 12
    num_decoder_layers: int = 12
    num_heads: int = 12
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    dropout_rate: float = 0.0
    layer_norm_epsilon: float = 1e-6
    feed_forward_proj: str = "gated-gelu"      # or "relu"
    tie_word_embeddings: bool = False
    is_decoder: bool = False
    decoder_start_token_id: int = 0
    attention_type: str = "flash"              # encoder self-attention: "flash" (full) or "local" (block-local)
    sliding_window: int = 512                  # block length of the "local" type


class _FusedOps:
    """Library operators behind `T5Stack.forward_fused`."""
    from .sequence_parallel import _DeviceOps as _sp
    rms_layer_norm = staticmethod(rms_layer_norm)
    add_rms_layer_norm = staticmethod(add_rms_layer_norm)
    gated_gelu = staticmethod(gated_gelu)
    attention = _sp.attention
    partial = _sp.partial
    merge = _sp.merge


class T5DenseGatedActDense(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.wi_0 = nn.Linear(cfg.d_model, cfg.d_ff, bias=False)
        self.wi_1 = nn.Linear(cfg.d_model, cfg.d_ff, bias=False)
        self.wo = nn.Linear(cfg.d_ff, cfg.d_model, bias=False)

    def forward(self, x):
        return self.wo(nn.functional.gelu(self.wi_0(x), approximate="tanh") * self.wi_1(x))


class T5DenseActDense(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.wi = nn.Linear(cfg.d_model, cfg.d_ff, bias=False)
        self.wo = nn.Linear(cfg.d_ff, cfg.d_model, bias=False)

    def forward(self, x):
        return self.wo(torch.relu(self.wi(x)))


class T5LayerFF(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        gated = cfg.feed_forward_proj.startswith("gated")
        self.DenseReluDense = T5DenseGatedActDense(cfg) if gated else T5DenseActDense(cfg)
        self.layer_norm = T5LayerNorm(cfg.d_model, eps=cfg.layer_norm_epsilon)

    def forward(self, hidden):
        return hidden + self.DenseReluDense(self.layer_norm(hidden).to(hidden.dtype))


class T5LayerSelfAttention(nn.Module):
    def __init__(self, cfg, has_relative_attention_bias):
        super().__init__()
        # the decoder always attends fully (as in the reference, src/turbot5/model/modeling.py:134-135)
        kind = T5FlashAttention if cfg.is_decoder else T5ATTENTION_TYPES[cfg.attention_type]
        self.SelfAttention = kind(cfg, has_relative_attention_bias=has_relative_attention_bias)
        self.layer_norm = T5LayerNorm(cfg.d_model, eps=cfg.layer_norm_epsilon)


class T5LayerCrossAttention(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.EncDecAttention = T5FlashAttention(cfg, cross_attention=True, has_relative_attention_bias=False)
        self.layer_norm = T5LayerNorm(cfg.d_model, eps=cfg.layer_norm_epsilon)


class T5Block(nn.Module):
    def __init__(self, cfg, has_relative_attention_bias):
        super().__init__()
        layers = [T5LayerSelfAttention(cfg, has_relative_attention_bias)]
        if cfg.is_decoder:
            layers.append(T5LayerCrossAttention(cfg))
        layers.append(T5LayerFF(cfg))
        self.layer = nn.ModuleList(layers)


class DecoderCache:
    """Preallocated K/V cache of one generation: self-attention keys/values grow in place,
    cross-attention keys/values are projected once from the encoder output.  Keys and values of a
    layer's self-attention live in ONE tensor (2, B, H, max_len, D), so that a decoding step appends
    both with one copy; `self_k[i]` / `self_v[i]` are its two halves."""

    def __init__(self, n_layers, batch, heads, d_kv, max_len, dtype, device):
        self.self_kv = [torch.empty((2, batch, heads, max_len, d_kv), dtype=dtype, device=device) for _ in range(n_layers)]
        self.self_k = [kv[0] for kv in self.self_kv]
        self.self_v = [kv[1] for kv in self.self_kv]
        self.cross_k: List[Optional[torch.Tensor]] = [None] * n_layers
        self.cross_v: List[Optional[torch.Tensor]] = [None] * n_layers
        self.length = 0
        self.max_len = max_len


class T5Stack(nn.Module):
    def __init__(self, cfg: T5StackConfig, embed_tokens: nn.Embedding, is_decoder: bool):
        super().__init__()
        cfg = T5StackConfig(**{**cfg.__dict__, "is_decoder": is_decoder})
        self.cfg = cfg
        self.is_decoder = is_decoder
        self.embed_tokens = embed_tokens
        n = cfg.num_decoder_layers if is_decoder else cfg.num_layers
        self.block = nn.ModuleList([T5Block(cfg, has_relative_attention_bias=(i == 0)) for i in range(n)])
        self.final_layer_norm = T5LayerNorm(cfg.d_model, eps=cfg.layer_norm_epsilon)

    def _table(self):
        return self.block[0].layer[0].SelfAttention.relative_attention_bias.weight

    def forward(self, input_ids=None, attention_mask=None, inputs_embeds=None, encoder_hidden_states=None,
                encoder_attention_mask=None):
        """Full (uncached) pass.  `attention_mask` is the raw 0/1 (B, L) mask or None."""
        hidden = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        table = self._table()
        for blk in self.block:
            sa = blk.layer[0]
            normed = sa.layer_norm(hidden).to(hidden.dtype)
            hidden = hidden + sa.SelfAttention(normed, mask=None if self.is_decoder else attention_mask,
                                               position_bias=table)[0]
            if self.is_decoder:
                ca = blk.layer[1]
                normed = ca.layer_norm(hidden).to(hidden.dtype)
                hidden = hidden + ca.EncDecAttention(normed, mask=encoder_attention_mask,
                                                     key_value_states=encoder_hidden_states)[0]
            hidden = blk.layer[-1](hidden)
        return self.final_layer_norm(hidden).to(hidden.dtype)

    # ---- inference pass of an encoder with the token-wise work fused around the attention path
    def _stacked_weights(self, i):
        """Per block: [q; k; v], [k; v], the cross-attention [k; v] and [wi_0; wi_1] weights stacked once,
        so each group is one matrix product.  Rebuilt when a parameter has been modified in place or
        replaced."""
        blk = self.block[i]
        att, ff = blk.layer[0].SelfAttention, blk.layer[-1].DenseReluDense
        gated = hasattr(ff, "wi_0")
        groups = dict(qkv=[att.q.weight, att.k.weight, att.v.weight], kv=[att.k.weight, att.v.weight])
        if self.is_decoder:
            catt = blk.layer[1].EncDecAttention
            groups["ckv"] = [catt.k.weight, catt.v.weight]
        if gated:
            groups["wi"] = [ff.wi_0.weight, ff.wi_1.weight]
        key = tuple((w.data_ptr(), w._version, w.dtype, w.device) for ws in groups.values() for w in ws)
        cache = self.__dict__.setdefault("_stacked", {})
        hit = cache.get(i)
        if hit is None or hit[0] != key:
            with torch.no_grad():
                cache[i] = hit = (key, {name: torch.cat(ws, 0) for name, ws in groups.items()})
        return hit[1]

    @torch.no_grad()
    def forward_fused(self, input_ids=None, inputs_embeds=None, seq_len=None, group=None, overlap=True, ops=None,
                      encoder_hidden_states=None, attention_mask=None, packed_rows=None, return_packed=False,
                      encoder_plan=None):
        """Forward pass without padding masks and without gradients, with the token-wise work fused
        around the attention path: per encoder block eight launches -- stacked q/k/v projection,
        attention, output projection, residual add fused with the next RMSNorm, stacked wi_0|wi_1
        projection, gated GELU, wo projection, residual add + RMSNorm -- and five more per decoder
        block for the cross attention (q projection, stacked k/v projection of the encoder states,
        attention, output projection, residual add + RMSNorm).  Same arithmetic and rounding points
        as `forward` (the blocks of src/turbot5/model/modeling.py:124-128,142-164,166-219,221-342).

        With `seq_len` given the pass is sequence parallel (encoder stacks): `input_ids` /
        `inputs_embeds` hold this rank's token shard (B, S), S = ceil(seq_len / world), every
        token-wise operation runs on the shard, and each attention layer gathers the other ranks'
        keys and values (see `sequence_parallel_attention_overlapped`; `overlap=False` gathers first
        and attends once).  Returns the normed hidden states of the rows this call was given.
        With `attention_mask` (encoder stacks; the raw 0/1 (B, L) mask, right-padded) the valid tokens
        are packed ONCE, after the embedding: every projection, norm and feed-forward layer then runs
        on the packed rows only, the attention layers use the packed-sequence kernel, and the result is
        scattered back at the end (zeros at padded positions) -- where the reference unpads and pads
        around every attention call and does everything else on the padded batch
        (src/turbot5/model/attentions.py:405-470, model/padding.py:113-150).  `packed_rows` is an
        upper bound on the number of valid tokens known to the caller (e.g. from the tokenizer; with a bound
        below the true count the result is all NaN); without it the count is read back from the device once
        per call.
        `return_packed=True` skips the final scatter and returns (packed states (T, d_model), plan): a
        decoder stack takes them as `encoder_hidden_states` (2-D) with `encoder_plan=plan` and its cross
        attention then reads the packed keys directly (packed-sequence kernel, no bias), so the encoder
        output is never padded again.

        `ops` replaces the library operators (an object with rms_layer_norm, add_rms_layer_norm,
        gated_gelu, attention and the partial / merge pair of the sequence-parallel path): tests of
        the sharding logic on CPU ranks pass reference implementations.
        """
        ops = ops or _FusedOps
        cfg = self.cfg
        if self.is_decoder and (encoder_hidden_states is None or seq_len is not None):
            raise ValueError("a decoder stack needs encoder_hidden_states and is not sequence parallel")
        if (encoder_plan is not None) != (encoder_hidden_states is not None and encoder_hidden_states.dim() == 2):
            raise ValueError("packed encoder states (T, d_model) go together with encoder_plan")
        x = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        plan = None
        if attention_mask is not None:
            if self.is_decoder or seq_len is not None:
                raise ValueError("attention_mask is taken by unsharded encoder stacks")
            from .padding import get_unpad_plan, pad_rows, unpad_rows
            plan = get_unpad_plan(attention_mask)
            pad_shape = x.shape
            n_valid = int(plan.cu_seqlens[-1]) if packed_rows is None else int(packed_rows)
            n_valid = min(max(n_valid, 1), pad_shape[0] * pad_shape[1])
            x = unpad_rows(x, plan)[:n_valid].unsqueeze(0)                  # (1, T, d_model): kept tokens, zero tail
            # With a caller's bound there may be rows past the last token.  The attention kernel does not
            # write them, and whatever the allocation held there must not reach a later matrix product
            # as the value row of a masked key (0 x NaN): those rows are zeroed after every attention call.
            tail_rows = None
            cu_att = plan.cu_seqlens
            if packed_rows is not None:
                tail_rows = (torch.arange(n_valid, device=x.device) >= plan.cu_seqlens[-1])[:, None, None]
                # no row past the buffers is ever touched, whatever the bound: the attention calls see the
                # sequences cut at it (the result is then marked below)
                cu_att = plan.cu_seqlens.clamp(max=n_valid)
        B, S, _ = x.shape
        H, D = cfg.num_heads, cfg.d_kv
        HD = H * D
        nb, md = cfg.relative_attention_num_buckets, cfg.relative_attention_max_distance
        eps = cfg.layer_norm_epsilon
        table = self._table()
        heads = lambda t: t.unflatten(-1, (H, D)).transpose(1, 2)        # (B, L, H*D) -> (B, H, L, D) view
        x = x.contiguous() if (inputs_embeds is None or plan is not None) else x.clone(memory_format=torch.contiguous_format)
        normed = ops.rms_layer_norm(x, self.block[0].layer[0].layer_norm.weight, eps).to(x.dtype)
        if seq_len is not None:
            from . import sequence_parallel as sp
        if encoder_plan is not None:
            if encoder_plan.batch != B:
                raise ValueError("encoder_plan was made for another batch size")
            cu_dec = torch.arange(B + 1, dtype=torch.int32, device=x.device) * S
        for i, blk in enumerate(self.block):
            att, ffl = blk.layer[0].SelfAttention, blk.layer[-1]
            if type(att) is not T5FlashAttention:
                raise ValueError("forward_fused covers full attention (attention_type='flash')")
            w = self._stacked_weights(i)
            if plan is not None:
                qkv = nn.functional.linear(normed, w["qkv"])[0]                           # (T, 3*H*D)
                q, k, v = (qkv[:, j * HD:(j + 1) * HD].unflatten(-1, (H, D)) for j in range(3))
                attn = flash_attention_with_fusing_bias_varlen(q, k, v, table, cu_att, cu_att,
                                                               plan.seqlen, plan.seqlen, causal=False, sm_scale=1.0,
                                                               NUM_BUCKETS=nb, MAX_DISTANCE=md)
                if tail_rows is not None:
                    attn = attn.masked_fill(tail_rows, 0)
            elif seq_len is None:
                qkv = nn.functional.linear(normed, w["qkv"])
                q, k, v = (heads(qkv[..., j * HD:(j + 1) * HD]) for j in range(3))
                attn = ops.attention(q, k, v, table, self.is_decoder, 1.0, nb, md, 0).transpose(1, 2)
            else:
                q = nn.functional.linear(normed, att.q.weight).view(B, S, H, D)
                kv = nn.functional.linear(normed, w["kv"])
                if overlap:
                    attn = sp.sequence_parallel_attention_overlapped(q, kv, table, seq_len, sm_scale=1.0, NUM_BUCKETS=nb,
                                                                     MAX_DISTANCE=md, group=group, ops=ops)
                else:
                    k, v = kv[..., :HD].reshape(B, S, H, D), kv[..., HD:].reshape(B, S, H, D)
                    attn = sp.sequence_parallel_attention(
                        q, k, v, table, seq_len, sm_scale=1.0, NUM_BUCKETS=nb, MAX_DISTANCE=md, group=group,
                        attention_fn=lambda q_, k_, v_, b_, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE, q_pos_offset:
                        ops.attention(q_, k_, v_, b_, causal, sm_scale, NUM_BUCKETS, MAX_DISTANCE, q_pos_offset))
            o = nn.functional.linear(attn.reshape(B, S, HD), att.o.weight)
            if self.is_decoder:
                ca = blk.layer[1]
                x, normed = ops.add_rms_layer_norm(x, o, ca.layer_norm.weight, eps, inplace=True)
                catt = ca.EncDecAttention
                ckv = nn.functional.linear(encoder_hidden_states, w["ckv"])
                if encoder_plan is None:
                    q = heads(nn.functional.linear(normed, catt.q.weight))
                    attn = ops.attention(q, heads(ckv[..., :HD]), heads(ckv[..., HD:]), None, False, 1.0, nb, md, 0)
                    attn = attn.transpose(1, 2)
                else:
                    # packed encoder states: every decoder sequence has S query rows, its keys are the valid
                    # encoder tokens of the same batch row
                    q = nn.functional.linear(normed, catt.q.weight).view(B * S, H, D)
                    attn = flash_attention_with_fusing_bias_varlen(
                        q, ckv[:, :HD].unflatten(-1, (H, D)), ckv[:, HD:].unflatten(-1, (H, D)), None, cu_dec,
                        encoder_plan.cu_seqlens, S, encoder_plan.seqlen, causal=False, sm_scale=1.0)
                o = nn.functional.linear(attn.reshape(B, S, HD), catt.o.weight)
            x, normed = ops.add_rms_layer_norm(x, o, ffl.layer_norm.weight, eps, inplace=True)
            ff = ffl.DenseReluDense
            if "wi" in w:
                f = nn.functional.linear(ops.gated_gelu(nn.functional.linear(normed, w["wi"])), ff.wo.weight)
            else:
                f = ff(normed)
            nxt = self.block[i + 1].layer[0].layer_norm if i + 1 < len(self.block) else self.final_layer_norm
            x, normed = ops.add_rms_layer_norm(x, f, nxt.weight, eps, inplace=True)
        if plan is not None:
            if packed_rows is not None:
                # a bound below the true token count would silently drop tokens: make that loud (NaN
                # everywhere) without reading anything back
                normed = normed.masked_fill(plan.cu_seqlens[-1] > S, float("nan"))
            if return_packed:
                return normed[0], plan
            if packed_rows is not None and S < pad_shape[0] * pad_shape[1]:
                # the scatter reads the packed row of every valid token: give it all of them
                full = normed.new_full((pad_shape[0] * pad_shape[1], normed.shape[-1]), float("nan"))
                full[:S] = normed[0]
                return pad_rows(full, plan)
            return pad_rows(normed[0], plan)          # (B, L, d_model), zeros at padded positions
        return normed

    # ---- generation with a preallocated cache (decoder only)
    def new_cache(self, encoder_hidden_states, max_len) -> DecoderCache:
        cfg = self.cfg
        B = encoder_hidden_states.shape[0]
        cache = DecoderCache(len(self.block), B, cfg.num_heads, cfg.d_kv, max_len, encoder_hidden_states.dtype,
                             encoder_hidden_states.device)
        for i, blk in enumerate(self.block):
            att = blk.layer[1].EncDecAttention
            shape = lambda x: x.view(B, -1, cfg.num_heads, cfg.d_kv).transpose(1, 2)
            cache.cross_k[i] = shape(att.k(encoder_hidden_states))
            cache.cross_v[i] = shape(att.v(encoder_hidden_states))
        return cache

    def decode_step_static(self, input_ids, cache: DecoderCache, pos, seqlens, encoder_seqlens=None):
        """One cached single-token step whose position lives on the device.

        `pos` (int64, shape (1,)) is the slot of the new token in the cache and `seqlens` (int32,
        shape (B,)) the number of cached keys including it; nothing in the launch sequence
        depends on their values, so the step can be captured once in a CUDA graph and replayed
        (the caller advances both tensors between replays).  Returns (B, 1, d_model).

        For 16-bit weights the step is fused like `forward_fused`: one stacked q|k|v projection, one
        copy that appends the new key and value to the cache, the split-KV kernel, the output
        projection, residual add + RMSNorm in one kernel -- thirteen launches per layer instead of
        twenty.
        """
        cfg = self.cfg
        B = input_ids.shape[0]
        H, D = cfg.num_heads, cfg.d_kv
        HD = H * D
        nb, md = cfg.relative_attention_num_buckets, cfg.relative_attention_max_distance
        eps = cfg.layer_norm_epsilon
        hidden = self.embed_tokens(input_ids)
        table = self._table()
        fused = hidden.dtype in (torch.bfloat16, torch.float16) and cfg.d_model % 8 == 0
        shape = lambda x: x.view(B, 1, H, D).transpose(1, 2)
        # The split count of the self-attention launch comes from the cache CAPACITY, not from the
        # current length, so it is the same in every replay (a split beyond the cached keys is empty
        # and merges as such); a small batch then still fills the GPU late in a long generation.
        from . import _native as nat
        self_splits = max(1, nat.lib().t5b_decode_num_splits(B, H, cache.max_len))
        if fused:
            hidden = hidden.contiguous()
            normed = rms_layer_norm(hidden, self.block[0].layer[0].layer_norm.weight, eps)
        for i, blk in enumerate(self.block):
            sa, ca, ffl = blk.layer[0], blk.layer[1], blk.layer[-1]
            att, catt = sa.SelfAttention, ca.EncDecAttention
            if fused:
                w = self._stacked_weights(i)
                qkv = nn.functional.linear(normed, w["qkv"])                       # (B, 1, 3*H*D)
                q = shape(qkv[..., :HD])
                # new key and value -> slot `pos` of the stacked cache, one copy: (2, B, H, 1, D)
                cache.self_kv[i].index_copy_(3, pos, qkv[..., HD:].view(B, 1, 2, H, D).permute(2, 0, 3, 1, 4))
            else:
                normed = sa.layer_norm(hidden).to(hidden.dtype)
                q = shape(att.q(normed))
                cache.self_k[i].index_copy_(2, pos, shape(att.k(normed)))
                cache.self_v[i].index_copy_(2, pos, shape(att.v(normed)))
            o = flash_decoding_with_fusing_bias(q, cache.self_k[i], cache.self_v[i], table, causal=True, sm_scale=1.0,
                                                NUM_BUCKETS=nb, MAX_DISTANCE=md, seqlens_k=seqlens,
                                                num_splits=self_splits)
            o = att.o(o.transpose(1, 2).reshape(B, 1, HD))
            if fused:
                hidden, normed = add_rms_layer_norm(hidden, o, ca.layer_norm.weight, eps, inplace=True)
            else:
                hidden = hidden + o
                normed = ca.layer_norm(hidden).to(hidden.dtype)
            q = shape(catt.q(normed))
            o = flash_decoding_with_fusing_bias(q, cache.cross_k[i], cache.cross_v[i], None, causal=False,
                                                sm_scale=1.0, seqlens_k=encoder_seqlens, q_pos_offset=0)
            o = catt.o(o.transpose(1, 2).reshape(B, 1, HD))
            if fused:
                hidden, normed = add_rms_layer_norm(hidden, o, ffl.layer_norm.weight, eps, inplace=True)
                ff = ffl.DenseReluDense
                if "wi" in w:
                    f = nn.functional.linear(gated_gelu(nn.functional.linear(normed, w["wi"])), ff.wo.weight)
                else:
                    f = ff(normed)
                nxt = self.block[i + 1].layer[0].layer_norm if i + 1 < len(self.block) else self.final_layer_norm
                hidden, normed = add_rms_layer_norm(hidden, f, nxt.weight, eps, inplace=True)
            else:
                hidden = hidden + o
                hidden = ffl(hidden)
        return normed if fused else self.final_layer_norm(hidden).to(hidden.dtype)

    def decode_step(self, input_ids, cache: DecoderCache, encoder_seqlens=None):
        """One cached step for `input_ids` (B, M) (M new tokens, usually 1); returns (B, M, d_model)."""
        cfg = self.cfg
        B, M = input_ids.shape
        H, D = cfg.num_heads, cfg.d_kv
        t0 = cache.length
        if t0 + M > cache.max_len:
            raise ValueError("decoder cache is full")
        hidden = self.embed_tokens(input_ids)
        table = self._table()
        shape = lambda x: x.view(B, M, H, D).transpose(1, 2)
        for i, blk in enumerate(self.block):
            sa, ca = blk.layer[0], blk.layer[1]
            att = sa.SelfAttention
            normed = sa.layer_norm(hidden).to(hidden.dtype)
            q = shape(att.q(normed))
            cache.self_k[i][:, :, t0:t0 + M] = shape(att.k(normed))
            cache.self_v[i][:, :, t0:t0 + M] = shape(att.v(normed))
            if M <= att.decode_max_rows:
                o = flash_decoding_with_fusing_bias(q, cache.self_k[i], cache.self_v[i], table, causal=True,
                                                    sm_scale=1.0, NUM_BUCKETS=cfg.relative_attention_num_buckets,
                                                    MAX_DISTANCE=cfg.relative_attention_max_distance, kv_len=t0 + M)
            else:
                o = flash_attention_with_fusing_bias(q, cache.self_k[i][:, :, :t0 + M], cache.self_v[i][:, :, :t0 + M],
                                                     table, causal=True, sm_scale=1.0,
                                                     NUM_BUCKETS=cfg.relative_attention_num_buckets,
                                                     MAX_DISTANCE=cfg.relative_attention_max_distance)
            hidden = hidden + att.o(o.transpose(1, 2).reshape(B, M, H * D))
            catt = ca.EncDecAttention
            normed = ca.layer_norm(hidden).to(hidden.dtype)
            q = shape(catt.q(normed))
            if M <= catt.decode_max_rows:
                o = flash_decoding_with_fusing_bias(q, cache.cross_k[i], cache.cross_v[i], None, causal=False,
                                                    sm_scale=1.0, seqlens_k=encoder_seqlens, q_pos_offset=0)
            else:
                o = flash_attention_with_fusing_bias(q, cache.cross_k[i], cache.cross_v[i], None, causal=False,
                                                     sm_scale=1.0, q_pos_offset=0)
            hidden = hidden + catt.o(o.transpose(1, 2).reshape(B, M, H * D))
            hidden = blk.layer[-1](hidden)
        cache.length = t0 + M
        return self.final_layer_norm(hidden).to(hidden.dtype)


class GraphedDecoding:
    """Greedy generation whose single-token step is one CUDA graph.

    The step (all decoder layers, LM head, argmax, token write-back, position update) is run
    once eagerly on a side stream (cuBLAS handles and stacked weights then exist), rewound,
    captured, and rewound again; `step()` then replays it.  The library's split scratch is kept
    per stream: the capture stream gets its own, allocated and zeroed inside the graph's memory
    pool during capture.  The token position and the cached
    length live in device tensors that the graph itself advances, so no launch argument
    changes between replays.
    """

    def __init__(self, model, encoder_hidden_states, max_len, encoder_seqlens=None):
        B = encoder_hidden_states.shape[0]
        dev = encoder_hidden_states.device
        self.model = model
        self.max_len = max_len
        self.cache = model.decoder.new_cache(encoder_hidden_states, max_len)
        self.cur = torch.empty((B, 1), dtype=torch.long, device=dev)
        self.pos = torch.empty(1, dtype=torch.long, device=dev)
        self.seqlens = torch.empty(B, dtype=torch.int32, device=dev)
        self.tokens = torch.zeros((B, max_len), dtype=torch.long, device=dev)
        self.encoder_seqlens = encoder_seqlens
        self.steps_done = 0
        self.rewind()
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            self._step()
        torch.cuda.current_stream(dev).wait_stream(side)
        self.rewind()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.last_logits = self._step()
        self.rewind()

    def rewind(self):
        self.cur.fill_(self.model.cfg.decoder_start_token_id)
        self.pos.zero_()
        self.seqlens.fill_(1)
        self.steps_done = 0

    def _step(self):
        m = self.model
        logits = m.logits(m.decoder.decode_step_static(self.cur, self.cache, self.pos, self.seqlens,
                                                       self.encoder_seqlens))
        nxt = logits[:, -1:].argmax(-1)
        self.tokens.index_copy_(1, self.pos, nxt)
        self.cur.copy_(nxt)
        self.pos.add_(1)
        self.seqlens.add_(1)
        return logits

    def step(self):
        if self.steps_done >= self.max_len:
            raise RuntimeError("the cache is full: %d steps" % self.max_len)
        self.graph.replay()
        self.steps_done += 1


class GraphedForward:
    """A whole teacher-forced forward pass (encoder, decoder, LM head) of fixed shapes as one CUDA graph.

    At small batches the pass is a few hundred short kernels and the host's launch rate, not the
    GPU, sets its duration (twelve decoder layers over 4 x 128 tokens: 4.4 ms of launches for well
    under 2 ms of work).  The pass is run once on a side stream (cuBLAS handles, stacked weights
    and the library's per-stream scratch then exist), captured, and replayed by `__call__`, which
    copies the token ids into the graph's input buffers and returns the graph's logits buffer (a
    static tensor: it is overwritten by the next call).  Inference only, unpadded inputs.
    """

    def __init__(self, model, batch, enc_len, dec_len, device=None):
        dev = torch.device(device) if device is not None else model.shared.weight.device
        self.model = model
        self.input_ids = torch.zeros((batch, enc_len), dtype=torch.long, device=dev)
        self.decoder_input_ids = torch.zeros((batch, dec_len), dtype=torch.long, device=dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side), torch.no_grad():
            model(self.input_ids, self.decoder_input_ids)
        torch.cuda.current_stream(dev).wait_stream(side)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.logits = model(self.input_ids, self.decoder_input_ids)

    def __call__(self, input_ids, decoder_input_ids):
        if input_ids.shape != self.input_ids.shape or decoder_input_ids.shape != self.decoder_input_ids.shape:
            raise ValueError("GraphedForward was captured for ids of shapes %s and %s" %
                             (tuple(self.input_ids.shape), tuple(self.decoder_input_ids.shape)))
        self.input_ids.copy_(input_ids, non_blocking=True)
        self.decoder_input_ids.copy_(decoder_input_ids, non_blocking=True)
        self.graph.replay()
        return self.logits


class T5ForConditionalGeneration(nn.Module):
    def __init__(self, cfg: T5StackConfig):
        super().__init__()
        self.cfg = cfg
        self.shared = nn.Embedding(cfg.vocab_size, cfg.d_model)
        self.encoder = T5Stack(cfg, self.shared, is_decoder=False)
        self.decoder = T5Stack(cfg, self.shared, is_decoder=True)
        self.lm_head = nn.Linear(cfg.d_model, cfg.vocab_size, bias=False)

    def logits(self, decoder_hidden):
        if self.cfg.tie_word_embeddings:
            decoder_hidden = decoder_hidden * (self.cfg.d_model ** -0.5)
        return self.lm_head(decoder_hidden)

    def forward(self, input_ids, decoder_input_ids, attention_mask=None):
        if not torch.is_grad_enabled() and self.cfg.attention_type == "flash" and \
                input_ids.is_cuda and self.shared.weight.dtype in (torch.bfloat16, torch.float16):
            # inference: fused token-wise kernels in both stacks; a padded batch is packed once and the
            # decoder's cross attention reads the packed encoder states
            if attention_mask is None:
                enc = self.encoder.forward_fused(input_ids)
                return self.logits(self.decoder.forward_fused(decoder_input_ids, encoder_hidden_states=enc))
            enc, plan = self.encoder.forward_fused(input_ids, attention_mask=attention_mask, return_packed=True)
            return self.logits(self.decoder.forward_fused(decoder_input_ids, encoder_hidden_states=enc,
                                                          encoder_plan=plan))
        enc = self.encoder(input_ids, attention_mask=attention_mask)
        dec = self.decoder(decoder_input_ids, encoder_hidden_states=enc, encoder_attention_mask=attention_mask)
        return self.logits(dec)

    @torch.no_grad()
    def forward_cuda_graph(self, input_ids, decoder_input_ids):
        """`forward` for unpadded inference inputs through a CUDA graph kept per input shape (captured on
        first use; the returned logits live in the graph's buffer until the next call with that shape)."""
        key = (tuple(input_ids.shape), tuple(decoder_input_ids.shape), input_ids.device)
        graphs = self.__dict__.setdefault("_forward_graphs", {})
        if key not in graphs:
            graphs[key] = GraphedForward(self, input_ids.shape[0], input_ids.shape[1], decoder_input_ids.shape[1],
                                         input_ids.device)
        return graphs[key](input_ids, decoder_input_ids)

    @torch.no_grad()
    def generate(self, input_ids, attention_mask=None, max_new_tokens=32, use_cuda_graph=True):
        """Greedy generation for a (padded) batch of prompts: the encoder pass on the packed valid tokens
        (`forward_fused`), the cross-attention keys and values projected once into the preallocated cache,
        then one captured single-token step per new token.  Returns the generated ids (B, max_new_tokens)."""
        fused = self.cfg.attention_type == "flash" and input_ids.is_cuda and \
            self.shared.weight.dtype in (torch.bfloat16, torch.float16)
        seqlens = None
        if attention_mask is not None:
            seqlens = attention_mask.to(torch.int32).sum(-1).to(torch.int32)
        if fused:
            enc = self.encoder.forward_fused(input_ids, attention_mask=attention_mask)
        else:
            enc = self.encoder(input_ids, attention_mask=attention_mask)
        tokens, _ = self.greedy_decode(enc, max_new_tokens, encoder_seqlens=seqlens, use_cuda_graph=use_cuda_graph)
        return tokens

    @torch.no_grad()
    def greedy_decode(self, encoder_hidden_states, steps, encoder_seqlens=None, use_cuda_graph=False):
        """Greedy generation from `decoder_start_token_id` with the preallocated cache.

        With `use_cuda_graph` the whole single-token step (all layers, LM head, argmax, position
        update) is captured once after a warm-up step and replayed: one graph launch per token
        instead of a few hundred kernel launches issued from Python.
        """
        B = encoder_hidden_states.shape[0]
        dev = encoder_hidden_states.device
        cache = self.decoder.new_cache(encoder_hidden_states, steps)
        cur = torch.full((B, 1), self.cfg.decoder_start_token_id, dtype=torch.long, device=dev)
        if not use_cuda_graph:
            tokens, last_logits = [], None
            for _ in range(steps):
                last_logits = self.logits(self.decoder.decode_step(cur, cache, encoder_seqlens))
                cur = last_logits[:, -1:].argmax(-1)
                tokens.append(cur)
            return torch.cat(tokens, dim=1), last_logits

        session = GraphedDecoding(self, encoder_hidden_states, steps, encoder_seqlens)
        for _ in range(steps):
            session.step()
        return session.tokens, session.last_logits
