"""CPU oracle for the T5 fused-relative-position-bias attention path.

TEST INFRASTRUCTURE ONLY.  This module restates, on the CPU, the arithmetic of
the reference's `basic` attention path and of its torch RMSNorm.  It is the
checker the CUDA kernels are compared against; nothing in the shipped package
imports it, and it is never used as a compute fallback.  Only the test-suite,
the smoke check and the CPU-baseline leg of the benchmark may call it.

Parity status: PINNED.  Every function below is checked against outputs of the
reference's own code (imported from its source tree through a small
compatibility shim and executed on CPU), stored as fixtures under
`tests/golden/` together with the script that generated them
(`tests/golden/make_golden.py`).  The reference's own test-suite holds no golden
vectors for this path (its tests assert shapes only), so the fixtures generated
from the live reference are the anchor.

Each function cites the reference source (path inside the reference project)
it follows.  Integer work (bucket indices) is numpy int64/float32; floating
point work uses torch CPU tensors so that the rounding points of the reference
(which is torch code) are reproduced exactly.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------- #
# a1: relative position -> bucket index (integer, must be bit-exact)
# --------------------------------------------------------------------------- #
def relative_position_bucket(relative_position, bidirectional: bool = True,
                             num_buckets: int = 32, max_distance: int = 128) -> np.ndarray:
    """Bucket index of `relative_position = key_pos - query_pos`.

    Follows `T5Attention._relative_position_bucket`
    (src/turbot5/model/attentions.py:78-124): half of the buckets per sign when
    bidirectional, `max_exact = nb // 2` exact buckets, the rest logarithmic in
    float32 (`log(d / max_exact) / log(max_distance / max_exact) * (nb - max_exact)`
    truncated toward zero) and clamped to `nb - 1`.
    """
    rel = np.asarray(relative_position, dtype=np.int64)
    buckets = np.zeros_like(rel)
    nb = int(num_buckets)
    if bidirectional:
        nb //= 2
        buckets = buckets + (rel > 0).astype(np.int64) * nb
        dist = np.abs(rel)
    else:
        dist = -np.minimum(rel, 0)
    max_exact = nb // 2
    is_small = dist < max_exact
    # float32 chain exactly as the reference: int -> float32, / int scalar,
    # log, / python-double scalar (rounded to float32), * int scalar, trunc.
    # torch is used for the three float ops so the same libm/SIMD log is hit.
    d_t = torch.from_numpy(np.where(is_small, max(max_exact, 1), dist).astype(np.int64))
    val = (torch.log(d_t.float() / max_exact)
           / math.log(max_distance / max_exact)
           * (nb - max_exact))
    large = max_exact + val.to(torch.long).numpy()
    large = np.minimum(large, nb - 1)
    return buckets + np.where(is_small, dist, large)


def bucket_of_delta(deltas: Sequence[int], bidirectional: bool, num_buckets: int,
                    max_distance: int) -> np.ndarray:
    """Bucket for each delta in `deltas` (convenience for table tests)."""
    return relative_position_bucket(np.asarray(list(deltas), dtype=np.int64),
                                    bidirectional, num_buckets, max_distance)


# --------------------------------------------------------------------------- #
# a2: bias tensor (1, H, M, N) from the [num_buckets, H] table
# --------------------------------------------------------------------------- #
def compute_bias(table: torch.Tensor, query_length: int, key_length: int,
                 bidirectional: bool, num_buckets: int, max_distance: int,
                 q_pos_offset: int = 0, rows: Optional[slice] = None) -> torch.Tensor:
    """`T5Attention.compute_bias` (src/turbot5/model/attentions.py:126-141).

    `q_pos_offset` is the absolute position of query row 0 in key coordinates;
    the reference gets the same effect by building the bias for
    `real_seq_length` rows and keeping the last rows (attentions.py:229-234),
    i.e. offset = key_length - query_length for cached decoding.  `rows`
    restricts the computation to a slab of query rows (long sequences).
    """
    r0, r1 = (0, query_length) if rows is None else (rows.start, rows.stop)
    ctx = np.arange(r0, r1, dtype=np.int64)[:, None] + q_pos_offset
    mem = np.arange(key_length, dtype=np.int64)[None, :]
    bucket = relative_position_bucket(mem - ctx, bidirectional, num_buckets, max_distance)
    values = table[torch.from_numpy(bucket)]            # (m, N, H) embedding lookup
    return values.permute(2, 0, 1).unsqueeze(0)          # (1, H, m, N)


# --------------------------------------------------------------------------- #
# a3: naive attention with bias
# --------------------------------------------------------------------------- #
def naive_attention_with_bias(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                              position_bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """`naive_torch_attention_with_bias` (src/turbot5/ops/naive_attention.py:4-23).

    Scores and bias-add in the input dtype, softmax in float32, probabilities
    cast back to the input dtype, no 1/sqrt(d).  Dropout and head mask are off
    (inference).
    """
    scores = torch.einsum("...qd,...kd->...qk", q, k)
    if position_bias is not None:
        scores = scores + position_bias
    w = torch.softmax(scores.float(), dim=-1).type_as(scores)
    return torch.einsum("...hqk,...hkd->...hqd", w, v)


def attention_basic(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                    table: Optional[torch.Tensor], causal: bool = False,
                    sm_scale: float = 1.0, num_buckets: int = 32, max_distance: int = 128,
                    q_pos_offset: Optional[int] = None, slab: int = 1024,
                    compute_dtype: torch.dtype = torch.float32,
                    rows: Optional[slice] = None) -> torch.Tensor:
    """Whole `basic` attention core for (B,H,M,D) x (B,H,N,D), slab by slab.

    This is a1+a2+a3 chained as `T5Attention.forward` does
    (src/turbot5/model/attentions.py:229-247) with the same meaning the fused
    kernel's arguments have: `causal` selects both the causal mask and
    unidirectional bucketing (src/turbot5/ops/fused_bias_attention.py:294-299,
    330-332), `sm_scale` multiplies QK^T, `table` may be None.  Inputs are
    upcast to `compute_dtype` (float32 by default: the float32 run of `basic`
    on the same values is the parity anchor; the bf16 run of `basic` rounds the
    scores to bf16 before softmax and is itself far from its float32 result).
    Query rows are processed in slabs so the L x L tensors never exist whole.
    `rows` limits the work to a slice of query rows (long-sequence spot checks).
    """
    B, H, M, D = q.shape
    N = k.shape[2]
    if q_pos_offset is None:
        q_pos_offset = N - M
    r0, r1 = (0, M) if rows is None else (rows.start, rows.stop)
    kf, vf = k.to(compute_dtype), v.to(compute_dtype)
    tf = None if table is None else table.to(compute_dtype)
    out = torch.zeros((B, H, r1 - r0, D), dtype=compute_dtype)
    keys = torch.arange(N)[None, :]
    for s0 in range(r0, r1, slab):
        s1 = min(s0 + slab, r1)
        qs = q[:, :, s0:s1].to(compute_dtype) * sm_scale
        bias = None
        if tf is not None:
            bias = compute_bias(tf, M, N, not causal, num_buckets, max_distance,
                                q_pos_offset=q_pos_offset, rows=slice(s0, s1))
        if causal:
            qpos = torch.arange(s0, s1)[:, None] + q_pos_offset
            mask = torch.where(keys <= qpos, 0.0, float("-inf")).to(compute_dtype)[None, None]
            bias = mask if bias is None else bias + mask
        o = naive_attention_with_bias(qs, kf, vf, bias)
        # rows with no visible key come out of softmax as NaN in torch; the
        # fused kernel defines them as zero (fused_bias_attention.py:351-354).
        out[:, :, s0 - r0:s1 - r0] = torch.nan_to_num(o, nan=0.0)
    return out


def local_attention_basic(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, table: Optional[torch.Tensor],
                          block_len: int, num_buckets: int = 32, max_distance: int = 128,
                          key_padding_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Block-local attention core of `T5LocalAttention.forward`
    (src/turbot5/model/attentions.py:553-650, helpers src/turbot5/model/utils.py:99-140).

    (B,H,L,D) float tensors.  The sequence is zero-padded to a multiple of `block_len` (a shorter
    sequence is a single block of its own length), split into blocks, and the queries of block i
    attend to the keys of blocks i-1, i, i+1; the missing neighbours of the first and last block
    are all-zero blocks that are NOT masked (score = bias only), exactly as the reference
    concatenates them.  Bias: bidirectional buckets of (key position - query position) inside the
    3-block window (`compute_bias(block_len)`, attentions.py:529-551).

    With `key_padding_mask` (raw 0/1 (B, L)) the mask `T5Stack` builds for this module is applied
    (`_get_local_attention_mask`, src/turbot5/model/utils.py:149-155,174-188; added as -1e10,
    attentions.py:600-603,619-621): a pair is visible when query and key are both valid AND
    |key - query| < block_len -- with a mask the three blocks shrink to a sliding window, and the
    zero blocks beyond the ends are masked.  Rows of padded queries see nothing but -1e10 and come
    out as the mean of all values in the window (callers compare valid rows only).
    """
    B, H, L, D = q.shape
    bl = block_len if L >= block_len else L
    pad = (-L) % bl
    f = lambda x: torch.nn.functional.pad(x.float(), (0, 0, 0, pad))
    qp, kp, vp = f(q), f(k), f(v)
    nblk = (L + pad) // bl
    qb = qp.view(B, H, nblk, bl, D)

    def three(x):
        xb = x.view(B, H, nblk, bl, D)
        z = torch.zeros_like(xb[:, :, :1])
        ext = torch.cat([z, xb, z], dim=2)                      # blocks -1 .. nblk
        return torch.cat([ext[:, :, 0:nblk], ext[:, :, 1:nblk + 1], ext[:, :, 2:nblk + 2]], dim=3)   # (B,H,nblk,3bl,D)
    kc, vc = three(kp), three(vp)
    scores = torch.einsum("bhnqd,bhnkd->bhnqk", qb, kc)
    if table is not None:
        mem = torch.arange(3 * bl)
        ctx = mem[bl:2 * bl]
        bucket = relative_position_bucket(mem[None, :] - ctx[:, None], True, num_buckets, max_distance)
        bias = table.float()[torch.as_tensor(bucket, dtype=torch.long)]     # (bl, 3bl, H)
        scores = scores + bias.permute(2, 0, 1)[None, :, None]
    if key_padding_mask is not None:
        mp = torch.nn.functional.pad(key_padding_mask.float(), (0, pad)).view(B, nblk, bl)
        z = torch.zeros_like(mp[:, :1])
        ext = torch.cat([z, mp, z], dim=1)
        m3 = torch.cat([ext[:, 0:nblk], ext[:, 1:nblk + 1], ext[:, 2:nblk + 2]], dim=2)         # (B, nblk, 3bl)
        rel = torch.arange(3 * bl)[None, :] - torch.arange(bl, 2 * bl)[:, None]
        vis = (mp[:, :, :, None] > 0) & (m3[:, :, None, :] > 0) & (rel.abs() < bl)[None, None]   # (B, nblk, bl, 3bl)
        scores = scores + torch.where(vis, 0.0, -1e10)[:, None]
    out = torch.einsum("bhnqk,bhnkd->bhnqd", torch.softmax(scores, dim=-1), vc)
    return out.reshape(B, H, nblk * bl, D)[:, :, :L]


def attention_basic_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                           table: Optional[torch.Tensor], cu_seqlens_q, cu_seqlens_k,
                           causal: bool = False, sm_scale: float = 1.0,
                           num_buckets: int = 32, max_distance: int = 128) -> torch.Tensor:
    """Packed (T,H,D) attention: `basic` on every unpadded sequence.

    Positions are sequence-relative as in the reference varlen kernel
    (src/turbot5/ops/varlen_fused_bias_attn.py:254,303); for causal the query
    rows are aligned to the end of the keys as in `basic`.
    """
    cq = [int(x) for x in cu_seqlens_q]
    ck = [int(x) for x in cu_seqlens_k]
    out = torch.zeros(q.shape, dtype=torch.float32)
    for b in range(len(cq) - 1):
        qs = q[cq[b]:cq[b + 1]].transpose(0, 1).unsqueeze(0)
        ks = k[ck[b]:ck[b + 1]].transpose(0, 1).unsqueeze(0)
        vs = v[ck[b]:ck[b + 1]].transpose(0, 1).unsqueeze(0)
        if qs.shape[2] == 0:
            continue
        if ks.shape[2] == 0:
            continue
        o = attention_basic(qs, ks, vs, table, causal, sm_scale, num_buckets, max_distance)
        out[cq[b]:cq[b + 1]] = o[0].transpose(0, 1)
    return out


# --------------------------------------------------------------------------- #
# a7: split-KV merge semantics
# --------------------------------------------------------------------------- #
def merge_splits(part_o: torch.Tensor, part_l: torch.Tensor, part_m: torch.Tensor) -> torch.Tensor:
    """Combine per-split partial results (src/turbot5/ops/flash_decoding.py:50-54).

    part_o: (..., S, D) normalised partial outputs acc/l; part_l, part_m: (..., S)
    partial normaliser and running max (natural-log domain).
    """
    a_max = torch.max(part_m, dim=-1, keepdim=True).values
    alpha = torch.exp(part_m - a_max)
    w = torch.softmax(torch.log(alpha * part_l), dim=-1)
    return torch.sum(w.unsqueeze(-1) * part_o, dim=-2)


# --------------------------------------------------------------------------- #
# a8: T5 RMSNorm
# --------------------------------------------------------------------------- #
def t5_layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """`T5LayerNorm._forward` (src/turbot5/model/modules.py:52-60).

    float32 variance without mean subtraction; x * rsqrt promotes to float32;
    if the weight is half precision the normalised value is rounded to that
    dtype before the multiply (two roundings).
    """
    variance = x.to(torch.float32).pow(2).mean(-1, keepdim=True)
    y = x * torch.rsqrt(variance + eps)
    if weight.dtype in (torch.float16, torch.bfloat16):
        y = y.to(weight.dtype)
    return weight * y


# --------------------------------------------------------------------------- #
# a9: unpad / pad glue
# --------------------------------------------------------------------------- #
def get_unpad_data(attention_mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """`_get_unpad_data` (src/turbot5/model/padding.py:79-88)."""
    seqlens = attention_mask.sum(dim=-1, dtype=torch.int32)
    indices = torch.nonzero(attention_mask.flatten(), as_tuple=False).flatten()
    cu = torch.nn.functional.pad(torch.cumsum(seqlens, dim=0, dtype=torch.int32), (1, 0))
    return indices, cu, int(seqlens.max())


def pad_rows(values: torch.Tensor, indices: torch.Tensor, batch: int, seqlen: int) -> torch.Tensor:
    """`pad_input` (src/turbot5/model/padding.py:30-44): scatter rows into zeros."""
    out = torch.zeros((batch * seqlen,) + tuple(values.shape[1:]), dtype=values.dtype)
    out[indices] = values
    return out.view(batch, seqlen, *values.shape[1:])


# --------------------------------------------------------------------------- #
# a6: attention module forward (basic) -- projections + core + output proj
# --------------------------------------------------------------------------- #
def t5_attention_layer(hidden: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor,
                       wv: torch.Tensor, wo: torch.Tensor, table: Optional[torch.Tensor],
                       n_heads: int, d_kv: int, is_decoder: bool = False,
                       num_buckets: int = 32, max_distance: int = 128,
                       key_value_states: Optional[torch.Tensor] = None,
                       key_padding_mask: Optional[torch.Tensor] = None,
                       past_key_value: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                       causal: Optional[bool] = None, round_to: Optional[torch.dtype] = None):
    """`T5Attention.forward` (src/turbot5/model/attentions.py:144-257) on CPU.

    `key_padding_mask` is the raw 0/1 (B, N) mask; padded keys get -inf-like
    additive bias (the stack's extended mask, finfo.min) and padded query rows
    are returned as the reference would compute them (callers compare valid
    rows only, since the flash module returns zeros there).  `causal` defaults
    to `is_decoder and key_value_states is None`.  Returns (out, (k, v)).  With `round_to`
    (bfloat16 / float16) the projections q, k, v and the attention output are rounded to that type
    where the module running in that type stores them (its linears return that type); all
    arithmetic stays float32.
    """
    B, L, _ = hidden.shape
    if causal is None:
        causal = is_decoder and key_value_states is None

    def shape(x):
        return x.view(B, -1, n_heads, d_kv).transpose(1, 2)

    rnd = (lambda x: x) if round_to is None else (lambda x: x.to(round_to).to(hidden.dtype))
    qh = shape(rnd(hidden @ wq.t()))
    src = hidden if key_value_states is None else key_value_states
    kh, vh = shape(rnd(src @ wk.t())), shape(rnd(src @ wv.t()))
    if past_key_value is not None and key_value_states is None:
        kh = torch.cat([past_key_value[0], kh], dim=2)
        vh = torch.cat([past_key_value[1], vh], dim=2)
    elif past_key_value is not None:
        kh, vh = past_key_value
    M, N = qh.shape[2], kh.shape[2]
    bias = None
    if table is not None:
        bias = compute_bias(table, M, N, not is_decoder, num_buckets, max_distance,
                            q_pos_offset=(N - M) if key_value_states is None else 0)
    if causal:
        qpos = torch.arange(M)[:, None] + (N - M)
        cm = torch.where(torch.arange(N)[None, :] <= qpos, 0.0,
                         torch.finfo(hidden.dtype).min).to(hidden.dtype)[None, None]
        bias = cm if bias is None else bias + cm
    if key_padding_mask is not None:
        pm = (1.0 - key_padding_mask.to(hidden.dtype))[:, None, None, :] * torch.finfo(hidden.dtype).min
        bias = pm if bias is None else bias + pm
    o = naive_attention_with_bias(qh, kh, vh, bias)
    o = rnd(o.transpose(1, 2).contiguous().view(B, -1, n_heads * d_kv))
    return o @ wo.t(), (kh, vh)


# --------------------------------------------------------------------------- #
# next row: the encoder / decoder stack around the attention path
# --------------------------------------------------------------------------- #
def _ffn(w, prefix, x, gated=True):
    """T5LayerFF (src/turbot5/model/modeling.py:63-128): pre-norm, gated-GELU (tanh) or ReLU, residual."""
    h = t5_layer_norm(x, w[prefix + "layer_norm.weight"])
    if gated:
        a = torch.nn.functional.gelu(h @ w[prefix + "DenseReluDense.wi_0.weight"].t(), approximate="tanh")
        h = (a * (h @ w[prefix + "DenseReluDense.wi_1.weight"].t())) @ w[prefix + "DenseReluDense.wo.weight"].t()
    else:
        h = torch.relu(h @ w[prefix + "DenseReluDense.wi.weight"].t()) @ w[prefix + "DenseReluDense.wo.weight"].t()
    return x + h


def t5_stack_forward(w, cfg, input_ids, is_decoder=False, mask=None, encoder_hidden=None, encoder_mask=None):
    """`T5Stack.forward` without a cache (src/turbot5/model/modeling.py:421-632) on a dict of
    weights with the Hugging Face parameter names.  `cfg`: dict with num_heads, d_kv, the bucket
    settings and the layer counts."""
    side = "decoder" if is_decoder else "encoder"
    n_layers = cfg["num_decoder_layers"] if is_decoder else cfg["num_layers"]
    H, D = cfg["num_heads"], cfg["d_kv"]
    nb, md = cfg["relative_attention_num_buckets"], cfg["relative_attention_max_distance"]
    x = w["shared.weight"][input_ids]
    table = w[f"{side}.block.0.layer.0.SelfAttention.relative_attention_bias.weight"]
    for i in range(n_layers):
        pre = f"{side}.block.{i}.layer.0."
        a = pre + "SelfAttention."
        h = t5_layer_norm(x, w[pre + "layer_norm.weight"])
        o, _ = t5_attention_layer(h, w[a + "q.weight"], w[a + "k.weight"], w[a + "v.weight"], w[a + "o.weight"],
                                  table, H, D, is_decoder=is_decoder, num_buckets=nb, max_distance=md,
                                  key_padding_mask=None if is_decoder else mask)
        x = x + o
        if is_decoder:
            pre = f"{side}.block.{i}.layer.1."
            a = pre + "EncDecAttention."
            h = t5_layer_norm(x, w[pre + "layer_norm.weight"])
            o, _ = t5_attention_layer(h, w[a + "q.weight"], w[a + "k.weight"], w[a + "v.weight"], w[a + "o.weight"],
                                      None, H, D, is_decoder=True, key_value_states=encoder_hidden,
                                      key_padding_mask=encoder_mask, causal=False)
            x = x + o
        ff = f"{side}.block.{i}.layer.{2 if is_decoder else 1}."
        x = _ffn(w, ff, x, gated=(ff + "DenseReluDense.wi_0.weight") in w)
    return t5_layer_norm(x, w[f"{side}.final_layer_norm.weight"])


def t5_model_logits(w, cfg, input_ids, decoder_input_ids, mask=None, tie_word_embeddings=False):
    """Encoder + decoder + LM head (src/turbot5/heads/t5_heads.py:132-260)."""
    enc = t5_stack_forward(w, cfg, input_ids, mask=mask)
    dec = t5_stack_forward(w, cfg, decoder_input_ids, is_decoder=True, encoder_hidden=enc, encoder_mask=mask)
    if tie_word_embeddings:
        dec = dec * (w["shared.weight"].shape[1] ** -0.5)
    return enc, dec @ w["lm_head.weight"].t()
