"""Query-block sequence parallelism for one long sequence on one multi-GPU node.

Rank r owns the token shard [r*S, (r+1)*S) (S = ceil(L / world)) for every
token-wise operation.  For attention each rank keeps its own query rows,
all-gathers the key and value shards of all ranks into a buffer in its OWN
memory (NCCL over NVLink; `torch.distributed.all_gather_into_tensor`) and runs
the fused-bias kernel on `q_local x all keys` with `q_pos_offset = r*S`, the
position of its first query row.  Every rank holds complete softmax rows, so no
reduction follows.  Remote keys are always read from local memory by the
kernel's ordinary per-block TMA loads.

The reference has no multi-GPU path; this is the partitioning of its single-GPU
call (src/turbot5/model/attentions.py:486-490) whose bias depends only on
absolute positions (src/turbot5/model/attentions.py:126-141).
"""
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_size(seq_len: int, world: int) -> int:
    """Tokens per rank (the last rank may own fewer real tokens; shards are padded to this size)."""
    return -(-seq_len // world)


def shard_bounds(seq_len: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, stop) of the real tokens owned by `rank`."""
    s = shard_size(seq_len, world)
    return min(rank * s, seq_len), min((rank + 1) * s, seq_len)


def all_gather_sequence(x_local: torch.Tensor, group=None) -> torch.Tensor:
    """(B, S, H, D) shard per rank -> (B, world*S, H, D) in this rank's memory.

    One collective per batch row, each into a contiguous slice of the output, so
    that the gathered buffer is directly addressable as (B, H, L, D) by strides.
    """
    world = dist.get_world_size(group)
    B, S = x_local.shape[:2]
    x_local = x_local.contiguous()
    out = torch.empty((B, world * S) + tuple(x_local.shape[2:]), dtype=x_local.dtype, device=x_local.device)
    if world == 1:
        out.copy_(x_local)
        return out
    for b in range(B):
        dist.all_gather_into_tensor(out[b], x_local[b], group=group)
    return out


def sequence_parallel_attention(q_local: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor,
                                bias: Optional[torch.Tensor], seq_len: int, causal: bool = False,
                                sm_scale: Optional[float] = None, NUM_BUCKETS: int = 32,
                                MAX_DISTANCE: int = 128, group=None,
                                attention_fn: Optional[Callable] = None) -> torch.Tensor:
    """Attention of this rank's query rows against the whole sequence.

    q_local, k_local, v_local: (B, S, H, D) token-major shards, S = shard_size(seq_len, world);
    rows of the last shard beyond `seq_len` are padding (their outputs are unspecified and
    their keys are never attended).  Returns (B, S, H, D).  `attention_fn` defaults to
    `flash_attention_with_fusing_bias`; tests on CPU ranks pass a reference implementation
    with the same signature.
    """
    if attention_fn is None:
        from .attention import flash_attention_with_fusing_bias as attention_fn
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    S = q_local.shape[1]
    if S != shard_size(seq_len, world):
        raise ValueError(f"shard length {S} does not match ceil({seq_len} / {world})")
    if world > 1:
        k_all = all_gather_sequence(k_local, group)
        v_all = all_gather_sequence(v_local, group)
    else:
        k_all, v_all = k_local, v_local
    # (B, H, rows, D) views of the token-major buffers; only the real keys are attended
    q = q_local.transpose(1, 2)
    k = k_all[:, :seq_len].transpose(1, 2)
    v = v_all[:, :seq_len].transpose(1, 2)
    out = attention_fn(q, k, v, bias, causal=causal, sm_scale=sm_scale, NUM_BUCKETS=NUM_BUCKETS,
                       MAX_DISTANCE=MAX_DISTANCE, q_pos_offset=rank * S)
    return out.transpose(1, 2)


class _DeviceOps:
    """The library operators the overlapped path is built from (tests on CPU ranks pass stand-ins
    with the same three functions)."""

    @staticmethod
    def attention(q, k, v, bias, causal, sm_scale, nb, md, q_pos_offset):
        from .attention import flash_attention_with_fusing_bias
        return flash_attention_with_fusing_bias(q, k, v, bias, causal=causal, sm_scale=sm_scale, NUM_BUCKETS=nb,
                                                MAX_DISTANCE=md, q_pos_offset=q_pos_offset)

    @staticmethod
    def partial(q, k, v, bias, causal, sm_scale, nb, md, q_pos_offset):
        from .attention import flash_attention_partial
        return flash_attention_partial(q, k, v, bias, causal=causal, sm_scale=sm_scale, NUM_BUCKETS=nb,
                                       MAX_DISTANCE=md, q_pos_offset=q_pos_offset)

    @staticmethod
    def merge(parts, dtype):
        from .attention import merge_attention_partials
        return merge_attention_partials(parts, dtype)


def high_priority_group(ranks=None):
    """An NCCL process group whose collectives run on a high-priority stream.  The all-gather of
    `sequence_parallel_attention_overlapped` is a kernel of a few blocks that has to start while the
    attention over the local keys already fills every SM; on a stream of normal priority its blocks
    queue behind the attention blocks that are still waiting for an SM and most of the gather ends
    up exposed (4 GPUs, one layer over 100 000 tokens: 0.25 ms exposed, against 0.03 ms with this)."""
    from torch.distributed import ProcessGroupNCCL
    opts = ProcessGroupNCCL.Options()
    opts.is_high_priority_stream = True
    return dist.new_group(ranks=ranks, pg_options=opts)


def sequence_parallel_attention_overlapped(q_local: torch.Tensor, kv_local: torch.Tensor,
                                           bias: Optional[torch.Tensor], seq_len: int, causal: bool = False,
                                           sm_scale: Optional[float] = None, NUM_BUCKETS: int = 32,
                                           MAX_DISTANCE: int = 128, group=None, ops=None) -> torch.Tensor:
    """Attention of this rank's query rows against the whole sequence, with the all-gather of the
    other ranks' keys and values hidden behind the attention over the keys this rank already holds.

    q_local (B, S, H, D); kv_local (B, S, 2*H*D) contiguous, each row the keys of all heads followed
    by the values of all heads (the output of ONE projection with the k and v weights stacked), so
    one collective moves both and the gathered buffer is addressable as K and V by strides.
    The gather is issued first and runs on the communication stream; meanwhile the kernel computes
    the partial result over the local keys (float32 output + log-sum-exp).  When the gather has
    landed in this rank's memory, the keys before and after the local shard are attended and the
    (up to three) partials are merged -- softmax over disjoint key sets combines exactly through
    the log-sum-exps, in any order.  Returns (B, S, H, D) in q's dtype; rows of the last shard
    beyond `seq_len` are unspecified.  Give it a `group` whose collectives run on a high-priority
    stream (`high_priority_group()`, or `init_process_group(..., pg_options=...)`), otherwise the
    gather starts late.
    """
    ops = ops or _DeviceOps
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    B, S, H, D = q_local.shape
    HD = H * D
    if S != shard_size(seq_len, world):
        raise ValueError(f"shard length {S} does not match ceil({seq_len} / {world})")
    if kv_local.shape != (B, S, 2 * HD) or not kv_local.is_contiguous():
        raise ValueError("kv_local must be a contiguous (B, S, 2*H*D) tensor")
    lo, hi = shard_bounds(seq_len, world, rank)

    def heads(buf, first, start, stop):
        # (B, H, stop-start, D) view of the keys (first=0) or values (first=HD) of rows [start, stop)
        return buf[:, start:stop, first:first + HD].unflatten(-1, (H, D)).transpose(1, 2)

    q = q_local.transpose(1, 2)
    args = (causal, 1.0 / (D ** 0.5) if sm_scale is None else sm_scale, NUM_BUCKETS, MAX_DISTANCE)
    if world == 1:
        out = ops.attention(q, heads(kv_local, 0, 0, hi), heads(kv_local, HD, 0, hi), bias, *args, 0)
        return out.transpose(1, 2)
    kv_all = torch.empty((B, world * S, 2 * HD), dtype=kv_local.dtype, device=kv_local.device)
    works = [dist.all_gather_into_tensor(kv_all[b], kv_local[b], group=group, async_op=True) for b in range(B)]
    parts = []
    if hi > lo:
        # local keys: query row 0 sits at the slice's first key
        parts.append(ops.partial(q, heads(kv_local, 0, 0, hi - lo), heads(kv_local, HD, 0, hi - lo), bias, *args, 0))
    for w in works:
        w.wait()
    if lo > 0:
        parts.append(ops.partial(q, heads(kv_all, 0, 0, lo), heads(kv_all, HD, 0, lo), bias, *args, lo))
    if hi < seq_len and not causal:      # under a causal mask no key after the shard is visible
        parts.append(ops.partial(q, heads(kv_all, 0, hi, seq_len), heads(kv_all, HD, hi, seq_len), bias, *args, lo - hi))
    if not parts:
        return torch.zeros_like(q_local)
    return ops.merge(parts, q_local.dtype).transpose(1, 2)
