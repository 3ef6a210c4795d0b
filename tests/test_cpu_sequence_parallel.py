"""Host-side logic of the sequence-parallel path on two CPU ranks (gloo).

The CUDA operator is replaced by the CPU oracle through the `attention_fn` hook, so the
test covers sharding, the all-gather layout and the position offsets: the concatenation of
the ranks' outputs must equal the unsharded result.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_attention(q, k, v, bias, causal=False, sm_scale=None, NUM_BUCKETS=32, MAX_DISTANCE=128,
                      q_pos_offset=None):
    from oracle import t5_oracle as orc
    return orc.attention_basic(q, k, v, bias, causal=causal, sm_scale=1.0 if sm_scale is None else sm_scale,
                               num_buckets=NUM_BUCKETS, max_distance=MAX_DISTANCE, q_pos_offset=q_pos_offset)


def _worker(rank, world, port, seq_len, causal, B, out_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from turbot5_b200 import sequence_parallel as sp
        H, D = 2, 16
        g = torch.Generator().manual_seed(0)
        q = torch.randn((B, seq_len, H, D), generator=g)
        k = torch.randn((B, seq_len, H, D), generator=g)
        v = torch.randn((B, seq_len, H, D), generator=g)
        table = torch.randn((32, H), generator=g) * 0.1
        S = sp.shard_size(seq_len, world)
        lo, hi = sp.shard_bounds(seq_len, world, rank)

        def shard(x):
            out = torch.zeros((B, S, H, D))
            out[:, :hi - lo] = x[:, lo:hi]
            return out
        o_local = sp.sequence_parallel_attention(shard(q), shard(k), shard(v), table, seq_len, causal=causal,
                                                 sm_scale=1.0, attention_fn=_oracle_attention)
        full = _oracle_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), table, causal=causal,
                                 sm_scale=1.0, q_pos_offset=0).transpose(1, 2)
        err = (o_local[:, :hi - lo] - full[:, lo:hi]).abs().max().item()
        out_queue.put((rank, err, tuple(o_local.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq_len,causal,B", [(64, False, 1), (61, False, 2), (61, True, 1)])
def test_two_rank_sequence_parallel_matches_unsharded(seq_len, causal, B):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, seq_len, causal, B, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, shape in results:
        assert shape == (B, -(-seq_len // world), 2, 16)
        assert err < 1e-5, (rank, err)


def test_shard_bounds_cover_the_sequence():
    from turbot5_b200 import sequence_parallel as sp
    for L in (1, 7, 64, 100000):
        for world in (1, 2, 3, 8):
            spans = [sp.shard_bounds(L, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == L
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(hi - lo <= sp.shard_size(L, world) for lo, hi in spans)
