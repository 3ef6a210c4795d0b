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


# ---------------------------------------------------------------------------
# the token-sharded encoder stack on two CPU ranks against the unsharded stack oracle
# ---------------------------------------------------------------------------
class _CpuOps:
    """Stand-ins for the library operators, built from the oracle (float32 on the CPU)."""

    @staticmethod
    def rms_layer_norm(x, w, eps):
        from oracle import t5_oracle as orc
        return orc.t5_layer_norm(x, w, eps)

    @staticmethod
    def add_rms_layer_norm(hidden, branch, w, eps, inplace=False):
        from oracle import t5_oracle as orc
        s = hidden + branch
        return s, orc.t5_layer_norm(s, w, eps)

    @staticmethod
    def gated_gelu(x):
        f = x.shape[-1] // 2
        return torch.nn.functional.gelu(x[..., :f], approximate="tanh") * x[..., f:]

    @staticmethod
    def attention(q, k, v, bias, causal, sm_scale, nb, md, q_pos_offset):
        return _oracle_attention(q, k, v, bias, causal=causal, sm_scale=sm_scale, NUM_BUCKETS=nb, MAX_DISTANCE=md,
                                 q_pos_offset=q_pos_offset)

    @staticmethod
    def partial(q, k, v, bias, causal, sm_scale, nb, md, q_pos_offset):
        # (normalised output, log-sum-exp) over a slice of the keys, written out plainly
        from oracle import t5_oracle as orc
        M, N = q.shape[2], k.shape[2]
        s = torch.einsum("bhmd,bhnd->bhmn", q.float(), k.float()) * sm_scale
        if bias is not None:
            s = s + orc.compute_bias(bias.float(), M, N, not causal, nb, md, q_pos_offset=q_pos_offset)
        if causal:
            qpos = torch.arange(M)[:, None] + q_pos_offset
            s = s.masked_fill(torch.arange(N)[None, :] > qpos, float("-inf"))
        lse = torch.logsumexp(s, dim=-1)
        p = torch.exp(s - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
        return torch.einsum("bhmn,bhnd->bhmd", p, v.float()), lse

    @staticmethod
    def merge(parts, dtype):
        lse = torch.stack([l for _, l in parts])
        mx = lse.max(0).values
        w = torch.exp(lse - torch.where(torch.isinf(mx), torch.zeros_like(mx), mx))
        out = sum(wi[..., None] * o for wi, (o, _) in zip(w, parts)) / w.sum(0).clamp_min(1e-38)[..., None]
        return out.to(dtype)


def _stack_worker(rank, world, port, seq_len, overlap, out_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import t5_oracle as orc
        from tests.helpers import seed_named_parameters
        from turbot5_b200 import sequence_parallel as sp
        from turbot5_b200.t5 import T5Stack, T5StackConfig
        cfgd = dict(vocab_size=64, d_model=32, d_kv=8, num_heads=4, d_ff=48, num_layers=3, num_decoder_layers=0,
                    relative_attention_num_buckets=32, relative_attention_max_distance=16)
        cfg = T5StackConfig(**cfgd)
        enc = seed_named_parameters(T5Stack(cfg, torch.nn.Embedding(cfg.vocab_size, cfg.d_model), is_decoder=False), 0).eval()
        ids = torch.randint(0, cfg.vocab_size, (1, seq_len), generator=torch.Generator().manual_seed(5))
        S = sp.shard_size(seq_len, world)
        lo, hi = sp.shard_bounds(seq_len, world, rank)
        local = torch.zeros((1, S), dtype=torch.long)
        local[:, :hi - lo] = ids[:, lo:hi]
        got = enc.forward_fused(local, seq_len=seq_len, overlap=overlap, ops=_CpuOps)
        w = {"encoder." + k: v.detach() for k, v in enc.state_dict().items()}
        w["shared.weight"] = enc.embed_tokens.weight.detach()
        want = orc.t5_stack_forward(w, cfgd, ids)
        err = (got[:, :hi - lo] - want[:, lo:hi]).abs().max().item()
        single = enc.forward_fused(ids, ops=_CpuOps) if rank == 0 else None
        err1 = (single - want).abs().max().item() if single is not None else 0.0
        out_queue.put((rank, err, err1))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq_len,overlap", [(48, True), (45, True), (45, False)])
def test_two_rank_sharded_encoder_matches_unsharded_oracle(seq_len, overlap):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_stack_worker, args=(r, world, port, seq_len, overlap, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, err1 in results:
        assert err < 1e-4 and err1 < 1e-4, (rank, err, err1)
