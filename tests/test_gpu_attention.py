"""CUDA attention kernels (through the C ABI) against the CPU oracle and the golden fixtures."""
import numpy as np
import pytest
import torch

from oracle import t5_oracle as orc
from tests.helpers import attention_case, check_close, load, local_case, local_masked_case, seeded

pytestmark = pytest.mark.gpu


def _ops():
    import turbot5_b200 as t5b
    return t5b


def _run_dense(q, k, v, table, dtype, kernel, causal=False, nb=32, md=128, q_pos_offset=None, sm_scale=1.0):
    t5b = _ops()
    dev = "cuda"
    out = t5b.flash_attention_with_fusing_bias(
        q.to(dev, dtype), k.to(dev, dtype), v.to(dev, dtype),
        None if table is None else table.to(dev, dtype), causal=causal, sm_scale=sm_scale,
        NUM_BUCKETS=nb, MAX_DISTANCE=md, q_pos_offset=q_pos_offset, kernel=kernel)
    torch.cuda.synchronize()
    t5b.check_device_status()
    return out


KERNELS_16BIT = ["tcgen05", "simt"]


@pytest.mark.parametrize("nb,md,bidir", [(32, 128, True), (32, 128, False), (64, 256, True),
                                          (16, 32, False), (24, 100, True), (128, 1024, False)])
def test_bucket_grid_bit_exact(nb, md, bidir):
    t5b = _ops()
    M, N, off = 257, 1500, 611
    got = t5b.relative_position_bucket_grid(M, N, off, bidir, nb, md).cpu().numpy()
    rel = np.arange(N)[None, :] - (np.arange(M)[:, None] + off)
    want = orc.relative_position_bucket(rel, bidir, nb, md)
    assert np.array_equal(got, want)


def test_bucket_grid_matches_reference_fixture():
    t5b = _ops()
    z = load("buckets.npz")
    got = t5b.relative_position_bucket_grid(300, 280, 0, True, 32, 128).cpu().numpy()
    assert np.array_equal(got, z["grid_bi"])
    got = t5b.relative_position_bucket_grid(300, 280, 0, False, 32, 128).cpu().numpy()
    assert np.array_equal(got, z["grid_uni"])


@pytest.mark.parametrize("kernel", KERNELS_16BIT)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", ["enc_small", "enc_ragged", "enc_long", "cross_mn"])
def test_golden_bidirectional(name, dtype, kernel):
    c = attention_case(load("attention.npz"), name)
    off = 0 if name == "cross_mn" else None
    out = _run_dense(c["q"], c["k"], c["v"], c["table"], dtype, kernel, nb=c["nb"], md=c["md"],
                     q_pos_offset=off)
    check_close(out, c["out"], dtype, name)


@pytest.mark.parametrize("name", ["enc_small", "enc_d32", "enc_d128", "cross_mn"])
def test_golden_fp32(name):
    c = attention_case(load("attention.npz"), name)
    off = 0 if name == "cross_mn" else None
    out = _run_dense(c["q"], c["k"], c["v"], c["table"], torch.float32, "auto", nb=c["nb"], md=c["md"],
                     q_pos_offset=off)
    check_close(out, c["out"], torch.float32, name)


@pytest.mark.parametrize("name", ["enc_d32", "enc_d128"])
def test_golden_other_head_dims_bf16(name):
    c = attention_case(load("attention.npz"), name)
    out = _run_dense(c["q"], c["k"], c["v"], c["table"], torch.bfloat16, "auto", nb=c["nb"], md=c["md"])
    check_close(out, c["out"], torch.bfloat16, name)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [16, 32])
@pytest.mark.parametrize("B,H,M,N,causal,off", [(2, 3, 300, 300, False, None), (1, 2, 128, 1024, False, 0),
                                                 (1, 2, 640, 640, True, None), (1, 1, 1, 300, True, None),
                                                 (1, 16, 2048, 2048, False, None)])
def test_narrow_head_dims_on_the_tensor_core_kernel(B, H, M, N, causal, off, D, dtype):
    # head dims 16 and 32 run as head dim 64 with zero-filled columns; forced onto the
    # tensor-core kernel, non-contiguous (B, L, H, D) storage as the modules produce it
    q = seeded((B, M, H, D), 1, dtype=dtype).transpose(1, 2)
    k = seeded((B, N, H, D), 2, dtype=dtype).transpose(1, 2)
    v = seeded((B, N, H, D), 3, dtype=dtype).transpose(1, 2)
    table = seeded((32, H), 4, 0.1, dtype=dtype)
    out = _run_dense(q, k, v, table, dtype, "tcgen05", causal=causal, q_pos_offset=off)
    assert out.shape == (B, H, M, D)
    if M * N > 1024 * 1024:
        rows = [0, 777, M - 1]
        want = orc.attention_basic(q[:, :2, rows] if off is not None else q[:, :2], k[:, :2], v[:, :2], table[:, :2],
                                   causal=causal, q_pos_offset=off)[:, :, rows]
        check_close(out[:, :2, rows], want, dtype)
    else:
        want = orc.attention_basic(q, k, v, table, causal=causal, q_pos_offset=off)
        check_close(out, want, dtype, f"{(B, H, M, N, causal, off, D)}")


@pytest.mark.parametrize("D", [16, 32])
def test_narrow_head_dims_packed_and_token_major(D):
    t5b = _ops()
    dt = torch.bfloat16
    lens = [5, 128, 0, 129, 300, 1]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    T, H = int(cu[-1]), 3
    q, k, v = seeded((T, H, D), 1, dtype=dt), seeded((T, H, D), 2, dtype=dt), seeded((T, H, D), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = orc.attention_basic_varlen(q, k, v, table, cu, cu, causal=False)
    out = t5b.flash_attention_with_fusing_bias_varlen(
        q.cuda(), k.cuda(), v.cuda(), table.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
        sm_scale=1.0, kernel="tcgen05")
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out, want, dt)
    # token-major storage: the heads of one token are neighbours in the output, so a store wider
    # than the head would land in the next head
    B, L = 2, 200
    qd, kd, vd = (seeded((B, L, H, D), s, dtype=dt).cuda().transpose(1, 2) for s in (5, 6, 7))
    got = t5b.flash_attention_with_fusing_bias(qd, kd, vd, table.cuda(), sm_scale=1.0, kernel="tcgen05")
    ref = t5b.flash_attention_with_fusing_bias(qd, kd, vd, table.cuda(), sm_scale=1.0, kernel="simt")
    torch.cuda.synchronize()
    assert got.transpose(1, 2).is_contiguous()
    assert (got.float() - ref.float()).abs().max().item() < 2e-2


@pytest.mark.parametrize("kernel", KERNELS_16BIT)
def test_golden_cached_decode_rows(kernel):
    # unidirectional bias, query rows at the end of the keys.  The fixture has no
    # causal mask, so only rows that see every key are comparable: the last row.
    z = load("attention.npz")
    for name in ("dec_cached", "dec_step"):
        c = attention_case(z, name)
        out = _run_dense(c["q"], c["k"], c["v"], c["table"], torch.bfloat16, kernel, causal=True)
        check_close(out[:, :, -1], c["out"][:, :, -1], torch.bfloat16, name)


CASES = [
    # B, H, M, N, causal, q_pos_offset
    (2, 3, 1024, 1024, False, None),
    (1, 2, 777, 777, False, None),
    (1, 2, 777, 777, True, None),
    (2, 2, 128, 1024, False, 0),        # cross-attention shape
    (1, 2, 200, 555, True, None),       # cached prefill: queries aligned to the end
    (1, 2, 300, 300, False, 4000),      # sequence-parallel shard offset
    (1, 1, 1, 300, True, None),
    (1, 2, 640, 130, True, None),       # more queries than keys: leading rows see nothing
]


@pytest.mark.parametrize("kernel", KERNELS_16BIT)
@pytest.mark.parametrize("B,H,M,N,causal,off", CASES)
def test_seeded_vs_oracle_bf16(B, H, M, N, causal, off, kernel):
    dt = torch.bfloat16
    q = seeded((B, H, M, 64), 1, dtype=dt)
    k = seeded((B, H, N, 64), 2, dtype=dt)
    v = seeded((B, H, N, 64), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = orc.attention_basic(q, k, v, table, causal=causal, q_pos_offset=off)
    out = _run_dense(q, k, v, table, dt, kernel, causal=causal, q_pos_offset=off)
    check_close(out, want, dt, f"{(B, H, M, N, causal, off)}")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,M,N,causal,off", [(2, 3, 1024, 1024, False, None), (1, 2, 512, 1536, False, 0),
                                                 (1, 2, 640, 640, True, None), (1, 2, 384, 384, False, 4000)])
def test_every_exponential_on_the_fma_pipe(B, H, M, N, causal, off, dtype):
    """kernel='tcgen05_polyexp' sends every exponential of an unmasked tile through the
    range-reduction + cubic path that the default kernel may use for a share of the columns;
    same tolerances as the hardware ex2 path."""
    q = seeded((B, H, M, 64), 11, dtype=dtype)
    k = seeded((B, H, N, 64), 12, dtype=dtype)
    v = seeded((B, H, N, 64), 13, dtype=dtype)
    table = seeded((32, H), 14, 0.1, dtype=dtype)
    want = orc.attention_basic(q, k, v, table, causal=causal, q_pos_offset=off)
    out = _run_dense(q, k, v, table, dtype, "tcgen05_polyexp", causal=causal, q_pos_offset=off)
    check_close(out, want, dtype, f"polyexp {(B, H, M, N, causal, off)}")
    # far-apart scores: exponents down to the clamp (2^-123) and a rescale of the running maximum
    q2 = q * 6.0
    want = orc.attention_basic(q2, k, v, table, causal=causal, q_pos_offset=off)
    out = _run_dense(q2, k, v, table, dtype, "tcgen05_polyexp", causal=causal, q_pos_offset=off)
    check_close(out, want, dtype, f"polyexp wide {(B, H, M, N, causal, off)}")


@pytest.mark.parametrize("kernel", KERNELS_16BIT)
def test_no_bias_and_scale(kernel):
    dt = torch.bfloat16
    q, k, v = seeded((1, 2, 300, 64), 1, dtype=dt), seeded((1, 2, 300, 64), 2, dtype=dt), seeded((1, 2, 300, 64), 3, dtype=dt)
    want = orc.attention_basic(q, k, v, None, sm_scale=0.125)
    out = _run_dense(q, k, v, None, dt, kernel, sm_scale=0.125)
    check_close(out, want, dt)


@pytest.mark.parametrize("kernel", KERNELS_16BIT)
def test_strided_views_keep_strides(kernel):
    # (B,H,L,D) views of (B,L,H,D) buffers, as the attention module passes them
    t5b = _ops()
    dt = torch.bfloat16
    B, L, H, D = 2, 384, 4, 64
    qb, kb, vb = (seeded((B, L, H, D), s, dtype=dt).cuda() for s in (1, 2, 3))
    table = seeded((32, H), 4, 0.1, dtype=dt).cuda()
    q, k, v = qb.transpose(1, 2), kb.transpose(1, 2), vb.transpose(1, 2)
    out = t5b.flash_attention_with_fusing_bias(q, k, v, table, sm_scale=1.0, kernel=kernel)
    torch.cuda.synchronize()
    t5b.check_device_status()
    assert out.stride() == q.stride() and out.shape == q.shape
    want = orc.attention_basic(q.cpu(), k.cpu(), v.cpu(), table.cpu())
    check_close(out, want, dt)


def test_layer_config1_fp32_matches_reference_layer():
    # batch 2, seq 512, 8 heads x 64, d_model 512, float32, seed 0: projections in
    # torch, attention core through the library, against the reference layer output
    t5b = _ops()
    z = load("layer.npz")
    g = torch.Generator().manual_seed(0)
    hidden = torch.randn((2, 512, 512), generator=g)
    ws = [torch.randn((512, 512), generator=g) * 0.05 for _ in range(3)]
    wo = torch.randn((512, 512), generator=g) * 0.05
    table = torch.randn((32, 8), generator=g) * 0.1
    sums = np.asarray([x.double().sum().item() for x in (hidden, *ws, wo, table)])
    if not np.allclose(sums, z["full_checks"], rtol=0, atol=1e-6):
        pytest.skip("torch RNG stream differs from the one that generated the fixture")
    shape = lambda x: x.view(2, 512, 8, 64).transpose(1, 2)
    q, k, v = (shape(hidden @ w.t()).cuda() for w in ws)
    out = t5b.flash_attention_with_fusing_bias(q, k, v, table.cuda(), sm_scale=1.0)
    o = out.transpose(1, 2).reshape(2, 512, 512).cpu() @ wo.t()
    diff = (o[:, ::16, ::16] - torch.from_numpy(z["full_out_sub"])).abs()
    assert diff.max().item() < 1e-4, diff.max().item()


@pytest.mark.parametrize("kernel", KERNELS_16BIT + ["fp32"])
@pytest.mark.parametrize("causal", [False, True])
def test_varlen_vs_oracle(kernel, causal):
    t5b = _ops()
    dt = torch.float32 if kernel == "fp32" else torch.bfloat16
    lens = [5, 128, 0, 129, 300, 1, 257, 64]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    T, H = int(cu[-1]), 3
    q, k, v = seeded((T, H, 64), 1, dtype=dt), seeded((T, H, 64), 2, dtype=dt), seeded((T, H, 64), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = orc.attention_basic_varlen(q, k, v, table, cu, cu, causal=causal)
    out = t5b.flash_attention_with_fusing_bias_varlen(
        q.cuda(), k.cuda(), v.cuda(), table.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
        causal=causal, sm_scale=1.0, kernel="auto" if kernel == "fp32" else kernel)
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out, want, dt)


@pytest.mark.parametrize("kernel", KERNELS_16BIT)
def test_varlen_different_q_and_k_lengths(kernel):
    t5b = _ops()
    dt = torch.bfloat16
    lq, lk = [3, 130, 40], [200, 130, 17]
    cq = torch.tensor(np.concatenate([[0], np.cumsum(lq)]), dtype=torch.int32)
    ck = torch.tensor(np.concatenate([[0], np.cumsum(lk)]), dtype=torch.int32)
    H = 2
    q = seeded((int(cq[-1]), H, 64), 1, dtype=dt)
    k, v = seeded((int(ck[-1]), H, 64), 2, dtype=dt), seeded((int(ck[-1]), H, 64), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = orc.attention_basic_varlen(q, k, v, table, cq, ck, causal=False)
    out = t5b.flash_attention_with_fusing_bias_varlen(q.cuda(), k.cuda(), v.cuda(), table.cuda(), cq.cuda(),
                                                      ck.cuda(), max(lq), max(lk), sm_scale=1.0, kernel=kernel)
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out, want, dt)


def test_lse_matches_logsumexp():
    t5b = _ops()
    dt = torch.bfloat16
    q, k, v = seeded((1, 2, 200, 64), 1, dtype=dt), seeded((1, 2, 333, 64), 2, dtype=dt), seeded((1, 2, 333, 64), 3, dtype=dt)
    table = seeded((32, 2), 4, 0.1, dtype=dt)
    bias = orc.compute_bias(table.float(), 200, 333, True, 32, 128, q_pos_offset=133)
    want = torch.logsumexp(torch.einsum("bhqd,bhkd->bhqk", q.float(), k.float()) + bias, dim=-1)
    for kernel in KERNELS_16BIT:
        _, lse = t5b.flash_attention_with_fusing_bias(q.cuda(), k.cuda(), v.cuda(), table.cuda(), sm_scale=1.0,
                                                      return_lse=True, kernel=kernel)
        # the tensor-core kernel normalises by the sum of the bf16-rounded probabilities
        # (each within 2^-9 of its value), so its LSE carries that rounding
        assert (lse.cpu() - want).abs().max().item() < (5e-3 if kernel == "tcgen05" else 1e-3)


def test_empty_and_argument_errors():
    t5b = _ops()
    dt = torch.bfloat16
    q = torch.zeros((1, 2, 0, 64), dtype=dt, device="cuda")
    k = torch.zeros((1, 2, 10, 64), dtype=dt, device="cuda")
    assert t5b.flash_attention_with_fusing_bias(q, k, k, None, sm_scale=1.0).shape == (1, 2, 0, 64)
    q = torch.zeros((1, 2, 4, 64), dtype=dt, device="cuda")
    k0 = torch.zeros((1, 2, 0, 64), dtype=dt, device="cuda")
    out = t5b.flash_attention_with_fusing_bias(q, k0, k0, None, sm_scale=1.0)   # no keys: zeros
    assert torch.count_nonzero(out) == 0
    with pytest.raises(AssertionError):
        bad = torch.zeros((1, 2, 4, 48), dtype=dt, device="cuda")
        t5b.flash_attention_with_fusing_bias(bad, bad, bad, None)
    with pytest.raises(RuntimeError):
        t5b.flash_attention_with_fusing_bias(q.cpu(), k.cpu(), k.cpu(), None)
    with pytest.raises(RuntimeError):   # bucket settings the reference formula cannot express
        t5b.flash_attention_with_fusing_bias(q, k, k, torch.zeros((2, 2), dtype=dt, device="cuda"),
                                             NUM_BUCKETS=2, MAX_DISTANCE=128)


def test_full_size_8k_properties():
    # B=2, H=12, L=8192, D=64 bf16: spot rows against the oracle plus two
    # size-independent properties (softmax weights sum to one; shift of all keys'
    # values by a constant shifts the output by that constant).
    t5b = _ops()
    dt = torch.bfloat16
    B, H, L, D = 2, 12, 8192, 64
    g = torch.Generator(device="cuda").manual_seed(0)
    qb = torch.randn((B, L, H, D), generator=g, device="cuda", dtype=torch.float32).to(dt)
    kb = torch.randn((B, L, H, D), generator=g, device="cuda", dtype=torch.float32).to(dt)
    vb = torch.randn((B, L, H, D), generator=g, device="cuda", dtype=torch.float32).to(dt)
    table = (torch.randn((32, H), generator=g, device="cuda") * 0.1).to(dt)
    q, k, v = qb.transpose(1, 2), kb.transpose(1, 2), vb.transpose(1, 2)
    out = t5b.flash_attention_with_fusing_bias(q, k, v, table, sm_scale=1.0)
    ones = torch.ones_like(v)
    out1 = t5b.flash_attention_with_fusing_bias(q, k, ones, table, sm_scale=1.0)
    torch.cuda.synchronize()
    t5b.check_device_status()
    assert (out1.float() - 1).abs().max().item() < 1e-2          # rows of P sum to one
    rows = slice(4000, 4160)
    want = orc.attention_basic(q[:1, :2].cpu(), k[:1, :2].cpu(), v[:1, :2].cpu(), table[:, :2].cpu(), rows=rows)
    check_close(out[:1, :2, rows], want, dt, "8k rows 4000:4160")
    rows = slice(8100, 8192)
    want = orc.attention_basic(q[1:, 10:].cpu(), k[1:, 10:].cpu(), v[1:, 10:].cpu(), table[:, 10:].cpu(), rows=rows)
    check_close(out[1:, 10:, rows], want, dt, "8k rows 8100:8192")


# ------------------------------------------------------------------ configured full sizes
def test_config3_varlen_full_size_spot_sequences():
    # 32 sequences with lengths uniform in [128, 4096] (seed 0), T5-base heads, bf16: every
    # sequence is compared on a band of rows; the shortest and two others in full.
    t5b = _ops()
    dt = torch.bfloat16
    lens = torch.randint(128, 4097, (32,), generator=torch.Generator().manual_seed(0))
    cu = torch.zeros(33, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    T, H = int(cu[-1]), 12
    g = torch.Generator(device="cuda").manual_seed(0)
    q, k, v = (torch.randn((T, H, 64), generator=g, device="cuda", dtype=torch.float32).to(dt) for _ in range(3))
    table = (torch.randn((32, H), generator=g, device="cuda") * 0.1).to(dt)
    out = t5b.flash_attention_with_fusing_bias_varlen(q, k, v, table, cu.cuda(), cu.cuda(), int(lens.max()),
                                                      int(lens.max()), sm_scale=1.0)
    torch.cuda.synchronize()
    t5b.check_device_status()
    order = torch.argsort(lens)
    full = {int(order[0]), int(order[1]), 7}
    for b in range(32):
        a, e = int(cu[b]), int(cu[b + 1])
        n = e - a
        rows = slice(0, n) if b in full else slice(max(0, n - 96), n)
        heads = slice(0, 12) if b in full else slice(3, 5)
        qs = q[a:e, heads].transpose(0, 1)[None].cpu()
        ks = k[a:e, heads].transpose(0, 1)[None].cpu()
        vs = v[a:e, heads].transpose(0, 1)[None].cpu()
        want = orc.attention_basic(qs, ks, vs, table[:, heads].cpu(), rows=rows)
        got = out[a:e, heads].transpose(0, 1)[None][:, :, rows]
        check_close(got, want, dt, f"sequence {b} (len {n})")


def test_config4_long_sequence_spot_rows():
    # one sequence of 100 000 tokens, T5-base heads: query slabs at the start, across the
    # middle and at the end against all keys (the oracle never builds L x L)
    t5b = _ops()
    dt = torch.bfloat16
    L, H = 100000, 12
    g = torch.Generator(device="cuda").manual_seed(0)
    q, k, v = (torch.randn((1, L, H, 64), generator=g, device="cuda", dtype=torch.float32).to(dt).transpose(1, 2)
               for _ in range(3))
    table = (torch.randn((32, H), generator=g, device="cuda") * 0.1).to(dt)
    out = t5b.flash_attention_with_fusing_bias(q, k, v, table, sm_scale=1.0)
    torch.cuda.synchronize()
    t5b.check_device_status()
    heads = slice(4, 6)
    kc, vc, tc = k[:, heads].cpu(), v[:, heads].cpu(), table[:, heads].cpu()
    for rows in (slice(0, 64), slice(49990, 50054), slice(99936, 100000)):
        want = orc.attention_basic(q[:, heads].cpu(), kc, vc, tc, rows=rows, slab=64)
        check_close(out[:, heads, rows], want, dt, f"rows {rows.start}:{rows.stop}")
    # a sequence-parallel shard (rows 87500.. of 8 ranks) gives the same rows as the whole.  Not
    # bit for bit: the shard's rows sit in other tiles/warps, so the running maxima that the
    # probabilities are rounded against may differ; both are within tolerance of the oracle.
    lo = 7 * 12500
    shard = t5b.flash_attention_with_fusing_bias(q[:, :, lo:lo + 12500], k, v, table, sm_scale=1.0, q_pos_offset=lo)
    diff = (shard.float() - out[:, :, lo:lo + 12500].float()).abs()
    assert diff.max().item() <= 2e-2 and diff.mean().item() <= 5e-4


@pytest.mark.parametrize("B,H,M,N", [(1, 2, 2048, 2048), (1, 3, 300, 4096), (2, 2, 1000, 1500)])
def test_last_wave_split_matches_unsplit_and_oracle(B, H, M, N):
    # few query tiles: the key range of every tile is split over several blocks and merged in
    # the same launch; results and LSE must agree with the unsplit launch and the oracle
    t5b = _ops()
    dt = torch.bfloat16
    q, k, v = seeded((B, H, M, 64), 1, dtype=dt), seeded((B, H, N, 64), 2, dtype=dt), seeded((B, H, N, 64), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    args = (q.cuda(), k.cuda(), v.cuda(), table.cuda())
    for _ in range(2):      # second call reuses the scratch: its counters were left at zero
        split, lse_s = t5b.flash_attention_with_fusing_bias(*args, sm_scale=1.0, q_pos_offset=0, return_lse=True,
                                                            kernel="tcgen05")
    plain, lse_p = t5b.flash_attention_with_fusing_bias(*args, sm_scale=1.0, q_pos_offset=0, return_lse=True,
                                                        kernel="tcgen05", balance_last_wave=False)
    torch.cuda.synchronize()
    t5b.check_device_status()
    want = orc.attention_basic(q, k, v, table, q_pos_offset=0)
    check_close(split, want, dt, "split")
    check_close(plain, want, dt, "unsplit")
    assert (lse_s - lse_p).abs().max().item() < 1e-2      # each carries the bf16 rounding of its row sums


# ---- head dim 128 on the tensor-core kernel (64-key tiles, two 64-dim sub-tiles per row)
CASES_D128 = [
    (2, 3, 1024, 1024, False, None),
    (1, 2, 777, 777, True, None),
    (2, 2, 128, 1024, False, 0),
    (1, 2, 200, 555, True, None),
    (1, 2, 300, 300, False, 4000),
    (1, 1, 1, 300, True, None),
    (1, 2, 640, 130, True, None),
    (1, 3, 300, 4096, False, 0),        # few query tiles: keys split over several blocks and merged
]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,M,N,causal,off", CASES_D128)
def test_head_dim_128_tensor_core_vs_oracle(B, H, M, N, causal, off, dt):
    q = seeded((B, H, M, 128), 1, dtype=dt)
    k = seeded((B, H, N, 128), 2, dtype=dt)
    v = seeded((B, H, N, 128), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = orc.attention_basic(q, k, v, table, causal=causal, q_pos_offset=off, sm_scale=0.5)
    out = _run_dense(q, k, v, table, dt, "tcgen05", causal=causal, q_pos_offset=off, sm_scale=0.5)
    check_close(out, want, dt, f"d128 {(B, H, M, N, causal, off)}")


def test_head_dim_128_golden_and_varlen():
    t5b = _ops()
    c = attention_case(load("attention.npz"), "enc_d128")
    out = _run_dense(c["q"], c["k"], c["v"], c["table"], torch.bfloat16, "tcgen05", nb=c["nb"], md=c["md"])
    check_close(out, c["out"], torch.bfloat16, "enc_d128")
    dt = torch.bfloat16
    lens = [5, 128, 0, 129, 300, 1, 257, 64]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    T, H = int(cu[-1]), 3
    q, k, v = seeded((T, H, 128), 1, 0.5, dtype=dt), seeded((T, H, 128), 2, 0.5, dtype=dt), seeded((T, H, 128), 3, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    for causal in (False, True):
        want = orc.attention_basic_varlen(q, k, v, table, cu, cu, causal=causal)
        got = t5b.flash_attention_with_fusing_bias_varlen(
            q.cuda(), k.cuda(), v.cuda(), table.cuda(), cu.cuda(), cu.cuda(), max(lens), max(lens),
            causal=causal, sm_scale=1.0, kernel="tcgen05")
        torch.cuda.synchronize()
        t5b.check_device_status()
        check_close(got, want, dt, f"varlen d128 causal={causal}")


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("dt,step", [(torch.bfloat16, 30.0), (torch.bfloat16, -30.0), (torch.float16, 9.0)])
def test_scores_that_keep_growing_take_the_rescale_path(dt, step, D):
    # The scores climb (or fall) by `step` every 37 keys, so the running maximum outgrows the
    # lazy-rescale threshold inside nearly every tile, by a different whole number of powers
    # of two in the two halves of a row and in different rows: O, l and the packed P are
    # rescaled.  The result is dominated by the top block of keys, whose weights differ by a
    # few units of noise.
    B, H, M, N = 1, 2, 300, 1000
    g = torch.Generator().manual_seed(11)
    q = torch.randn((B, H, M, D), generator=g) * 0.05
    k = torch.randn((B, H, N, D), generator=g) * 0.05
    q[..., 0] = 1.0 + 0.5 * torch.rand((B, H, M), generator=g)
    k[..., 0] = step * torch.floor(torch.arange(N) / 37.0) + 2.0 * torch.randn((B, H, N), generator=g)
    v = torch.randn((B, H, N, D), generator=g)
    q, k, v = q.to(dt), k.to(dt), v.to(dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = orc.attention_basic(q, k, v, table, q_pos_offset=0)
    for kernel in ("tcgen05",):
        out = _run_dense(q, k, v, table, dt, kernel, q_pos_offset=0)
        check_close(out, want, dt, f"growing scores {dt} {step} d{D}")


# ---- block-local attention (T5LocalAttention): keys of the three neighbouring blocks only
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", ["loc_ragged", "loc_short", "loc_even", "loc_long"])
def test_block_local_attention_vs_reference_fixture(name, dt):
    t5b = _ops()
    q, k, v, table, bl, want = local_case(load("local.npz"), name)
    out = t5b.flash_attention_with_fusing_bias(q.to("cuda", dt), k.to("cuda", dt), v.to("cuda", dt),
                                               table.to("cuda", dt), sm_scale=1.0, local_block=bl)
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out, want, dt, name)


@pytest.mark.parametrize("D,L,bl", [(64, 4096, 512), (128, 2048, 256), (64, 1000, 128), (64, 700, 1024)])
def test_block_local_attention_seeded_vs_oracle(D, L, bl):
    t5b = _ops()
    dt = torch.bfloat16
    q, k, v = (seeded((2, 3, L, D), s, 0.5 if D == 128 else 1.0, dtype=dt) for s in (1, 2, 3))
    table = seeded((32, 3), 4, 0.1, dtype=dt)
    want = orc.local_attention_basic(q, k, v, table, bl)
    out = t5b.flash_attention_with_fusing_bias(q.cuda(), k.cuda(), v.cuda(), table.cuda(), sm_scale=1.0, local_block=bl)
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out, want, dt, f"local d{D} L{L} block {bl}")


def test_block_local_attention_refuses_what_it_cannot_do():
    t5b = _ops()
    q = torch.randn(1, 2, 600, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):      # blocks of 100 rows would cut through the 128-row query tiles
        t5b.flash_attention_with_fusing_bias(q, q, q, None, sm_scale=1.0, local_block=100)
    with pytest.raises(RuntimeError):
        t5b.flash_attention_with_fusing_bias(q.float(), q.float(), q.float(), None, sm_scale=1.0, local_block=128)


# ---- T5LocalAttention with its padding mask: a sliding window |n - m| < block over the valid keys
def _window_oracle(q, k, v, table, bl, lens):
    mask = torch.zeros((q.shape[0], q.shape[2]))
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    return orc.local_attention_basic(q, k, v, table, bl, key_padding_mask=mask)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", ["locm_ragged", "locm_short", "locm_even", "locm_long", "locm_full"])
def test_sliding_window_vs_masked_reference_fixture(name, dt):
    """The valid prefix of the fixture's sequence as a dense call with window = block length."""
    t5b = _ops()
    q, k, v, table, bl, want, lens = local_masked_case(load("local_masked.npz"), name)
    n = lens[0]
    out = t5b.flash_attention_with_fusing_bias(q[:, :, :n].to("cuda", dt), k[:, :, :n].to("cuda", dt),
                                               v[:, :, :n].to("cuda", dt), table.to("cuda", dt), sm_scale=1.0, window=bl)
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out, want[:, :, :n], dt, name)


@pytest.mark.parametrize("D,L,bl,lens", [(64, 3000, 512, [3000, 1717, 1]), (128, 1500, 256, [900, 1500]),
                                         (64, 700, 128, [700, 129, 128]), (64, 300, 1024, [300, 77])])
def test_local_module_with_padding_mask_vs_oracle(D, L, bl, lens):
    """T5LocalFlashAttention with the raw mask: unpad, packed kernel with the window, pad."""
    t5b = _ops()
    dt = torch.bfloat16
    H, B = 2, len(lens)

    class Cfg:
        is_decoder = False
        relative_attention_num_buckets = 32
        relative_attention_max_distance = 128
        d_model = H * D
        d_kv = D
        num_heads = H
        dropout_rate = 0.0
        sliding_window = bl
    mod = t5b.T5ATTENTION_TYPES["local"](Cfg(), has_relative_attention_bias=True)
    eye = torch.eye(H * D)
    g = torch.Generator().manual_seed(3)
    pk_, pv_ = torch.randperm(H * D, generator=g), torch.randperm(H * D, generator=g)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    with torch.no_grad():
        mod.q.weight.copy_(eye); mod.k.weight.copy_(eye[pk_]); mod.v.weight.copy_(eye[pv_]); mod.o.weight.copy_(eye)
        mod.relative_attention_bias.weight.copy_(table.float())
    mod = mod.cuda().to(dt).eval()
    hidden = seeded((B, L, H * D), 5, 0.5 if D == 128 else 1.0, dtype=dt)
    mask = torch.zeros((B, L), dtype=torch.int64)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    with torch.no_grad():
        out = mod(hidden.cuda(), mask=mask.cuda())[0]
    torch.cuda.synchronize()
    t5b.check_device_status()
    shape = lambda x: x.view(B, L, H, D).transpose(1, 2)
    hf = hidden.float()
    want = _window_oracle(shape(hf), shape(hf[..., pk_]), shape(hf[..., pv_]), table.float(), bl, lens)
    want = want.transpose(1, 2).reshape(B, L, H * D)
    for b, n in enumerate(lens):
        check_close(out[b, :n], want[b, :n], dt, f"masked local row {b}")
        assert torch.count_nonzero(out[b, n:]) == 0          # padded rows come back as zeros


def test_sliding_window_refuses_what_it_cannot_do():
    t5b = _ops()
    q = torch.randn(1, 2, 600, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):       # no CUDA-core kernel for it
        t5b.flash_attention_with_fusing_bias(q.float(), q.float(), q.float(), None, sm_scale=1.0, window=128)
    with pytest.raises(NotImplementedError):       # not together with the causal mask
        t5b.flash_attention_with_fusing_bias(q, q, q, None, causal=True, sm_scale=1.0, window=128)
