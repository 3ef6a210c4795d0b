"""Backward of the fused-bias attention (through the C ABI and torch.autograd) against the
CPU oracle under autograd and the gradient fixtures generated from the reference."""
import numpy as np
import pytest
import torch

from oracle import t5_oracle as orc
from tests.helpers import check_close, check_grad_close, from_bf16_bits, load, seeded

pytestmark = pytest.mark.gpu


def _ops():
    import turbot5_b200 as t5b
    return t5b


def _cuda_grads(q, k, v, table, dout, dt, **kw):
    t5b = _ops()
    qc, kc, vc = (t.detach().to("cuda", dt).requires_grad_(True) for t in (q, k, v))
    tc = None if table is None else table.detach().to("cuda", dt).requires_grad_(True)
    out = t5b.flash_attention_with_fusing_bias(qc, kc, vc, tc, sm_scale=kw.pop("sm_scale", 1.0), **kw)
    out.backward(dout.to("cuda", dt))
    torch.cuda.synchronize()
    t5b.check_device_status()
    return out.detach(), qc.grad, kc.grad, vc.grad, (None if tc is None else tc.grad)


def _oracle_grads(q, k, v, table, dout, **kw):
    qf, kf, vf = (t.detach().float().clone().requires_grad_(True) for t in (q, k, v))
    tf = None if table is None else table.detach().float().clone().requires_grad_(True)
    out = orc.attention_basic(qf, kf, vf, tf, **kw)
    (out * dout.float()).sum().backward()
    return out.detach(), qf.grad, kf.grad, vf.grad, (None if tf is None else tf.grad)


@pytest.mark.parametrize("name", ["g_enc", "g_cross", "g_long"])
def test_gradients_match_reference_fixture(name):
    z = load("attention_grad.npz")
    B, H, M, N, D, dec, nb, md = [int(x) for x in z[name + "_meta"]]
    q, k, v, table, dout = (from_bf16_bits(z[name + s]) for s in ("_q", "_k", "_v", "_table", "_dout"))
    _, dq, dk, dv, dt_ = _cuda_grads(q, k, v, table, dout, torch.bfloat16, q_pos_offset=0, NUM_BUCKETS=nb,
                                     MAX_DISTANCE=md)
    check_grad_close(dq, torch.from_numpy(z[name + "_dq"]), name + " dq")
    check_grad_close(dk, torch.from_numpy(z[name + "_dk"]), name + " dk")
    check_grad_close(dv, torch.from_numpy(z[name + "_dv"]), name + " dv")
    check_grad_close(dt_, torch.from_numpy(z[name + "_dtable"]), name + " dtable")


CASES = [
    # B, H, M, N, causal, q_pos_offset
    (2, 3, 512, 512, False, None),
    (1, 2, 777, 777, False, None),
    (1, 2, 777, 777, True, None),
    (2, 2, 128, 1024, False, 0),        # cross-attention shape
    (1, 2, 200, 555, True, None),       # cached prefill: queries aligned to the end
    (1, 2, 300, 300, False, 4000),      # far from the diagonal: one bucket only
    (1, 1, 1, 300, True, None),
    (1, 2, 1000, 70, False, 0),
    (1, 2, 2048, 2048, False, None),    # few tiles: the last wave is split 8 ways and summed in scratch
    (2, 2, 1000, 1500, False, 0),
]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,M,N,causal,off", CASES)
def test_seeded_gradients_vs_oracle(B, H, M, N, causal, off, dt):
    q = seeded((B, H, M, 64), 1, 0.5, dtype=dt)
    k = seeded((B, H, N, 64), 2, 0.5, dtype=dt)
    v = seeded((B, H, N, 64), 3, dtype=dt)
    dout = seeded((B, H, M, 64), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = _oracle_grads(q, k, v, table, dout, causal=causal, q_pos_offset=off)
    got = _cuda_grads(q, k, v, table, dout, dt, causal=causal, q_pos_offset=off)
    what = f"{(B, H, M, N, causal, off)}"
    check_close(got[0], want[0], dt, what + " out")
    for g, w, nm in zip(got[1:], want[1:], ("dq", "dk", "dv", "dtable")):
        check_grad_close(g, w, what + " " + nm, floor=2.0 if nm == "dtable" else 1e-6)


BUCKET_CASES = [
    # num_buckets, max_distance, causal, L: the per-delta tables, their padding and the fold of the
    # bias-table gradient into buckets, for geometries other than T5's 32 / 128
    (32, 128, True, 1100),      # unidirectional buckets over many tiles
    (64, 256, False, 900),      # the window around the diagonal is wider than a tile pair
    (16, 32, False, 700),       # narrow window: most tiles lie beyond +-max_distance
    (128, 1024, False, 640),    # every tile is inside the window
    (8, 20, True, 333),
]


@pytest.mark.parametrize("nb,md,causal,L", BUCKET_CASES)
def test_bucket_geometries_gradients_vs_oracle(nb, md, causal, L):
    dt = torch.bfloat16
    B, H = 1, 2
    q = seeded((B, H, L, 64), 11, 0.5, dtype=dt)
    k = seeded((B, H, L, 64), 12, 0.5, dtype=dt)
    v = seeded((B, H, L, 64), 13, dtype=dt)
    dout = seeded((B, H, L, 64), 15, dtype=dt)
    table = seeded((nb, H), 14, 0.2, dtype=dt)
    want = _oracle_grads(q, k, v, table, dout, causal=causal, num_buckets=nb, max_distance=md)
    got = _cuda_grads(q, k, v, table, dout, dt, causal=causal, NUM_BUCKETS=nb, MAX_DISTANCE=md)
    what = f"{(nb, md, causal, L)}"
    check_close(got[0], want[0], dt, what + " out")
    for g, w, nm in zip(got[1:], want[1:], ("dq", "dk", "dv", "dtable")):
        check_grad_close(g, w, what + " " + nm, floor=2.0 if nm == "dtable" else 1e-6)


def test_no_bias_scale_and_strided_views():
    # BHLD views of BLHD buffers, sm_scale != 1, no table: gradients keep the inputs' layout
    t5b = _ops()
    dt = torch.bfloat16
    B, H, L, D = 2, 3, 300, 64
    base = [seeded((B, L, H, D), s, 0.7, dtype=dt) for s in (1, 2, 3)]
    dout = seeded((B, H, L, D), 5, dtype=dt)
    want = _oracle_grads(*(t.transpose(1, 2) for t in base), None, dout, sm_scale=0.25)
    leaves = [t.cuda().requires_grad_(True) for t in base]
    out = t5b.flash_attention_with_fusing_bias(*(t.transpose(1, 2) for t in leaves), None, sm_scale=0.25)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    for leaf, w, nm in zip(leaves, want[1:4], ("dq", "dk", "dv")):
        check_grad_close(leaf.grad.transpose(1, 2), w, nm)


@pytest.mark.parametrize("causal", [False, True])
def test_varlen_gradients_vs_oracle(causal):
    t5b = _ops()
    dt = torch.bfloat16
    lens = [5, 128, 0, 129, 300, 1, 257, 64]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    T, H = int(cu[-1]), 3
    q, k, v = seeded((T, H, 64), 1, 0.5, dtype=dt), seeded((T, H, 64), 2, 0.5, dtype=dt), seeded((T, H, 64), 3, dtype=dt)
    dout = seeded((T, H, 64), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    qf, kf, vf, tf = (t.float().requires_grad_(True) for t in (q, k, v, table))
    want = orc.attention_basic_varlen(qf, kf, vf, tf, cu, cu, causal=causal)
    (want * dout.float()).sum().backward()
    qc, kc, vc, tc = (t.cuda().requires_grad_(True) for t in (q, k, v, table))
    out = t5b.flash_attention_with_fusing_bias_varlen(qc, kc, vc, tc, cu.cuda(), cu.cuda(), max(lens), max(lens),
                                                      causal=causal, sm_scale=1.0)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out.detach(), want.detach(), dt, "varlen out")
    for g, w, nm in ((qc.grad, qf.grad, "dq"), (kc.grad, kf.grad, "dk"), (vc.grad, vf.grad, "dv"),
                     (tc.grad, tf.grad, "dtable")):
        check_grad_close(g, w, f"varlen causal={causal} {nm}")


SIMT_CASES = [
    # dtype, D, B, H, M, N, causal, q_pos_offset
    (torch.float32, 64, 2, 8, 512, 512, False, None),     # the reference's float32 parity config
    (torch.float32, 64, 1, 2, 200, 333, True, None),
    (torch.float32, 16, 1, 2, 100, 100, False, None),
    (torch.float32, 128, 1, 2, 70, 150, False, 0),
    (torch.bfloat16, 32, 1, 2, 130, 130, True, None),
    (torch.bfloat16, 128, 1, 2, 300, 300, False, None),
    (torch.float16, 64, 1, 2, 100, 100, False, None),       # kernel="simt" on a tensor-core shape
]


@pytest.mark.parametrize("dt,D,B,H,M,N,causal,off", SIMT_CASES)
def test_cuda_core_backward_vs_oracle(dt, D, B, H, M, N, causal, off):
    # float32 tensors, rows that are not 16-byte aligned and kernel="simt" take the CUDA-core backward
    # (float32 arithmetic)
    q = seeded((B, H, M, D), 1, 0.5, dtype=dt)
    k = seeded((B, H, N, D), 2, 0.5, dtype=dt)
    v = seeded((B, H, N, D), 3, dtype=dt)
    dout = seeded((B, H, M, D), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = _oracle_grads(q, k, v, table, dout, causal=causal, q_pos_offset=off)
    kw = dict(kernel="simt") if dt != torch.float32 else {}
    got = _cuda_grads(q, k, v, table, dout, dt, causal=causal, q_pos_offset=off, **kw)
    rel = 2e-4 if dt == torch.float32 else 1e-2
    check_close(got[0], want[0], dt, "out")
    for g, w, nm in zip(got[1:], want[1:], ("dq", "dk", "dv", "dtable")):
        check_grad_close(g, w, f"{dt} d{D} {nm}", rel=rel, floor=(0.05 if dt == torch.float32 else 2.0) if nm == "dtable" else 1e-6)


CASES_D128 = [
    (2, 3, 512, 512, False, None),
    (1, 2, 777, 777, True, None),
    (2, 2, 128, 1024, False, 0),
    (1, 2, 200, 555, True, None),
    (1, 2, 300, 300, False, 4000),
    (1, 2, 2048, 2048, False, None),     # last wave split
]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,M,N,causal,off", CASES_D128)
def test_head_dim_128_tensor_core_backward_vs_oracle(B, H, M, N, causal, off, dt):
    q = seeded((B, H, M, 128), 1, 0.35, dtype=dt)
    k = seeded((B, H, N, 128), 2, 0.35, dtype=dt)
    v = seeded((B, H, N, 128), 3, dtype=dt)
    dout = seeded((B, H, M, 128), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = _oracle_grads(q, k, v, table, dout, causal=causal, q_pos_offset=off)
    got = _cuda_grads(q, k, v, table, dout, dt, causal=causal, q_pos_offset=off, kernel="tcgen05")
    what = f"d128 {(B, H, M, N, causal, off)}"
    check_close(got[0], want[0], dt, what + " out")
    for g, w, nm in zip(got[1:], want[1:], ("dq", "dk", "dv", "dtable")):
        check_grad_close(g, w, what + " " + nm, floor=2.0 if nm == "dtable" else 1e-6)


CASES_NARROW = [
    (2, 3, 512, 512, False, None),
    (1, 2, 777, 777, True, None),
    (2, 2, 128, 1024, False, 0),
    (1, 2, 300, 300, False, 4000),
    (1, 5, 2048, 2048, False, None),     # last wave split
]


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("D", [16, 32])
@pytest.mark.parametrize("B,H,M,N,causal,off", CASES_NARROW)
def test_narrow_head_dims_tensor_core_backward_vs_oracle(B, H, M, N, causal, off, D, dt):
    # head dims 16 and 32 run as head dim 64 with zero-filled columns; token-major storage, so a
    # gradient store wider than the head would land in the next head
    q = seeded((B, M, H, D), 1, 0.5, dtype=dt).transpose(1, 2)
    k = seeded((B, N, H, D), 2, 0.5, dtype=dt).transpose(1, 2)
    v = seeded((B, N, H, D), 3, dtype=dt).transpose(1, 2)
    dout = seeded((B, M, H, D), 5, dtype=dt).transpose(1, 2)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = _oracle_grads(q, k, v, table, dout, causal=causal, q_pos_offset=off)
    got = _cuda_grads(q, k, v, table, dout, dt, causal=causal, q_pos_offset=off, kernel="tcgen05")
    what = f"d{D} {(B, H, M, N, causal, off)}"
    check_close(got[0], want[0], dt, what + " out")
    for g, w, nm in zip(got[1:], want[1:], ("dq", "dk", "dv", "dtable")):
        assert g.shape == w.shape
        # with every key in one bucket (offset 4000) the table gradient is 180 000 rounded terms that
        # cancel to zero: the scale of its error is the sum of their magnitudes, not the result
        check_grad_close(g, w, what + " " + nm, floor=4.0 if nm == "dtable" else 1e-6)


@pytest.mark.parametrize("D", [16, 32])
def test_narrow_head_dims_backward_packed_sequences(D):
    t5b = _ops()
    dt = torch.bfloat16
    lens = [5, 128, 0, 129, 300, 1, 257, 64]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    T, H = int(cu[-1]), 3
    q, k, v = seeded((T, H, D), 1, 0.7, dtype=dt), seeded((T, H, D), 2, 0.7, dtype=dt), seeded((T, H, D), 3, dtype=dt)
    dout = seeded((T, H, D), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    qf, kf, vf, tf = (t.float().clone().requires_grad_(True) for t in (q, k, v, table))
    want = orc.attention_basic_varlen(qf, kf, vf, tf, cu, cu, causal=False)
    (want * dout.float()).sum().backward()
    qc, kc, vc, tc = (t.cuda().requires_grad_(True) for t in (q, k, v, table))
    out = t5b.flash_attention_with_fusing_bias_varlen(qc, kc, vc, tc, cu.cuda(), cu.cuda(), max(lens), max(lens),
                                                      sm_scale=1.0, kernel="tcgen05")
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    for g, w, nm in ((qc.grad, qf.grad, "dq"), (kc.grad, kf.grad, "dk"), (vc.grad, vf.grad, "dv"),
                     (tc.grad, tf.grad, "dtable")):
        check_grad_close(g, w, f"d{D} packed " + nm, floor=2.0 if nm == "dtable" else 1e-6)


def test_head_dim_128_backward_packed_sequences():
    t5b = _ops()
    dt = torch.bfloat16
    lens = [5, 128, 0, 129, 300, 1, 257, 64]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32)
    T, H = int(cu[-1]), 2
    q, k, v = seeded((T, H, 128), 1, 0.35, dtype=dt), seeded((T, H, 128), 2, 0.35, dtype=dt), seeded((T, H, 128), 3, dtype=dt)
    dout = seeded((T, H, 128), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    qf, kf, vf, tf = (t.float().clone().requires_grad_(True) for t in (q, k, v, table))
    want = orc.attention_basic_varlen(qf, kf, vf, tf, cu, cu, causal=True)
    (want * dout.float()).sum().backward()
    qc, kc, vc, tc = (t.cuda().requires_grad_(True) for t in (q, k, v, table))
    out = t5b.flash_attention_with_fusing_bias_varlen(qc, kc, vc, tc, cu.cuda(), cu.cuda(), max(lens), max(lens),
                                                      causal=True, sm_scale=1.0, kernel="tcgen05")
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    for g, w, nm in ((qc.grad, qf.grad, "dq"), (kc.grad, kf.grad, "dk"), (vc.grad, vf.grad, "dv"),
                     (tc.grad, tf.grad, "dtable")):
        check_grad_close(g, w, "d128 packed " + nm, floor=2.0 if nm == "dtable" else 1e-6)


def test_cuda_core_backward_packed_sequences_float32():
    t5b = _ops()
    lens_q, lens_k = [5, 40, 0, 33], [9, 40, 7, 70]
    cq = torch.tensor(np.concatenate([[0], np.cumsum(lens_q)]), dtype=torch.int32)
    ck = torch.tensor(np.concatenate([[0], np.cumsum(lens_k)]), dtype=torch.int32)
    H = 2
    q = seeded((int(cq[-1]), H, 32), 1, 0.5)
    k, v = seeded((int(ck[-1]), H, 32), 2, 0.5), seeded((int(ck[-1]), H, 32), 3)
    dout = seeded((int(cq[-1]), H, 32), 5)
    table = seeded((32, H), 4, 0.1)
    qf, kf, vf, tf = (t.clone().requires_grad_(True) for t in (q, k, v, table))
    want = orc.attention_basic_varlen(qf, kf, vf, tf, cq, ck, causal=False)
    (want * dout).sum().backward()
    qc, kc, vc, tc = (t.cuda().requires_grad_(True) for t in (q, k, v, table))
    out = t5b.flash_attention_with_fusing_bias_varlen(qc, kc, vc, tc, cq.cuda(), ck.cuda(), max(lens_q), max(lens_k),
                                                      sm_scale=1.0)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    for g, w, nm in ((qc.grad, qf.grad, "dq"), (kc.grad, kf.grad, "dk"), (vc.grad, vf.grad, "dv"),
                     (tc.grad, tf.grad, "dtable")):
        check_grad_close(g, w, "packed float32 " + nm, rel=2e-4, floor=0.05 if nm == "dtable" else 1e-6)


def test_backward_with_empty_sides_returns_zero_gradients():
    t5b = _ops()
    dt = torch.bfloat16
    q = torch.randn(1, 2, 5, 64, device="cuda", dtype=dt, requires_grad=True)
    k = torch.randn(1, 2, 0, 64, device="cuda", dtype=dt, requires_grad=True)
    v = torch.randn(1, 2, 0, 64, device="cuda", dtype=dt, requires_grad=True)
    table = torch.randn(32, 2, device="cuda", dtype=dt, requires_grad=True)
    out = t5b.flash_attention_with_fusing_bias(q, k, v, table, sm_scale=1.0)
    assert torch.count_nonzero(out) == 0
    out.sum().backward()
    assert torch.count_nonzero(q.grad) == 0 and k.grad.shape == k.shape and torch.count_nonzero(table.grad) == 0


def test_gradients_do_not_depend_on_how_dout_is_laid_out():
    # a transposed (non-contiguous) upstream gradient is accepted as it is or copied; same result
    t5b = _ops()
    dt = torch.bfloat16
    q, k, v = (seeded((1, 2, 200, 64), s, 0.5, dtype=dt).cuda().requires_grad_(True) for s in (1, 2, 3))
    dout = seeded((1, 200, 2, 64), 5, dtype=dt).cuda()
    grads = []
    for d in (dout.transpose(1, 2), dout.transpose(1, 2).contiguous()):
        for t in (q, k, v):
            t.grad = None
        t5b.flash_attention_with_fusing_bias(q, k, v, None, sm_scale=1.0).backward(d)
        grads.append([t.grad.clone() for t in (q, k, v)])
    torch.cuda.synchronize()
    for a, b in zip(*grads):
        assert torch.equal(a, b)


def test_last_wave_split_leaves_its_scratch_clean():
    # two different shapes after each other share the scratch buffer: the second must not see
    # anything of the first (counters and float32 rows are zeroed by the last part to arrive)
    dt = torch.bfloat16
    for (M, N) in ((2048, 2048), (1000, 1500), (2048, 2048)):
        q = seeded((1, 2, M, 64), 1, 0.5, dtype=dt)
        k = seeded((1, 2, N, 64), 2, 0.5, dtype=dt)
        v = seeded((1, 2, N, 64), 3, dtype=dt)
        dout = seeded((1, 2, M, 64), 5, dtype=dt)
        table = seeded((32, 2), 4, 0.1, dtype=dt)
        want = _oracle_grads(q, k, v, table, dout, q_pos_offset=0)
        got = _cuda_grads(q, k, v, table, dout, dt, q_pos_offset=0)
        for g, w, nm in zip(got[1:], want[1:], ("dq", "dk", "dv", "dtable")):
            check_grad_close(g, w, f"{(M, N)} {nm}", floor=2.0 if nm == "dtable" else 1e-6)
    from turbot5_b200 import attention as att
    for key, ws in att._workspaces.items():
        if key[0] == "attn_bwd":
            assert torch.count_nonzero(ws) == 0


@pytest.mark.parametrize("D,L,bl", [(64, 1024, 256), (64, 300, 128), (64, 200, 512), (128, 768, 128), (32, 640, 128),
                                    (16, 300, 128)])
def test_block_local_attention_gradients_vs_oracle(D, L, bl):
    t5b = _ops()
    dt = torch.bfloat16
    q, k, v = (seeded((1, 2, L, D), s, 0.5 if D == 64 else 0.35, dtype=dt) for s in (1, 2, 3))
    dout = seeded((1, 2, L, D), 5, dtype=dt)
    table = seeded((32, 2), 4, 0.1, dtype=dt)
    ref = [t.float().clone().requires_grad_(True) for t in (q, k, v, table)]
    want = orc.local_attention_basic(*ref, bl)
    (want * dout.float()).sum().backward()
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, table)]
    out = t5b.flash_attention_with_fusing_bias(*leaves, sm_scale=1.0, local_block=bl)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out.detach(), want.detach(), dt, "local out")
    for g, w, nm in zip(leaves, ref, ("dq", "dk", "dv", "dtable")):
        check_grad_close(g.grad, w.grad, f"local d{D} L{L} block {bl} {nm}", floor=2.0 if nm == "dtable" else 1e-6)


@pytest.mark.parametrize("D,bl,lens", [(64, 256, [1500, 700, 1]), (64, 128, [700, 129, 128]), (128, 256, [900, 300]),
                                       (64, 1024, [300, 77]), (64, 512, [3000]), (32, 128, [700, 129, 128]), (16, 256, [900, 300])])
def test_sliding_window_gradients_vs_oracle(D, bl, lens):
    """Packed sequences with the sliding window |key - query| < window (T5LocalAttention with its
    padding mask): dq, dk, dv and the bias-table gradient against float32 autograd of the oracle."""
    t5b = _ops()
    dt = torch.bfloat16
    H, T = 2, sum(lens)
    q, k, v = (seeded((T, H, D), s, 0.5 if D == 64 else 0.35, dtype=dt) for s in (1, 2, 3))
    dout = seeded((T, H, D), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    ref = [t.float().clone().requires_grad_(True) for t in (q, k, v, table)]
    outs, lo = [], 0
    for n in lens:
        seq = [t[lo:lo + n].transpose(0, 1).unsqueeze(0) for t in ref[:3]]          # (1, H, n, D)
        outs.append(orc.local_attention_basic(*seq, ref[3], bl, key_padding_mask=torch.ones((1, n)))[0].transpose(0, 1))
        lo += n
    want = torch.cat(outs)
    (want * dout.float()).sum().backward()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, table)]
    out = t5b.flash_attention_with_fusing_bias_varlen(*leaves, cu, cu, max(lens), max(lens), sm_scale=1.0, window=bl)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out.detach(), want.detach(), dt, "window out")
    for g, w, nm in zip(leaves, ref, ("dq", "dk", "dv", "dtable")):
        check_grad_close(g.grad, w.grad, f"window d{D} block {bl} {nm}", floor=2.0 if nm == "dtable" else 1e-6)


@pytest.mark.parametrize("D,L,bl", [(64, 1100, 256), (128, 640, 128), (32, 640, 128)])
def test_dense_sliding_window_gradients_vs_oracle(D, L, bl):
    t5b = _ops()
    dt = torch.bfloat16
    q, k, v = (seeded((2, 2, L, D), s, 0.5 if D == 64 else 0.35, dtype=dt) for s in (1, 2, 3))
    dout = seeded((2, 2, L, D), 5, dtype=dt)
    table = seeded((32, 2), 4, 0.1, dtype=dt)
    ref = [t.float().clone().requires_grad_(True) for t in (q, k, v, table)]
    want = orc.local_attention_basic(*ref, bl, key_padding_mask=torch.ones((2, L)))
    (want * dout.float()).sum().backward()
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, table)]
    out = t5b.flash_attention_with_fusing_bias(*leaves, sm_scale=1.0, window=bl)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    check_close(out.detach(), want.detach(), dt, "window out")
    for g, w, nm in zip(leaves, ref, ("dq", "dk", "dv", "dtable")):
        check_grad_close(g.grad, w.grad, f"dense window d{D} L{L} block {bl} {nm}", floor=2.0 if nm == "dtable" else 1e-6)


def test_local_module_with_padding_mask_trains():
    """T5LocalFlashAttention with the raw mask under autograd: unpad, packed kernel with the window, pad;
    gradient of the hidden states against float32 autograd of the oracle (valid rows; padded rows get none)."""
    t5b = _ops()
    dt = torch.bfloat16
    H, D, L, bl, lens = 2, 64, 900, 256, [900, 411]
    B = len(lens)

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
    mod = mod.cuda().to(dt).train()
    hidden = seeded((B, L, H * D), 5, 0.5, dtype=dt)
    dout = seeded((B, L, H * D), 6, dtype=dt)
    mask = torch.zeros((B, L), dtype=torch.int64)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    hid = hidden.cuda().requires_grad_(True)
    out = mod(hid, mask=mask.cuda())[0]
    (out.float() * (dout.cuda().float() * mask.cuda()[..., None])).sum().backward()
    torch.cuda.synchronize()
    t5b.check_device_status()
    href = hidden.float().clone().requires_grad_(True)
    tref = table.float().clone().requires_grad_(True)
    shape = lambda x: x.view(B, L, H, D).transpose(1, 2)
    want = orc.local_attention_basic(shape(href), shape(href[..., pk_]), shape(href[..., pv_]), tref, bl,
                                     key_padding_mask=mask.float())
    want = want.transpose(1, 2).reshape(B, L, H * D)
    (want * (dout.float() * mask[..., None])).sum().backward()
    for b, n in enumerate(lens):
        check_grad_close(hid.grad[b, :n], href.grad[b, :n], f"masked local hidden grad row {b}", rel=3e-2)
        assert torch.count_nonzero(hid.grad[b, n:]) == 0
    check_grad_close(mod.relative_attention_bias.weight.grad, tref.grad, "masked local dtable", floor=2.0)


def test_gradients_at_a_long_sequence():
    # 4096 x 4096 keys, two heads: every tile class of the backward kernels (far tiles with one bias
    # bucket, diagonal tiles with per-element bias, the split last wave) in one call, against float32
    # autograd of the oracle on the whole problem
    dt = torch.bfloat16
    B, H, L = 1, 2, 4096
    q = seeded((B, H, L, 64), 1, 0.5, dtype=dt)
    k = seeded((B, H, L, 64), 2, 0.5, dtype=dt)
    v = seeded((B, H, L, 64), 3, dtype=dt)
    dout = seeded((B, H, L, 64), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    want = _oracle_grads(q, k, v, table, dout)
    got = _cuda_grads(q, k, v, table, dout, dt)
    check_close(got[0], want[0], dt, "out")
    for g, w, nm in zip(got[1:], want[1:], ("dq", "dk", "dv", "dtable")):
        check_grad_close(g, w, "4k " + nm, floor=2.0 if nm == "dtable" else 1e-6)
