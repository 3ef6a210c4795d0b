"""Right-padded dense batches read in place (per-row lengths) against the oracle."""
import pytest
import torch

from oracle import t5_oracle as orc
from tests.helpers import check_close, check_grad_close, seeded

pytestmark = pytest.mark.gpu


def _ops():
    import turbot5_b200 as t5b
    return t5b


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_self_attention_with_row_lengths_forward_and_backward(D, causal):
    t5b = _ops()
    dt = torch.bfloat16
    B, H, L = 4, 2, 300
    lens = [300, 37, 129, 0]
    q, k, v = (seeded((B, H, L, D), s, 0.5 if D == 64 else 0.35, dtype=dt) for s in (1, 2, 3))
    dout = seeded((B, H, L, D), 5, dtype=dt)
    table = seeded((32, H), 4, 0.1, dtype=dt)
    sl = torch.tensor(lens, dtype=torch.int32).cuda()
    leaves = [t.cuda().requires_grad_(True) for t in (q, k, v, table)]
    out = t5b.flash_attention_with_fusing_bias(*leaves, causal=causal, sm_scale=1.0, seqlens_q=sl, seqlens_k=sl)
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    dtable = torch.zeros((32, H))
    for b, n in enumerate(lens):
        # padding rows: zeros out, zero gradients
        assert torch.count_nonzero(out[b, :, n:]) == 0
        for g in leaves[:3]:
            assert torch.count_nonzero(g.grad[b, :, n:]) == 0
        if n == 0:
            continue
        ref = [t[b:b + 1, :, :n].float().clone().requires_grad_(True) for t in (q, k, v)]
        tref = table.float().clone().requires_grad_(True)
        want = orc.attention_basic(*ref, tref, causal=causal)
        (want * dout[b:b + 1, :, :n].float()).sum().backward()
        check_close(out[b:b + 1, :, :n].detach(), want.detach(), dt, f"row {b}")
        for g, w, nm in zip(leaves[:3], ref, ("dq", "dk", "dv")):
            check_grad_close(g.grad[b:b + 1, :, :n], w.grad, f"row {b} {nm}")
        dtable += tref.grad
    check_grad_close(leaves[3].grad, dtable, "dtable", floor=2.0)


def test_cross_attention_with_key_lengths():
    t5b = _ops()
    dt = torch.bfloat16
    B, H, M, N = 3, 2, 70, 260
    lens = [260, 1, 131]
    q = seeded((B, H, M, 64), 1, 0.5, dtype=dt)
    k, v = seeded((B, H, N, 64), 2, 0.5, dtype=dt), seeded((B, H, N, 64), 3, dtype=dt)
    sl = torch.tensor(lens, dtype=torch.int32).cuda()
    out = t5b.flash_attention_with_fusing_bias(q.cuda(), k.cuda(), v.cuda(), None, sm_scale=1.0, q_pos_offset=0,
                                               seqlens_k=sl)
    torch.cuda.synchronize()
    for b, n in enumerate(lens):
        want = orc.attention_basic(q[b:b + 1], k[b:b + 1, :, :n], v[b:b + 1, :, :n], None, q_pos_offset=0)
        check_close(out[b:b + 1], want, dt, f"row {b}")


def test_module_reads_right_padded_batches_in_place():
    # the in-place path and the packing path of the module agree with each other and with the oracle layer
    from tests.test_gpu_other_kernels import _Cfg, _make_module, _oracle_layer
    dt = torch.bfloat16
    hidden = seeded((3, 200, 128), 2, dtype=dt)
    lens = [200, 37, 129]
    mask = torch.zeros((3, 200), dtype=torch.int64)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    packed = _make_module(_Cfg(), dt, 1)
    inplace = _make_module(_Cfg(right_padded_masks=True), dt, 1)
    with torch.no_grad():
        a = packed(hidden.cuda(), mask=mask.cuda())[0]
        b_ = inplace(hidden.cuda(), mask=mask.cuda())[0]
    want, _ = _oracle_layer(inplace, hidden, key_padding_mask=mask)
    for b, n in enumerate(lens):
        check_close(b_[b, :n], want[b, :n], dt, f"in place, batch row {b}")
        assert (a[b, :n].float() - b_[b, :n].float()).abs().max().item() <= 2e-2
        assert torch.count_nonzero(b_[b, n:]) == 0


@pytest.mark.parametrize("L,bl", [(600, 256), (300, 512)])
def test_block_local_attention_with_key_lengths(L, bl):
    t5b = _ops()
    dt = torch.bfloat16
    B, H = 3, 2
    lens = [L, 45, L - 130]
    q, k, v = (seeded((B, H, L, 64), s, 0.5, dtype=dt) for s in (1, 2, 3))
    table = seeded((32, H), 4, 0.1, dtype=dt)
    mask = torch.zeros((B, L), dtype=torch.int64)
    for b, n in enumerate(lens):
        mask[b, :n] = 1
    want = orc.local_attention_basic(q, k, v, table, bl, key_padding_mask=mask)
    out = t5b.flash_attention_with_fusing_bias(q.cuda(), k.cuda(), v.cuda(), table.cuda(), sm_scale=1.0, local_block=bl,
                                               seqlens_k=torch.tensor(lens, dtype=torch.int32).cuda())
    torch.cuda.synchronize()
    t5b.check_device_status()
    for b, n in enumerate(lens):
        check_close(out[b, :, :n], want[b, :, :n], dt, f"row {b}")
