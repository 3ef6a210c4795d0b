"""Failure reporting without a fault: a bounded device-side wait that runs out is reported through
the status word, the kernel returns, and the GPU keeps working."""
import ctypes

import pytest
import torch

from oracle import t5_oracle as orc
from tests.helpers import check_close, seeded

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_is_reported():
    import turbot5_b200 as t5b
    from turbot5_b200 import _native as nat
    from turbot5_b200.attention import device_status
    L = nat.lib()
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    t5b.check_device_status(dev)                       # clean before the test
    word = device_status(dev)
    # a barrier nobody arrives at, limit 200 000 SM cycles (about 0.1 ms)
    assert L.t5b_selftest_bounded_wait(word.data_ptr(), 200000, stream) == 0
    code = ctypes.c_int32(0)
    assert L.t5b_check_status(word.data_ptr(), ctypes.byref(code), stream) == nat.ERR_DEVICE_TIMEOUT
    assert code.value == 9001                          # the single waiting thread gave up first
    assert b"wait ran out" in L.t5b_status_string(nat.ERR_DEVICE_TIMEOUT)
    assert int(word.item()) == 0                       # reading clears the word
    # the Python wrapper raises on it
    assert L.t5b_selftest_bounded_wait(word.data_ptr(), 50000, stream) == 0
    with pytest.raises(RuntimeError, match="gave up waiting"):
        t5b.check_device_status(dev)
    t5b.check_device_status(dev)                       # cleared again
    # arguments out of range are refused without a launch
    assert L.t5b_selftest_bounded_wait(word.data_ptr(), 0, stream) == 5
    assert L.t5b_selftest_bounded_wait(None, 1000, stream) == 5
    # and the next ordinary launches are correct
    dt = torch.bfloat16
    q, k, v = seeded((1, 2, 300, 64), 1, dtype=dt), seeded((1, 2, 300, 64), 2, dtype=dt), seeded((1, 2, 300, 64), 3, dtype=dt)
    table = seeded((32, 2), 4, 0.1, dtype=dt)
    out = t5b.flash_attention_with_fusing_bias(q.cuda(), k.cuda(), v.cuda(), table.cuda(), sm_scale=1.0)
    torch.cuda.synchronize()
    t5b.check_device_status(dev)
    check_close(out, orc.attention_basic(q, k, v, table), dt, "launch after a reported give-up")


def test_cu_seqlens_past_the_tensors_touch_nothing_beyond_them():
    """A cumulative-length array that runs past the row count of the packed tensors (a caller's mistake)
    is cut at the tensors: rows that exist are computed, nothing after them is read as data or written.
    The tensors are views into larger buffers whose remaining rows hold a sentinel (so even a wrong
    kernel would stay inside an allocation)."""
    import turbot5_b200 as t5b
    dt = torch.bfloat16
    H, D, rows, spare = 2, 64, 300, 200
    g = torch.Generator(device="cuda").manual_seed(3)
    bufs = [torch.randn((rows + spare, H, D), generator=g, device="cuda").to(dt) for _ in range(3)]
    for b in bufs:
        b[rows:] = 777.0
    q, k, v = (b[:rows] for b in bufs)
    table = (torch.randn((32, H), generator=g, device="cuda") * 0.1).to(dt)
    cu = torch.tensor([0, 200, 450], dtype=torch.int32, device="cuda")       # second sequence claims 250 rows, 100 exist
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
    out = t5b.flash_attention_with_fusing_bias_varlen(*leaves, table, cu, cu, 256, 256, sm_scale=1.0)
    dout = torch.randn((rows, H, D), generator=g, device="cuda").to(dt)
    grads = torch.autograd.grad(out, leaves, dout)
    torch.cuda.synchronize()
    t5b.check_device_status()
    # the same call with the lengths as they really are gives the same rows
    cu_ok = torch.tensor([0, 200, 300], dtype=torch.int32, device="cuda")
    want = t5b.flash_attention_with_fusing_bias_varlen(q, k, v, table, cu_ok, cu_ok, 256, 256, sm_scale=1.0)
    assert torch.equal(out.detach(), want)
    assert all(torch.isfinite(x).all() for x in grads)
    for b in bufs:
        assert (b[rows:] == 777.0).all()
