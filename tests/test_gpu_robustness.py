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
