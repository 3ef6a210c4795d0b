"""The allocation-free decoding entry point against the ordinary one.

Some callers cannot allocate device memory at the point where they decode (a
serving loop with a frozen memory budget, a latency-critical thread where an
allocation could block, C code that was given only inputs and outputs).  `t5b_decode_fwd_static_scratch` keeps
the split-KV scratch in a fixed array inside the library instead.  This test
drives it through the C ABI with caller-owned input and output buffers and
checks it against `t5b_decode_fwd` on two consecutive calls (the second call
sees whatever the first one left in the shared array).  It runs last so that a
failure here cannot hide any other test's result.
"""
import pytest
import torch

from tests.helpers import seeded

pytestmark = pytest.mark.gpu


def _args(nat, q, k, v, out, table, N, splits, causal):
    a = nat.DecodeArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.table = None if table is None else table.data_ptr()
    a.seqlens_k = None
    a.workspace, a.workspace_bytes = None, 0
    a.q_stride_b, a.q_stride_h, a.q_stride_m = q.stride(0), q.stride(1), q.stride(2)
    a.k_stride_b, a.k_stride_h, a.k_stride_n = k.stride(0), k.stride(1), k.stride(2)
    a.v_stride_b, a.v_stride_h, a.v_stride_n = v.stride(0), v.stride(1), v.stride(2)
    a.o_stride_b, a.o_stride_h, a.o_stride_m = out.stride(0), out.stride(1), out.stride(2)
    a.table_stride0 = 0 if table is None else table.stride(0)
    a.dtype = nat.dtype_code(q.dtype)
    a.table_dtype = nat.F32 if table is None else nat.dtype_code(table.dtype)
    a.B, a.H, a.M, a.N, a.D = q.shape[0], q.shape[1], q.shape[2], N, q.shape[3]
    a.causal = int(causal)
    a.num_buckets, a.max_distance = 32, 128
    a.q_pos_offset = -1
    a.num_splits = splits
    a.sm_scale = 1.0
    return a


@pytest.mark.parametrize("B,H,M,N,causal,splits", [(3, 4, 1, 2000, True, 6), (2, 2, 3, 1500, True, 0),
                                                    (4, 16, 1, 8192, False, 0),
                                                    (2, 3, 7, 1800, True, 5),      # more rows than one launch takes:
                                                    (1, 2, 8, 3000, False, 0)])    # the counters serve several launches
def test_static_scratch_matches_workspace_entry_point(B, H, M, N, causal, splits):
    from turbot5_b200 import _native as nat
    L = nat.lib()
    dt = torch.bfloat16
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for call in range(2):                       # two calls in a row share the library's array
        q = seeded((B, H, M, 64), 10 + call, dtype=dt).to(dev)
        k = seeded((B, H, N, 64), 20 + call, dtype=dt).to(dev)
        v = seeded((B, H, N, 64), 30 + call, dtype=dt).to(dev)
        table = seeded((32, H), 40 + call, 0.1, dtype=dt).to(dev) if causal else None
        out_static = torch.full((B, H, M, 64), float("nan"), dtype=dt, device=dev)
        out_ws = torch.full((B, H, M, 64), float("nan"), dtype=dt, device=dev)
        n_splits = splits or L.t5b_decode_num_splits(B, H, N)
        ws = torch.zeros(L.t5b_decode_workspace_bytes(B, H, M, 64, n_splits), dtype=torch.uint8, device=dev)
        a = _args(nat, q, k, v, out_ws, table, N, n_splits, causal)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        assert L.t5b_decode_fwd(a, stream) == 0
        b = _args(nat, q, k, v, out_static, table, N, splits, causal)
        assert L.t5b_decode_fwd_static_scratch(b, stream) == 0
        torch.cuda.synchronize()
        assert not torch.isnan(out_static).any()
        # same kernel, same split count: the results agree to the tolerance of the other
        # decoding tests (max-abs 2e-2 for bf16); in practice they are identical
        assert (out_static.float() - out_ws.float()).abs().max().item() <= 2e-2
        assert torch.equal(out_static, out_ws)


def test_static_scratch_refuses_oversized_problems():
    from turbot5_b200 import _native as nat
    L = nat.lib()
    cap = L.t5b_decode_static_scratch_bytes()
    assert cap == 4 << 20
    dt = torch.bfloat16
    dev = torch.device("cuda", 0)
    B, H, N, splits = 64, 64, 4096, 8            # scratch need far above the built-in array
    assert L.t5b_decode_workspace_bytes(B, H, 1, 64, splits) > cap
    q = torch.zeros((B, H, 1, 64), dtype=dt, device=dev)
    k = torch.zeros((B, H, N, 64), dtype=dt, device=dev)
    out = torch.zeros_like(q)
    a = _args(nat, q, k, k, out, None, N, splits, False)
    status = L.t5b_decode_fwd_static_scratch(a, torch.cuda.current_stream(dev).cuda_stream)
    assert status == 8                            # T5B_ERR_WORKSPACE
    assert b"workspace" in L.t5b_status_string(status)


def test_static_scratch_checks_arguments_before_touching_the_array():
    """A call that is refused for its arguments reports that reason (not a scratch problem) and
    queues nothing on the shared array."""
    from turbot5_b200 import _native as nat
    L = nat.lib()
    dt = torch.bfloat16
    dev = torch.device("cuda", 0)
    stream = torch.cuda.current_stream(dev).cuda_stream
    q = torch.zeros((2, 2, 1, 64), dtype=dt, device=dev)
    k = torch.zeros((2, 2, 4096, 64), dtype=dt, device=dev)
    out = torch.zeros_like(q)
    a = _args(nat, q, k, k, out, None, 4096, 300, False)          # more than 256 splits
    assert L.t5b_decode_fwd_static_scratch(a, stream) == 5        # T5B_ERR_ARG, as t5b_decode_fwd answers
    a = _args(nat, q, k, k, out, None, 4096, 4, False)
    a.k = None
    assert L.t5b_decode_fwd_static_scratch(a, stream) == 5
    a = _args(nat, q, k, k, out, None, 4096, 4, False)
    a.D = 48
    assert L.t5b_decode_fwd_static_scratch(a, stream) == 4        # T5B_ERR_HEAD_DIM
    torch.cuda.synchronize()
