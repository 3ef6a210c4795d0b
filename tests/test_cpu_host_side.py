"""CPU-only checks of the C ABI library and the host-side logic (no kernel launches)."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from tests.helpers import load

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from turbot5_b200 import _native as nat
    header = open(os.path.join(ROOT, "include", "turbot5_b200.h")).read()
    declared = set(re.findall(r"T5B_API[^;(]*?\b(t5b_\w+)\s*\(", header))
    assert declared == set(nat.SYMBOLS), declared ^ set(nat.SYMBOLS)
    L = ctypes.CDLL(nat.LIB_PATH)
    for name in declared:
        assert hasattr(L, name), name
    assert nat.lib().t5b_abi_version() == 1
    assert nat.lib().t5b_status_string(0) == b"ok"


def test_struct_layouts_match_header_field_order():
    from turbot5_b200 import _native as nat
    header = open(os.path.join(ROOT, "include", "turbot5_b200.h")).read()
    for cname, cls in (("t5b_attn_args", nat.AttnArgs), ("t5b_decode_args", nat.DecodeArgs),
                       ("t5b_attn_bwd_args", nat.AttnBwdArgs)):
        end = header.index("} " + cname + ";")
        body = header[header.rindex("typedef struct {", 0, end) + len("typedef struct {"):end]
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            parts = decl.replace("*", " ").split(",")
            names.append(parts[0].split()[-1])
            names += [p.strip() for p in parts[1:]]
        assert names == [f[0] for f in cls._fields_], cname


def _header_fields(cname):
    header = open(os.path.join(ROOT, "include", "turbot5_b200.h")).read()
    end = header.index("} " + cname + ";")
    body = header[header.rindex("typedef struct {", 0, end) + len("typedef struct {"):end]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        ctype = "ptr" if "*" in decl else decl.split()[0]
        parts = decl.replace("*", " ").split(",")
        fields.append((parts[0].split()[-1], ctype))
        fields += [(p.strip(), ctype) for p in parts[1:]]
    return fields


def test_integration_stub_struct_matches_header():
    """The ctypes struct a maintainer would paste from INTEGRATION.md has the header's fields, in
    order and with the header's types (a struct that is short or reordered corrupts calls)."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    start = text.index("class _AttnArgs(C.Structure)")
    end = text.index("_lib.t5b_attention_fwd.argtypes")
    scope = {"C": ctypes}
    exec(text[start:end], scope)
    stub = scope["_AttnArgs"]
    ctype_of = {"ptr": ctypes.c_void_p, "int64_t": ctypes.c_int64, "int32_t": ctypes.c_int32, "float": ctypes.c_float}
    want = [(n, ctype_of[t]) for n, t in _header_fields("t5b_attn_args")]
    assert [(n, t) for n, t in stub._fields_] == want
    from turbot5_b200 import _native as nat
    assert ctypes.sizeof(stub) == ctypes.sizeof(nat.AttnArgs)


def test_host_bucket_table_bit_exact_vs_reference_fixture():
    import turbot5_b200 as t5b
    z = load("buckets.npz")
    for nb, md, bidir, lo, hi in z["settings"]:
        key = f"nb{nb}_md{md}_{'bi' if bidir else 'uni'}"
        got = t5b.relative_position_bucket_table(int(nb), int(md), bool(bidir), int(lo), int(hi)).numpy()
        assert np.array_equal(got, z[key]), key


def test_host_bucket_table_rejects_bad_settings():
    import turbot5_b200 as t5b
    for nb, md in ((2, 128), (32, 0), (32, 4), (1024, 128)):
        with pytest.raises(RuntimeError):
            t5b.relative_position_bucket_table(nb, md, True)


def test_decode_split_heuristic_and_workspace_size():
    from turbot5_b200 import _native as nat
    L = nat.lib()
    assert L.t5b_decode_num_splits(64, 16, 8192) >= 2
    assert L.t5b_decode_num_splits(64, 16, 100) == 1
    assert L.t5b_decode_num_splits(1, 1, 1 << 20) == 64
    n = L.t5b_decode_workspace_bytes(64, 16, 1, 64, 8)
    assert n % 256 == 0 and n >= 64 * 16 * 8 * (64 + 2) * 4
    assert L.t5b_decode_workspace_bytes(0, 16, 1, 64, 8) == 0


def test_cpu_tensors_are_refused_not_silently_computed():
    import turbot5_b200 as t5b
    q = torch.zeros((1, 1, 4, 64))
    with pytest.raises(RuntimeError, match="CUDA"):
        t5b.flash_attention_with_fusing_bias(q, q, q, None)
    with pytest.raises(RuntimeError, match="CUDA"):
        t5b.rms_layer_norm(torch.zeros(2, 8), torch.ones(8))
    with pytest.raises(RuntimeError, match="CUDA"):
        t5b.get_unpad_plan(torch.ones((2, 3), dtype=torch.int64))


def test_entry_points_validate_arguments_without_a_device():
    from turbot5_b200 import _native as nat
    L = nat.lib()
    assert L.t5b_attention_fwd(None, None) == 5
    a = nat.AttnArgs()
    a.dtype, a.D, a.B, a.H, a.M, a.N = 7, 64, 1, 1, 1, 1
    assert L.t5b_attention_fwd(a, None) == 1           # dtype
    a.dtype, a.D = nat.BF16, 48
    assert L.t5b_attention_fwd(a, None) == 4           # head dim
    a.D, a.M = 64, -1
    assert L.t5b_attention_fwd(a, None) == 2           # shape
    a.M = 0
    assert L.t5b_attention_fwd(a, None) == 0           # empty problem: nothing to do
    a.M = 1
    assert L.t5b_attention_fwd(a, None) == 5           # null pointers
    assert L.t5b_rmsnorm_fwd(None, None, None, None, 1, 8, 8, 8, 0, 0, 1e-6, None) == 5
    assert L.t5b_decode_fwd(None, None) == 5
    assert L.t5b_unpad_plan(None, 1, 1, 1, None, None, None, None) == 5
    assert L.t5b_gather_rows(None, 16, None, 16, None, 1, 16, None) == 5


def test_registry_and_module_signature():
    import inspect
    import turbot5_b200 as t5b
    assert t5b.T5ATTENTION_TYPES["flash"] is t5b.T5FlashAttention
    sig = inspect.signature(t5b.T5FlashAttention.forward)
    assert list(sig.parameters)[1:] == ["hidden_states", "mask", "key_value_states", "position_bias",
                                        "past_key_value", "layer_head_mask", "query_length", "use_cache",
                                        "output_attentions"]
    sig = inspect.signature(t5b.flash_attention_with_fusing_bias)
    assert list(sig.parameters)[:8] == ["q", "k", "v", "bias", "causal", "sm_scale", "NUM_BUCKETS", "MAX_DISTANCE"]
    sig = inspect.signature(t5b.flash_attention_with_fusing_bias_varlen)
    assert list(sig.parameters)[:12] == ["q", "k", "v", "bias", "cu_seqlens_q", "cu_seqlens_k", "max_seqlen_q",
                                         "max_seqlen_k", "causal", "sm_scale", "NUM_BUCKETS", "MAX_DISTANCE"]


def test_host_bucket_table_matches_oracle_on_random_settings():
    # property test over (num_buckets, max_distance, direction): the library's host table (glibc
    # logf, float32 chain) and the oracle (the reference's torch expression) agree bit for bit
    from hypothesis import given, settings, strategies as st
    import turbot5_b200 as t5b
    from oracle import t5_oracle as orc

    @settings(max_examples=150, deadline=None)
    @given(st.sampled_from([4, 6, 8, 12, 16, 24, 32, 40, 64, 96, 128, 256]), st.integers(2, 2048), st.booleans())
    def check(nb, md, bidir):
        n_side = nb // 2 if bidir else nb
        if n_side < 2 or md <= n_side // 2:
            with pytest.raises(RuntimeError):
                t5b.relative_position_bucket_table(nb, md, bidir)
            return
        got = t5b.relative_position_bucket_table(nb, md, bidir, -md - 3, md + 3).numpy()
        want = orc.bucket_of_delta(range(-md - 3, md + 4), bidir, nb, md)
        assert np.array_equal(got, want), (nb, md, bidir)
        # monotone in distance on each side and saturating at max_distance
        neg = got[:md + 4][::-1]
        assert np.all(np.diff(neg) >= 0) and neg[md] == neg[-1]
    check()


def test_attention_workspace_query_is_zero_without_a_device_or_when_not_applicable():
    from turbot5_b200 import _native as nat
    L = nat.lib()
    a = nat.AttnArgs()
    assert L.t5b_attention_workspace_bytes(None) == 0
    a.dtype, a.D, a.B, a.H, a.M, a.N = nat.F32, 64, 1, 1, 4096, 4096
    assert L.t5b_attention_workspace_bytes(a) == 0        # float32 never takes the tensor-core kernel


def test_hot_kernels_stay_within_their_register_and_spill_budget():
    """ptxas's own report for the tensor-core kernels of the bench workload (bf16, head dim 64, no window):
    two blocks per SM need <= 96 registers, and the softmax loops are written to (almost) fit in them.
    Extra loop-live values show up here as spills long before any numerical test notices."""
    from turbot5_b200 import build
    fwd = build.resource_report("attn_fwd_sm100.cu")
    bwd = build.resource_report("attn_bwd_sm100.cu")

    def pick(report, *parts):
        names = [n for n in report if all(p in n for p in parts)]
        assert len(names) == 1, (parts, names)
        return report[names[0]]
    # mangled template arguments: Lb1 = bf16, Li64 = head dim, Li0 = no FMA-pipe exponentials, then Lb0 = no
    # window and Lb0 / Lb1 = head dim 64 itself / the kernel that also takes head dims 16 and 32
    for narrow in ("Lb0E", "Lb1E"):
        k = pick(fwd, "attn_fwd_kernel", "ILb1ELi64ELi0ELb0E" + narrow)
        assert k["registers"] <= 96 and k["spill_stores"] <= 128, k
    k = pick(bwd, "attn_bwd_dq_kernel", "ILb1ELi64ELb0E")
    assert k["registers"] <= 96 and k["spill_stores"] <= 16, k
    k = pick(bwd, "attn_bwd_dkv_wide_kernel", "ILb1ELb0E")
    assert k["registers"] <= 96 and k["spill_stores"] <= 64, k
