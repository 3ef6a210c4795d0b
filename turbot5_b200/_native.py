"""ctypes binding of `libturbot5_b200.so` (the C ABI in include/turbot5_b200.h).

The library is the only compute path: if it cannot be loaded the import of any
operator raises, there is no fallback.  `torch` is used here only to read
pointers, strides and the current stream.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libturbot5_b200.so")

OK = 0
ERR_DEVICE_TIMEOUT = 7
ERR_UNSUPPORTED = 10
F32, F16, BF16 = 0, 1, 2
KERNEL_AUTO, KERNEL_TCGEN05, KERNEL_SIMT, KERNEL_TCGEN05_POLYEXP, KERNEL_TCGEN05_2TILE = 0, 1, 2, 3, 4
KERNELS = {"auto": KERNEL_AUTO, "tcgen05": KERNEL_TCGEN05, "simt": KERNEL_SIMT,
           "tcgen05_polyexp": KERNEL_TCGEN05_POLYEXP, "tcgen05_2tile": KERNEL_TCGEN05_2TILE}

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}

SYMBOLS = ("t5b_status_string", "t5b_abi_version", "t5b_bucket_table_host", "t5b_bucket_indices",
           "t5b_attention_fwd", "t5b_attention_workspace_bytes", "t5b_attention_bwd", "t5b_attention_bwd_workspace_bytes", "t5b_decode_workspace_bytes", "t5b_decode_num_splits",
           "t5b_decode_fwd", "t5b_decode_static_scratch_bytes", "t5b_decode_fwd_static_scratch",
           "t5b_rmsnorm_fwd", "t5b_rmsnorm_bwd", "t5b_unpad_plan", "t5b_gather_rows",
           "t5b_scatter_rows", "t5b_attention_merge", "t5b_add_rmsnorm_fwd", "t5b_gated_gelu_fwd",
           "t5b_check_status", "t5b_selftest_bounded_wait")


class AttnArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("lse", C.c_void_p), ("table", C.c_void_p),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p), ("device_status", C.c_void_p),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_m", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64), ("k_stride_n", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64), ("v_stride_n", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64), ("o_stride_m", C.c_int64),
        ("table_stride0", C.c_int64),
        ("dtype", C.c_int32), ("table_dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("total_q", C.c_int32), ("total_k", C.c_int32),
        ("causal", C.c_int32), ("num_buckets", C.c_int32), ("max_distance", C.c_int32),
        ("q_pos_offset", C.c_int32), ("kernel", C.c_int32), ("sm_scale", C.c_float),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("local_block", C.c_int32), ("out_f32", C.c_int32), ("window", C.c_int32),
    ]


class AttnBwdArgs(C.Structure):
    _fields_ = [
        ("fwd", AttnArgs), ("dout", C.c_void_p),
        ("do_stride_b", C.c_int64), ("do_stride_h", C.c_int64), ("do_stride_m", C.c_int64),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dtable", C.c_void_p), ("delta", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
    ]


MERGE_MAX_PARTS = 8


class MergeArgs(C.Structure):
    _fields_ = [
        ("part_out", C.c_void_p * MERGE_MAX_PARTS), ("part_lse", C.c_void_p * MERGE_MAX_PARTS),
        ("out", C.c_void_p), ("lse_out", C.c_void_p),
        ("part_stride_b", C.c_int64), ("part_stride_h", C.c_int64), ("part_stride_m", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64), ("o_stride_m", C.c_int64),
        ("n_parts", C.c_int32), ("out_dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("M", C.c_int32), ("D", C.c_int32),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("table", C.c_void_p), ("seqlens_k", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_m", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_h", C.c_int64), ("k_stride_n", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_h", C.c_int64), ("v_stride_n", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64), ("o_stride_m", C.c_int64),
        ("table_stride0", C.c_int64),
        ("dtype", C.c_int32), ("table_dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("M", C.c_int32), ("N", C.c_int32), ("D", C.c_int32),
        ("causal", C.c_int32), ("num_buckets", C.c_int32), ("max_distance", C.c_int32),
        ("q_pos_offset", C.c_int32), ("num_splits", C.c_int32), ("sm_scale", C.c_float),
    ]


_lib = None


def lib():
    """The loaded library.  Raises if it has not been built (no fallback path)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m turbot5_b200.build` "
            "(nvcc, sm_100a).  turbot5_b200 has no CPU or PyTorch fallback.")
    L = C.CDLL(LIB_PATH)
    L.t5b_status_string.restype = C.c_char_p
    L.t5b_status_string.argtypes = [C.c_int]
    L.t5b_abi_version.restype = C.c_int
    L.t5b_bucket_table_host.restype = C.c_int
    L.t5b_bucket_table_host.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    L.t5b_bucket_indices.restype = C.c_int
    L.t5b_bucket_indices.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
    L.t5b_attention_fwd.restype = C.c_int
    L.t5b_attention_fwd.argtypes = [C.POINTER(AttnArgs), C.c_void_p]
    L.t5b_attention_bwd.restype = C.c_int
    L.t5b_attention_bwd.argtypes = [C.POINTER(AttnBwdArgs), C.c_void_p]
    L.t5b_attention_bwd_workspace_bytes.restype = C.c_int64
    L.t5b_attention_bwd_workspace_bytes.argtypes = [C.POINTER(AttnBwdArgs)]
    L.t5b_attention_workspace_bytes.restype = C.c_int64
    L.t5b_attention_workspace_bytes.argtypes = [C.POINTER(AttnArgs)]
    L.t5b_decode_workspace_bytes.restype = C.c_int64
    L.t5b_decode_workspace_bytes.argtypes = [C.c_int] * 5
    L.t5b_decode_num_splits.restype = C.c_int
    L.t5b_decode_num_splits.argtypes = [C.c_int] * 3
    L.t5b_decode_fwd.restype = C.c_int
    L.t5b_decode_fwd.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
    L.t5b_decode_static_scratch_bytes.restype = C.c_int64
    L.t5b_decode_static_scratch_bytes.argtypes = []
    L.t5b_decode_fwd_static_scratch.restype = C.c_int
    L.t5b_decode_fwd_static_scratch.argtypes = [C.POINTER(DecodeArgs), C.c_void_p]
    L.t5b_rmsnorm_fwd.restype = C.c_int
    L.t5b_rmsnorm_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                  C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_void_p]
    L.t5b_rmsnorm_bwd.restype = C.c_int
    L.t5b_rmsnorm_bwd.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                                  C.c_int64, C.c_int64, C.c_int64, C.c_int32, C.c_int32, C.c_float, C.c_void_p]
    L.t5b_unpad_plan.restype = C.c_int
    L.t5b_unpad_plan.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_void_p]
    L.t5b_check_status.restype = C.c_int
    L.t5b_check_status.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_void_p]
    L.t5b_selftest_bounded_wait.restype = C.c_int
    L.t5b_selftest_bounded_wait.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
    L.t5b_attention_merge.restype = C.c_int
    L.t5b_attention_merge.argtypes = [C.POINTER(MergeArgs), C.c_void_p]
    L.t5b_add_rmsnorm_fwd.restype = C.c_int
    L.t5b_add_rmsnorm_fwd.argtypes = [C.c_void_p] * 5 + [C.c_int64, C.c_int32] + [C.c_int64] * 4 + \
                                      [C.c_int32, C.c_int32, C.c_float, C.c_void_p]
    L.t5b_gated_gelu_fwd.restype = C.c_int
    L.t5b_gated_gelu_fwd.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int64, C.c_int64, C.c_int32,
                                     C.c_void_p]
    for name in ("t5b_gather_rows", "t5b_scatter_rows"):
        fn = getattr(L, name)
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]
    _lib = L
    return L


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise TypeError(f"turbot5_b200 supports float32, float16 and bfloat16, got {dt}") from None


def check(status: int, what: str):
    if status != OK:
        msg = lib().t5b_status_string(status).decode()
        raise RuntimeError(f"{what}: {msg} (t5b_status {status})")


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("turbot5_b200 operators need CUDA tensors: there is no CPU path")


def stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t):
    return None if t is None else t.data_ptr()
