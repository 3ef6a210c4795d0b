"""turbot5_b200: B200 (sm_100a) kernels for T5's relative-position-bias attention path.

Drop-in for the `attention_type='flash'` path of TurboT5: the same module and
function names, backed by hand-written CUDA behind a C ABI
(`include/turbot5_b200.h`, `libturbot5_b200.so`).  There is no CPU path and no
other backend: operators raise if the library is missing or a tensor is not on a
CUDA device.
"""
from .attention import (check_device_status, flash_attention_partial, flash_attention_with_fusing_bias,
                        flash_attention_with_fusing_bias_varlen, flash_decoding_with_fusing_bias,
                        merge_attention_partials, relative_position_bucket_grid, relative_position_bucket_table)

from .modules import (RMSLayerNorm, T5ATTENTION_TYPES, T5FlashAttention, T5LayerNorm, T5LocalFlashAttention,
                      add_rms_layer_norm, gated_gelu, rms_layer_norm)
from .padding import get_unpad_plan, pad_rows, unpad_rows
from .sequence_parallel import (sequence_parallel_attention, sequence_parallel_attention_overlapped, shard_bounds,
                                shard_size)

__all__ = [
    "T5ATTENTION_TYPES", "T5FlashAttention", "T5LocalFlashAttention", "T5LayerNorm", "RMSLayerNorm", "rms_layer_norm",
    "get_unpad_plan", "unpad_rows", "pad_rows",
    "add_rms_layer_norm", "gated_gelu", "flash_attention_partial", "merge_attention_partials",
    "sequence_parallel_attention", "sequence_parallel_attention_overlapped", "shard_bounds", "shard_size",
    "flash_attention_with_fusing_bias", "flash_attention_with_fusing_bias_varlen",
    "flash_decoding_with_fusing_bias", "relative_position_bucket_table",
    "relative_position_bucket_grid", "check_device_status",
]
