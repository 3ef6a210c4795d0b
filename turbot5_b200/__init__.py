"""turbot5_b200: B200 (sm_100a) kernels for T5's relative-position-bias attention path.

Drop-in for the `attention_type='flash'` path of TurboT5: the same module and
function names, backed by hand-written CUDA behind a C ABI
(`include/turbot5_b200.h`, `libturbot5_b200.so`).  There is no CPU path and no
other backend: operators raise if the library is missing or a tensor is not on a
CUDA device.
"""
from .attention import (check_device_status, flash_attention_with_fusing_bias,
                        flash_attention_with_fusing_bias_varlen, flash_decoding_with_fusing_bias,
                        relative_position_bucket_grid, relative_position_bucket_table)

__all__ = [
    "flash_attention_with_fusing_bias", "flash_attention_with_fusing_bias_varlen",
    "flash_decoding_with_fusing_bias", "relative_position_bucket_table",
    "relative_position_bucket_grid", "check_device_status",
]
