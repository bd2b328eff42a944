"""B200-native attention for TinyTensor: forward, autograd backward and single-query decode.

The GPU work lives in `lib/libtt_attn.so` (hand-written sm_100a CUDA behind the C ABI of
`include/tt_attn.h`); `capi` binds it with ctypes, `functional` wraps it for torch CUDA
tensors, `sharder` spreads the independent (batch, head) slices over ranks.
The directory name contains a hyphen, so import it with
`importlib.import_module("pku-aiprogramming_b200")`.
"""
from . import capi  # noqa: F401  (raises NativeLibraryMissing with the build command if absent)
from .capi import TTError, NativeLibraryMissing, shard_range, launch_count  # noqa: F401
from .functional import (  # noqa: F401
    attention_forward, attention_backward, attention_decode, decode_workspace_bytes,
    attention_forward_host, attention_backward_host, attention_decode_host, attention_step_host,
    check_device_status, softmax_forward, softmax_backward, fc_forward, fc_backward, attention_decode_paged,
    set_backward_deterministic, attention_forward_varlen, attention_backward_varlen,
)
