"""ctypes binding of `lib/libtt_attn.so` (the C ABI declared in `include/tt_attn.h`).

Everything the Python side of this package does on a GPU goes through these entry
points; there is no alternative implementation to fall back to.  If the shared library
has not been built, importing this module raises with the build command.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libtt_attn.so")

TT_OK = 0
TT_ERR_NULL, TT_ERR_BAD_SHAPE, TT_ERR_BAD_DTYPE, TT_ERR_BAD_DEVICE = 1, 2, 3, 4
TT_ERR_WORKSPACE, TT_ERR_CUDA, TT_ERR_TIMEOUT, TT_ERR_UNSUPPORTED, TT_ERR_NCCL = 5, 6, 7, 8, 9
TT_F32, TT_BF16 = 0, 1

STATUS_NAMES = {
    0: "TT_OK", 1: "TT_ERR_NULL", 2: "TT_ERR_BAD_SHAPE", 3: "TT_ERR_BAD_DTYPE", 4: "TT_ERR_BAD_DEVICE",
    5: "TT_ERR_WORKSPACE", 6: "TT_ERR_CUDA", 7: "TT_ERR_TIMEOUT", 8: "TT_ERR_UNSUPPORTED", 9: "TT_ERR_NCCL",
}

# every symbol include/tt_attn.h declares: name -> (restype, argtypes)
class Desc(ctypes.Structure):
    _fields_ = [("B", c_int32), ("H", c_int32), ("S", c_int32), ("L", c_int32), ("D", c_int32),
                ("dtype", c_int32), ("causal", c_int32), ("scale", c_float), ("Hkv", c_int32)]


class VarlenDesc(ctypes.Structure):
    _fields_ = [("n_seq", c_int32), ("H", c_int32), ("Hkv", c_int32), ("D", c_int32), ("dtype", c_int32),
                ("causal", c_int32), ("scale", c_float), ("max_q", c_int32), ("max_k", c_int32),
                ("total_q", c_int64), ("total_k", c_int64)]


_P = c_void_p
_DP = POINTER(Desc)
_VP = POINTER(VarlenDesc)
SIGNATURES = {
    "tt_attn_fwd": (c_int, [_DP, _P, _P, _P, _P, _P, _P]),
    "tt_attn_bwd_workspace_bytes": (c_size_t, [_DP]),
    "tt_attn_bwd_set_deterministic": (c_int, [c_int]),
    "tt_attn_bwd": (c_int, [_DP, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_size_t, _P]),
    "tt_attn_fwd_padded": (c_int, [_DP, _P, _P, _P, _P, _P, _P, _P]),
    "tt_attn_bwd_padded": (c_int, [_DP, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_size_t, _P]),
    "tt_attn_fwd_varlen": (c_int, [_VP, _P, _P, _P, _P, _P, _P, _P, _P]),
    "tt_attn_bwd_varlen_workspace_bytes": (c_size_t, [_VP]),
    "tt_attn_bwd_varlen": (c_int, [_VP, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_size_t, _P]),
    "tt_attn_decode_workspace_bytes": (c_size_t, [_DP]),
    "tt_attn_decode": (c_int, [_DP, _P, _P, _P, _P, _P, _P, c_size_t, _P]),
    "tt_attn_decode_paged": (c_int, [_DP, _P, _P, _P, _P, _P, c_int32, c_int32, _P, _P, _P, c_size_t, _P]),
    "tt_attn_decode_static": (c_int, [_DP, _P, _P, _P, _P, _P, _P]),
    "tt_softmax_fwd": (c_int, [_P, _P, c_int64, c_int32, c_int32, _P]),
    "tt_softmax_bwd": (c_int, [_P, _P, _P, c_int64, c_int32, c_int32, _P]),
    "tt_fc_fwd": (c_int, [_P, _P, _P, _P, c_int64, c_int32, c_int32, c_int32, _P]),
    "tt_fc_bwd_workspace_bytes": (c_size_t, [c_int64, c_int32, c_int32, c_int32]),
    "tt_fc_bwd": (c_int, [_P, _P, _P, _P, _P, _P, c_int32, c_int64, c_int32, c_int32, c_int32, _P, c_size_t, _P]),
    "tt_fc_path": (c_int, [c_int64, c_int32, c_int32, c_int32]),
    "tt_attn_fwd_host": (c_int, [_DP, _P, _P, _P, _P, _P]),
    "tt_attn_bwd_host": (c_int, [_DP, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "tt_attn_decode_host": (c_int, [_DP, _P, _P, _P, _P, _P]),
    "tt_attn_fwd_bwd_host": (c_int, [_DP, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "tt_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "tt_free": (c_int, [_P]),
    "tt_host_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "tt_host_free": (c_int, [_P]),
    "tt_buffer_retain": (c_int, [_P]),
    "tt_buffer_release": (c_int, [_P]),
    "tt_pool_trim": (c_int, []),
    "tt_pool_stats": (c_int, [POINTER(c_size_t), POINTER(c_size_t), POINTER(c_uint64)]),
    "tt_shard_range": (c_int, [c_int64, c_int32, c_int32, POINTER(c_int64), POINTER(c_int64)]),
    "tt_mgpu_unique_id": (c_int, [_P]),
    "tt_mgpu_init": (c_int, [POINTER(c_void_p), c_int32, c_int32, _P]),
    "tt_mgpu_destroy": (c_int, [_P]),
    "tt_mgpu_shard": (c_int, [_P, _DP, POINTER(c_int64), POINTER(c_int64)]),
    "tt_mgpu_attn_fwd": (c_int, [_P, _DP, _P, _P, _P, _P, _P, _P, _P]),
    "tt_mgpu_bwd_workspace_bytes": (c_size_t, [_P, _DP]),
    "tt_mgpu_attn_bwd": (c_int, [_P, _DP, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, c_size_t, _P]),
    "tt_mgpu_wait": (c_int, [_P, _P]),
    "tt_last_error": (c_char_p, []),
    "tt_kernel_launch_count": (c_uint64, []),
    "tt_attn_fwd_path": (c_char_p, [_DP]),
    "tt_attn_bwd_path": (c_char_p, [_DP]),
    "tt_check_device_status": (c_int, [_P]),
    "tt_profile_enable": (c_int, [c_int]),
    "tt_profile_reset": (c_int, []),
    "tt_profile_kernel_count": (c_int, []),
    "tt_profile_kernel_name": (c_char_p, [c_int]),
    "tt_profile_read": (c_int, [c_int, POINTER(ctypes.c_double), POINTER(c_uint64)]),
    "tt_debug_wait_timeout": (c_int, [c_int64, _P]),
    "tt_debug_umma_probe": (c_int, [_P, _P, _P, c_int32, _P, _P, _P]),
}


# tuning aids declared in csrc/tt_debug.h (not part of the boundary)
DEBUG_SIGNATURES = {
    "tt_debug_fwd_trace": (c_int, [_P, c_int32, c_int32]),
    "tt_debug_bwd_trace": (c_int, [_P, c_int32, c_int32]),
    "tt_mgpu_set_collectives": (c_int, [_P]),
    "tt_debug_fail_host_call_after": (c_int, [c_int64]),
    "tt_debug_guard_syncs": (c_int64, []),
}


class NativeLibraryMissing(ImportError):
    pass


class TTError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise NativeLibraryMissing(
            f"{LIB_PATH} not found. Build it with `python {os.path.join(_PKG, 'build.py')}` "
            "(needs nvcc; there is no non-CUDA implementation of this package).")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in list(SIGNATURES.items()) + list(DEBUG_SIGNATURES.items()):
        fn = getattr(lib, name)   # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    return (lib.tt_last_error() or b"").decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != TT_OK:
        code = int(rc)
        if code in (TT_ERR_NULL, TT_ERR_BAD_SHAPE, TT_ERR_BAD_DTYPE, TT_ERR_BAD_DEVICE, TT_ERR_WORKSPACE):
            # argument errors surface as ValueError, like the reference's std::invalid_argument
            err = TTError(code, last_error())
            raise ValueError(str(err)) from err
        raise TTError(code, last_error())


def make_desc(B, H, S, L, D, dtype, causal=False, scale=None, Hkv=None) -> Desc:
    return Desc(int(B), int(H), int(S), int(L), int(D), int(dtype), 1 if causal else 0,
                float(scale) if scale is not None else 0.0, int(Hkv) if Hkv else 0)


def shard_range(n_slices: int, world: int, rank: int):
    b, c = c_int64(0), c_int64(0)
    check(lib.tt_shard_range(int(n_slices), int(world), int(rank), ctypes.byref(b), ctypes.byref(c)))
    return int(b.value), int(c.value)


def launch_count() -> int:
    return int(lib.tt_kernel_launch_count())


def profile_enable(on: bool = True) -> None:
    check(lib.tt_profile_enable(1 if on else 0))


def profile_reset() -> None:
    check(lib.tt_profile_reset())


def profile_read() -> dict:
    """{kernel name: (total device ms, timed launches)} for every kernel family with launches."""
    res = {}
    for i in range(int(lib.tt_profile_kernel_count())):
        ms, n = ctypes.c_double(0.0), c_uint64(0)
        check(lib.tt_profile_read(i, ctypes.byref(ms), ctypes.byref(n)))
        if n.value:
            res[lib.tt_profile_kernel_name(i).decode()] = (float(ms.value), int(n.value))
    return res
