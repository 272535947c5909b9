"""ctypes binding of libxfb200.so (the C-ABI library with every CUDA kernel).

There is no fallback: if the library is missing or a symbol cannot be found,
importing the operators raises, and calling an operator without a CUDA device
raises.  The structures mirror ``include/xfb200.h`` field by field.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

ABI_VERSION = 4

XFB200_OK = 0
XFB200_E_INVALID = -1
XFB200_E_UNSUPPORTED = -2
XFB200_E_CUDA = -3
XFB200_E_DEVICE = -4

BF16, F16, F32 = 0, 1, 2
MASK_NONE, MASK_CAUSAL_TOP_LEFT, MASK_CAUSAL_BOTTOM_RIGHT, MASK_LOCAL_BOTTOM_RIGHT = 0, 1, 2, 3
PREFILL_AUTO, PREFILL_MMA_SYNC, PREFILL_TCGEN05, PREFILL_TCGEN05_CTA, PREFILL_TCGEN05_PERSISTENT = 0, 1, 2, 4, 6
KV_PLAIN, KV_INT4_ROWWISE, KV_FP8_ROWWISE = 0, 1, 2
MERGE_MAX_PTRS = 32
DECODE_STATIC_SCRATCH_BYTES = 16 << 20

EXPORTED_SYMBOLS = (
    "xfb200_abi_version",
    "xfb200_last_error",
    "xfb200_prefill_forward",
    "xfb200_prefill_device_status",
    "xfb200_decode_device_status",
    "xfb200_decode_scratch_bytes",
    "xfb200_decode_forward",
    "xfb200_decode_forward_static_scratch",
    "xfb200_merge_attentions",
    "xfb200_rope_padded",
)


class Strides(C.Structure):
    _fields_ = [("b", C.c_int64), ("m", C.c_int64), ("g", C.c_int64), ("h", C.c_int64)]


class PrefillParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("out", C.c_void_p),
        ("lse", C.c_void_p),
        ("seqstart_q", C.c_void_p),
        ("seqstart_k", C.c_void_p),
        ("seqlen_k", C.c_void_p),
        ("dtype", C.c_int32),
        ("batch", C.c_int32),
        ("mq", C.c_int32),
        ("mkv", C.c_int32),
        ("total_q", C.c_int32),
        ("groups", C.c_int32),
        ("heads_per_group", C.c_int32),
        ("head_dim", C.c_int32),
        ("q_strides", Strides),
        ("k_strides", Strides),
        ("v_strides", Strides),
        ("o_strides", Strides),
        ("lse_stride_b", C.c_int64),
        ("lse_stride_g", C.c_int64),
        ("lse_stride_h", C.c_int64),
        ("mask_type", C.c_int32),
        ("kv_offset", C.c_int32),
        ("window_left", C.c_int32),
        ("scale", C.c_float),
        ("out_dtype", C.c_int32),
        ("kernel_path", C.c_int32),
        ("bias", C.c_void_p),
        ("bias_dtype", C.c_int32),
        ("window_right", C.c_int32),
        ("bias_stride_b", C.c_int64),
        ("bias_stride_g", C.c_int64),
        ("bias_stride_h", C.c_int64),
        ("bias_stride_m", C.c_int64),
        ("wait_budget_kcycles", C.c_int32),
        ("debug_flags", C.c_int32),
        ("kv_split", C.c_int32),
        ("kv_offset2", C.c_int32),
        ("sm_margin", C.c_int32),
        ("reserved", C.c_int32),
    ]


class DecodeParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("k", C.c_void_p),
        ("v", C.c_void_p),
        ("out", C.c_void_p),
        ("lse", C.c_void_p),
        ("scratch", C.c_void_p),
        ("seqlen_k", C.c_void_p),
        ("block_tables", C.c_void_p),
        ("dtype", C.c_int32),
        ("kv_format", C.c_int32),
        ("num_quant_groups", C.c_int32),
        ("batch", C.c_int32),
        ("mq", C.c_int32),
        ("kv_heads", C.c_int32),
        ("q_per_kv", C.c_int32),
        ("head_dim", C.c_int32),
        ("kv_padding", C.c_int32),
        ("page_size", C.c_int32),
        ("block_table_stride", C.c_int32),
        ("split_k", C.c_int32),
        ("q_stride_m", C.c_int64),
        ("q_stride_g", C.c_int64),
        ("q_stride_h", C.c_int64),
        ("k_stride_m", C.c_int64),
        ("k_stride_g", C.c_int64),
        ("v_stride_m", C.c_int64),
        ("v_stride_g", C.c_int64),
        ("o_stride_m", C.c_int64),
        ("o_stride_g", C.c_int64),
        ("o_stride_h", C.c_int64),
        ("lse_stride_g", C.c_int64),
        ("lse_stride_h", C.c_int64),
        ("mask_type", C.c_int32),
        ("scale", C.c_float),
        ("out_dtype", C.c_int32),
        ("ss_words", C.c_int32),
        ("k_scale_shift", C.c_void_p),
        ("v_scale_shift", C.c_void_p),
        ("ks_stride_m", C.c_int64),
        ("ks_stride_g", C.c_int64),
        ("vs_stride_m", C.c_int64),
        ("vs_stride_g", C.c_int64),
        ("kv_seqstart", C.c_void_p),
        ("kv_rows", C.c_int64),
        ("window_size", C.c_int32),
        ("reserved", C.c_int32),
        ("bias", C.c_void_p),
        ("bias_dtype", C.c_int32),
        ("reserved2", C.c_int32),
        ("bias_stride_b", C.c_int64),
        ("bias_stride_kvh", C.c_int64),
        ("bias_stride_q", C.c_int64),
        ("bias_stride_m", C.c_int64),
    ]


class MergeParams(C.Structure):
    _fields_ = [
        ("attn_ptrs", C.POINTER(C.c_void_p)),
        ("lse_ptrs", C.POINTER(C.c_void_p)),
        ("num_splits", C.c_int32),
        ("stacked", C.c_int32),
        ("attn_stride_s", C.c_int64),
        ("lse_stride_s", C.c_int64),
        ("attn_strides", Strides),
        ("lse_in_stride_b", C.c_int64),
        ("lse_in_stride_g", C.c_int64),
        ("lse_in_stride_h", C.c_int64),
        ("out", C.c_void_p),
        ("lse_out", C.c_void_p),
        ("out_strides", Strides),
        ("lse_out_stride_b", C.c_int64),
        ("lse_out_stride_g", C.c_int64),
        ("lse_out_stride_h", C.c_int64),
        ("B", C.c_int32),
        ("M", C.c_int32),
        ("G", C.c_int32),
        ("H", C.c_int32),
        ("D", C.c_int32),
        ("in_dtype", C.c_int32),
        ("out_dtype", C.c_int32),
        ("reserved", C.c_int32),
    ]


class RopeParams(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("xq", "xk", "xv", "out_q", "cache_k", "cache_v", "seqstart_q", "seqstart_k", "seqlen_k", "first_seqpos", "seqpos")]
        + [("seqpos_stride", C.c_int64)]
        + [
            (n, C.c_int32)
            for n in ("dtype", "batch", "max_q_per_seq", "q_heads", "kv_heads", "groups", "dim", "adjacents", "use_dynamic_scaling", "internal_f64", "seqpos_i64")
        ]
        + [
            (n, C.c_float)
            for n in ("theta", "linear_scale", "dynamic_old_context_len", "dynamic_scale_factor", "dynamic_low_freq_factor", "dynamic_high_freq_factor")
        ]
        + [(f"{t}_{a}", C.c_int64) for t in ("xq", "xk", "xv", "oq", "ck", "cv") for a in "mgh"]
        + [("block_tables", C.c_void_p), ("block_tables_stride", C.c_int64), ("page_size", C.c_int32), ("cache_format", C.c_int32)]
        + [("k_scale_shift", C.c_void_p), ("v_scale_shift", C.c_void_p)]
        + [(f"{t}_{a}", C.c_int64) for t in ("kss", "vss") for a in "mgh"]
        + [("pages_per_seq", C.c_int32), ("reserved", C.c_int32)]
    )


def library_path() -> Path:
    override = os.environ.get("XFB200_LIBRARY")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent / "csrc" / "libxfb200.so"


_LIB: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Load the library once; raise a clear error if it is absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = library_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m xformers_b200.build` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback for these operators."
        )
    lib = C.CDLL(str(path))
    for name in EXPORTED_SYMBOLS:
        if not hasattr(lib, name):
            raise RuntimeError(f"{path} does not export {name}")
    lib.xfb200_abi_version.restype = C.c_int
    lib.xfb200_last_error.restype = C.c_char_p
    lib.xfb200_prefill_forward.argtypes = [C.POINTER(PrefillParams), C.c_void_p]
    lib.xfb200_prefill_forward.restype = C.c_int
    lib.xfb200_prefill_device_status.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    lib.xfb200_prefill_device_status.restype = C.c_int
    lib.xfb200_decode_device_status.argtypes = [C.c_void_p, C.POINTER(C.c_int32)]
    lib.xfb200_decode_device_status.restype = C.c_int
    lib.xfb200_decode_scratch_bytes.argtypes = [C.c_int32] * 6
    lib.xfb200_decode_scratch_bytes.restype = C.c_size_t
    lib.xfb200_decode_forward.argtypes = [C.POINTER(DecodeParams), C.c_void_p]
    lib.xfb200_decode_forward.restype = C.c_int
    lib.xfb200_decode_forward_static_scratch.argtypes = [C.POINTER(DecodeParams), C.c_void_p]
    lib.xfb200_decode_forward_static_scratch.restype = C.c_int
    lib.xfb200_merge_attentions.argtypes = [C.POINTER(MergeParams), C.c_void_p]
    lib.xfb200_merge_attentions.restype = C.c_int
    lib.xfb200_rope_padded.argtypes = [C.POINTER(RopeParams), C.c_void_p]
    lib.xfb200_rope_padded.restype = C.c_int
    if lib.xfb200_abi_version() != ABI_VERSION:
        raise RuntimeError(f"{path}: ABI version {lib.xfb200_abi_version()} != {ABI_VERSION}")
    _LIB = lib
    return lib


def is_built() -> bool:
    return library_path().exists()


class Xfb200Error(RuntimeError):
    pass


def check_status_after_every_call() -> bool:
    """``XFB200_CHECK_STATUS=1``: the operators read the device status word after every
    launch (a stream synchronisation each time) and raise when a kernel gave up a wait."""
    return os.environ.get("XFB200_CHECK_STATUS", "0") not in ("", "0")


def debug_checks() -> bool:
    """``XFB200_DEBUG_CHECKS=1``: the operators validate page tables, sequence starts and
    lengths on the host before a launch (device-to-host copies: a debugging aid)."""
    return os.environ.get("XFB200_DEBUG_CHECKS", "0") not in ("", "0")


def check(rc: int, what: str) -> None:
    """Translate a C return code: invalid -> ValueError, unsupported ->
    NotImplementedError, CUDA failures and kernels that gave up a wait
    (``XFB200_E_DEVICE``) -> RuntimeError."""
    if rc == XFB200_OK:
        return
    msg = load().xfb200_last_error().decode(errors="replace")
    if rc == XFB200_E_INVALID:
        raise ValueError(f"{what}: {msg}")
    if rc == XFB200_E_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {msg}")
    raise Xfb200Error(f"{what}: {msg} (code {rc})")
