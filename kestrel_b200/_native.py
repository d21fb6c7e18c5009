"""ctypes binding of ``libkestrel_b200.so`` (the C ABI in ``include/kestrel_b200.h``).

There is no CPU fallback: if the shared library is missing, was built for a
different ABI version, or a call fails, the caller gets an exception.
"""

from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libkestrel_b200.so"
ABI_VERSION = 4

DTYPE_F32, DTYPE_F16, DTYPE_BF16, DTYPE_E4M3 = 0, 1, 2, 3
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024  # KB200_STATIC_SCRATCH_BYTES

STATUS_BAD_SLOT, STATUS_BAD_PAGE, STATUS_BAD_ROW, STATUS_WAIT_TIMEOUT, STATUS_BAD_POSITION, STATUS_BAD_PREFIX = 1, 2, 4, 8, 16, 32

# Every symbol include/kestrel_b200.h declares.
EXPORTS = (
    "kb200_abi_version",
    "kb200_last_error",
    "kb200_device_status",
    "kb200_reshape_and_cache_flash",
    "kb200_build_slot_mapping",
    "kb200_build_paged_kv_metadata",
    "kb200_build_decode_step_metadata",
    "kb200_rope_append",
    "kb200_copy_pages",
    "kb200_attn_workspace_bytes",
    "kb200_attn_workspace_bytes_for",
    "kb200_paged_attention",
    "kb200_block_visibility",
    "kb200_paged_attention_static",
    "kb200_sample_step_from_logits",
)


class NativeLibraryError(RuntimeError):
    """The CUDA library is missing or unusable."""


class AttnArgs(C.Structure):
    """Mirror of ``kb200_attn_args``."""

    _fields_ = [
        ("struct_bytes", C.c_uint32),
        ("device", C.c_int32),
        ("stream", C.c_void_p),
        ("q", C.c_void_p),
        ("out", C.c_void_p),
        ("lse", C.c_void_p),
        ("q_batch_stride", C.c_int64),
        ("q_row_stride", C.c_int64),
        ("q_head_stride", C.c_int64),
        ("o_batch_stride", C.c_int64),
        ("o_row_stride", C.c_int64),
        ("o_head_stride", C.c_int64),
        ("k_cache", C.c_void_p),
        ("v_cache", C.c_void_p),
        ("kv_page_stride", C.c_int64),
        ("kv_token_stride", C.c_int64),
        ("kv_head_stride", C.c_int64),
        ("n_pages", C.c_int64),
        ("page_table", C.c_void_p),
        ("pt_row_stride", C.c_int64),
        ("seqused_k", C.c_void_p),
        ("seqused_q", C.c_void_p),
        ("cu_seqlens_q", C.c_void_p),
        ("batch", C.c_int64),
        ("total_q", C.c_int64),
        ("seqlen_q", C.c_int32),
        ("n_q_heads", C.c_int32),
        ("n_kv_heads", C.c_int32),
        ("head_dim", C.c_int32),
        ("page_size", C.c_int32),
        ("q_dtype", C.c_int32),
        ("kv_dtype", C.c_int32),
        ("softmax_scale", C.c_float),
        ("causal", C.c_int32),
        ("window_left", C.c_int32),
        ("k_scale", C.c_float),
        ("v_scale", C.c_float),
        ("k_scale_per_head", C.c_void_p),
        ("v_scale_per_head", C.c_void_p),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_uint64),
        ("q_visible_until", C.c_void_p),
        ("q_visible_batch_stride", C.c_int64),
        ("shared_prefix_pages", C.c_int32),
        ("reserved0", C.c_int32),
    ]


_lib = None
_lock = threading.Lock()


def _declare(lib: C.CDLL) -> None:
    i32, i64, vp = C.c_int32, C.c_int64, C.c_void_p
    lib.kb200_abi_version.restype = C.c_int
    lib.kb200_abi_version.argtypes = []
    lib.kb200_last_error.restype = C.c_char_p
    lib.kb200_last_error.argtypes = []
    lib.kb200_device_status.restype = C.c_int
    lib.kb200_device_status.argtypes = [C.c_int, C.POINTER(i32), C.c_int]
    lib.kb200_reshape_and_cache_flash.restype = C.c_int
    lib.kb200_reshape_and_cache_flash.argtypes = [
        vp, vp, i64, i64, vp, vp, i64, i64, i64, vp, i64, i64,
        i32, i32, i32, i32, i32, vp, vp, i32, i32, vp,
    ]
    lib.kb200_build_slot_mapping.restype = C.c_int
    lib.kb200_build_slot_mapping.argtypes = [
        vp, i64, i64, i64, vp, i32, i32, i64, vp, i32, vp, i64, i32, i32, vp,
    ]
    lib.kb200_build_paged_kv_metadata.restype = C.c_int
    lib.kb200_build_paged_kv_metadata.argtypes = [
        vp, i64, i64, i64, vp, i32, vp, vp, i64, i64, vp, i64, i32, i32, vp,
    ]
    lib.kb200_build_decode_step_metadata.restype = C.c_int
    lib.kb200_build_decode_step_metadata.argtypes = [
        vp, i64, i64, i64, vp, i32, vp, vp, i64, i64, vp, vp, vp, i64, i32, i32, i32, vp,
    ]
    lib.kb200_rope_append.restype = C.c_int
    lib.kb200_rope_append.argtypes = [
        vp, vp, vp, i64, i64, i64, i64, i32, i32, i32, i32, vp, i32, vp, i64, i64,
        vp, vp, i64, i64, i64, vp, i64, i32, i32, i32, vp, vp, i32, i32, i32, vp,
    ]
    lib.kb200_copy_pages.restype = C.c_int
    lib.kb200_copy_pages.argtypes = [C.POINTER(vp), i32, i64, i64, i64, vp, vp, i64, i32, vp]
    lib.kb200_attn_workspace_bytes.restype = C.c_uint64
    lib.kb200_attn_workspace_bytes.argtypes = [i64, i64, i32, i32, i32, i32]
    lib.kb200_attn_workspace_bytes_for.restype = C.c_uint64
    lib.kb200_attn_workspace_bytes_for.argtypes = [C.POINTER(AttnArgs)]
    lib.kb200_block_visibility.restype = C.c_int
    lib.kb200_block_visibility.argtypes = [vp, i64, i64, i64, vp, i64, i32, vp]
    lib.kb200_paged_attention.restype = C.c_int
    lib.kb200_paged_attention.argtypes = [C.POINTER(AttnArgs)]
    lib.kb200_sample_step_from_logits.restype = C.c_int
    lib.kb200_sample_step_from_logits.argtypes = [vp, i32, i64, i64, i64, vp, vp, vp, vp, vp, i32, vp]
    lib.kb200_paged_attention_static.restype = C.c_int
    lib.kb200_paged_attention_static.argtypes = [C.POINTER(AttnArgs)]


def load() -> C.CDLL:
    """Load the library once; raises :class:`NativeLibraryError` when it cannot be used."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise NativeLibraryError(
                f"{LIB_PATH} is missing: build it with `python -m kestrel_b200.build` "
                "(there is no CPU or PyTorch fallback for the paged-KV kernels)"
            )
        try:
            lib = C.CDLL(str(LIB_PATH))
        except OSError as exc:  # pragma: no cover - depends on the host
            raise NativeLibraryError(f"cannot load {LIB_PATH}: {exc}") from exc
        missing = [name for name in EXPORTS if not hasattr(lib, name)]
        if missing:
            raise NativeLibraryError(f"{LIB_PATH} lacks symbols: {missing}")
        _declare(lib)
        got = lib.kb200_abi_version()
        if got != ABI_VERSION:
            raise NativeLibraryError(f"{LIB_PATH} has ABI version {got}, expected {ABI_VERSION}")
        if C.sizeof(AttnArgs) <= 0:
            raise NativeLibraryError("bad AttnArgs layout")
        _lib = lib
    return _lib


def check(rc: int) -> None:
    """Turn a negative return code into an exception carrying the library's message."""
    if rc == 0:
        return
    msg = load().kb200_last_error().decode("utf-8", "replace")
    if rc == -3:
        raise NotImplementedError(msg)
    if rc == -1:
        raise ValueError(msg)
    raise RuntimeError(f"kestrel_b200 native call failed ({rc}): {msg}")


def device_status(device: int, clear: bool = True) -> tuple[int, int, int, int]:
    """(flags, first bad value, kernel id, count) recorded by kernels on ``device``; synchronises."""
    out = (C.c_int32 * 4)()
    check(load().kb200_device_status(int(device), out, 1 if clear else 0))
    return tuple(int(v) for v in out)
