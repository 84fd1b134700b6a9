"""ctypes binding of ``csrc/liboeq_b200.so`` (the C ABI declared in ``include/oeq_b200.h``).

Plays the part of the reference's extension loader (openequivariance/openequivariance/_torch/extlib/__init__.py:36-182):
it locates the in-tree shared library, loads it, and exposes ``BUILT_EXTENSION`` / ``BUILT_EXTENSION_ERROR``.
There is no fallback: if the library is missing every kernel call raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "liboeq_b200.so")


class KernelProp(Structure):
    """``oeqb_kernel_prop`` of include/oeq_b200.h."""

    _fields_ = [("L1_dim", c_int64), ("L2_dim", c_int64), ("L3_dim", c_int64), ("weight_numel", c_int64),
                ("shared_weights", c_int32), ("irrep_dtype", c_int32), ("weight_dtype", c_int32),
                ("idx_dtype", c_int32), ("is_conv", c_int32), ("deterministic", c_int32), ("kahan", c_int32),
                ("is_uvw", c_int32), ("fast_path", c_int32), ("reserved", c_int32)]


_P = c_void_p
_DESC = [c_char_p, c_size_t, c_int64]
_PROTOTYPES = {
    "oeqb_query": (c_int, _DESC + [POINTER(KernelProp)]),
    "oeqb_tp_forward": (c_int, _DESC + [c_int64] + [_P] * 5),
    "oeqb_tp_backward": (c_int, _DESC + [c_int64] + [_P] * 8),
    "oeqb_tp_double_backward": (c_int, _DESC + [c_int64] + [_P] * 12),
    "oeqb_conv_workspace_bytes": (c_int64, _DESC + [c_int, c_int64, c_int64]),
    "oeqb_conv_forward": (c_int, _DESC + [c_int64, c_int64] + [_P] * 8 + [c_int64, _P]),
    "oeqb_conv_forward_rect": (c_int, _DESC + [c_int64, c_int64, c_int64] + [_P] * 8 + [c_int64, _P]),
    "oeqb_conv_backward": (c_int, _DESC + [c_int64, c_int64] + [_P] * 11 + [c_int64, _P]),
    "oeqb_conv_backward_rect": (c_int, _DESC + [c_int64, c_int64, c_int64] + [_P] * 11 + [c_int64, _P]),
    "oeqb_conv_backward_edges": (c_int, _DESC + [c_int64, c_int64, c_int64] + [_P] * 10 + [c_int64, _P]),
    "oeqb_conv_backward_rows": (c_int, _DESC + [c_int64, c_int64, c_int64, c_int64, _P, _P, c_int64, _P, _P]),
    "oeqb_conv_double_backward": (c_int, _DESC + [c_int64, c_int64] + [_P] * 15 + [c_int64, _P]),
    "oeqb_conv_backward_noalloc": (c_int, _DESC + [c_int64, c_int64] + [_P] * 11),
    "oeqb_noalloc_status": (c_int, []),
    "oeqb_check_status": (c_int, []),
    "oeqb_selftest_bounded_wait": (c_int, [c_char_p, c_size_t, c_int64, _P]),
    "oeqb_group_mm": (c_int, [c_int, c_int, c_int64, c_int64, c_int64, c_int64, POINTER(c_int64), _P, _P, _P, _P]),
    "oeqb_slow_path_count": (c_int64, []),
    "oeqb_graph_workspace_bytes": (c_int64, [c_int64, c_int64]),
    "oeqb_prepare_graph": (c_int, [c_int, c_int64, c_int64] + [_P] * 7 + [c_int64, _P]),
    "oeqb_plan_workspace_bytes": (c_int64, [c_int64, c_int64, c_int64, c_int64, c_int]),
    "oeqb_plan_count": (c_int, [c_int64, c_int64, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int, c_int, _P, _P, c_int64, _P, _P]),
    "oeqb_plan_fill": (c_int, [c_int64, c_int64, _P, _P, c_int64, c_int64, c_int64, c_int64, c_int, _P, c_int64, c_int64, c_int64,
                               _P, c_int64, _P, _P, _P, _P, _P, _P]),
    "oeqb_emit_source": (c_int, [c_char_p, c_size_t, c_char_p, c_char_p, c_size_t, POINTER(c_size_t)]),
    "oeqb_precompile": (c_int, _DESC),
    "oeqb_set_option": (c_int, [c_char_p, c_char_p]),
    "oeqb_launch_count": (c_int64, []),
    "oeqb_last_error": (c_char_p, []),
    "oeqb_version": (c_char_p, []),
}

BUILT_EXTENSION = False
BUILT_EXTENSION_ERROR = None
_lib = None


def exported_symbols():
    """Names every C-ABI entry point the header declares (used by the CPU test-suite)."""
    return sorted(_PROTOTYPES)


def load(build_if_missing: bool = True):
    """Loads (building first if the .so is absent and nvcc is available) and returns the ctypes library."""
    global _lib, BUILT_EXTENSION, BUILT_EXTENSION_ERROR
    if _lib is not None:
        return _lib
    try:
        if build_if_missing:
            # rebuild when the library is missing or older than its sources (only where a compiler is at hand:
            # a machine that received the built library keeps it)
            from . import build_native
            nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
            if not os.path.exists(LIB_PATH):
                build_native.build(verbose=False)
            elif os.path.exists(nvcc) and os.environ.get("OEQB_NO_REBUILD") != "1" and build_native.needs_build():
                try:
                    build_native.build(verbose=False)
                except Exception as exc:  # noqa: BLE001 - a library exists: use it, but say that it is out of date
                    import sys
                    print(f"[oeq_b200] WARNING: {LIB_PATH} is older than its sources and rebuilding failed ({exc}); "
                          "loading the existing library", file=sys.stderr)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _PROTOTYPES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
        BUILT_EXTENSION, BUILT_EXTENSION_ERROR = True, None
        if os.environ.get("OEQB_LOG") == "1":
            lib.oeqb_set_option(b"log", b"1")
        # OEQB_OPTIONS="name=value,name=value": library options (see oeqb_set_option) applied at load time
        for item in filter(None, os.environ.get("OEQB_OPTIONS", "").split(",")):
            name, _, value = item.partition("=")
            lib.oeqb_set_option(name.strip().encode(), value.strip().encode())
    except Exception as exc:  # noqa: BLE001 - surfaced through BUILT_EXTENSION_ERROR and re-raised on use
        BUILT_EXTENSION, BUILT_EXTENSION_ERROR = False, exc
        raise RuntimeError(f"oeq_b200 native library unavailable ({LIB_PATH}): {exc}") from exc
    return _lib


def last_error() -> str:
    return load().oeqb_last_error().decode("utf-8", "replace")


def check(rc: int, what: str):
    """Turns a non-zero C-ABI return code into ``RuntimeError`` carrying the library's message."""
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc}): {last_error()}")


def query(desc: bytes, key: int) -> KernelProp:
    prop = KernelProp()
    check(load().oeqb_query(desc, len(desc), key, ctypes.byref(prop)), "oeqb_query")
    return prop


def emit_source(desc: bytes, kind: str) -> str:
    lib = load()
    need = c_size_t(0)
    check(lib.oeqb_emit_source(desc, len(desc), kind.encode(), None, 0, ctypes.byref(need)), "oeqb_emit_source")
    buf = ctypes.create_string_buffer(need.value)
    check(lib.oeqb_emit_source(desc, len(desc), kind.encode(), buf, need.value, ctypes.byref(need)), "oeqb_emit_source")
    return buf.value.decode()


def precompile(desc: bytes, key: int = 0) -> int:
    n = load().oeqb_precompile(desc, len(desc), key)
    if n < 0:
        raise RuntimeError(f"oeqb_precompile failed (code {-n}): {last_error()}")
    return n


def launch_count() -> int:
    return int(load().oeqb_launch_count())


def set_option(name: str, value: str):
    check(load().oeqb_set_option(name.encode(), value.encode()), "oeqb_set_option")
