"""ctypes binding of libwe_b200.so (the C ABI declared in include/we_b200.h).

The library is the product: there is no Python or CPU fallback.  If the shared
object is missing or does not export the expected symbols, loading raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libwe_b200.so"
ABI_VERSION = 1

BF16, F16, F32 = 0, 1, 2

# Every symbol include/we_b200.h declares.
EXPORTS = (
    "we_b200_abi_version",
    "we_b200_strerror",
    "we_b200_kv_append",
    "we_b200_block_mask",
    "we_b200_attn_workspace_bytes",
    "we_b200_frame_attn",
    "we_b200_append_attend",
    "we_b200_append_attend_gated",
    "we_b200_frame_attn_static",
    "we_b200_qkv_prologue",
    "we_b200_launch_count",
)


class CacheGeom(ctypes.Structure):
    """Mirror of `we_b200_cache_geom`."""
    _fields_ = [
        ("B", c_int32), ("Hkv", c_int32), ("T", c_int32), ("Dh", c_int32),
        ("L", c_int64), ("dilation", c_int32), ("dtype", c_int32),
        ("kv_plane_stride", c_int64), ("kv_batch_stride", c_int64),
        ("written_batch_stride", c_int64), ("frame_t_stride", c_int64),
    ]


Strides3 = c_int64 * 3


class PrologueArgs(ctypes.Structure):
    """Mirror of `we_b200_prologue_args`."""
    _fields_ = [
        ("q_in", c_void_p), ("k_in", c_void_p), ("v_in", c_void_p), ("v1", c_void_p),
        ("q_out", c_void_p), ("k_out", c_void_p), ("v_out", c_void_p),
        ("q_in_strides", Strides3), ("k_in_strides", Strides3), ("v_in_strides", Strides3), ("v1_strides", Strides3),
        ("q_out_strides", Strides3), ("k_out_strides", Strides3), ("v_out_strides", Strides3),
        ("v_lamb", c_void_p), ("v_lamb_dtype", c_int32),
        ("cos_table", c_void_p), ("sin_table", c_void_p), ("table_rows", c_int64),
        ("t_pos", c_void_p), ("y_pos", c_void_p), ("x_pos", c_void_p), ("pos_batch_stride", c_int64),
        ("height", c_int32), ("width", c_int32),
        ("B", c_int32), ("T", c_int32), ("Hq", c_int32), ("Hkv", c_int32), ("Dh", c_int32),
        ("dtype", c_int32), ("eps", c_float),
    ]


class WeB200Error(RuntimeError):
    def __init__(self, code: int, where: str, msg: str):
        super().__init__(f"{where}: {msg} (code {code})")
        self.code = code


_lib = None


def lib_path() -> str:
    return os.environ.get("WE_B200_LIB", os.path.join(_PKG, LIB_NAME))


def load() -> ctypes.CDLL:
    """Loads the shared library once; raises if it is absent or incomplete."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} not found: build it with `python -m world_engine_b200.csrc.build` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    lib = ctypes.CDLL(path)
    missing = [s for s in EXPORTS if not hasattr(lib, s)]
    if missing:
        raise ImportError(f"{path} does not export {missing}")

    lib.we_b200_abi_version.restype = c_int
    lib.we_b200_abi_version.argtypes = []
    lib.we_b200_strerror.restype = c_char_p
    lib.we_b200_strerror.argtypes = [c_int]
    lib.we_b200_launch_count.restype = c_uint64
    lib.we_b200_launch_count.argtypes = []
    lib.we_b200_attn_workspace_bytes.restype = c_size_t
    lib.we_b200_attn_workspace_bytes.argtypes = [c_int32, c_int32, c_int32, c_int32, c_int64]
    lib.we_b200_kv_append.restype = c_int
    lib.we_b200_kv_append.argtypes = [
        c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_void_p, c_void_p, c_void_p,
        c_void_p, POINTER(CacheGeom), c_int, c_void_p]
    lib.we_b200_block_mask.restype = c_int
    lib.we_b200_block_mask.argtypes = [
        c_void_p, c_int64, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.we_b200_frame_attn.restype = c_int
    lib.we_b200_frame_attn.argtypes = [
        c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_int32,
        c_void_p, c_void_p, c_void_p, POINTER(CacheGeom), c_float,
        c_void_p, c_size_t, c_void_p, c_void_p]
    lib.we_b200_append_attend.restype = c_int
    lib.we_b200_append_attend.argtypes = [
        c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_int32,
        c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64),
        c_void_p, c_void_p, c_void_p, c_void_p, POINTER(CacheGeom), c_int, c_float,
        c_void_p, c_size_t, c_void_p, c_void_p]

    lib.we_b200_append_attend_gated.restype = c_int
    lib.we_b200_append_attend_gated.argtypes = [
        c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_int32,
        c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64),
        c_void_p, c_void_p, c_void_p, c_void_p, POINTER(CacheGeom), c_int, c_float,
        c_void_p, POINTER(c_int64), c_int,
        c_void_p, c_size_t, c_void_p, c_void_p]

    lib.we_b200_frame_attn_static.restype = c_int
    lib.we_b200_frame_attn_static.argtypes = [
        c_void_p, POINTER(c_int64), c_void_p, POINTER(c_int64), c_int32,
        c_void_p, c_void_p, c_void_p, POINTER(CacheGeom), c_float, c_void_p, c_void_p]

    lib.we_b200_qkv_prologue.restype = c_int
    lib.we_b200_qkv_prologue.argtypes = [POINTER(PrologueArgs), c_void_p, c_void_p]

    got = lib.we_b200_abi_version()
    if got != ABI_VERSION:
        raise ImportError(f"{path}: ABI version {got}, this package expects {ABI_VERSION}")
    _lib = lib
    return lib


def check(code: int, where: str) -> None:
    """Raises WeB200Error for a non-zero return code of the library."""
    if code != 0:
        msg = load().we_b200_strerror(code)
        raise WeB200Error(code, where, msg.decode() if msg else "?")
