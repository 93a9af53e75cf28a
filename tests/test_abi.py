"""CPU-side checks of the C-ABI boundary: the library builds, loads, exports
every symbol the header declares, and rejects bad arguments on the host before
any launch (these calls never reach a kernel, so they run without a GPU)."""
import ctypes
import os
import re

import pytest

from world_engine_b200 import _lib
from world_engine_b200._lib import CacheGeom, Strides3
from world_engine_b200.csrc import build as csrc_build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    csrc_build.build()
    return _lib.load()


def test_header_symbols_are_all_exported(lib):
    header = open(os.path.join(ROOT, "include", "we_b200.h")).read()
    declared = set(re.findall(r"\b(we_b200_[a-z_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_abi_version_and_messages(lib):
    assert lib.we_b200_abi_version() == _lib.ABI_VERSION
    assert lib.we_b200_strerror(0) == b"ok"
    for code in range(-7, 0):
        assert b"unknown" not in lib.we_b200_strerror(code)
    assert b"unknown" in lib.we_b200_strerror(-99)


def _geom(**kw):
    g = CacheGeom()
    g.B, g.Hkv, g.T, g.Dh, g.L, g.dilation, g.dtype = 1, 4, 64, 64, 256, 1, _lib.BF16
    g.kv_plane_stride = 1 * 4 * 320 * 64
    g.kv_batch_stride = 4 * 320 * 64
    g.written_batch_stride = 0
    g.frame_t_stride = 0
    for k, v in kw.items():
        setattr(g, k, v)
    return g


FAKE = 0x10000  # a 16-byte aligned, never dereferenced "device pointer"


def _append(lib, g, k=FAKE, v=FAKE, kv=FAKE, written=FAKE, ft=FAKE, ks=None, vs=None):
    ks = ks or Strides3(4 * 64 * 64, 64 * 64, 64)
    vs = vs or Strides3(4 * 64 * 64, 64 * 64, 64)
    return lib.we_b200_kv_append(k, ks, v, vs, kv, written, None, ft, ctypes.byref(g), 1, None)


def test_append_rejects_bad_arguments(lib):
    assert _append(lib, _geom(), k=None) == -1                       # null
    assert _append(lib, _geom(), k=FAKE + 2) == -2                   # misaligned pointer
    assert _append(lib, _geom(), ks=Strides3(4 * 64 * 64, 64 * 64, 60)) == -2   # stride not 16-byte
    assert _append(lib, _geom(L=200)) == -3                          # L % T != 0
    assert _append(lib, _geom(T=512, L=256)) == -3                   # frame longer than ring
    assert _append(lib, _geom(dilation=3)) == -3                     # (L/T) % dilation != 0
    assert _append(lib, _geom(dtype=9)) == -4                        # unknown dtype
    assert _append(lib, _geom(frame_t_stride=1)) == -3               # per-row frame_t needs per-row written


def test_attention_rejects_bad_arguments(lib):
    s = Strides3(4 * 64 * 64, 64 * 64, 64)
    def call(g, q=FAKE, Hq=4, ws=FAKE, ws_bytes=1 << 30):
        return lib.we_b200_frame_attn(q, s, FAKE, s, Hq, FAKE, FAKE, FAKE, ctypes.byref(g), 0.0, ws, ws_bytes,
                                      None, None)
    assert call(_geom(), q=None) == -1
    assert call(_geom(dtype=_lib.F32)) == -4                         # attention is bf16 / f16 only
    assert call(_geom(Dh=96, kv_plane_stride=4 * 320 * 96, kv_batch_stride=4 * 320 * 96)) == -4
    assert call(_geom(), Hq=6) == -3                                 # Hq % Hkv != 0
    # a long ring is split over several CTAs; where they cannot merge through cluster shared memory (no device
    # here), the split needs the caller's workspace
    long_ring = dict(L=64 * 64, kv_plane_stride=4 * 65 * 64 * 64, kv_batch_stride=4 * 65 * 64 * 64)
    assert call(_geom(**long_ring), ws=None, ws_bytes=0) == -5
    assert call(_geom(L=64 * 4096, kv_plane_stride=4 * 64 * 4097 * 64, kv_batch_stride=4 * 64 * 4097 * 64)) == -7


def test_workspace_size_is_monotone(lib):
    a = lib.we_b200_attn_workspace_bytes(1, 16, 256, 128, 4096)
    b = lib.we_b200_attn_workspace_bytes(64, 16, 256, 128, 8192)
    assert a > 0 and b > 0
    assert lib.we_b200_attn_workspace_bytes(0, 16, 256, 128, 4096) == 0


def test_ops_refuse_cpu_tensors():
    import torch
    from world_engine_b200 import B200LayerKVCache
    cache = B200LayerKVCache(1, 2, 128, 64, torch.bfloat16, 64)
    x = torch.zeros(1, 2, 64, 64, dtype=torch.bfloat16)
    pos = {"t_pos": torch.zeros(1, 64, dtype=torch.long)}
    with pytest.raises(RuntimeError, match="no CPU path"):
        cache.append_and_attend(x, x, x, pos, True)


def test_prologue_and_gate_reject_bad_arguments(lib):
    from world_engine_b200._lib import PrologueArgs
    def args(**kw):
        a = PrologueArgs()
        for name in ("q_in", "k_in", "v_in", "q_out", "k_out", "v_out", "cos_table", "sin_table", "t_pos", "y_pos",
                     "x_pos"):
            setattr(a, name, FAKE)
        s = Strides3(256 * 48 * 128, 128, 48 * 128)
        for name in ("q_in_strides", "k_in_strides", "v_in_strides", "q_out_strides", "k_out_strides",
                     "v_out_strides"):
            setattr(a, name, s)
        a.table_rows, a.pos_batch_stride, a.height, a.width = 1024, 256, 16, 16
        a.B, a.T, a.Hq, a.Hkv, a.Dh, a.dtype, a.eps = 1, 256, 16, 16, 128, _lib.BF16, 1e-6
        for k, v in kw.items():
            setattr(a, k, v)
        return a
    call = lambda a: lib.we_b200_qkv_prologue(ctypes.byref(a), None, None)
    assert lib.we_b200_qkv_prologue(None, None, None) == -1
    assert call(args(q_in=None)) == -1
    assert call(args(v1=FAKE)) == -1                                 # a residual source needs its weight
    assert call(args(dtype=_lib.F32)) == -4                          # 16-bit tensors only
    assert call(args(Dh=96)) == -4
    assert call(args(T=0)) == -3
    assert call(args(q_in=FAKE + 4)) == -2                           # rows of Dh=128 are read as 8-byte words
    assert call(args(k_in_strides=Strides3(256 * 48 * 128, 128, 48 * 128 + 2))) == -2
    # the gated layer-step needs its gate
    s = Strides3(4 * 64 * 64, 64 * 64, 64)
    g = _geom()
    rc = lib.we_b200_append_attend_gated(FAKE, s, FAKE, s, 4, FAKE, s, FAKE, s, FAKE, FAKE, None, FAKE,
                                         ctypes.byref(g), 1, 0.0, None, None, 1, FAKE, 1 << 30, None, None)
    assert rc == -1
