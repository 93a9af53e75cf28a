"""Tensor-level entry points over the C ABI, plus their `torch.library` custom
ops so that the calls survive `torch.compile(fullgraph=True)` -- the way the
reference wraps its own native kernel (src/quantize.py:17-42).

Every function here enqueues on the caller's current CUDA stream, performs no
host synchronisation and allocates nothing except (once per device) the
split-KV workspace and the status word.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import CacheGeom, PrologueArgs, Strides3

_DTYPE_CODE = {torch.bfloat16: _lib.BF16, torch.float16: _lib.F16, torch.float32: _lib.F32}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise TypeError(f"world_engine_b200: unsupported cache dtype {dtype}") from None


def _require_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "world_engine_b200 runs on CUDA tensors only (sm_100a); there is no CPU path")


def _strides3(t: torch.Tensor) -> Strides3:
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError("expected a [B, H, T, Dh] tensor whose last axis is contiguous")
    return Strides3(t.stride(0), t.stride(1), t.stride(2))


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def make_geom(kv: torch.Tensor, written: torch.Tensor, tokens_per_frame: int, dilation: int,
              frame_t_stride: int = 0) -> CacheGeom:
    """Geometry of a reference-layout cache tensor kv[2, B, H, L+T, Dh]
    (src/model/kv_cache.py:81-84)."""
    if kv.dim() != 5 or kv.size(0) != 2:
        raise ValueError("kv must be [2, B, H, L + tokens_per_frame, Dh]")
    if kv.stride(4) != 1 or kv.stride(3) != kv.size(4) or kv.stride(2) != kv.size(3) * kv.size(4):
        raise ValueError("kv must be contiguous over (head, token, head_dim)")
    _, B, H, C, Dh = kv.shape
    g = CacheGeom()
    g.B, g.Hkv, g.T, g.Dh = B, H, tokens_per_frame, Dh
    g.L = C - tokens_per_frame
    g.dilation = dilation
    g.dtype = dtype_code(kv.dtype)
    g.kv_plane_stride = kv.stride(0)
    g.kv_batch_stride = kv.stride(1)
    g.written_batch_stride = written.stride(0) if written.dim() == 2 else 0
    g.frame_t_stride = frame_t_stride
    return g


# ------------------------------------------------------------------ workspace
_workspaces = {}
_status_words = {}


def workspace_for(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised split-KV workspace of the device (grown on demand).
    Calls that share it must be ordered on one stream."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def status_word(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    st = _status_words.get(key)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = st
    return st


def check_status(device: torch.device) -> None:
    """Synchronising health check: raises if a kernel on `device` reported a device-side anomaly."""
    st = int(status_word(device).item())
    if st != 0:
        status_word(device).zero_()
        what = {1: "a bounded wait of the attention kernel expired; the output of that call is invalid",
                2: "a token position points outside the RoPE table (IndexError in the reference)"}.get(st & 0xFF, "unknown")
        where = f" (debug build: wait at source line {st >> 8})" if st >> 8 else ""
        raise RuntimeError(f"world_engine_b200: device status {st & 0xFF}: {what}{where}")


def kv_append_(kv: torch.Tensor, written: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
               frame_t: torch.Tensor, tokens_per_frame: int, dilation: int, is_frozen: bool,
               mask_written: Optional[torch.Tensor] = None, frame_t_stride: int = 0) -> None:
    """In-place append of one frame (we_b200_kv_append)."""
    _require_cuda(kv, written, k_new, v_new, frame_t, mask_written)
    g = make_geom(kv, written, tokens_per_frame, dilation, frame_t_stride)
    lib = _lib.load()
    with torch.cuda.device(kv.device):
        rc = lib.we_b200_kv_append(
            k_new.data_ptr(), _strides3(k_new), v_new.data_ptr(), _strides3(v_new),
            kv.data_ptr(), written.data_ptr(),
            mask_written.data_ptr() if mask_written is not None else None,
            frame_t.data_ptr(), ctypes.byref(g), int(bool(is_frozen)), _stream_ptr(kv.device))
    _lib.check(rc, "we_b200_kv_append")


def frame_attn(q: torch.Tensor, kv: torch.Tensor, written: torch.Tensor, frame_t: torch.Tensor,
               tokens_per_frame: int, dilation: int, scale: float = 0.0,
               out: Optional[torch.Tensor] = None, frame_t_stride: int = 0) -> torch.Tensor:
    """Attention of the new frame's queries over the cache (we_b200_frame_attn).
    The output has q's shape and strides, like flex_attention's."""
    _require_cuda(q, kv, written, frame_t)
    g = make_geom(kv, written, tokens_per_frame, dilation, frame_t_stride)
    if out is None:
        out = torch.empty_like(q)
    lib = _lib.load()
    B, Hq, T, Dh = q.shape
    with torch.cuda.device(q.device):
        need = lib.we_b200_attn_workspace_bytes(B, Hq, T, Dh, g.L)
        ws = workspace_for(q.device, need)
        rc = lib.we_b200_frame_attn(
            q.data_ptr(), _strides3(q), out.data_ptr(), _strides3(out), Hq,
            kv.data_ptr(), written.data_ptr(), frame_t.data_ptr(), ctypes.byref(g), float(scale),
            ws.data_ptr(), ws.numel(), status_word(q.device).data_ptr(), _stream_ptr(q.device))
    _lib.check(rc, "we_b200_frame_attn")
    return out


def frame_attn_no_alloc(q: torch.Tensor, out: torch.Tensor, status: torch.Tensor, kv: torch.Tensor,
                        written: torch.Tensor, frame_t: torch.Tensor, tokens_per_frame: int, dilation: int,
                        scale: float = 0.0, frame_t_stride: int = 0) -> torch.Tensor:
    """`frame_attn` for hosts that must not allocate device memory while running (an engine that gave
    the whole GPU to its own arena, a plug-in limited to the buffers it receives): binds
    we_b200_frame_attn_static, whose split-KV scratch is a fixed 12 MiB array inside the library.
    Nothing is allocated here either, so `out` (q's shape) and `status` (one int32) are the caller's.
    Raises WeB200Error (code -8) for shapes that need more scratch.  Calls share that one array:
    keep them on one stream per device, and make the first call on a device outside stream capture."""
    _require_cuda(q, out, status, kv, written, frame_t)
    g = make_geom(kv, written, tokens_per_frame, dilation, frame_t_stride)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        rc = lib.we_b200_frame_attn_static(
            q.data_ptr(), _strides3(q), out.data_ptr(), _strides3(out), q.size(1),
            kv.data_ptr(), written.data_ptr(), frame_t.data_ptr(), ctypes.byref(g), float(scale),
            status.data_ptr(), _stream_ptr(q.device))
    _lib.check(rc, "we_b200_frame_attn_static")
    return out


def append_attend(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, kv: torch.Tensor,
                  written: torch.Tensor, frame_t: torch.Tensor, tokens_per_frame: int, dilation: int,
                  is_frozen: bool, scale: float = 0.0, out: Optional[torch.Tensor] = None,
                  mask_written: Optional[torch.Tensor] = None, frame_t_stride: int = 0,
                  gate: Optional[torch.Tensor] = None, gate_is_logits: bool = False) -> torch.Tensor:
    """One layer-step: append the frame, then attend (we_b200_append_attend).  With `gate` (a `[B,Hq,T]` view of
    q's dtype) the output rows are multiplied by it, or by its sigmoid when `gate_is_logits`, on their way out
    (we_b200_append_attend_gated; src/model/attn.py:117-119)."""
    _require_cuda(q, k_new, v_new, kv, written, frame_t, mask_written, gate)
    g = make_geom(kv, written, tokens_per_frame, dilation, frame_t_stride)
    if out is None:
        out = torch.empty_like(q)
    lib = _lib.load()
    B, Hq, T, Dh = q.shape
    if gate is not None and (gate.shape != (B, Hq, T) or gate.dtype != q.dtype):
        raise ValueError("gate must be a [B, Hq, T] view of q's dtype")
    with torch.cuda.device(q.device):
        need = lib.we_b200_attn_workspace_bytes(B, Hq, T, Dh, g.L)
        ws = workspace_for(q.device, need)
        head = (q.data_ptr(), _strides3(q), out.data_ptr(), _strides3(out), Hq,
                k_new.data_ptr(), _strides3(k_new), v_new.data_ptr(), _strides3(v_new),
                kv.data_ptr(), written.data_ptr(),
                mask_written.data_ptr() if mask_written is not None else None,
                frame_t.data_ptr(), ctypes.byref(g), int(bool(is_frozen)), float(scale))
        tail = (ws.data_ptr(), ws.numel(), status_word(q.device).data_ptr(), _stream_ptr(q.device))
        if gate is None:
            rc = lib.we_b200_append_attend(*head, *tail)
        else:
            rc = lib.we_b200_append_attend_gated(*head, gate.data_ptr(), Strides3(*gate.stride()),
                                                 int(bool(gate_is_logits)), *tail)
    _lib.check(rc, "we_b200_append_attend")
    return out


def qkv_prologue(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, v1: Optional[torch.Tensor],
                 v_lamb: Optional[torch.Tensor], cos_table: torch.Tensor, sin_table: torch.Tensor,
                 t_pos: torch.Tensor, y_pos: torch.Tensor, x_pos: torch.Tensor, height: int, width: int,
                 eps: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """q, k, v `[B,H,T,Dh]` views (any strides, head dim contiguous) -> (q', k', v') as the attention and the
    cache receive them: value residual, weightless RMS norm and RoPE in one pass (we_b200_qkv_prologue;
    src/model/attn.py:105-110).  `v1=None` skips the residual.  Outputs are fresh `[B,T,H,Dh]`-ordered
    buffers viewed as `[B,H,T,Dh]`, the layout the merged-QKV slices have."""
    _require_cuda(q, k, v, v1, v_lamb, cos_table, sin_table, t_pos, y_pos, x_pos)
    B, Hq, T, Dh = q.shape
    Hkv = k.shape[1]
    if cos_table.dtype != torch.float32 or sin_table.dtype != torch.float32 or not cos_table.is_contiguous() \
            or not sin_table.is_contiguous() or cos_table.shape != sin_table.shape or cos_table.shape[-1] != Dh // 2:
        raise ValueError("cos / sin tables must be contiguous float32 [rows, Dh/2]")
    for name, t in (("t_pos", t_pos), ("y_pos", y_pos), ("x_pos", x_pos)):
        if t.dtype != torch.int64 or t.shape != (B, T) or t.stride() != t_pos.stride() or t.stride(1) != 1:
            raise ValueError(f"{name} must be int64 [B, T] with contiguous rows")
    q_out = torch.empty((B, T, Hq, Dh), dtype=q.dtype, device=q.device).transpose(1, 2)
    k_out = torch.empty((B, T, Hkv, Dh), dtype=k.dtype, device=k.device).transpose(1, 2)
    v_out = torch.empty((B, T, Hkv, Dh), dtype=v.dtype, device=v.device).transpose(1, 2)
    a = PrologueArgs()
    a.q_in, a.k_in, a.v_in = q.data_ptr(), k.data_ptr(), v.data_ptr()
    a.v1 = v1.data_ptr() if v1 is not None else None
    a.q_out, a.k_out, a.v_out = q_out.data_ptr(), k_out.data_ptr(), v_out.data_ptr()
    a.q_in_strides, a.k_in_strides, a.v_in_strides = _strides3(q), _strides3(k), _strides3(v)
    a.v1_strides = _strides3(v1) if v1 is not None else Strides3(0, 0, 0)
    a.q_out_strides, a.k_out_strides, a.v_out_strides = _strides3(q_out), _strides3(k_out), _strides3(v_out)
    if v1 is not None:
        if v_lamb is None or v_lamb.numel() != 1:
            raise ValueError("v_lamb must be a one-element tensor when v1 is given")
        a.v_lamb, a.v_lamb_dtype = v_lamb.data_ptr(), dtype_code(v_lamb.dtype)
    a.cos_table, a.sin_table, a.table_rows = cos_table.data_ptr(), sin_table.data_ptr(), cos_table.shape[0]
    a.t_pos, a.y_pos, a.x_pos = t_pos.data_ptr(), y_pos.data_ptr(), x_pos.data_ptr()
    a.pos_batch_stride = t_pos.stride(0)
    a.height, a.width = int(height), int(width)
    a.B, a.T, a.Hq, a.Hkv, a.Dh = B, T, Hq, Hkv, Dh
    a.dtype = dtype_code(q.dtype)
    a.eps = float(torch.finfo(torch.float32).eps if eps is None else eps)
    lib = _lib.load()
    with torch.cuda.device(q.device):
        rc = lib.we_b200_qkv_prologue(ctypes.byref(a), status_word(q.device).data_ptr(), _stream_ptr(q.device))
    _lib.check(rc, "we_b200_qkv_prologue")
    return q_out, k_out, v_out


def block_mask_tables(mask_written: torch.Tensor, tokens_per_frame: int
                      ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """int32 tables of the flex BlockMask for a visibility vector (we_b200_block_mask)."""
    _require_cuda(mask_written)
    C = mask_written.numel()
    qb = (tokens_per_frame + 127) // 128
    kb = (C + 127) // 128
    dev = mask_written.device
    kv_num = torch.empty((1, 1, qb), dtype=torch.int32, device=dev)
    kv_idx = torch.empty((1, 1, qb, kb), dtype=torch.int32, device=dev)
    full_num = torch.empty((1, 1, qb), dtype=torch.int32, device=dev)
    full_idx = torch.empty((1, 1, qb, kb), dtype=torch.int32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        rc = lib.we_b200_block_mask(mask_written.data_ptr(), C, tokens_per_frame, kv_num.data_ptr(),
                                    kv_idx.data_ptr(), full_num.data_ptr(), full_idx.data_ptr(),
                                    _stream_ptr(dev))
    _lib.check(rc, "we_b200_block_mask")
    return kv_num, kv_idx, full_num, full_idx


# ----------------------------------------------------------------- custom ops
# Registered under the reference's own namespace style ("world_engine::...").
@torch.library.custom_op("world_engine_b200::append_attend", mutates_args=("kv", "written"))
def append_attend_op(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, kv: torch.Tensor,
                     written: torch.Tensor, frame_t: torch.Tensor, tokens_per_frame: int,
                     dilation: int, is_frozen: bool, scale: float) -> torch.Tensor:
    return append_attend(q, k_new, v_new, kv, written, frame_t, tokens_per_frame, dilation,
                         is_frozen, scale)


@append_attend_op.register_fake
def _append_attend_fake(q, k_new, v_new, kv, written, frame_t, tokens_per_frame, dilation,
                        is_frozen, scale):
    return torch.empty_like(q)


@torch.library.custom_op("world_engine_b200::kv_append", mutates_args=("kv", "written", "mask_written"))
def kv_append_op(kv: torch.Tensor, written: torch.Tensor, mask_written: torch.Tensor,
                 k_new: torch.Tensor, v_new: torch.Tensor, frame_t: torch.Tensor,
                 tokens_per_frame: int, dilation: int, is_frozen: bool) -> None:
    kv_append_(kv, written, k_new, v_new, frame_t, tokens_per_frame, dilation, is_frozen,
               mask_written=mask_written)


@kv_append_op.register_fake
def _kv_append_fake(kv, written, mask_written, k_new, v_new, frame_t, tokens_per_frame, dilation,
                    is_frozen):
    return None


@torch.library.custom_op("world_engine_b200::frame_attn", mutates_args=())
def frame_attn_op(q: torch.Tensor, kv: torch.Tensor, written: torch.Tensor, frame_t: torch.Tensor,
                  tokens_per_frame: int, dilation: int, scale: float) -> torch.Tensor:
    return frame_attn(q, kv, written, frame_t, tokens_per_frame, dilation, scale)


@frame_attn_op.register_fake
def _frame_attn_fake(q, kv, written, frame_t, tokens_per_frame, dilation, scale):
    return torch.empty_like(q)


@torch.library.custom_op("world_engine_b200::qkv_prologue", mutates_args=())
def qkv_prologue_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, v1: Optional[torch.Tensor],
                    v_lamb: Optional[torch.Tensor], cos_table: torch.Tensor, sin_table: torch.Tensor,
                    t_pos: torch.Tensor, y_pos: torch.Tensor, x_pos: torch.Tensor, height: int,
                    width: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return qkv_prologue(q, k, v, v1, v_lamb, cos_table, sin_table, t_pos, y_pos, x_pos, height, width)


@qkv_prologue_op.register_fake
def _qkv_prologue_fake(q, k, v, v1, v_lamb, cos_table, sin_table, t_pos, y_pos, x_pos, height, width):
    def like(t):
        B, H, T, Dh = t.shape
        return torch.empty((B, T, H, Dh), dtype=t.dtype, device=t.device).transpose(1, 2)
    return like(q), like(k), like(v)


@torch.library.custom_op("world_engine_b200::append_attend_gated", mutates_args=("kv", "written"))
def append_attend_gated_op(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, kv: torch.Tensor,
                           written: torch.Tensor, frame_t: torch.Tensor, gate: torch.Tensor,
                           tokens_per_frame: int, dilation: int, is_frozen: bool, scale: float,
                           gate_is_logits: bool) -> torch.Tensor:
    return append_attend(q, k_new, v_new, kv, written, frame_t, tokens_per_frame, dilation, is_frozen, scale,
                         gate=gate, gate_is_logits=gate_is_logits)


@append_attend_gated_op.register_fake
def _append_attend_gated_fake(q, k_new, v_new, kv, written, frame_t, gate, tokens_per_frame, dilation, is_frozen,
                              scale, gate_is_logits):
    return torch.empty_like(q)
