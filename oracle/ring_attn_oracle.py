"""CPU oracle for the frame-causal attention over the KV ring-buffer cache.

TEST INFRASTRUCTURE ONLY.  This module is a numpy restatement of the
reference's algorithm.  It is the checker for the CUDA path: only the test
suite, the smoke entry and the benchmark's CPU-baseline leg may import it.
The shipped package never does; the product path has no CPU fallback.

Parity pin: the reference holds no tests, golden vectors or fixtures for
this path.  The oracle is pinned instead against outputs of the reference's
own code (`src/model/kv_cache.py` + torch's eager `flex_attention`) executed
on CPU; those outputs are committed as fixtures under `tests/golden/`
together with the script that produced them.

Every function names the reference lines it restates (paths are relative to
the reference project root).
"""
from __future__ import annotations

import math

import numpy as np

SPARSE_BLOCK = 128  # torch.nn.attention.flex_attention._DEFAULT_SPARSE_BLOCK_SIZE


# --------------------------------------------------------------------------
# bf16 helpers (numpy has no bfloat16; caches hold the raw 16-bit patterns)
# --------------------------------------------------------------------------
def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (uint16), NaN kept quiet."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    rounding = ((u >> 16) & 1) + np.uint32(0x7FFF)
    r = ((u + rounding) >> 16).astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, np.uint16(0x7FC0), r)
    return r


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_to_bf16(x: np.ndarray) -> np.ndarray:
    """fp32 values rounded to the nearest bf16-representable fp32."""
    return bf16_bits_to_f32(f32_to_bf16_bits(x))


# --------------------------------------------------------------------------
# slot arithmetic
# --------------------------------------------------------------------------
def slot_arithmetic(frame_t: int, tokens_per_frame: int, L: int, pinned_dilation: int = 1):
    """Ring slot of a frame.  Restates src/model/kv_cache.py:129-131,140.

    Returns (bucket, slot, base, write_step) as Python ints / bool, computed
    with int64 floor semantics exactly like the reference's tensor ops.
    """
    d = int(pinned_dilation)
    num_buckets = (L // tokens_per_frame) // d          # kv_cache.py:77
    t = int(frame_t)
    bucket = (t + (d - 1)) // d                          # kv_cache.py:129
    slot = bucket % num_buckets                          # kv_cache.py:130
    base = slot * tokens_per_frame                       # kv_cache.py:131
    write_step = (t % d) == 0                            # kv_cache.py:140
    return bucket, slot, base, write_step


# --------------------------------------------------------------------------
# block-mask tables
# --------------------------------------------------------------------------
def block_mask_tables(T: int, capacity: int, mask_written: np.ndarray):
    """The four int32 tables of the flex BlockMask.  Restates
    src/model/kv_cache.py:12-39 (make_block_mask, dense_to_ordered).

    Returns kv_num_blocks[1,1,Qb], kv_indices[1,1,Qb,KVb],
    full_kv_num_blocks[1,1,Qb], full_kv_indices[1,1,Qb,KVb].
    """
    BS = SPARSE_BLOCK
    kv_blocks = (capacity + BS - 1) // BS
    q_blocks = (T + BS - 1) // BS
    padded = np.zeros(kv_blocks * BS, dtype=bool)
    padded[:capacity] = mask_written
    blocks = padded.reshape(kv_blocks, BS)
    block_any = blocks.any(-1)
    block_all = blocks.all(-1)
    full = block_all
    partial = block_any & ~block_all

    def ordered(dense_row):
        num = np.int32(dense_row.sum())
        # stable descending argsort of a bool row == True indices ascending, then False ascending
        idx = np.argsort(~dense_row, kind="stable").astype(np.int32)
        nums = np.full((1, 1, q_blocks), num, dtype=np.int32)
        idxs = np.broadcast_to(idx, (1, 1, q_blocks, kv_blocks)).copy()
        return nums, idxs

    kv_num, kv_idx = ordered(partial)
    full_num, full_idx = ordered(full)
    return kv_num, kv_idx, full_num, full_idx


# --------------------------------------------------------------------------
# the cache
# --------------------------------------------------------------------------
class OracleLayerKVCache:
    """numpy twin of LayerKVCache (src/model/kv_cache.py:64-154).

    `kv` has the reference's shape [2, B, H, L + tpf, Dh]; its numpy dtype is
    whatever element container the caller chose (float32, or uint16 holding
    bf16 bit patterns) because the cache only ever copies elements.
    """

    def __init__(self, B, H, L, Dh, np_dtype, tokens_per_frame, pinned_dilation=1):
        self.tpf = int(tokens_per_frame)
        self.L = int(L)
        self.capacity = self.L + self.tpf                              # :74-75
        self.pinned_dilation = int(pinned_dilation)
        self.num_buckets = (self.L // self.tpf) // self.pinned_dilation  # :77
        assert (self.L // self.tpf) % self.pinned_dilation == 0 and self.L % self.tpf == 0  # :78
        self.kv = np.zeros((2, B, H, self.capacity, Dh), dtype=np_dtype)  # :81-84
        self.written = np.zeros(self.capacity, dtype=bool)              # :88-90
        self.written[self.L:] = True
        self.mask_written = np.zeros(self.capacity, dtype=bool)         # :91

    def reset(self):                                                    # :99-102
        self.kv[...] = 0
        self.written[:] = False
        self.written[self.L:] = True

    def upsert(self, kv_new: np.ndarray, frame_t: int, is_frozen: bool):
        """kv_new [2,B,H,T,Dh]; restates src/model/kv_cache.py:126-154.

        Returns (k_full, v_full, mask_written): views of the whole buffer and
        the per-token visibility used for this call's attention.
        """
        T = self.tpf
        if kv_new.shape[3] != T:
            raise ValueError("KV cache expects exactly one frame per upsert")    # :113
        if frame_t < 0:
            raise ValueError("t_pos must be non-negative during inference")      # :120-123
        _, _, base, write_step = slot_arithmetic(frame_t, T, self.L, self.pinned_dilation)
        ring = slice(base, base + T)                                     # :134
        tail = slice(self.L, self.L + T)                                 # :97
        self.kv[:, :, :, tail, :] = kv_new                               # :138
        self.mask_written[:] = self.written                              # :141-142
        if write_step:
            self.mask_written[ring] = False                              # :143
        if not is_frozen:                                                # :147-151
            dst = ring if write_step else tail
            self.kv[:, :, :, dst, :] = kv_new
            self.written[dst] = True
        return self.kv[0], self.kv[1], self.mask_written                 # :153-154


# --------------------------------------------------------------------------
# the attention
# --------------------------------------------------------------------------
def frame_attention(q: np.ndarray, k_full: np.ndarray, v_full: np.ndarray,
                    mask_written: np.ndarray, scale: float | None = None) -> np.ndarray:
    """softmax(q k^T * scale, masked to mask_written) v in fp32.

    q [B,Hq,T,Dh], k_full/v_full [B,Hkv,C,Dh] (fp32 values), mask_written [C]
    bool.  Restates what flex_attention computes at src/model/attn.py:116
    with the mask of src/model/kv_cache.py:47-48 (`written[kv]`), the default
    scale 1/sqrt(Dh), GQA by repeating kv heads, and the fp32 eager order of
    operations: scores -> scale -> -inf mask -> softmax -> P @ V.
    """
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k_full, dtype=np.float32)
    v = np.asarray(v_full, dtype=np.float32)
    B, Hq, T, Dh = q.shape
    Hkv = k.shape[1]
    G = Hq // Hkv
    if scale is None:
        scale = 1.0 / math.sqrt(Dh)
    vis = np.flatnonzero(mask_written)
    out = np.empty((B, Hq, T, Dh), dtype=np.float32)
    for b in range(B):
        for h in range(Hq):
            kh = k[b, h // G][vis]                                       # gather only what is visible
            vh = v[b, h // G][vis]
            s = (q[b, h] @ kh.T) * np.float32(scale)
            m = s.max(axis=-1, keepdims=True)
            p = np.exp(s - m)
            p /= p.sum(axis=-1, keepdims=True)
            out[b, h] = p @ vh
    return out


def frame_step(cache: OracleLayerKVCache, q_f32: np.ndarray, kv_new: np.ndarray,
               frame_t: int, is_frozen: bool, scale: float | None = None,
               to_f32=lambda a: a) -> np.ndarray:
    """One layer-step of the hot path: upsert then attend
    (src/model/attn.py:113-116 / src/patch_model.py:131-133).

    `to_f32` converts the cache's element container to fp32 values
    (identity for float32 caches, `bf16_bits_to_f32` for uint16 caches).
    """
    k_full, v_full, mask = cache.upsert(kv_new, frame_t, is_frozen)
    return frame_attention(q_f32, to_f32(k_full), to_f32(v_full), mask, scale)


# --------------------------------------------------------------------------
# what happens to q, k, v between the projections and the cache
# (src/model/attn.py:105-110, src/patch_model.py:124-129)
# --------------------------------------------------------------------------
F32_EPS = float(np.finfo(np.float32).eps)


def unit_rms_norm(x_f32: np.ndarray, eps: float = F32_EPS) -> np.ndarray:
    """Weightless RMS norm over the last axis in fp32: x * rsqrt(mean(x^2) + eps)
    (`rms_norm`, src/model/nn.py:55-56: F.rms_norm without weight and with the
    default eps, which for 16-bit inputs is the fp32 machine epsilon because the
    op computes in fp32).  The caller rounds the result to the tensor's dtype."""
    x = np.asarray(x_f32, dtype=np.float32)
    ms = np.mean(x * x, axis=-1, keepdims=True, dtype=np.float32)
    return (x * (np.float32(1.0) / np.sqrt(ms + np.float32(eps)))).astype(np.float32)


def rope_rotate(x_f32: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """RoPE.forward (src/model/attn.py:33-40) in fp32: consecutive pairs
    (x[2j], x[2j+1]) are rotated by the angle j of the token and the result is
    laid out as [all first components | all second components].
    x [..., T, Dh]; cos, sin [..., T, Dh/2] (broadcast over heads by the caller)."""
    x = np.asarray(x_f32, dtype=np.float32)
    x0, x1 = x[..., 0::2], x[..., 1::2]
    c, s = np.asarray(cos, dtype=np.float32), np.asarray(sin, dtype=np.float32)
    y0 = (x0 * c).astype(np.float32) - (x1 * s).astype(np.float32)
    y1 = (x1 * c).astype(np.float32) + (x0 * s).astype(np.float32)
    return np.concatenate([y0, y1], axis=-1).astype(np.float32)


def rope_angles(cos_table: np.ndarray, sin_table: np.ndarray, t_pos, y_pos, x_pos, height: int, width: int):
    """RoPE.get_angles (src/model/attn.py:22-31): row t*(H*W) + y*W + x of the
    tables for every token; returns cos, sin [B, 1, T, Dh/2]."""
    flat = np.asarray(t_pos, dtype=np.int64) * (height * width) + np.asarray(y_pos, dtype=np.int64) * width \
        + np.asarray(x_pos, dtype=np.int64)
    if flat.min() < 0 or flat.max() >= cos_table.shape[0]:
        raise IndexError("position outside the RoPE table")
    return cos_table[flat][:, None], sin_table[flat][:, None]


def value_residual(v_f32: np.ndarray, v1_f32: np.ndarray, lamb: float) -> np.ndarray:
    """torch.lerp(v, v1, lamb) in fp32 (src/model/attn.py:105-107), with the
    two-sided form torch uses: start + w*diff below 0.5, end - diff*(1-w) from 0.5 on."""
    v = np.asarray(v_f32, dtype=np.float32)
    d = np.asarray(v1_f32, dtype=np.float32) - v
    w = np.float32(lamb)
    if abs(float(lamb)) < 0.5:
        return (v + w * d).astype(np.float32)
    return (np.asarray(v1_f32, dtype=np.float32) - d * (np.float32(1.0) - w)).astype(np.float32)


def qkv_prologue(q, k, v, v1, lamb, cos, sin, rounder=round_to_bf16):
    """q, k, v [B,H,T,Dh] fp32 values of 16-bit tensors -> (q', k', v') as the
    attention and the cache receive them: v' = lerp(v, v1, lamb) (skipped when
    v1 is None), q' = rope(rms_norm(q)), k' = rope(rms_norm(k)); `rounder`
    rounds to the tensors' dtype after every step that materialises a tensor in
    the reference (the norm, the rotation, the lerp)."""
    vo = np.asarray(v, dtype=np.float32) if v1 is None else rounder(value_residual(v, v1, lamb))
    qn, kn = rounder(unit_rms_norm(q)), rounder(unit_rms_norm(k))
    return rounder(rope_rotate(qn, cos, sin)), rounder(rope_rotate(kn, cos, sin)), vo
