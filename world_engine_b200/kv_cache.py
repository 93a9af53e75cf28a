"""KV ring-buffer cache with the reference's call surface, backed by the
sm_100a kernels.

`B200LayerKVCache` / `B200StaticKVCache` stand in for `LayerKVCache` /
`StaticKVCache` (src/model/kv_cache.py:64-193): same constructor arguments,
same buffer names, shapes and dtypes (`kv[2,B,H,L+tpf,Dh]`, `written[L+tpf]`),
same methods (`reset`, `set_frozen`, `upsert`).  State after any sequence of
calls is bit-identical to the reference's.  On top of that surface they offer
`append_and_attend`, which does the whole layer-step (append + attention) in
the library without building a BlockMask.
"""
from __future__ import annotations

from typing import Mapping, Optional, Tuple

import torch
from torch import Tensor, nn

from . import ops

SPARSE_BLOCK = 128  # flex-attention's default sparse block size


def block_mask_from_tables(tables, mask_written: Tensor, T: int, capacity: int):
    """flex-attention BlockMask over precomputed tables; same construction the
    reference ends make_block_mask with (src/model/kv_cache.py:47-59)."""
    from torch.nn.attention.flex_attention import BlockMask

    kv_num, kv_idx, full_num, full_idx = tables

    def visible(b, h, q, kv):
        return mask_written[kv]

    return BlockMask.from_kv_blocks(
        kv_num, kv_idx, full_num, full_idx,
        BLOCK_SIZE=SPARSE_BLOCK, mask_mod=visible, seq_lengths=(T, capacity),
        compute_q_blocks=False)


class B200LayerKVCache(nn.Module):
    """One layer's ring of L tokens plus a tail frame (drop-in for LayerKVCache)."""

    def __init__(self, B: int, H: int, L: int, Dh: int, dtype: torch.dtype,
                 tokens_per_frame: int, pinned_dilation: int = 1):
        super().__init__()
        if L % tokens_per_frame != 0 or (L // tokens_per_frame) % pinned_dilation != 0:
            raise ValueError("L must be a multiple of tokens_per_frame, and the frame count a "
                             "multiple of pinned_dilation")
        self.tpf = tokens_per_frame
        self.L = L
        self.capacity = L + tokens_per_frame
        self.pinned_dilation = pinned_dilation
        self.num_buckets = (L // tokens_per_frame) // pinned_dilation
        self.kv = nn.Buffer(torch.zeros(2, B, H, self.capacity, Dh, dtype=dtype), persistent=False)
        flags = torch.zeros(self.capacity, dtype=torch.bool)
        flags[L:] = True  # the tail always holds the current frame
        self.written = nn.Buffer(flags, persistent=False)
        self._mask_written = nn.Buffer(torch.zeros_like(flags), persistent=False)
        self.validate = True  # eager-only argument checks (they synchronise, like the reference's)

    # -- lifecycle ---------------------------------------------------------
    def reset(self) -> None:
        self.kv.zero_()
        self.written.zero_()
        self.written[self.L:] = True

    # -- checks (src/model/kv_cache.py:112-124; skipped while compiling or capturing)
    def _check(self, k: Tensor, t_pos: Tensor) -> None:
        if not self.validate or torch.compiler.is_compiling():
            return
        if k.is_cuda and torch.cuda.is_current_stream_capturing():
            return
        if k.size(2) != self.tpf:
            raise RuntimeError("KV cache expects exactly one frame per upsert")
        if tuple(t_pos.shape) != (k.size(0), self.tpf):
            raise RuntimeError("t_pos must be [B, T]")
        if bool((t_pos < 0).any().item()):
            raise RuntimeError("t_pos must be non-negative during inference")
        if not bool((t_pos == t_pos[:, :1]).all().item()):
            raise RuntimeError("t_pos must be constant within frame")

    @staticmethod
    def _frame_t(pos_ids: Mapping[str, Tensor]) -> Tensor:
        t_pos = pos_ids["t_pos"]
        if t_pos.dtype != torch.int64:
            raise TypeError("t_pos must be int64")
        return t_pos

    # -- reference surface --------------------------------------------------
    def upsert_kv(self, k: Tensor, v: Tensor, pos_ids: Mapping[str, Tensor], is_frozen: bool
                  ) -> Tuple[Tensor, Tensor, object]:
        """`upsert` without the packed [2,...] copy: k, v are [B,H,T,Dh] views."""
        t_pos = self._frame_t(pos_ids)
        self._check(k, t_pos)
        ops.kv_append_op(self.kv, self.written, self._mask_written, k, v, t_pos,
                         self.tpf, self.pinned_dilation, bool(is_frozen))
        tables = ops.block_mask_tables(self._mask_written, self.tpf)
        bm = block_mask_from_tables(tables, self._mask_written, self.tpf, self.capacity)
        k_full, v_full = self.kv.unbind(0)
        return k_full, v_full, bm

    def upsert(self, kv: Tensor, pos_ids: Mapping[str, Tensor], is_frozen: bool):
        """kv [2,B,H,T,Dh] for one frame -> (k_full, v_full, BlockMask), the
        reference's signature (src/model/kv_cache.py:104)."""
        return self.upsert_kv(kv[0], kv[1], pos_ids, is_frozen)

    # -- fused layer-step ---------------------------------------------------
    def append_and_attend(self, q: Tensor, k: Tensor, v: Tensor, pos_ids: Mapping[str, Tensor],
                          is_frozen: bool, scale: float = 0.0, gate: Optional[Tensor] = None,
                          gate_is_logits: bool = False) -> Tensor:
        """Append the frame and attend to the cache: what upsert + flex_attention
        do at src/model/attn.py:113-116, without a BlockMask (one launch when the
        tail frame is made of whole 128-key tiles, else append + attention).
        `gate` ([B,Hq,T], q's dtype) multiplies the output rows, after a sigmoid
        when `gate_is_logits` (the head gate of src/model/attn.py:117-119)."""
        t_pos = self._frame_t(pos_ids)
        self._check(k, t_pos)
        if gate is not None:
            return ops.append_attend_gated_op(q, k, v, self.kv, self.written, t_pos, gate,
                                              self.tpf, self.pinned_dilation, bool(is_frozen), float(scale),
                                              bool(gate_is_logits))
        return ops.append_attend_op(q, k, v, self.kv, self.written, t_pos,
                                    self.tpf, self.pinned_dilation, bool(is_frozen), float(scale))

    def attend(self, q: Tensor, pos_ids: Mapping[str, Tensor], scale: float = 0.0) -> Tensor:
        """Attention only (the frame must already be appended)."""
        return ops.frame_attn_op(q, self.kv, self.written, self._frame_t(pos_ids),
                                 self.tpf, self.pinned_dilation, float(scale))


class B200StaticKVCache(nn.Module):
    """Per-layer caches chosen like StaticKVCache (src/model/kv_cache.py:157-181):
    every `global_attn_period`-th layer (offset `global_attn_offset`) gets the
    global window and the pinned dilation, the others the local window."""

    def __init__(self, config, batch_size: int, dtype: torch.dtype):
        super().__init__()
        self.tpf = config.tokens_per_frame
        period = config.global_attn_period
        offset = getattr(config, "global_attn_offset", 0) % period
        kv_heads = getattr(config, "n_kv_heads", config.n_heads)
        head_dim = config.d_model // config.n_heads
        layers = []
        for idx in range(config.n_layers):
            is_global = (idx - offset) % period == 0
            window = config.global_window if is_global else config.local_window
            dilation = config.global_pinned_dilation if is_global else 1
            layers.append(B200LayerKVCache(batch_size, kv_heads, window * self.tpf, head_dim, dtype,
                                           self.tpf, dilation))
        self.layers = nn.ModuleList(layers)
        self._is_frozen = True

    def reset(self) -> None:
        for layer in self.layers:
            layer.reset()
        self._is_frozen = True

    def set_frozen(self, is_frozen: bool) -> None:
        self._is_frozen = is_frozen

    def upsert(self, k: Tensor, v: Tensor, pos_ids: Mapping[str, Tensor], layer: int):
        return self.layers[layer].upsert_kv(k, v, pos_ids, self._is_frozen)

    def append_and_attend(self, q: Tensor, k: Tensor, v: Tensor, pos_ids: Mapping[str, Tensor],
                          layer: int, scale: float = 0.0, gate: Optional[Tensor] = None,
                          gate_is_logits: bool = False) -> Tensor:
        return self.layers[layer].append_and_attend(q, k, v, pos_ids, self._is_frozen, scale, gate, gate_is_logits)
