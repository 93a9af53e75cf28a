"""Frame-causal self-attention module and its installer.

The reference swaps modules in place: `apply_inference_patches` walks the
model and calls `model.set_submodule(name, Replacement(old, ...))`
(src/patch_model.py:144-147,182-185).  `patch_Attn_b200` is one more function
of that chain.  It replaces every self-attention module (`Attn`,
src/model/attn.py:70-122, or its merged-QKV form `MergedQKVAttn`,
src/patch_model.py:92-141) by `B200Attn`, whose forward keeps the projections,
value residual, QK-norm, RoPE, head gate and output projection of the original
and hands the cache update + attention to the sm_100a library in one call.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from . import ops
from .kv_cache import B200StaticKVCache


def _unit_rms(x: torch.Tensor) -> torch.Tensor:
    # weightless RMS norm over the head dim (src/model/nn.py:55-56)
    return F.rms_norm(x, (x.size(-1),))


class B200Attn(nn.Module):
    """Drop-in for Attn / MergedQKVAttn with the same forward signature
    `(x, pos_ids, v1, kv_cache) -> (y, v1)` (src/model/world_model.py:166)."""

    def __init__(self, src: nn.Module):
        super().__init__()
        self.layer_idx = src.layer_idx
        self.n_heads = src.n_heads
        self.n_kv_heads = src.n_kv_heads
        self.d_head = src.d_head
        self.value_residual = bool(getattr(src, "value_residual", False))
        self.gated_attn = bool(getattr(src, "gated_attn", False))
        if self.value_residual:
            self.v_lamb = src.v_lamb
        if self.gated_attn:
            self.gate_proj = src.gate_proj
        self.rope = src.rope
        self.out_proj = src.out_proj
        self.q_out = self.n_heads * self.d_head
        self.kv_out = self.n_kv_heads * self.d_head
        if hasattr(src, "qkv_proj"):
            self.qkv_proj = src.qkv_proj
        else:
            # merge the three projections the way src/patch_model.py:102-112 does
            w = src.q_proj.weight
            self.qkv_proj = nn.Linear(src.q_proj.in_features, self.q_out + 2 * self.kv_out, bias=False,
                                      device=w.device, dtype=w.dtype)
            with torch.no_grad():
                self.qkv_proj.weight.copy_(torch.cat(
                    [src.q_proj.weight, src.k_proj.weight, src.v_proj.weight], dim=0))
        self.train(src.training)

    def _fused_prologue(self, q: torch.Tensor, pos_ids) -> bool:
        """The one-pass prologue needs the table form of RoPE (`cos` / `sin` buffers indexed by
        t*(H*W) + y*W + x, src/model/attn.py:12-31), 16-bit CUDA tensors and a head dim of 64 or 128; any
        other RoPE module is applied through its own forward."""
        rope = self.rope
        if not (hasattr(rope, "cos") and hasattr(rope, "sin") and hasattr(rope, "config")):
            return False
        if not (q.is_cuda and q.dtype in (torch.bfloat16, torch.float16) and self.d_head in (64, 128)):
            return False
        if rope.cos.dtype != torch.float32 or rope.cos.shape[-1] != self.d_head // 2:
            return False
        return all(key in pos_ids for key in ("t_pos", "y_pos", "x_pos"))

    def forward(self, x, pos_ids, v1, kv_cache: B200StaticKVCache):
        B, T = x.shape[:2]
        q, k, v = self.qkv_proj(x).split((self.q_out, self.kv_out, self.kv_out), dim=-1)
        q = q.reshape(B, T, self.n_heads, self.d_head).transpose(1, 2)
        k = k.reshape(B, T, self.n_kv_heads, self.d_head).transpose(1, 2)
        v = v.reshape(B, T, self.n_kv_heads, self.d_head).transpose(1, 2)

        if self._fused_prologue(q, pos_ids):
            # value residual + QK-norm + RoPE in one pass over q, k, v (src/patch_model.py:124-129)
            residual = None
            if self.value_residual:
                residual = None if v1 is None else v1.view_as(v)     # lerp(v, v, w) == v: nothing to do
                v1 = v if v1 is None else v1
            cfg = self.rope.config
            q, k, v = ops.qkv_prologue_op(q, k, v, residual, self.v_lamb if residual is not None else None,
                                          self.rope.cos, self.rope.sin, pos_ids["t_pos"], pos_ids["y_pos"],
                                          pos_ids["x_pos"], int(cfg.height), int(cfg.width))
        else:
            if self.value_residual:
                v1 = v if v1 is None else v1
                v = torch.lerp(v, v1.view_as(v), self.v_lamb)

            q, k = _unit_rms(q), _unit_rms(k)
            q, k = self.rope(q, pos_ids), self.rope(k, pos_ids)

        # cache update + attention: replaces upsert + flex_attention
        # (src/patch_model.py:131-133)
        # with the head gate (src/patch_model.py:135-137) applied to the rows on their way out of the kernel:
        # sigmoid(gate_proj(x[..., :H])) as a [B, H, T] view of the [B, T, H] logits
        if self.gated_attn and q.is_cuda and q.dtype in (torch.bfloat16, torch.float16):
            logits = self.gate_proj(x[..., : self.n_heads])
            y = kv_cache.append_and_attend(q, k, v, pos_ids, self.layer_idx, gate=logits.permute(0, 2, 1),
                                           gate_is_logits=True)
        else:
            y = kv_cache.append_and_attend(q, k, v, pos_ids, self.layer_idx)
            if self.gated_attn:
                gates = torch.sigmoid(self.gate_proj(x[..., : self.n_heads]))
                y = y * gates.permute(0, 2, 1).unsqueeze(-1)

        y = y.transpose(1, 2).reshape(B, T, -1)
        return self.out_proj(y), v1


def _is_self_attention(mod: nn.Module) -> bool:
    if isinstance(mod, B200Attn):
        return False
    names = {c.__name__ for c in type(mod).__mro__}
    return "Attn" in names  # Attn and its subclass MergedQKVAttn; CrossAttention is a different class


def patch_Attn_b200(model: nn.Module) -> None:
    """Installs B200Attn on every self-attention module of `model`.  Call it
    after (or instead of) the reference's patch_Attn_merge_qkv; the engine must
    then own a B200StaticKVCache."""
    for name, mod in list(model.named_modules()):
        if _is_self_attention(mod):
            model.set_submodule(name, B200Attn(mod))
