"""The reference's CPU code path for one layer-step, for timing on host cores.

TEST / BENCHMARK INFRASTRUCTURE ONLY (the CPU-baseline legs of bench.py and
the CPU tests import it; the shipped package never does).

On a CPU the reference executes, per layer-step, `LayerKVCache.upsert`
(src/model/kv_cache.py:104-154: torch index arithmetic, two `index_copy_`,
`make_block_mask`) and then torch's un-compiled `flex_attention`
(src/model/attn.py:116), which dispatches to the eager dense path of the
installed PyTorch.  The reference tree is not shipped with this repository,
so the cache update is restated here with the same torch operators on the
same buffer layout, and the attention call is the very same library call:
`torch.nn.attention.flex_attention.flex_attention(q, k, v, block_mask=...,
enable_gqa=...)` with a `BlockMask` built from the four index tables and
the `mask_mod` the reference builds.  What is timed is therefore torch's own
operators on this host, in the order the reference issues them.
"""
from __future__ import annotations

import torch
from torch.nn.attention.flex_attention import BlockMask, flex_attention

SPARSE_BLOCK = 128  # _DEFAULT_SPARSE_BLOCK_SIZE of torch.nn.attention.flex_attention


class TorchLayerKVCache:
    """Buffers and update rule of LayerKVCache (src/model/kv_cache.py:64-154) on CPU tensors."""

    def __init__(self, B: int, H: int, L: int, Dh: int, dtype: torch.dtype, tokens_per_frame: int, dilation: int = 1):
        self.T, self.L, self.C, self.d = tokens_per_frame, L, L + tokens_per_frame, dilation
        self.buckets = (L // tokens_per_frame) // dilation                       # :77
        self.kv = torch.zeros(2, B, H, self.C, Dh, dtype=dtype)                   # :81-84
        self.written = torch.zeros(self.C, dtype=torch.bool)                      # :86-90
        self.written[L:] = True
        self.offsets = torch.arange(tokens_per_frame, dtype=torch.long)           # :92

    def _block_mask(self, visible: torch.Tensor) -> BlockMask:
        """make_block_mask (src/model/kv_cache.py:12-61): per 128-token block any / all, ordered index tables."""
        nblk = (self.C + SPARSE_BLOCK - 1) // SPARSE_BLOCK
        qblk = (self.T + SPARSE_BLOCK - 1) // SPARSE_BLOCK
        rows = torch.nn.functional.pad(visible, (0, nblk * SPARSE_BLOCK - self.C)).view(nblk, SPARSE_BLOCK)
        some, every = rows.any(-1), rows.all(-1)

        def tables(dense):                                                       # :36-41
            dense = dense[None, :].expand(qblk, nblk)
            count = dense.sum(-1, dtype=torch.int32)
            order = dense.argsort(dim=-1, descending=True, stable=True).to(torch.int32)
            return count[None, None].contiguous(), order[None, None].contiguous()

        part_n, part_i = tables(some & ~every)
        full_n, full_i = tables(every)
        return BlockMask.from_kv_blocks(part_n, part_i, full_n, full_i, BLOCK_SIZE=SPARSE_BLOCK,
                                        mask_mod=lambda b, h, q, kv: visible[kv],
                                        seq_lengths=(self.T, self.C), compute_q_blocks=False)

    def upsert(self, kv_new: torch.Tensor, frame_t: torch.Tensor, is_frozen: bool):
        """kv_new [2,B,H,T,Dh], frame_t a 0-d int64 tensor (src/model/kv_cache.py:126-154)."""
        bucket = (frame_t + (self.d - 1)) // self.d                              # :129
        base = (bucket % self.buckets) * self.T                                  # :130-131
        ring_idx = base + self.offsets                                           # :132
        tail_idx = self.L + self.offsets                                         # :134
        self.kv.index_copy_(3, tail_idx, kv_new)                                 # :138
        write_step = (frame_t % self.d) == 0                                     # :140
        visible = self.written.clone()                                           # :141-143
        visible[ring_idx] = visible[ring_idx] & ~write_step
        bm = self._block_mask(visible)                                           # :144
        if not is_frozen:                                                        # :147-151
            dst = torch.where(write_step, ring_idx, tail_idx)
            self.kv.index_copy_(3, dst, kv_new)
            self.written[dst] = True
        k, v = self.kv.unbind(0)                                                 # :153
        return k, v, bm


def layer_step(cache: TorchLayerKVCache, q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
               frame_t: int, is_frozen: bool) -> torch.Tensor:
    """StaticKVCache.upsert (the stack of k and v, src/model/kv_cache.py:191-193) + flex_attention
    (src/model/attn.py:113-116)."""
    k, v, bm = cache.upsert(torch.stack([k_new, v_new], 0), torch.tensor(frame_t, dtype=torch.long), is_frozen)
    return flex_attention(q, k, v, block_mask=bm, enable_gqa=q.shape[1] != k.shape[1])
