"""Many independent generation sessions on one GPU, and their placement on GPUs.

The reference runs one session per engine with batch 1 (src/world_engine.py:69,
src/model/world_model.py:279).  Sessions share nothing, so a server batches them:
`SessionSlab` keeps the per-layer caches of S sessions in one HBM slab
`[S, 2, H, L+T, Dh]` and runs the layer-step of all of them in one launch, each
session with its own frame counter and its own `written` vector (ring wrap
offsets differ between sessions).  Every session still sees exactly the
reference's cache layout: `slab.session_kv(i)` is a `[2, 1, H, L+T, Dh]` view
and `slab.session_written(i)` a `[L+T]` view, bit-comparable with a
`LayerKVCache` that replayed the same calls.

Across GPUs sessions are sharded round-robin (`shard_sessions`); there is no
exchange step, hence no collective on the data path.
"""
from __future__ import annotations

from typing import List

import torch
from torch import Tensor

from . import ops


def shard_sessions(n_sessions: int, world_size: int, rank: int) -> List[int]:
    """Sessions owned by `rank`: session i lives on GPU i mod world_size."""
    if not (0 <= rank < world_size):
        raise ValueError("rank out of range")
    return list(range(rank, n_sessions, world_size))


class SessionSlab:
    """One layer's KV ring caches of `n_sessions` independent sessions."""

    def __init__(self, n_sessions: int, H: int, L: int, Dh: int, dtype: torch.dtype, tokens_per_frame: int,
                 pinned_dilation: int = 1, device="cuda"):
        if L % tokens_per_frame != 0 or (L // tokens_per_frame) % pinned_dilation != 0:
            raise ValueError("L must be a multiple of tokens_per_frame, and the frame count a multiple of "
                             "pinned_dilation")
        self.n_sessions = n_sessions
        self.tpf = tokens_per_frame
        self.L = L
        self.capacity = L + tokens_per_frame
        self.pinned_dilation = pinned_dilation
        self._slab = torch.zeros(n_sessions, 2, H, self.capacity, Dh, dtype=dtype, device=device)
        # K plane / V plane first, sessions second: the [2, B, H, C, Dh] shape the kernels take, as a strided view
        self.kv = self._slab.transpose(0, 1)
        pitch = (self.capacity + 15) // 16 * 16                 # rows of `written` start 16-byte aligned
        self._written = torch.zeros(n_sessions, pitch, dtype=torch.bool, device=device)
        self._written[:, L:self.capacity] = True                # the tail is always visible (kv_cache.py:88-90)
        self.frame_t = torch.zeros(n_sessions, dtype=torch.int64, device=device)

    # -- per-session views in the reference's layout ------------------------
    def session_kv(self, i: int) -> Tensor:
        return self._slab[i].unsqueeze(1)                        # [2, 1, H, C, Dh]

    def session_written(self, i: int) -> Tensor:
        return self._written[i, :self.capacity]

    def reset(self, i: int | None = None) -> None:
        """LayerKVCache.reset (src/model/kv_cache.py:99-102) for one session or all."""
        sel = slice(None) if i is None else i
        self._slab[sel].zero_()
        self._written[sel].zero_()
        self._written[sel, self.L:self.capacity] = True
        self.frame_t[sel] = 0

    # -- the layer-step of every session, one launch each for append and attention
    def append_and_attend(self, q: Tensor, k: Tensor, v: Tensor, is_frozen: bool, scale: float = 0.0,
                          out: Tensor | None = None) -> Tensor:
        """q [S, Hq, T, Dh], k / v [S, H, T, Dh]; session i uses frame counter `frame_t[i]`."""
        return ops.append_attend(q, k, v, self.kv, self._written, self.frame_t, self.tpf,
                                 self.pinned_dilation, is_frozen, scale, out=out, frame_t_stride=1)

    def append(self, k: Tensor, v: Tensor, is_frozen: bool) -> None:
        ops.kv_append_(self.kv, self._written, k, v, self.frame_t, self.tpf,
                       self.pinned_dilation, is_frozen, frame_t_stride=1)
