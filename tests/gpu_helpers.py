"""Helpers of the GPU parity tests: build device tensors from the seeded host
inputs and compare device state with the oracle's."""
from __future__ import annotations

import hashlib
from dataclasses import replace

import numpy as np
import torch

from tests import helpers
from world_engine_b200 import B200LayerKVCache

TORCH_DTYPE = {"f32": torch.float32, "bf16": torch.bfloat16}


def dev_tensor(cfg, x: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(x)).to("cuda").to(TORCH_DTYPE[cfg.dtype])


def pos_ids(cfg, frame_t: int):
    return {"t_pos": torch.full((cfg.B, cfg.T), frame_t, dtype=torch.long, device="cuda")}


def new_gpu_cache(cfg) -> B200LayerKVCache:
    return B200LayerKVCache(cfg.B, cfg.Hkv, cfg.L, cfg.Dh, TORCH_DTYPE[cfg.dtype], cfg.T, cfg.dilation).to("cuda")


def kv_bytes(cache: B200LayerKVCache) -> bytes:
    kv = cache.kv.detach()
    if kv.dtype == torch.bfloat16:
        kv = kv.view(torch.int16)
    return kv.cpu().numpy().tobytes()


def kv_sha(cache: B200LayerKVCache) -> str:
    return hashlib.sha256(kv_bytes(cache)).hexdigest()


def as_bf16(cfg):
    return cfg if cfg.dtype == "bf16" else replace(cfg, dtype="bf16")
