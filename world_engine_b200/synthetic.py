"""Seeded synthetic workloads: the shapes and value distributions of the
benchmark configurations of this path (there is no dataset; the reference's
own benchmark drives real weights that are not redistributable here).

Everything is generated with numpy's PCG64 in fp32 on the host, so the CUDA
path and a CPU checker can be fed bit-identical inputs.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Dict, Tuple

import numpy as np


@dataclass(frozen=True)
class StepConfig:
    name: str
    B: int              # batch rows (sessions)
    Hq: int
    Hkv: int
    Dh: int
    T: int              # tokens per frame
    ring_frames: int    # L = ring_frames * T
    dilation: int
    frame_t: int        # frame index of the step under test
    dtype: str          # "bf16" | "f32"
    seed: int
    k_outlier_frac: float = 0.0   # fraction of (head, channel) pairs of K scaled by k_outlier_gain
    k_outlier_gain: float = 1.0

    @property
    def L(self) -> int:
        return self.ring_frames * self.T

    @property
    def capacity(self) -> int:
        return self.L + self.T

    def visible_keys(self) -> int:
        """Tokens the step attends to: written ring frames other than the slot being replaced, plus the tail."""
        d = self.dilation
        buckets = self.ring_frames // d
        persisted = min(buckets, (self.frame_t + d - 1) // d)       # frames t' < t with t' % d == 0
        hidden = 1 if (self.frame_t % d == 0 and persisted == buckets) else 0
        return (persisted - hidden + 1) * self.T

    def flops(self) -> float:
        return 4.0 * self.B * self.Hq * self.T * self.visible_keys() * self.Dh

    def algorithmic_bytes(self, frozen: bool = True, elem: int = 2) -> float:
        """K,V of every visible key + Q in + O out + read of the new K,V + cache writes
        (tail always; ring slot too on an unfrozen write step)."""
        w = 1 if (frozen or self.frame_t % self.dilation != 0) else 2
        kv_row = 2 * self.Hkv * self.Dh * elem
        return self.B * (kv_row * self.visible_keys() + 2 * self.Hq * self.T * self.Dh * elem
                         + kv_row * self.T + w * kv_row * self.T)


# The five configurations of the benchmark specification.
CONFIGS: Dict[str, StepConfig] = {
    # CPU-runnable fp32 layer; run pre-wrap (frame_t=2) and wrapped (frame_t=6)
    "cfg1": StepConfig("cfg1", 1, 4, 4, 64, 64, 4, 1, 6, "f32", 1235),
    "cfg1_prewrap": StepConfig("cfg1_prewrap", 1, 4, 4, 64, 64, 4, 1, 2, "f32", 1235),
    # single frame step at small-model scale, ring wrapped, write pointer at slot 11
    "cfg2": StepConfig("cfg2", 1, 16, 16, 128, 256, 16, 1, 27, "bf16", 1236),
    # one layer of the 24-layer denoise (cfg3 = 24 independent copies of this, 4 steps per frame)
    "cfg3_layer": StepConfig("cfg3_layer", 1, 16, 16, 128, 256, 16, 1, 20, "bf16", 1237),
    # one session of the 64-session throughput run (32-frame ring)
    "cfg4_session": StepConfig("cfg4_session", 1, 16, 16, 128, 256, 32, 1, 32 + 4711, "bf16", 1238),
    # high-resolution long-context run with K outliers
    "cfg5": StepConfig("cfg5", 4, 16, 16, 128, 1024, 16, 1, 21, "bf16", 1239,
                       k_outlier_frac=0.01, k_outlier_gain=3.0),
}


def scaled(cfg: StepConfig, **kw) -> StepConfig:
    return replace(cfg, **kw)


def _rng(cfg: StepConfig, *key: int) -> np.random.Generator:
    return np.random.default_rng([cfg.seed, *key])


def k_channel_gain(cfg: StepConfig) -> np.ndarray:
    """[Hkv, Dh] multiplier for K: 1 everywhere, `k_outlier_gain` on a seeded fraction of pairs."""
    g = np.ones((cfg.Hkv, cfg.Dh), dtype=np.float32)
    if cfg.k_outlier_frac > 0:
        pick = _rng(cfg, 3).random((cfg.Hkv, cfg.Dh)) < cfg.k_outlier_frac
        g[pick] = cfg.k_outlier_gain
    return g


def frame_kv(cfg: StepConfig, frame: int) -> Tuple[np.ndarray, np.ndarray]:
    """K, V of frame `frame`: [B, Hkv, T, Dh] fp32 ~ N(0,1) (K with the outlier gain)."""
    r = _rng(cfg, 1, frame)
    shape = (cfg.B, cfg.Hkv, cfg.T, cfg.Dh)
    k = r.standard_normal(shape, dtype=np.float32)
    v = r.standard_normal(shape, dtype=np.float32)
    if cfg.k_outlier_frac > 0:
        k *= k_channel_gain(cfg)[None, :, None, :]
    return k, v


def frame_q(cfg: StepConfig, frame: int, step: int = 0) -> np.ndarray:
    """Q of denoise step `step` of frame `frame`: [B, Hq, T, Dh] fp32 ~ N(0,1)."""
    return _rng(cfg, 2, frame, step).standard_normal((cfg.B, cfg.Hq, cfg.T, cfg.Dh), dtype=np.float32)


def history_frames(cfg: StepConfig):
    """Frames whose unfrozen upsert determines the cache state seen at `cfg.frame_t`.
    With dilation 1 only the last `ring_frames` frames survive; otherwise replay everything."""
    if cfg.dilation == 1:
        return range(max(0, cfg.frame_t - cfg.ring_frames), cfg.frame_t)
    return range(0, cfg.frame_t)
