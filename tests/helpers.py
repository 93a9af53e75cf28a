"""Shared helpers of the test-suite: golden fixtures, oracle replay, input builders."""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np

from oracle import ring_attn_oracle as oracle
from world_engine_b200 import synthetic
from world_engine_b200.synthetic import StepConfig

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
GOLDEN_CASES = ["cfg1", "cfg1_prewrap", "dilation2", "gqa_bf16", "outliers_bf16", "cfg2"]

# Tolerance of the attention output against the reference run in fp32 (the specification's bar).
MAX_ABS_TOL = 1e-2
MEAN_ABS_TOL = 1e-3


def load_golden(name: str):
    z = np.load(os.path.join(GOLDEN_DIR, f"{name}.npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    c = dict(meta["config"])
    cfg = StepConfig(**c)
    return cfg, meta, z


def step_inputs(cfg: StepConfig, frame_t: int, step: int):
    """(q, k, v) fp32 arrays rounded to the cache dtype's values."""
    k, v = synthetic.frame_kv(cfg, frame_t)
    q = synthetic.frame_q(cfg, frame_t, step)
    if cfg.dtype == "bf16":
        q, k, v = oracle.round_to_bf16(q), oracle.round_to_bf16(k), oracle.round_to_bf16(v)
    return q, k, v


def new_oracle_cache(cfg: StepConfig) -> oracle.OracleLayerKVCache:
    np_dtype = np.float32 if cfg.dtype == "f32" else np.uint16
    return oracle.OracleLayerKVCache(cfg.B, cfg.Hkv, cfg.L, cfg.Dh, np_dtype, cfg.T, cfg.dilation)


def to_container(cfg: StepConfig, x: np.ndarray) -> np.ndarray:
    return x if cfg.dtype == "f32" else oracle.f32_to_bf16_bits(x)


def from_container(cfg: StepConfig, x: np.ndarray) -> np.ndarray:
    return x if cfg.dtype == "f32" else oracle.bf16_bits_to_f32(x)


def kv_digest(kv: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(kv).tobytes()).hexdigest()


def oracle_step(cfg: StepConfig, cache, frame_t: int, step: int, is_frozen: bool, want_out: bool = True):
    q, k, v = step_inputs(cfg, frame_t, step)
    kv_new = np.stack([to_container(cfg, k), to_container(cfg, v)], 0)
    k_full, v_full, mask = cache.upsert(kv_new, frame_t, is_frozen)
    out = None
    if want_out:
        out = oracle.frame_attention(q, from_container(cfg, k_full), from_container(cfg, v_full), mask)
    return out, mask


def error_stats(got: np.ndarray, want: np.ndarray):
    d = np.abs(np.asarray(got, dtype=np.float64) - np.asarray(want, dtype=np.float64))
    return float(d.max()), float(d.mean())
