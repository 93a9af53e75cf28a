"""Generates the golden fixtures of this directory by RUNNING THE REFERENCE.

Runs only where a checkout of the reference is available (its location is
taken from the environment variable REFERENCE_ROOT): it imports the reference's own `src/model/kv_cache.py`
(LayerKVCache.upsert, make_block_mask) by path and calls torch's un-compiled
`flex_attention` exactly as `src/model/attn.py:116` does, on the seeded inputs
of `world_engine_b200.synthetic`.  The reference publishes no tests or golden
vectors for this path, so these recorded outputs are what pins the oracle.

`tensordict` (imported by kv_cache.py only for a type annotation) is not
installed; a stub module providing `TensorDict = dict` is injected.  Nothing
from the reference is copied into the repository: only its OUTPUTS are stored.

Usage:  REFERENCE_ROOT=<checkout of the reference> python tests/golden/make_golden.py
        (rewrites tests/golden/*.npz)
"""
from __future__ import annotations

import hashlib
import importlib
import json
import os
import sys
import types
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from world_engine_b200 import synthetic  # noqa: E402
from world_engine_b200.synthetic import StepConfig  # noqa: E402

REFERENCE_ROOT = os.environ.get("REFERENCE_ROOT", "")
if not os.path.isdir(os.path.join(REFERENCE_ROOT, "src", "model")):
    raise SystemExit("make_golden.py: set REFERENCE_ROOT to a checkout of the reference (it needs src/model/kv_cache.py)")


def load_reference_kv_cache():
    td = types.ModuleType("tensordict")
    td.TensorDict = dict
    sys.modules.setdefault("tensordict", td)
    pkg = types.ModuleType("_we_ref")
    pkg.__path__ = [os.path.join(REFERENCE_ROOT, "src")]
    sys.modules["_we_ref"] = pkg
    sub = types.ModuleType("_we_ref.model")
    sub.__path__ = [os.path.join(REFERENCE_ROOT, "src", "model")]
    sys.modules["_we_ref.model"] = sub
    return importlib.import_module("_we_ref.model.kv_cache")


# Each case: a config and the call sequence replayed from a freshly reset cache.
# calls = list of (frame_t, is_frozen, record_output)
def denoise_then_persist(frames, last_frozen_steps=1, record_from=None):
    """History frames persisted unfrozen; the last frame runs `last_frozen_steps` frozen steps then one unfrozen."""
    calls = []
    frames = list(frames)
    for f in frames[:-1]:
        calls.append((f, False, record_from is not None and f >= record_from))
    last = frames[-1]
    for _ in range(last_frozen_steps):
        calls.append((last, True, True))
    calls.append((last, False, True))
    return calls


CASES = {
    # benchmark config 1, wrapped and pre-wrap (fp32, the reference's own CPU-runnable case)
    "cfg1": (synthetic.CONFIGS["cfg1"], denoise_then_persist(range(0, 7), 2, record_from=3)),
    "cfg1_prewrap": (synthetic.CONFIGS["cfg1_prewrap"], denoise_then_persist(range(0, 3), 1, record_from=0)),
    # pinned dilation 2: write steps and non-write steps, slot quirk (only num_buckets slots used)
    "dilation2": (StepConfig("dilation2", 1, 2, 2, 64, 64, 4, 2, 9, "f32", 4321),
                  denoise_then_persist(range(0, 10), 1, record_from=0)),
    # grouped-query heads, bf16-rounded inputs, 128-token frames
    "gqa_bf16": (StepConfig("gqa_bf16", 2, 8, 2, 64, 128, 3, 1, 7, "bf16", 777),
                 denoise_then_persist(range(0, 8), 1, record_from=5)),
    # Dh=128, 256-token frames, small ring, K outliers (benchmark config 5 in miniature)
    "outliers_bf16": (StepConfig("outliers_bf16", 2, 4, 4, 128, 256, 3, 1, 4, "bf16", 999,
                                 k_outlier_frac=0.05, k_outlier_gain=3.0),
                      denoise_then_persist(range(0, 5), 1, record_from=2)),
    # benchmark config 2 at full size (outputs subsampled to keep the fixture small)
    "cfg2": (synthetic.CONFIGS["cfg2"], denoise_then_persist(range(27 - 16, 28), 1, record_from=27)),
}
SUBSAMPLE_ROWS = {"cfg2": [0, 37, 128, 255], "gqa_bf16": [0, 1, 31, 64, 77, 127],
                  "outliers_bf16": [0, 5, 127, 128, 200, 255]}


def sha(t: torch.Tensor) -> str:
    a = t.detach().contiguous()
    if a.dtype == torch.bfloat16:
        a = a.view(torch.int16)
    return hashlib.sha256(a.numpy().tobytes()).hexdigest()


def main():
    ref = load_reference_kv_cache()
    from torch.nn.attention.flex_attention import flex_attention
    warnings.filterwarnings("ignore")
    torch.manual_seed(0)
    for name, (cfg, calls) in CASES.items():
        tdtype = torch.float32 if cfg.dtype == "f32" else torch.bfloat16
        cache = ref.LayerKVCache(cfg.B, cfg.Hkv, cfg.L, cfg.Dh, tdtype, cfg.T, cfg.dilation)
        cache.reset()
        rec = {}
        meta = {"config": cfg.__dict__, "calls": [], "reference": "Overworldai/world_engine src/model/kv_cache.py + "
                f"torch {torch.__version__} eager flex_attention", "subsample_rows": SUBSAMPLE_ROWS.get(name)}
        step_of_frame = {}
        for ci, (t, frozen, record) in enumerate(calls):
            step = step_of_frame.get(t, 0)
            step_of_frame[t] = step + 1
            k_np, v_np = synthetic.frame_kv(cfg, t)
            q_np = synthetic.frame_q(cfg, t, step)
            k = torch.from_numpy(k_np).to(tdtype)
            v = torch.from_numpy(v_np).to(tdtype)
            q = torch.from_numpy(q_np).to(tdtype)
            pos = {"t_pos": torch.full((cfg.B, cfg.T), t, dtype=torch.long)}
            k_full, v_full, bm = cache.upsert(torch.stack([k, v], 0), pos, frozen)   # kv_cache.py:191-193
            entry = {"frame_t": t, "is_frozen": frozen, "step": step, "kv_sha256": sha(cache.kv),
                     "recorded": bool(record)}
            rec[f"written_{ci}"] = cache.written.numpy().copy()
            rec[f"mask_{ci}"] = cache._mask_written.numpy().copy()
            rec[f"kv_num_blocks_{ci}"] = bm.kv_num_blocks.numpy().copy()
            rec[f"kv_indices_{ci}"] = bm.kv_indices.numpy().copy()
            rec[f"full_kv_num_blocks_{ci}"] = bm.full_kv_num_blocks.numpy().copy()
            rec[f"full_kv_indices_{ci}"] = bm.full_kv_indices.numpy().copy()
            if record:
                # "the reference run in fp32": same (dtype-rounded) values, fp32 tensors
                out = flex_attention(q.float(), k_full.float(), v_full.float(), block_mask=bm,
                                     enable_gqa=cfg.Hq != cfg.Hkv)                   # attn.py:116
                out = out.numpy()
                rows = SUBSAMPLE_ROWS.get(name)
                rec[f"out_{ci}"] = out[:, :, rows, :].copy() if rows else out
                entry["out_sha256_full"] = hashlib.sha256(out.tobytes()).hexdigest()
            meta["calls"].append(entry)
        rec["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **rec)
        print(f"{name}: {len(calls)} calls -> {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
