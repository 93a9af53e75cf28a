"""Generates tests/golden/prologue_*.npz by RUNNING THE REFERENCE's own code for what happens to q, k, v
between the projections and the cache: `rms_norm` (src/model/nn.py:55-56), `RoPE.forward` / `get_angles`
(src/model/attn.py:22-40) and the value residual `torch.lerp` (src/model/attn.py:105-107), on seeded bf16
inputs and a seeded angle table.  (The table's real values come from the third-party package
`rotary_embedding_torch`, which is not installed; `RoPE.forward` only indexes and applies whatever table the
module holds, so a placeholder class lets the module import and the table is set by hand.)

Usage:  REFERENCE_ROOT=<checkout of the reference> python tests/golden/make_golden_prologue.py
"""
from __future__ import annotations

import importlib
import json
import os
import sys
import types

import numpy as np
import torch
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ring_attn_oracle as oracle  # noqa: E402  (bf16 bit helpers only)

REFERENCE_ROOT = os.environ.get("REFERENCE_ROOT", "")
if not os.path.isdir(os.path.join(REFERENCE_ROOT, "src", "model")):
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference (it needs src/model/attn.py)")


def load_reference_attn():
    td = types.ModuleType("tensordict")
    td.TensorDict = dict
    sys.modules.setdefault("tensordict", td)
    ret = types.ModuleType("rotary_embedding_torch")

    class RotaryEmbedding:      # placeholder: only get_freqs would use it, and that is not called here
        def __init__(self, *a, **k):
            raise RuntimeError("table generation is not part of this recording")
    ret.RotaryEmbedding = RotaryEmbedding
    sys.modules.setdefault("rotary_embedding_torch", ret)
    pkg = types.ModuleType("_we_ref")
    pkg.__path__ = [os.path.join(REFERENCE_ROOT, "src")]
    sys.modules["_we_ref"] = pkg
    sub = types.ModuleType("_we_ref.model")
    sub.__path__ = [os.path.join(REFERENCE_ROOT, "src", "model")]
    sys.modules["_we_ref.model"] = sub
    return importlib.import_module("_we_ref.model.attn"), importlib.import_module("_we_ref.model.nn")


CASES = {
    # name: B, Hq, Hkv, Dh, grid height, grid width, frames in the table, frame index, lerp weight, seed
    "prologue_dh64": (2, 4, 2, 64, 4, 8, 5, 3, 0.5, 31),
    "prologue_dh128_gqa": (1, 8, 2, 128, 8, 8, 3, 2, 0.296875, 32),
    "prologue_no_residual": (1, 2, 2, 128, 4, 4, 2, 0, None, 33),
}


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    attn, refnn = load_reference_attn()
    for name, (B, Hq, Hkv, Dh, Hh, Ww, n_frames, frame, lamb, seed) in CASES.items():
        rng = np.random.default_rng(seed)
        T = Hh * Ww
        q = torch.from_numpy(rng.standard_normal((B, Hq, T, Dh), dtype=np.float32) * 2.0).bfloat16()
        k = torch.from_numpy(rng.standard_normal((B, Hkv, T, Dh), dtype=np.float32) * 0.5).bfloat16()
        v = torch.from_numpy(rng.standard_normal((B, Hkv, T, Dh), dtype=np.float32)).bfloat16()
        v1 = torch.from_numpy(rng.standard_normal((B, Hkv, T, Dh), dtype=np.float32)).bfloat16()
        ang = torch.from_numpy(rng.uniform(-np.pi, np.pi, (n_frames * Hh * Ww, Dh // 2)).astype(np.float32))
        rope = object.__new__(attn.RoPE)          # the module without its table generation
        nn.Module.__init__(rope)
        rope.config = types.SimpleNamespace(height=Hh, width=Ww)
        rope.cos = nn.Buffer(ang.cos().contiguous(), persistent=False)
        rope.sin = nn.Buffer(ang.sin().contiguous(), persistent=False)
        yy, xx = torch.meshgrid(torch.arange(Hh), torch.arange(Ww), indexing="ij")
        pos = {"t_pos": torch.full((B, T), frame, dtype=torch.long),
               "y_pos": yy.reshape(1, T).expand(B, T).contiguous(),
               "x_pos": xx.reshape(1, T).expand(B, T).contiguous()}
        vo = v
        if lamb is not None:
            vo = torch.lerp(v, v1.view_as(v), torch.tensor(lamb, dtype=torch.bfloat16))     # attn.py:105-107
        qn, kn = refnn.rms_norm(q), refnn.rms_norm(k)                                        # attn.py:109
        qo, ko = rope(qn, pos), rope(kn, pos)                                                # attn.py:110
        meta = {"B": B, "Hq": Hq, "Hkv": Hkv, "Dh": Dh, "height": Hh, "width": Ww, "frames": n_frames,
                "frame": frame, "lamb": lamb, "seed": seed,
                "reference": f"Overworldai/world_engine src/model/attn.py RoPE + src/model/nn.py rms_norm, torch {torch.__version__} CPU"}
        rec = {"q": bits(q), "k": bits(k), "v": bits(v), "v1": bits(v1), "cos": rope.cos.numpy().copy(),
               "sin": rope.sin.numpy().copy(), "t_pos": pos["t_pos"].numpy(), "y_pos": pos["y_pos"].numpy(),
               "x_pos": pos["x_pos"].numpy(), "q_out": bits(qo), "k_out": bits(ko), "v_out": bits(vo),
               "meta": np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)}
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **rec)
        print(f"{name} -> {path} ({os.path.getsize(path) / 1024:.0f} KiB)")


if __name__ == "__main__":
    main()
