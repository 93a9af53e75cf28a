"""Seeded random geometries through the C ABI against the oracle: batch rows, grouped-query ratios, head dims,
frame lengths that are and are not multiples of the 128-key tile, ring lengths, dilations, both 16-bit types,
frozen and persisting calls over a run of frames that crosses the wrap.  Cache state bit-exact with
LayerKVCache.upsert (src/model/kv_cache.py:126-151) after every call; attention within the tolerance."""
import numpy as np
import pytest
import torch

from oracle import ring_attn_oracle as oracle
from tests import helpers
from world_engine_b200 import B200LayerKVCache, ops
from world_engine_b200.synthetic import StepConfig, frame_kv, frame_q

pytestmark = pytest.mark.gpu


def _cases(n=24, seed=20240607):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(n):
        Dh = int(rng.choice([64, 128]))
        Hkv = int(rng.choice([1, 2, 4]))
        group = int(rng.choice([1, 2, 4]))
        T = int(rng.choice([16, 64, 96, 128, 192, 256, 384]))
        dil = int(rng.choice([1, 1, 2, 3]))
        ring = dil * int(rng.integers(1, 5))
        B = int(rng.choice([1, 1, 2, 3]))
        dtype = str(rng.choice(["bf16", "f16"]))
        out.append((f"r{i}_B{B}_H{Hkv * group}k{Hkv}_D{Dh}_T{T}_ring{ring}_d{dil}_{dtype}",
                    B, Hkv * group, Hkv, Dh, T, ring, dil, dtype, 9000 + i))
    return out


CASES = _cases()


def _round(x, dtype):
    x = np.asarray(x, dtype=np.float32)
    return oracle.round_to_bf16(x) if dtype == "bf16" else x.astype(np.float16).astype(np.float32)


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_random_geometry(case):
    name, B, Hq, Hkv, Dh, T, ring, dil, dtype, seed = case
    cfg = StepConfig(name, B, Hq, Hkv, Dh, T, ring, dil, 0, "f32", seed)
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float16
    cache = B200LayerKVCache(B, Hkv, cfg.L, Dh, tdt, T, dil).to("cuda")
    ocache = oracle.OracleLayerKVCache(B, Hkv, cfg.L, Dh, np.float32, T, dil)   # fp32 container of rounded values
    n_frames = ring + 2
    for t in range(n_frames):
        for step, frozen in ((0, True), (1, False)):
            k, v = frame_kv(cfg, t)
            q = frame_q(cfg, t, step)
            q, k, v = _round(q, dtype), _round(k, dtype), _round(v, dtype)
            pos = {"t_pos": torch.full((B, T), t, dtype=torch.long, device="cuda")}
            out = cache.append_and_attend(torch.from_numpy(q).to("cuda", tdt), torch.from_numpy(k).to("cuda", tdt),
                                          torch.from_numpy(v).to("cuda", tdt), pos, frozen)
            k_full, v_full, mask = ocache.upsert(np.stack([k, v], 0), t, frozen)
            got_kv = cache.kv.float().cpu().numpy()
            assert np.array_equal(got_kv, ocache.kv), f"{name}: kv differs at frame {t} frozen={frozen}"
            assert np.array_equal(cache.written.cpu().numpy(), ocache.written), f"{name}: written, frame {t}"
            want = oracle.frame_attention(q, k_full, v_full, mask)
            mx, mean = helpers.error_stats(out.float().cpu().numpy(), want)
            assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"{name} frame {t}: {mx} {mean}"
    ops.check_status(torch.device("cuda"))
