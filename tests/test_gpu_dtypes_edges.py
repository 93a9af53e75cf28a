"""Cases the golden recordings do not reach: float16 caches (the kernel's second 16-bit type) and the first
frames of a session, when the ring is still empty or partly filled and only the tail frame (plus the few
written slots) is visible.  State bit-exact with LayerKVCache.upsert (src/model/kv_cache.py:126-151), attention
within the tolerance of the fp32 oracle."""
import numpy as np
import pytest
import torch

from oracle import ring_attn_oracle as oracle
from tests import helpers
from world_engine_b200 import B200LayerKVCache, ops
from world_engine_b200.synthetic import StepConfig, frame_kv, frame_q

pytestmark = pytest.mark.gpu


def _f16(x):
    return np.asarray(x, dtype=np.float32).astype(np.float16)


@pytest.mark.parametrize("shape", [
    # name, B, Hq, Hkv, Dh, T, ring_frames, dilation
    ("one_launch_dh128", 2, 4, 2, 128, 128, 3, 1),      # tail of whole 128-key tiles: append fused into the attention
    ("two_launch_dh64", 1, 4, 4, 64, 64, 4, 1),          # ragged tiles: append kernel + attention, keys masked per tile
], ids=lambda s: s[0])
def test_float16_cache_matches_oracle(shape):
    name, B, Hq, Hkv, Dh, T, ring, dil = shape
    cfg = StepConfig(name, B, Hq, Hkv, Dh, T, ring, dil, 0, "f32", 777)
    cache = B200LayerKVCache(B, Hkv, cfg.L, Dh, torch.float16, T, dil).to("cuda")
    ocache = oracle.OracleLayerKVCache(B, Hkv, cfg.L, Dh, np.float16, T, dil)
    for t in range(ring + 3):
        for step, frozen in ((0, True), (1, False)):
            k, v = frame_kv(cfg, t)
            q = frame_q(cfg, t, step)
            q, k, v = _f16(q), _f16(k), _f16(v)
            pos = {"t_pos": torch.full((B, T), t, dtype=torch.long, device="cuda")}
            out = cache.append_and_attend(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(),
                                          torch.from_numpy(v).cuda(), pos, frozen)
            k_full, v_full, mask = ocache.upsert(np.stack([k, v], 0), t, frozen)
            assert cache.kv.cpu().numpy().tobytes() == ocache.kv.tobytes(), f"{name}: kv differs at frame {t}"
            assert np.array_equal(cache.written.cpu().numpy(), ocache.written)
            want = oracle.frame_attention(q.astype(np.float32), k_full.astype(np.float32),
                                          v_full.astype(np.float32), mask)
            mx, mean = helpers.error_stats(out.float().cpu().numpy(), want)
            assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"{name} frame {t}: {mx} {mean}"
    ops.check_status(torch.device("cuda"))


def test_first_frames_of_a_session_at_layer_size():
    """cfg2 geometry from an empty cache: frame 0 sees only itself (256 keys in 2 of 34 tiles), then one more
    slot per frame; the split over CTAs leaves most of them without a single visible tile."""
    cfg = StepConfig("first_frames", 1, 16, 16, 128, 256, 16, 1, 0, "bf16", 99)
    from tests import gpu_helpers as gh
    cache = gh.new_gpu_cache(cfg)
    ocache = helpers.new_oracle_cache(cfg)
    rows = [0, 1, 127, 128, 255]
    heads = [0, 7, 15]
    for t in range(3):
        for step, frozen in ((0, True), (1, False)):
            q, k, v = helpers.step_inputs(cfg, t, step)
            out = cache.append_and_attend(gh.dev_tensor(cfg, q), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v),
                                          gh.pos_ids(cfg, t), frozen)
            kv_new = np.stack([helpers.to_container(cfg, k), helpers.to_container(cfg, v)], 0)
            k_full, v_full, mask = ocache.upsert(kv_new, t, frozen)
            assert int(mask.sum()) == (t + 1) * cfg.T
            assert gh.kv_bytes(cache) == ocache.kv.tobytes()
            assert np.array_equal(cache.written.cpu().numpy(), ocache.written)
            kf = helpers.from_container(cfg, k_full[:1, heads])
            vf = helpers.from_container(cfg, v_full[:1, heads])
            want = oracle.frame_attention(q[:1][:, heads][:, :, rows], kf, vf, mask)
            got = out[:1][:, heads][:, :, rows].float().cpu().numpy()
            mx, mean = helpers.error_stats(got, want)
            assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"frame {t} frozen={frozen}: {mx} {mean}"
            assert torch.isfinite(out.float()).all()
    ops.check_status(torch.device("cuda"))


def test_long_ring_near_the_tile_capacity():
    """65536-token ring (512 frames of 128 tokens) + tail = 513 key tiles for one head: the split over a cluster
    of 8 CTAs with 64 tiles each, half of the documented capacity of 1024 tiles per (row, head).  The ring is
    filled directly (replaying 512 frames would only exercise the append), then two steps are checked."""
    from tests import gpu_helpers as gh
    cfg = StepConfig("long_ring", 1, 2, 1, 128, 128, 512, 1, 512 + 37, "bf16", 123)
    cache = gh.new_gpu_cache(cfg)
    ocache = helpers.new_oracle_cache(cfg)
    g = torch.Generator(device="cuda").manual_seed(4)
    cache.kv.normal_(generator=g)
    cache.written.fill_(True)
    ocache.kv[...] = cache.kv.view(torch.int16).cpu().numpy().view(np.uint16)
    ocache.written[:] = True
    t = cfg.frame_t
    for step, frozen in ((0, True), (1, False)):
        q, k, v = helpers.step_inputs(cfg, t, step)
        out = cache.append_and_attend(gh.dev_tensor(cfg, q), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v),
                                      gh.pos_ids(cfg, t), frozen)
        kv_new = np.stack([helpers.to_container(cfg, k), helpers.to_container(cfg, v)], 0)
        k_full, v_full, mask = ocache.upsert(kv_new, t, frozen)
        assert int(mask.sum()) == cfg.L                      # 511 ring frames + the tail
        assert gh.kv_bytes(cache) == ocache.kv.tobytes()
        assert np.array_equal(cache.written.cpu().numpy(), ocache.written)
        want = oracle.frame_attention(q, helpers.from_container(cfg, k_full), helpers.from_container(cfg, v_full), mask)
        mx, mean = helpers.error_stats(out.float().cpu().numpy(), want)
        assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"step {step}: {mx} {mean}"
    ops.check_status(torch.device("cuda"))
