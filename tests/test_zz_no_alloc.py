"""The entry point for hosts that cannot allocate device memory (we_b200_frame_attn_static) must give
what the ordinary entry point gives.  Collected last on purpose: if it fails, a run that stops at the
first failure has already gone through every other test."""
import numpy as np
import pytest
import torch

from tests import helpers
from tests import gpu_helpers as gh
from world_engine_b200 import ops
from world_engine_b200.synthetic import StepConfig

pytestmark = pytest.mark.gpu


def test_no_alloc_entry_point_matches_the_workspace_entry_point_twice():
    # 2 rows x 4 heads x 2 query tiles = 16 units on a 148-SM part -> the KV tiles are split over several
    # CTAs.  Their partial results merge through cluster shared memory where the device can schedule such
    # clusters and through the built-in scratch array otherwise (tests/test_gpu_workspace_merge.py runs this
    # test once more with the merge forced through the array); either way nothing is allocated.
    cfg = StepConfig("noalloc", 2, 4, 4, 128, 256, 3, 1, 4, "bf16", 31337)
    cache = gh.new_gpu_cache(cfg)
    ocache = helpers.new_oracle_cache(cfg)
    for t in range(0, cfg.frame_t + 1):
        _, k, v = helpers.step_inputs(cfg, t, 0)
        ops.kv_append_(cache.kv, cache.written.view(torch.uint8), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v),
                       gh.pos_ids(cfg, t)["t_pos"], cfg.T, cfg.dilation, False)
        ocache.upsert(np.stack([helpers.to_container(cfg, k), helpers.to_container(cfg, v)], 0), t, False)
    lib = ops._lib.load()
    assert lib.we_b200_attn_workspace_bytes(cfg.B, cfg.Hq, cfg.T, cfg.Dh, cfg.L) > 4096   # split-KV plan
    t_pos = gh.pos_ids(cfg, cfg.frame_t)["t_pos"]
    written = cache.written.view(torch.uint8)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for call in range(2):                       # two calls in a row share the array
        q = gh.dev_tensor(cfg, helpers.step_inputs(cfg, cfg.frame_t, call)[0])
        out = torch.full_like(q, float("nan"))
        ops.frame_attn_no_alloc(q, out, status, cache.kv, written, t_pos, cfg.T, cfg.dilation)
        ref = ops.frame_attn(q, cache.kv, written, t_pos, cfg.T, cfg.dilation)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        got, want = out.float().cpu().numpy(), ref.float().cpu().numpy()
        mx, mean = helpers.error_stats(got, want)
        assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"call {call}: max {mx} mean {mean}"
        # and both agree with the CPU oracle (visibility of the last replayed call: slot hidden, tail visible)
        q_host = helpers.step_inputs(cfg, cfg.frame_t, call)[0]
        want_cpu = helpers.oracle.frame_attention(q_host, helpers.from_container(cfg, ocache.kv[0]),
                                                  helpers.from_container(cfg, ocache.kv[1]), ocache.mask_written)
        mx, mean = helpers.error_stats(got, want_cpu)
        assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"call {call} vs oracle: {mx} {mean}"


def test_no_alloc_entry_point_rejects_shapes_beyond_its_scratch():
    import ctypes
    from world_engine_b200._lib import CacheGeom, Strides3
    lib = ops._lib.load()
    # What outgrows the array here is the per-unit arrival counters of a very large batch (a split plan whose
    # partials need more than 12 MiB is rejected the same way when clusters are unavailable).  Nothing is
    # launched: the size check comes first, and should it ever be skipped the null frame counter below makes
    # the launcher refuse the call before any pointer is dereferenced.
    B, Hq, T, Dh, L = 65535, 64, 128, 128, 128 * 4
    need = lib.we_b200_attn_workspace_bytes(B, Hq, T, Dh, L)
    assert need > (12 << 20)
    g = CacheGeom()
    g.B, g.Hkv, g.T, g.Dh, g.L, g.dilation, g.dtype = B, Hq, T, Dh, L, 1, 0
    g.kv_plane_stride = B * Hq * (L + T) * Dh
    g.kv_batch_stride = Hq * (L + T) * Dh
    s = Strides3(Hq * T * Dh, T * Dh, Dh)
    fake = 0x10000
    rc = lib.we_b200_frame_attn_static(fake, s, fake, s, Hq, fake, fake, None, ctypes.byref(g), 0.0, None, None)
    assert rc == -8
    assert b"12 MiB" in lib.we_b200_strerror(rc)
