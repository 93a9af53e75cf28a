"""The one-launch append + attention path (tail made of whole 128-key tiles): the new frame's tiles are read
from k_new / v_new and persisted from the kernel's K / V rings.  Cache bytes and `written` must stay bit-exact
with LayerKVCache.upsert (src/model/kv_cache.py:126-151) over a run of frames that crosses the ring wrap, for
grouped-query heads, several batch rows, both head dims, frozen and unfrozen calls and a dilated ring; the
attention stays within the tolerance of the fp32 oracle."""
import numpy as np
import pytest
import torch

from tests import gpu_helpers as gh
from tests import helpers
from world_engine_b200 import ops
from world_engine_b200.synthetic import StepConfig

pytestmark = pytest.mark.gpu

CASES = [
    # name, B, Hq, Hkv, Dh, T, ring_frames, dilation
    ("gqa_batch", 3, 4, 2, 128, 128, 3, 1),
    ("dh64", 2, 4, 4, 64, 128, 4, 1),
    ("two_tail_tiles_gqa", 1, 8, 2, 128, 256, 3, 1),
    ("dilation2", 2, 2, 2, 128, 128, 4, 2),
    ("long_tail", 2, 16, 8, 128, 512, 2, 1),   # unsplit CTAs: more new-frame tiles than ring stages in one CTA
    # unsplit, two CTAs per kv head: four store jobs per CTA on a persisting step, more than the K ring has stages
    ("many_jobs_per_cta", 20, 4, 4, 128, 256, 3, 1),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_fused_append_keeps_cache_exact_across_the_wrap(case):
    name, B, Hq, Hkv, Dh, T, ring, dil = case
    cfg = StepConfig(name, B, Hq, Hkv, Dh, T, ring, dil, 0, "bf16", 4242)
    assert cfg.T % 128 == 0 and cfg.L % 128 == 0     # the geometry that takes the one-launch path
    cache = gh.new_gpu_cache(cfg)
    ocache = helpers.new_oracle_cache(cfg)
    n_frames = 2 * ring + 2
    for t in range(n_frames):
        # a frozen call first (tail only), then the call that persists the frame
        for step, frozen in ((0, True), (1, False)):
            q, k, v = helpers.step_inputs(cfg, t, step)
            out = cache.append_and_attend(gh.dev_tensor(cfg, q), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v),
                                          gh.pos_ids(cfg, t), frozen)
            want, _ = helpers.oracle_step(cfg, ocache, t, step, frozen)
            assert gh.kv_bytes(cache) == ocache.kv.tobytes(), f"{name}: kv differs at frame {t} frozen={frozen}"
            assert np.array_equal(cache.written.cpu().numpy(), ocache.written), f"{name}: written, frame {t}"
            mx, mean = helpers.error_stats(out.float().cpu().numpy(), want)
            assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, \
                f"{name} frame {t} frozen={frozen}: max {mx} mean {mean}"
    ops.check_status(torch.device("cuda"))
