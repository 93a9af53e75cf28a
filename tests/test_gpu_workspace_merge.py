"""The split merge through the caller's workspace (partials in global memory, arrival ticket, last CTA merges)
is the path a device takes on which thread-block clusters of the split count cannot be scheduled.  A B200 can
always schedule them, so the library is told to answer "clusters unavailable"
(WE_B200_FORCE_WORKSPACE_MERGE, read on every call) and the parity tests of the other files are run again
through that path: the recorded cases of the reference, the gated output on every store path, float16 caches,
random geometries, and the entry point that keeps its scratch in the library image."""
import numpy as np
import pytest
import torch

from tests import gpu_helpers as gh
from tests import helpers
from tests import test_gpu_dtypes_edges, test_gpu_gate, test_gpu_parity, test_zz_no_alloc
from world_engine_b200 import ops
from world_engine_b200.synthetic import StepConfig

pytestmark = pytest.mark.gpu


@pytest.fixture
def workspace_merge(monkeypatch):
    monkeypatch.setenv("WE_B200_FORCE_WORKSPACE_MERGE", "1")
    yield


def test_the_switch_changes_the_path(monkeypatch):
    """Same inputs through both merges: equal within the tolerance, and not bit-identical (the cluster merge
    exchanges fp16 rows, the workspace merge fp32 rows) -- which shows the switch is honoured."""
    cfg = StepConfig("switch", 1, 4, 4, 128, 256, 8, 1, 11, "bf16", 777)      # 8 units -> 8 splits
    cache = gh.new_gpu_cache(cfg)
    cache.kv.normal_(generator=torch.Generator(device="cuda").manual_seed(3))
    cache.written.fill_(True)
    q = gh.dev_tensor(cfg, helpers.step_inputs(cfg, cfg.frame_t, 0)[0])
    pos = gh.pos_ids(cfg, cfg.frame_t)
    a = cache.attend(q, pos).float()
    monkeypatch.setenv("WE_B200_FORCE_WORKSPACE_MERGE", "1")
    b = cache.attend(q, pos).float()
    b2 = cache.attend(q, pos).float()
    monkeypatch.setenv("WE_B200_FORCE_WORKSPACE_MERGE", "0")
    c = cache.attend(q, pos).float()
    assert torch.equal(b, b2) and torch.equal(a, c)             # each path is deterministic
    assert (a - b).abs().max().item() <= 4e-3
    assert not torch.equal(a, b)
    ops.check_status(torch.device("cuda"))


@pytest.mark.parametrize("case", helpers.GOLDEN_CASES)
def test_recorded_cases_through_the_workspace_merge(workspace_merge, case):
    test_gpu_parity.test_append_and_attend_matches_oracle_and_recording(case)


@pytest.mark.parametrize("case", test_gpu_gate.CASES, ids=[c[0] for c in test_gpu_gate.CASES])
def test_gated_output_through_the_workspace_merge(workspace_merge, case):
    test_gpu_gate.test_gated_output(case, True)


@pytest.mark.parametrize("shape", [("one_launch_dh128", 2, 4, 2, 128, 128, 3, 1), ("two_launch_dh64", 1, 4, 4, 64, 64, 4, 1)],
                         ids=lambda s: s[0])
def test_float16_caches_through_the_workspace_merge(workspace_merge, shape):
    test_gpu_dtypes_edges.test_float16_cache_matches_oracle(shape)


def test_first_frames_and_long_ring_through_the_workspace_merge(workspace_merge):
    test_gpu_dtypes_edges.test_first_frames_of_a_session_at_layer_size()     # most CTAs of a split find no tile
    test_gpu_dtypes_edges.test_long_ring_near_the_tile_capacity()            # 8 splits of 64 tiles


@pytest.mark.parametrize("shape", [
    # name, B, Hq, Hkv, Dh, T, ring frames: split counts 2, 4, 8; both head dims; a frame that is no multiple of 128
    ("ns2", 2, 8, 4, 128, 256, 6),
    ("ns4_dh64", 1, 16, 16, 64, 256, 12),
    ("ns8_ragged", 1, 2, 1, 128, 200, 12),
    ("ns8_dh64", 1, 4, 4, 64, 128, 30),
], ids=lambda s: s[0])
def test_split_counts_and_head_dims_through_the_workspace_merge(workspace_merge, shape):
    name, B, Hq, Hkv, Dh, T, ring = shape
    cfg = StepConfig(name, B, Hq, Hkv, Dh, T, ring, 1, ring + 3, "bf16", 9090)
    cache = gh.new_gpu_cache(cfg)
    ocache = helpers.new_oracle_cache(cfg)
    for f in range(cfg.frame_t - ring, cfg.frame_t):
        _, k, v = helpers.step_inputs(cfg, f, 0)
        ops.kv_append_(cache.kv, cache.written.view(torch.uint8), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v),
                       gh.pos_ids(cfg, f)["t_pos"], T, 1, False)
        ocache.upsert(np.stack([helpers.to_container(cfg, k), helpers.to_container(cfg, v)], 0), f, False)
    q, k, v = helpers.step_inputs(cfg, cfg.frame_t, 0)
    args = (gh.dev_tensor(cfg, q), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v), gh.pos_ids(cfg, cfg.frame_t), True)
    outs = [cache.append_and_attend(*args) for _ in range(2)]
    assert torch.equal(outs[0], outs[1])                            # the merge order is fixed: reruns are bit-identical
    want, _ = helpers.oracle_step(cfg, ocache, cfg.frame_t, 0, True)
    assert gh.kv_bytes(cache) == ocache.kv.tobytes()
    mx, mean = helpers.error_stats(outs[0].float().cpu().numpy(), want)
    assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"{name}: max {mx} mean {mean}"
    ops.check_status(torch.device("cuda"))


def test_no_alloc_entry_point_through_its_scratch_array(workspace_merge):
    """we_b200_frame_attn_static with the merge forced through the 12 MiB array of the library image: address
    look-up, counter clearing and the last-arriver merge all execute; two calls in a row, against the ordinary
    entry point and the oracle."""
    test_zz_no_alloc.test_no_alloc_entry_point_matches_the_workspace_entry_point_twice()
