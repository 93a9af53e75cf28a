"""The torch restatement of the reference's CPU code path (oracle/torch_eager_path.py, used by the CPU-baseline
legs of the benchmark) against the numpy oracle and the reference recordings: cache bytes and `written` bit-exact,
attention within fp32 summation order."""
import numpy as np
import pytest
import torch

from oracle import ring_attn_oracle as oracle
from oracle import torch_eager_path as tep
from tests import helpers


@pytest.mark.parametrize("case", ["cfg1", "cfg1_prewrap", "dilation2"])
def test_torch_eager_path_matches_the_oracle_and_the_recordings(case):
    cfg, meta, z = helpers.load_golden(case)
    assert cfg.dtype == "f32"
    tcache = tep.TorchLayerKVCache(cfg.B, cfg.Hkv, cfg.L, cfg.Dh, torch.float32, cfg.T, cfg.dilation)
    ocache = helpers.new_oracle_cache(cfg)
    for ci, call in enumerate(meta["calls"]):
        t, step, frozen = call["frame_t"], call["step"], call["is_frozen"]
        q, k, v = helpers.step_inputs(cfg, t, step)
        got = tep.layer_step(tcache, torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v), t, frozen)
        want, _ = helpers.oracle_step(cfg, ocache, t, step, frozen, want_out=True)
        assert tcache.kv.numpy().tobytes() == ocache.kv.tobytes(), f"kv differs after call {ci}"
        assert helpers.kv_digest(tcache.kv.numpy()) == call["kv_sha256"]
        assert np.array_equal(tcache.written.numpy(), ocache.written)
        mx, _ = helpers.error_stats(got.numpy(), want)
        assert mx <= 2e-5, f"call {ci}: {mx}"
