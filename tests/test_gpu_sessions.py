"""Independent sessions batched in one launch (per-session frame counters and `written` vectors):
each session must match its own oracle cache bit-for-bit and its own oracle attention."""
import numpy as np
import pytest
import torch

from oracle import ring_attn_oracle as oracle
from tests import helpers
from tests import gpu_helpers as gh
from world_engine_b200 import SessionSlab, ops
from world_engine_b200.synthetic import StepConfig, scaled

pytestmark = pytest.mark.gpu


def test_sessions_at_different_wrap_offsets_match_their_own_oracles():
    base = StepConfig("sess", 1, 4, 2, 128, 128, 3, 1, 0, "bf16", 4242)
    frame_ts = [0, 1, 2, 5, 9, 4, 7]                       # pre-wrap, just wrapped, wrapped at every slot
    S = len(frame_ts)
    cfgs = [scaled(base, seed=base.seed + i, frame_t=t) for i, t in enumerate(frame_ts)]
    slab = SessionSlab(S, base.Hkv, base.L, base.Dh, torch.bfloat16, base.T)
    ocaches = [helpers.new_oracle_cache(c) for c in cfgs]
    # history: every session replays its own frames 0..t-1 unfrozen, through its reference-layout view
    for i, c in enumerate(cfgs):
        for f in range(c.frame_t):
            _, k, v = helpers.step_inputs(c, f, 0)
            ocaches[i].upsert(np.stack([helpers.to_container(c, k), helpers.to_container(c, v)], 0), f, False)
            ops.kv_append_(slab.session_kv(i), slab.session_written(i).view(torch.uint8), gh.dev_tensor(c, k),
                           gh.dev_tensor(c, v), torch.tensor([f], device="cuda"), c.T, 1, False)
    slab.frame_t.copy_(torch.tensor(frame_ts, device="cuda"))
    # the step under test: all sessions in ONE launch, first frozen then unfrozen
    for frozen in (True, False):
        qs, ks, vs, wants = [], [], [], []
        for i, c in enumerate(cfgs):
            q, k, v = helpers.step_inputs(c, c.frame_t, 0 if frozen else 1)
            qs.append(q[0]); ks.append(k[0]); vs.append(v[0])
            want, _ = helpers.oracle_step(c, ocaches[i], c.frame_t, 0 if frozen else 1, frozen)
            wants.append(want[0])
        q = gh.dev_tensor(base, np.stack(qs)); k = gh.dev_tensor(base, np.stack(ks)); v = gh.dev_tensor(base, np.stack(vs))
        out = slab.append_and_attend(q, k, v, frozen).float().cpu().numpy()
        for i, c in enumerate(cfgs):
            kv = slab.session_kv(i).contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            assert kv.tobytes() == ocaches[i].kv.tobytes(), f"session {i} cache differs (frozen={frozen})"
            assert np.array_equal(slab.session_written(i).cpu().numpy(), ocaches[i].written), f"session {i} written"
            mx, mean = helpers.error_stats(out[i], wants[i])
            assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"session {i}: max {mx} mean {mean}"
    ops.check_status(torch.device("cuda"))
