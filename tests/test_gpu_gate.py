"""The head gate applied inside the attention kernel (we_b200_append_attend_gated): out = attention * sigmoid(logit)
per (batch row, head, token), src/model/attn.py:116-119.  Compared with the un-gated kernel's output times the
gate computed by torch in fp32 (the kernel rounds once, the reference twice: a last-place difference at most), and
with the oracle's attention times the same gate.  Shapes: no split, splits merged through the cluster, many
splits, queries past the end of the last tile (the merge through the workspace is covered by
tests/test_gpu_workspace_merge.py, which runs these cases again)."""
import numpy as np
import pytest
import torch

from oracle import ring_attn_oracle as oracle
from tests import gpu_helpers as gh
from tests import helpers
from world_engine_b200 import ops
from world_engine_b200.synthetic import StepConfig

pytestmark = pytest.mark.gpu

CASES = [
    # name, B, Hq, Hkv, Dh, T, ring_frames
    ("split4_layer_shape", 1, 16, 16, 128, 256, 16),
    ("unsplit_many_heads", 4, 64, 32, 128, 128, 3),
    ("split8_one_head", 1, 1, 1, 128, 128, 15),
    ("ragged_dh64", 2, 4, 2, 64, 96, 4),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
@pytest.mark.parametrize("logits", [True, False], ids=["sigmoid_of_logits", "plain_factor"])
def test_gated_output(case, logits):
    name, B, Hq, Hkv, Dh, T, ring = case
    cfg = StepConfig(name, B, Hq, Hkv, Dh, T, ring, 1, ring + 2, "bf16", 606)
    caches = [gh.new_gpu_cache(cfg) for _ in range(2)]
    for c in caches:
        c.kv.normal_(generator=torch.Generator(device="cuda").manual_seed(1))
        c.written.fill_(True)
    caches[1].kv.copy_(caches[0].kv)
    q, k, v = helpers.step_inputs(cfg, cfg.frame_t, 0)
    qd, kd, vd = gh.dev_tensor(cfg, q), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v)
    g = torch.Generator(device="cuda").manual_seed(2)
    raw = (torch.randn(B, T, Hq, device="cuda", generator=g) * 2).bfloat16()      # [B,T,H] like gate_proj's output
    gate_view = raw.permute(0, 2, 1)                                               # [B,H,T], strided
    pos = gh.pos_ids(cfg, cfg.frame_t)
    plain = caches[0].append_and_attend(qd, kd, vd, pos, False).float()
    gated = caches[1].append_and_attend(qd, kd, vd, pos, False, gate=gate_view, gate_is_logits=logits).float()
    factor = torch.sigmoid(gate_view.float()).bfloat16().float() if logits else gate_view.float()
    want = plain * factor.unsqueeze(-1)
    err = (gated - want).abs()
    bound = 2 ** -7 * want.abs().clamp_min(1e-3) + 1e-6          # one bf16 unit in the last place of the product, twice
    assert bool((err <= 2 * bound).all()), f"{name}: max excess {(err - 2 * bound).max().item()}"
    assert torch.equal(caches[0].kv.view(torch.int16), caches[1].kv.view(torch.int16))
    assert torch.equal(caches[0].written, caches[1].written)
    # against the oracle: its fp32 attention over the cache as it was (every ring frame written, this frame's slot
    # hidden, the new frame in the tail), times the gate rounded to bf16 as the reference's `gates` tensor is
    kv_host = caches[0].kv.float().cpu().numpy()
    mask = np.ones(cfg.capacity, dtype=bool)
    slot = (cfg.frame_t % ring) * T
    mask[slot:slot + T] = False
    want_cpu = oracle.frame_attention(q, kv_host[0], kv_host[1], mask) * factor.unsqueeze(-1).cpu().numpy()
    # the attention's error budget is absolute; a plain factor is not bounded by 1 like a sigmoid and scales it
    widen = max(1.0, float(factor.abs().max()))
    mx, mean = helpers.error_stats(gated.cpu().numpy(), want_cpu)
    assert mx <= widen * helpers.MAX_ABS_TOL and mean <= widen * helpers.MEAN_ABS_TOL, \
        f"{name} vs oracle: max {mx} mean {mean} (factor up to {widen})"
    ops.check_status(torch.device("cuda"))
