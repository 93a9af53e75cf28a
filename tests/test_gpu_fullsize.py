"""Full-size configurations on the GPU: parity with the oracle on a subset of rows (the oracle finishes in
seconds on those) plus size-independent properties of the operation on the whole output."""
import numpy as np
import pytest
import torch

from oracle import ring_attn_oracle as oracle
from tests import helpers
from tests import gpu_helpers as gh
from world_engine_b200 import ops
from world_engine_b200.synthetic import CONFIGS, frame_kv, frame_q, history_frames

pytestmark = pytest.mark.gpu

ROWS = [0, 1, 63, 64, 127, 128, 200, -1]


def _fill(cfg):
    """Replays the frames that determine the cache state at cfg.frame_t on the GPU and in the oracle."""
    cache = gh.new_gpu_cache(cfg)
    ocache = helpers.new_oracle_cache(cfg)
    for f in history_frames(cfg):
        _, k, v = helpers.step_inputs(cfg, f, 0)
        ops.kv_append_(cache.kv, cache.written.view(torch.uint8), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v),
                       gh.pos_ids(cfg, f)["t_pos"], cfg.T, cfg.dilation, False)
        ocache.upsert(np.stack([helpers.to_container(cfg, k), helpers.to_container(cfg, v)], 0), f, False)
    return cache, ocache


@pytest.mark.parametrize("name", ["cfg2", "cfg4_session", "cfg5"])
def test_fullsize_step_matches_oracle_on_row_subset_and_keeps_state_exact(name):
    cfg = CONFIGS[name]
    cache, ocache = _fill(cfg)
    t = cfg.frame_t
    for step, frozen in ((0, True), (1, False)):
        q, k, v = helpers.step_inputs(cfg, t, step)
        out = cache.append_and_attend(gh.dev_tensor(cfg, q), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v),
                                      gh.pos_ids(cfg, t), frozen)
        kv_new = np.stack([helpers.to_container(cfg, k), helpers.to_container(cfg, v)], 0)
        k_full, v_full, mask = ocache.upsert(kv_new, t, frozen)
        assert int(mask.sum()) == cfg.visible_keys()
        assert gh.kv_bytes(cache) == ocache.kv.tobytes(), "cache contents differ"
        assert np.array_equal(cache.written.cpu().numpy(), ocache.written)
        rows = sorted({r % cfg.T for r in ROWS})
        heads = sorted({0, cfg.Hq // 2, cfg.Hq - 1})
        kv_heads = [h * cfg.Hkv // cfg.Hq for h in heads]
        for b in range(cfg.B):                      # every batch row, a subset of query rows and heads of each
            kf = helpers.from_container(cfg, k_full[b:b + 1, kv_heads])
            vf = helpers.from_container(cfg, v_full[b:b + 1, kv_heads])
            want = oracle.frame_attention(q[b:b + 1][:, heads][:, :, rows], kf, vf, mask)
            got = out[b:b + 1][:, heads][:, :, rows].float().cpu().numpy()
            mx, mean = helpers.error_stats(got, want)
            assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, \
                f"{name} step {step} batch row {b}: max {mx} mean {mean}"
        assert torch.isfinite(out.float()).all()
    ops.check_status(torch.device("cuda"))


def test_slab_of_64_sessions_at_random_wrap_offsets():
    """The throughput configuration as the benchmark runs it: 64 sessions with 32-frame rings (8192 keys) in one
    slab, every session at its own frame counter, one launch per layer-step.  Three sessions (first, middle,
    last) are followed in the oracle: cache bytes and `written` bit-exact after a frozen and a persisting call,
    attention on a subset of rows and heads.  The rings are filled directly (replaying 64 x 32 frames would
    only exercise the append)."""
    from world_engine_b200 import SessionSlab
    from world_engine_b200.synthetic import scaled
    base = CONFIGS["cfg4_session"]
    S = 64
    gen = torch.Generator(device="cuda").manual_seed(5)
    slab = SessionSlab(S, base.Hkv, base.L, base.Dh, torch.bfloat16, base.T)
    slab._slab.normal_(generator=gen)
    slab._written.fill_(True)
    frame_ts = (32 + torch.randint(0, 10000, (S,), device="cuda", generator=gen)).tolist()
    slab.frame_t.copy_(torch.tensor(frame_ts, device="cuda"))
    followed = [0, 31, 63]
    cfgs = {i: scaled(base, seed=base.seed + i, frame_t=frame_ts[i]) for i in range(S)}
    ocaches = {}
    for i in followed:
        oc = helpers.new_oracle_cache(cfgs[i])
        oc.kv[...] = slab.session_kv(i).contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
        oc.written[:] = True
        ocaches[i] = oc
    rows = sorted({r % base.T for r in ROWS})
    heads = sorted({0, base.Hq // 2, base.Hq - 1})
    for step, frozen in ((0, True), (1, False)):
        qs, ks, vs = [], [], []
        for i in range(S):
            q, k, v = helpers.step_inputs(cfgs[i], frame_ts[i], step)
            qs.append(q[0]); ks.append(k[0]); vs.append(v[0])
        qd, kd, vd = (gh.dev_tensor(base, np.stack(x)) for x in (qs, ks, vs))
        out = slab.append_and_attend(qd, kd, vd, frozen)
        assert torch.isfinite(out.float()).all()
        for i in followed:
            c = cfgs[i]
            kv_new = np.stack([helpers.to_container(c, ks[i][None]), helpers.to_container(c, vs[i][None])], 0)
            k_full, v_full, mask = ocaches[i].upsert(kv_new, frame_ts[i], frozen)
            assert int(mask.sum()) == c.visible_keys()
            kv = slab.session_kv(i).contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
            assert kv.tobytes() == ocaches[i].kv.tobytes(), f"session {i}: cache differs (frozen={frozen})"
            assert np.array_equal(slab.session_written(i).cpu().numpy(), ocaches[i].written)
            kf = helpers.from_container(c, k_full[:1, heads])
            vf = helpers.from_container(c, v_full[:1, heads])
            want = oracle.frame_attention(qs[i][None][:, heads][:, :, rows], kf, vf, mask)
            got = out[i:i + 1][:, heads][:, :, rows].float().cpu().numpy()
            mx, mean = helpers.error_stats(got, want)
            assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"session {i} step {step}: {mx} {mean}"
    ops.check_status(torch.device("cuda"))


def test_properties_at_full_size():
    """cfg2 shape: (1) constant V gives that constant; (2) the output is linear in V; (3) the slot a frame sits
    in does not matter (keys are a set): shifting the whole history by one ring slot leaves the output unchanged
    up to summation order."""
    cfg = CONFIGS["cfg2"]
    cache, _ = _fill(cfg)
    t = cfg.frame_t
    q, k, v = helpers.step_inputs(cfg, t, 0)
    qd, kd, vd = gh.dev_tensor(cfg, q), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v)
    pos = gh.pos_ids(cfg, t)
    base = cache.append_and_attend(qd, kd, vd, pos, True).float()
    # (1) convexity: all V rows equal to c  ->  output equals c
    saved_v = cache.kv[1].clone()
    cache.kv[1].fill_(0.75)
    const = cache.append_and_attend(qd, kd, torch.full_like(vd, 0.75), pos, True).float()
    assert torch.allclose(const, torch.full_like(const, 0.75), atol=4e-3)
    # (2) linearity in V: out(V) - out(0.5 V) == out(0.5 V)   (0.5 V is exact in bf16)
    cache.kv[1].copy_(saved_v * 0.5)
    half = cache.append_and_attend(qd, kd, vd * 0.5, pos, True).float()
    assert (base - 2 * half).abs().max().item() <= 2e-2 * max(1.0, base.abs().max().item())
    assert (base - 2 * half).abs().mean().item() <= 1e-3
    # (3) permutation of ring slots: the same frame data persisted one slot later and queried one frame later
    #     leaves the same set of visible keys (the hidden slot again holds the oldest frame)
    cache.kv[1].copy_(saved_v)
    from dataclasses import replace
    cfg_b = replace(cfg, frame_t=t + 1)
    cache_b = gh.new_gpu_cache(cfg_b)
    for f in history_frames(cfg):
        _, kf, vf = helpers.step_inputs(cfg, f, 0)
        ops.kv_append_(cache_b.kv, cache_b.written.view(torch.uint8), gh.dev_tensor(cfg, kf), gh.dev_tensor(cfg, vf),
                       gh.pos_ids(cfg, f + 1)["t_pos"], cfg.T, cfg.dilation, False)
    shifted = cache_b.append_and_attend(qd, kd, vd, gh.pos_ids(cfg_b, t + 1), True).float()
    assert (shifted - base).abs().max().item() <= 8e-3      # only the summation order differs
    ops.check_status(torch.device("cuda"))


def test_denoise_protocol_over_twenty_frames_at_layer_size():
    """The call sequence of WorldEngine._denoise_pass / _cache_pass (src/world_engine.py:139-152) on one layer
    cache of the cfg3 shape: per frame four frozen steps, then one unfrozen step that persists the frame, for
    21 consecutive frames, so every ring slot is overwritten at least once.  The cache must equal the oracle's
    after every frame; the attention of the last frozen step and of the persisting step of selected frames is
    compared on a subset of rows and heads."""
    cfg = CONFIGS["cfg3_layer"]
    cache, ocache = _fill(cfg)
    rows = sorted({r % cfg.T for r in ROWS})
    heads = sorted({0, cfg.Hq // 2, cfg.Hq - 1})
    checked = {cfg.frame_t, cfg.frame_t + 7, cfg.frame_t + 20}
    for t in range(cfg.frame_t, cfg.frame_t + 21):
        _, k, v = helpers.step_inputs(cfg, t, 0)          # K/V of a frame are the same at every step of it
        kd, vd = gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v)
        kv_new = np.stack([helpers.to_container(cfg, k), helpers.to_container(cfg, v)], 0)
        pos = gh.pos_ids(cfg, t)
        for step in range(5):
            frozen = step < 4
            q = frame_q(cfg, t, step)
            q = oracle.round_to_bf16(q)
            out = cache.append_and_attend(gh.dev_tensor(cfg, q), kd, vd, pos, frozen)
            k_full, v_full, mask = ocache.upsert(kv_new, t, frozen)
            if t in checked and step >= 3:
                assert int(mask.sum()) == cfg.visible_keys()
                kf = helpers.from_container(cfg, k_full[:1, [h * cfg.Hkv // cfg.Hq for h in heads]])
                vf = helpers.from_container(cfg, v_full[:1, [h * cfg.Hkv // cfg.Hq for h in heads]])
                want = oracle.frame_attention(q[:1][:, heads][:, :, rows], kf, vf, mask)
                got = out[:1][:, heads][:, :, rows].float().cpu().numpy()
                mx, mean = helpers.error_stats(got, want)
                assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, f"frame {t} step {step}: {mx} {mean}"
        assert gh.kv_bytes(cache) == ocache.kv.tobytes(), f"cache differs after frame {t}"
        assert np.array_equal(cache.written.cpu().numpy(), ocache.written)
    ops.check_status(torch.device("cuda"))
