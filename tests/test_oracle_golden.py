"""Pins the CPU oracle to the reference: replays every golden call sequence
(recorded by running the reference's LayerKVCache.upsert + flex_attention, see
tests/golden/make_golden.py) through the oracle and compares cache state,
indices and masks bit-for-bit and attention outputs in fp32."""
import numpy as np
import pytest

from oracle import ring_attn_oracle as oracle
from tests import helpers


@pytest.mark.parametrize("case", helpers.GOLDEN_CASES)
def test_oracle_matches_reference_recording(case):
    cfg, meta, z = helpers.load_golden(case)
    cache = helpers.new_oracle_cache(cfg)
    rows = meta["subsample_rows"]
    for ci, call in enumerate(meta["calls"]):
        out, mask = helpers.oracle_step(cfg, cache, call["frame_t"], call["step"], call["is_frozen"],
                                        want_out=call["recorded"])
        # cache contents, written flags and visibility: bit-exact
        assert helpers.kv_digest(cache.kv) == call["kv_sha256"], f"kv differs after call {ci}"
        assert np.array_equal(cache.written, z[f"written_{ci}"]), f"written differs after call {ci}"
        assert np.array_equal(mask, z[f"mask_{ci}"]), f"mask differs at call {ci}"
        # block-mask index tables: bit-exact
        tables = oracle.block_mask_tables(cfg.T, cfg.capacity, mask)
        for got, key in zip(tables, ("kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices")):
            want = z[f"{key}_{ci}"]
            assert got.dtype == want.dtype and got.shape == want.shape
            assert np.array_equal(got, want), f"{key} differs at call {ci}"
        if call["recorded"]:
            want = z[f"out_{ci}"]
            got = out[:, :, rows, :] if rows else out
            mx, mean = helpers.error_stats(got, want)
            # both sides are fp32 on identical inputs; only summation order differs
            assert mx < 2e-5 and mean < 2e-6, f"call {ci}: max {mx} mean {mean}"


def test_slot_arithmetic_matches_recorded_writes():
    """The slot a frame is persisted to is visible in the recorded `written` vectors."""
    cfg, meta, z = helpers.load_golden("dilation2")
    prev = np.zeros(cfg.capacity, dtype=bool)
    prev[cfg.L:] = True
    for ci, call in enumerate(meta["calls"]):
        w = z[f"written_{ci}"]
        _, slot, base, write_step = oracle.slot_arithmetic(call["frame_t"], cfg.T, cfg.L, cfg.dilation)
        expect = prev.copy()
        if not call["is_frozen"] and write_step:
            expect[base:base + cfg.T] = True
        assert np.array_equal(w, expect)
        assert slot < (cfg.ring_frames // cfg.dilation)   # only the first num_buckets slots are ever used
        prev = w


def test_bf16_rounding_helper_matches_torch():
    import torch
    x = np.random.default_rng(0).standard_normal(100000, dtype=np.float32) * 37.0
    x[:4] = [0.0, -0.0, np.inf, -np.inf]
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16_bits(x), want)
    assert np.array_equal(oracle.bf16_bits_to_f32(want), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_visible_key_count_formula():
    for case in helpers.GOLDEN_CASES:
        cfg, meta, z = helpers.load_golden(case)
        last = len(meta["calls"]) - 1
        assert meta["calls"][last]["frame_t"] == cfg.frame_t
        assert int(z[f"mask_{last}"].sum()) == cfg.visible_keys()
