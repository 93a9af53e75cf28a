"""The oracle's restatement of the q/k/v prologue (weightless RMS norm, RoPE rotation, value residual) against
recordings of the reference's own code (tests/golden/make_golden_prologue.py): bit-exact in bf16."""
import json
import os

import numpy as np
import pytest

from oracle import ring_attn_oracle as oracle
from tests.helpers import GOLDEN_DIR

PROLOGUE_CASES = ["prologue_dh64", "prologue_dh128_gqa", "prologue_no_residual"]


def load_prologue(name):
    z = np.load(os.path.join(GOLDEN_DIR, f"{name}.npz"))
    meta = json.loads(bytes(z["meta"]).decode())
    return meta, z


@pytest.mark.parametrize("name", PROLOGUE_CASES)
def test_prologue_oracle_reproduces_the_reference_bit_for_bit(name):
    meta, z = load_prologue(name)
    f = oracle.bf16_bits_to_f32
    cos, sin = oracle.rope_angles(z["cos"], z["sin"], z["t_pos"], z["y_pos"], z["x_pos"], meta["height"], meta["width"])
    lamb = meta["lamb"]
    if lamb is not None:
        lamb = float(oracle.round_to_bf16(np.float32(lamb)))        # the parameter is a bf16 tensor in the recording
    q, k, v = oracle.qkv_prologue(f(z["q"]), f(z["k"]), f(z["v"]), None if lamb is None else f(z["v1"]), lamb, cos, sin)
    assert np.array_equal(oracle.f32_to_bf16_bits(q), z["q_out"])
    assert np.array_equal(oracle.f32_to_bf16_bits(k), z["k_out"])
    assert np.array_equal(oracle.f32_to_bf16_bits(v), z["v_out"])


def test_positions_outside_the_table_are_rejected():
    meta, z = load_prologue("prologue_dh64")
    with pytest.raises(IndexError):
        oracle.rope_angles(z["cos"], z["sin"], z["t_pos"] + 100, z["y_pos"], z["x_pos"], meta["height"], meta["width"])
