"""The fused q/k/v prologue kernel (value residual + weightless RMS norm + RoPE) through the C ABI: against the
recordings of the reference's own code, and against the oracle on the layer-sized shape with the strided
merged-QKV views the module hands it.  bf16 results may differ from the reference in the last place on a handful of elements (the fp32 sum of squares
is reduced in another order); nothing more."""
import numpy as np
import pytest
import torch

from oracle import ring_attn_oracle as oracle
from tests.test_oracle_prologue import PROLOGUE_CASES, load_prologue
from world_engine_b200 import ops

pytestmark = pytest.mark.gpu


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).cuda()


def _close(got: torch.Tensor, want: torch.Tensor, what: str):
    """Equal except for a handful of elements: a row whose fp32 sum of squares rounds differently can move the
    normalised values by one bf16 unit in the last place (2^-6 at the magnitudes a unit-RMS row reaches), and
    the rotation combines two of them."""
    d = (got.float() - want.float()).abs()
    assert float(d.max()) <= 2 ** -5, f"{what}: max difference {float(d.max())}"
    assert float((d > 0).float().mean()) <= 2e-3, f"{what}: too many elements differ"


@pytest.mark.parametrize("name", PROLOGUE_CASES)
def test_prologue_kernel_against_reference_recordings(name):
    meta, z = load_prologue(name)
    lamb = meta["lamb"]
    v1 = _bf16(z["v1"]) if lamb is not None else None
    w = torch.tensor(lamb, dtype=torch.bfloat16, device="cuda") if lamb is not None else None
    q, k, v = ops.qkv_prologue(_bf16(z["q"]), _bf16(z["k"]), _bf16(z["v"]), v1, w,
                               torch.from_numpy(z["cos"]).cuda(), torch.from_numpy(z["sin"]).cuda(),
                               torch.from_numpy(z["t_pos"]).cuda(), torch.from_numpy(z["y_pos"]).cuda(),
                               torch.from_numpy(z["x_pos"]).cuda(), meta["height"], meta["width"])
    _close(q, _bf16(z["q_out"]), "q")
    _close(k, _bf16(z["k_out"]), "k")
    assert torch.equal(v.contiguous().view(torch.int16), _bf16(z["v_out"]).view(torch.int16)), "v (lerp) must be exact"
    ops.check_status(torch.device("cuda"))


def test_prologue_on_merged_qkv_views_at_layer_size():
    """cfg2 layer shape: q, k, v are slices of one [B, T, (Hq + 2 Hkv) Dh] projection output viewed as
    [B, H, T, Dh] (src/patch_model.py:117-122); fp32 tables of 16 x 16 positions x 3 frames."""
    B, T, Hq, Hkv, Dh, Hh, Ww = 1, 256, 16, 16, 128, 16, 16
    g = torch.Generator(device="cuda").manual_seed(5)
    qkv = (torch.randn(B, T, (Hq + 2 * Hkv) * Dh, device="cuda", generator=g) * 1.5).bfloat16()
    q, k, v = qkv.split((Hq * Dh, Hkv * Dh, Hkv * Dh), dim=-1)
    q = q.reshape(B, T, Hq, Dh).transpose(1, 2)
    k = k.reshape(B, T, Hkv, Dh).transpose(1, 2)
    v = v.reshape(B, T, Hkv, Dh).transpose(1, 2)
    v1 = torch.randn(B, Hkv, T, Dh, device="cuda", generator=g).bfloat16()
    lamb = torch.tensor(0.625, dtype=torch.bfloat16, device="cuda")
    ang = torch.rand(3 * Hh * Ww, Dh // 2, device="cuda", generator=g) * 6.28 - 3.14
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    yy, xx = torch.meshgrid(torch.arange(Hh, device="cuda"), torch.arange(Ww, device="cuda"), indexing="ij")
    t_pos = torch.full((B, T), 2, dtype=torch.long, device="cuda")
    y_pos, x_pos = yy.reshape(1, T).contiguous(), xx.reshape(1, T).contiguous()
    qo, ko, vo = ops.qkv_prologue(q, k, v, v1, lamb, cos, sin, t_pos, y_pos, x_pos, Hh, Ww)
    c, s = oracle.rope_angles(cos.cpu().numpy(), sin.cpu().numpy(), t_pos.cpu().numpy(), y_pos.cpu().numpy(),
                              x_pos.cpu().numpy(), Hh, Ww)
    wq, wk, wv = oracle.qkv_prologue(q.float().cpu().numpy(), k.float().cpu().numpy(), v.float().cpu().numpy(),
                                     v1.float().cpu().numpy(), 0.625, c, s)
    _close(qo, torch.from_numpy(wq).bfloat16().cuda(), "q")
    _close(ko, torch.from_numpy(wk).bfloat16().cuda(), "k")
    assert torch.equal(vo.float().cpu(), torch.from_numpy(wv)), "v (lerp) must be exact"
    # the outputs have the memory order of the merged-QKV slices: [B, T, H, Dh]
    assert qo.transpose(1, 2).is_contiguous() and ko.transpose(1, 2).is_contiguous()
    ops.check_status(torch.device("cuda"))


def test_position_outside_the_table_is_reported_not_faulted():
    meta, z = load_prologue("prologue_no_residual")
    t_far = torch.from_numpy(z["t_pos"]).cuda() + 1000
    ops.qkv_prologue(_bf16(z["q"]), _bf16(z["k"]), _bf16(z["v"]), None, None,
                     torch.from_numpy(z["cos"]).cuda(), torch.from_numpy(z["sin"]).cuda(),
                     t_far, torch.from_numpy(z["y_pos"]).cuda(), torch.from_numpy(z["x_pos"]).cuda(),
                     meta["height"], meta["width"])
    with pytest.raises(RuntimeError, match="outside the RoPE table"):
        ops.check_status(torch.device("cuda"))
    ops.check_status(torch.device("cuda"))      # the word was cleared
