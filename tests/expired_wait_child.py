"""Child process of tests/test_gpu_expired_wait.py: runs with the debug build of the library (WE_B200_LIB), in
which one wait of the attention kernel can be made to run out on purpose.  Prints one line per check."""
import ctypes
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import numpy as np
import torch

from tests import gpu_helpers as gh
from tests import helpers
from world_engine_b200 import _lib, ops
from world_engine_b200.synthetic import StepConfig


def main() -> int:
    lib = _lib.load()
    lib.we_b200_debug_expire_wait.argtypes = [ctypes.c_int]
    # 2 rows x 32 heads x 2 query tiles = 128 units: no split, hence no cluster and no peer that waits for the CTA
    cfg = StepConfig("expire", 2, 32, 8, 128, 256, 3, 1, 5, "bf16", 515)
    assert lib.we_b200_attn_workspace_bytes(cfg.B, cfg.Hq, cfg.T, cfg.Dh, cfg.L) <= 4096, "shape must not split"
    cache = gh.new_gpu_cache(cfg)
    ocache = helpers.new_oracle_cache(cfg)
    for t in range(cfg.frame_t):
        _, k, v = helpers.step_inputs(cfg, t, 0)
        ops.kv_append_(cache.kv, cache.written, gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v),
                       gh.pos_ids(cfg, t)["t_pos"], cfg.T, 1, False)
        ocache.upsert(np.stack([helpers.to_container(cfg, k), helpers.to_container(cfg, v)], 0), t, False)
    q, k, v = helpers.step_inputs(cfg, cfg.frame_t, 0)
    args = (gh.dev_tensor(cfg, q), gh.dev_tensor(cfg, k), gh.dev_tensor(cfg, v), gh.pos_ids(cfg, cfg.frame_t), True)
    dev = torch.device("cuda")
    cache.append_and_attend(*args)
    torch.cuda.synchronize()
    ops.check_status(dev)
    print("CLEAN_BEFORE ok")

    assert lib.we_b200_debug_expire_wait(1) == 0
    cache.append_and_attend(*args)
    torch.cuda.synchronize()
    assert lib.we_b200_debug_expire_wait(0) == 0
    st = int(ops.status_word(dev).item())
    print("STATUS", st & 0xFF)
    try:
        ops.check_status(dev)
        print("RAISED no")
    except RuntimeError as e:
        print("RAISED yes:", "expired" in str(e))
    print("CLEARED", int(ops.status_word(dev).item()))

    out = cache.append_and_attend(*args)             # the context is intact: the next call is correct
    torch.cuda.synchronize()
    ops.check_status(dev)
    want, _ = helpers.oracle_step(cfg, ocache, cfg.frame_t, 0, True)
    mx, mean = helpers.error_stats(out.float().cpu().numpy(), want)
    print("AFTER", "ok" if (mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL) else f"bad {mx} {mean}")
    assert gh.kv_bytes(cache) == ocache.kv.tobytes()
    print("STATE ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())
