"""A whole generated frame under CUDA-graph replay, the way the reference runs it (src/world_engine.py:139-152:
`_denoise_pass` for every scheduler step with the cache frozen, then `_cache_pass` with the cache unfrozen, both
compiled with mode="max-autotune", i.e. replayed as CUDA graphs, with the frame index staying on the device,
src/model/kv_cache.py:126).  One graph holds the frame's layer-steps of a three-layer cache (one layer with the
global window and a pinned dilation) -- four frozen passes, one persisting pass -- and the increment of the
device-resident frame counter.  It is replayed for more frames than the longest ring has slots; after every
replay the cache bytes and `written` of every layer must equal the oracle's, and the attention outputs of the
last replayed frame are compared with the oracle's.  A wrong slot after replay cannot go unnoticed."""
import numpy as np
import pytest
import torch

from oracle import ring_attn_oracle as oracle
from tests import gpu_helpers as gh
from tests import helpers
from world_engine_b200 import B200StaticKVCache, ops
from world_engine_b200.synthetic import StepConfig

pytestmark = pytest.mark.gpu


class _ModelCfg:          # the reference's config keys that size the cache (src/model/kv_cache.py:161-179)
    tokens_per_frame = 128
    local_window = 4
    global_window = 6
    global_attn_period = 3
    global_attn_offset = 1
    global_pinned_dilation = 2
    n_layers = 3
    n_heads = 4
    n_kv_heads = 2
    d_model = 4 * 128


def test_whole_frames_replayed_from_one_cuda_graph_keep_the_caches_exact():
    mc = _ModelCfg
    B, T, Hq, Hkv, Dh = 1, mc.tokens_per_frame, mc.n_heads, mc.n_kv_heads, 128
    dev = torch.device("cuda")
    cache = B200StaticKVCache(mc, batch_size=B, dtype=torch.bfloat16).to(dev)
    n_layers, passes = mc.n_layers, [True, True, True, True, False]
    layer_cfgs, ocaches = [], []
    for li, layer in enumerate(cache.layers):
        layer.validate = False                       # the eager-only argument checks read values on the host
        ring = layer.L // T
        c = StepConfig(f"layer{li}", B, Hq, Hkv, Dh, T, ring, layer.pinned_dilation, 0, "bf16", 2000 + li)
        layer_cfgs.append(c)
        ocaches.append(helpers.new_oracle_cache(c))
    assert [c.dilation for c in layer_cfgs] == [1, 2, 1] and [c.ring_frames for c in layer_cfgs] == [4, 6, 4]

    # static buffers of the graph: inputs of every (pass, layer), outputs, the frame counter
    q_s = torch.zeros(len(passes), n_layers, B, Hq, T, Dh, device=dev, dtype=torch.bfloat16)
    k_s = torch.zeros(n_layers, B, Hkv, T, Dh, device=dev, dtype=torch.bfloat16)
    v_s = torch.zeros_like(k_s)
    out_s = torch.zeros_like(q_s)
    t_pos = torch.zeros(B, T, dtype=torch.long, device=dev)
    pos = {"t_pos": t_pos}

    def frame():
        for pi, frozen in enumerate(passes):
            cache.set_frozen(frozen)
            for li in range(n_layers):
                out_s[pi, li].copy_(cache.append_and_attend(q_s[pi, li], k_s[li], v_s[li], pos, li))
        t_pos.add_(1)                                # next frame: the counter every layer reads, on the device

    def host_inputs(t):
        qs = np.zeros((len(passes), n_layers, B, Hq, T, Dh), np.float32)
        ks = np.zeros((n_layers, B, Hkv, T, Dh), np.float32)
        vs = np.zeros_like(ks)
        for li, c in enumerate(layer_cfgs):
            for pi in range(len(passes)):
                q, k, v = helpers.step_inputs(c, t, pi)
                qs[pi, li] = q
            ks[li], vs[li] = k, v                    # K/V of a frame are the same at every pass of it
        return qs, ks, vs

    def load_inputs(t):
        qs, ks, vs = host_inputs(t)
        q_s.copy_(torch.from_numpy(qs).to(dev)); k_s.copy_(torch.from_numpy(ks).to(dev)); v_s.copy_(torch.from_numpy(vs).to(dev))
        return qs, ks, vs

    # warm-up outside the graph on frame 0 (sets function attributes, allocates the status word), then start over
    load_inputs(0)
    frame()
    torch.cuda.synchronize()
    cache.reset()
    t_pos.zero_()
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    load_inputs(0)
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            frame()
    torch.cuda.synchronize()
    # capture does not execute: the caches are still empty and the counter is still 0
    assert int(t_pos[0, 0].item()) == 0 and not bool(cache.layers[0].written[:cache.layers[0].L].any())

    n_frames = max(c.ring_frames for c in layer_cfgs) + 3
    for t in range(n_frames):
        qs, ks, vs = load_inputs(t)
        graph.replay()
        torch.cuda.synchronize()
        assert int(t_pos[0, 0].item()) == t + 1
        last = t == n_frames - 1
        for li, c in enumerate(layer_cfgs):
            kv_new = np.stack([helpers.to_container(c, ks[li]), helpers.to_container(c, vs[li])], 0)
            for pi, frozen in enumerate(passes):
                k_full, v_full, mask = ocaches[li].upsert(kv_new, t, frozen)
                if last:
                    want = oracle.frame_attention(qs[pi, li], helpers.from_container(c, k_full),
                                                  helpers.from_container(c, v_full), mask)
                    mx, mean = helpers.error_stats(out_s[pi, li].float().cpu().numpy(), want)
                    assert mx <= helpers.MAX_ABS_TOL and mean <= helpers.MEAN_ABS_TOL, \
                        f"frame {t} layer {li} pass {pi}: max {mx} mean {mean}"
            layer = cache.layers[li]
            assert gh.kv_bytes(layer) == ocaches[li].kv.tobytes(), f"frame {t}: cache of layer {li} differs"
            assert np.array_equal(layer.written.cpu().numpy(), ocaches[li].written), f"frame {t}: written, layer {li}"
    ops.check_status(dev)
