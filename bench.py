#!/usr/bin/env python
"""Benchmark of the frame-causal attention + KV ring-buffer append on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload cfg2|cfg3|cfg4|cfg5] [--gpu-baseline] [--profile]

Workload (N = 1 and per rank for N > 1): the single frame step at small-model
scale -- B=1, H=16, head_dim=128, 256 tokens per frame, 16-frame ring that has
wrapped (write pointer at slot 11), bf16, K/V append included.  That
layer-step is run over 24 distinct layer caches (the 24 layers of one DiT
forward; 24 x 35.65 MB of cache = 855 MB, far larger than L2, so every
layer-step reads its K/V from HBM), and one bench STEP is as many passes over
those 24 caches as make it last about 6 ms, so that the timed region of the
default run is above 100 ms (`config.layer_steps_per_step` tells how many
layer-steps that is).  Sessions are independent, so N GPUs run N replicas of
the workload with no collective on the data path (weak scaling); the only
communication is the barrier and the max-over-ranks of the timing.
`--workload cfg4` shards the 64 sessions of the throughput configuration over
the ranks (64 / N per rank) instead.

Printed JSON line (rank 0): `value` = layer-steps per second over all ranks
with inputs resident in HBM (CUDA-graph replay, CUDA events); `e2e` = the same
through the public Python API with q/k/v coming from pinned HOST memory and
the output read back every pass; `roofline` = the attention kernel's
algorithmic bytes per launch over its measured average launch duration against
the measured HBM copy peak; `cpu_baseline` = the reference's CPU code path
(torch operators of the cache update + torch's un-compiled flex_attention, see
oracle/torch_eager_path.py) timed on this box's host cores on a bounded sample,
with the numpy oracle beside it.

`--impl reference` times that CPU path alone, with every host thread.
`--gpu-baseline` adds the kernel this library replaces on the same GPU: the
cache update with torch index ops + Inductor-compiled flex_attention with the
BlockMask the cache returns, replayed from a CUDA graph over the same caches.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_LAYERS = 24
FALLBACK_HBM_GBS = 6650.0
STEP_TARGET_MS = 6.0          # a bench step is sized to last about this long on the device
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the attention kernel, from the ncu capture summarised in
# the named file under profiles/ (bytes).  The figure belongs to the kernel build the capture was taken of.
NCU_TRAFFIC = {
    "cfg2": {"bytes": 34.71e6, "source": "profiles/frame_attn_cfg2_ncu_full.md"},
    "cfg3": {"bytes": 34.71e6, "source": "profiles/frame_attn_cfg2_ncu_full.md"},
    "cfg5": {"bytes": 584.9e6, "source": "profiles/frame_attn_cfg5_ncu_full.md"},
}
METRIC = "frame-attn layer-steps/s (append + attention)"
WORKLOADS = {
    "cfg2": "cfg2: B=1 H=16 Dh=128 T=256, 16-frame ring wrapped (frame_t=27, slot 11), bf16, append included; "
            "24 distinct layer caches (855 MB > L2, no flush needed)",
    "cfg3": "cfg3: whole generated frames of a 24-layer model at the cfg2 layer shape: 4 frozen denoise passes + 1 "
            "unfrozen pass that persists the frame = 120 layer-steps per frame; the frame counter advances on the "
            "device after every frame, so the ring slot moves and wraps",
    "cfg4": "cfg4: 64 sessions x (H=16 Dh=128 T=256, 32-frame ring = 8192 keys) sharded over the ranks, random wrap "
            "offsets, bf16, append included; 2 distinct session slabs per rank (larger than L2)",
    "cfg5": "cfg5: B=4 H=16 Dh=128 T=1024, 16-frame ring wrapped (16384 keys), bf16, append included; 4 distinct layer "
            "caches (4 x 570 MB > L2)",
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, 1590.0, "fallback"


def config_dict(workload: str, layer_steps_per_step, sessions_per_gpu):
    """The `config` object both arms print (same keys, so the two lines can be compared field by field)."""
    return {"workload": WORKLOADS[workload], "layer_steps_per_step": layer_steps_per_step,
            "sessions_per_gpu": sessions_per_gpu,
            "l2": "inputs larger than L2 (distinct caches cycled within a step)"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed regions run."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.samples = []
        self._stop = threading.Event()
        self._thr = None

    def _run(self):
        while not self._stop.is_set():
            try:
                r = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                    "-i", str(self.gpu)], capture_output=True, text=True, timeout=5)
                if r.returncode == 0 and r.stdout.strip():
                    self.samples.append([x.strip() for x in r.stdout.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._thr = threading.Thread(target=self._run, daemon=True)
        self._thr.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thr.join(timeout=6)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[1]))
                mx.append(float(s[2]))
            except Exception:
                continue
            for name, val in zip(names, s[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- CPU legs
def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def use_host_threads(n: int) -> int:
    """Thread count of the CPU legs, whatever OMP_NUM_THREADS the launcher set (torchrun exports 1)."""
    try:
        import torch
        torch.set_num_threads(n)
    except Exception:
        pass
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=n)
    except Exception:
        pass
    return n


def cpu_numpy_layer_step_seconds(cfg, repeats: int):
    """The numpy oracle's layer-step (upsert + attention).  Returns median seconds per layer-step."""
    import numpy as np
    from oracle import ring_attn_oracle as oracle   # CPU baseline leg: one of the places bench.py may use oracle/
    rng = np.random.default_rng(cfg.seed)
    cache = oracle.OracleLayerKVCache(cfg.B, cfg.Hkv, cfg.L, cfg.Dh, np.uint16, cfg.T, cfg.dilation)
    cache.kv[...] = oracle.f32_to_bf16_bits(rng.standard_normal(cache.kv.shape, dtype=np.float32))
    cache.written[:] = True
    q = oracle.round_to_bf16(rng.standard_normal((cfg.B, cfg.Hq, cfg.T, cfg.Dh), dtype=np.float32))
    kv_new = oracle.f32_to_bf16_bits(rng.standard_normal((2, cfg.B, cfg.Hkv, cfg.T, cfg.Dh), dtype=np.float32))
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        k_full, v_full, mask = cache.upsert(kv_new, cfg.frame_t, True)
        oracle.frame_attention(q, oracle.bf16_bits_to_f32(k_full), oracle.bf16_bits_to_f32(v_full), mask)
        times.append(time.perf_counter() - t0)
    return statistics.median(times), times


class TorchEagerLeg:
    """The reference's CPU code path (torch cache update + un-compiled flex_attention) on the cfg2 layer shape."""

    def __init__(self, cfg, dtype="bf16"):
        import torch
        from oracle import torch_eager_path as tep   # CPU baseline leg (see the module's header)
        self.torch, self.tep, self.cfg = torch, tep, cfg
        tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
        g = torch.Generator().manual_seed(cfg.seed)
        self.cache = tep.TorchLayerKVCache(cfg.B, cfg.Hkv, cfg.L, cfg.Dh, tdt, cfg.T, cfg.dilation)
        self.cache.kv.copy_(torch.randn(self.cache.kv.shape, generator=g).to(tdt))
        self.cache.written[:] = True
        self.q = torch.randn(cfg.B, cfg.Hq, cfg.T, cfg.Dh, generator=g).to(tdt)
        self.k = torch.randn(cfg.B, cfg.Hkv, cfg.T, cfg.Dh, generator=g).to(tdt)
        self.v = torch.randn(cfg.B, cfg.Hkv, cfg.T, cfg.Dh, generator=g).to(tdt)

    def run(self, n: int):
        t0 = time.perf_counter()
        with self.torch.no_grad():
            for _ in range(n):
                self.tep.layer_step(self.cache, self.q, self.k, self.v, self.cfg.frame_t, True)
        return time.perf_counter() - t0


def run_reference(args):
    """`--impl reference`: the reference's CPU code path on this box's host cores, every thread."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import warnings
    warnings.filterwarnings("ignore")
    from world_engine_b200.synthetic import CONFIGS
    cfg = CONFIGS["cfg2"]
    cores = use_host_threads(host_threads())
    leg = TorchEagerLeg(cfg)
    leg.run(3)                                             # first calls trace the operator wrapper
    probe = leg.run(2) / 2
    budget = 150.0                                         # seconds for the whole run
    per_step = max(1, min(N_LAYERS, int(budget / max(probe, 1e-3) / max(1, args.steps + args.warmup))))
    for _ in range(args.warmup):
        leg.run(per_step)
    dt = sum(leg.run(per_step) for _ in range(args.steps))
    value = per_step * args.steps / dt
    sample = (f"{per_step} layer-step(s) of the cfg2 shape per step: torch index_copy_ cache update + torch's "
              f"un-compiled flex_attention, bf16 tensors, {cores} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value,
        "unit": "layer-steps/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": config_dict("cfg2", per_step, cfg.B),
        "us_per_layer_step": 1e6 / value,
        "cpu_baseline": {"value": value, "unit": "layer-steps/s", "cores": cores, "kind": "port", "sample": sample,
                         "what": "the reference's CPU code path restated with the same torch operators "
                                 "(oracle/torch_eager_path.py); the attention is torch's own eager flex_attention"},
        "e2e": {"value": value, "unit": "layer-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------- ours
def time_graph(torch, graph, stream, reps: int) -> float:
    """Milliseconds for `reps` replays (CUDA events on the launching stream)."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(reps):
        graph.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def gpu_baseline_leg(torch, cfg, cache, q, k, v, t_pos, steps: int, dev):
    """The kernel this library replaces, on the same caches and the same GPU: the cache update with torch index
    ops (src/model/kv_cache.py:126-151) + flex_attention compiled by Inductor (src/world_engine.py:139 compiles
    the whole model with mode="max-autotune"; src/model/attn.py:116 is the call), with the BlockMask that
    B200LayerKVCache.upsert returns for the same visibility, replayed from a CUDA graph over the 24 caches."""
    from torch.nn.attention.flex_attention import flex_attention
    n_layers = len(cache.layers)
    T, L = cfg.T, cfg.L
    offs = torch.arange(T, device=dev)
    pos = {"t_pos": t_pos}
    # the BlockMask of this step (identical for every layer: same frame, every ring slot written); built once, as
    # the tables do not change between replays of the frozen step
    _, _, bm = cache.layers[0].upsert_kv(k[0], v[0], pos, True)
    out = torch.empty_like(q)
    try:
        flex = torch.compile(flex_attention, dynamic=False, mode="max-autotune-no-cudagraphs")
        flex(q[0], cache.layers[0].kv[0], cache.layers[0].kv[1], block_mask=bm)
        mode = "max-autotune-no-cudagraphs"
    except Exception:
        torch._dynamo.reset()
        flex = torch.compile(flex_attention, dynamic=False)
        flex(q[0], cache.layers[0].kv[0], cache.layers[0].kv[1], block_mask=bm)
        mode = "default"

    def layer_steps():
        tail = L + offs
        for li, layer in enumerate(cache.layers):
            kv_new = torch.stack([k[li], v[li]], 0)                     # StaticKVCache.upsert, kv_cache.py:191-193
            layer.kv.index_copy_(3, tail, kv_new)                       # tail write, kv_cache.py:138
            out[li].copy_(flex(q[li], layer.kv[0], layer.kv[1], block_mask=bm))

    layer_steps()
    torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            layer_steps()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream(dev)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    reps = max(steps, 10)
    ms = time_graph(torch, graph, stream, reps)
    return {"kind": "torch-inductor-flex", "compile_mode": mode, "us_per_layer_step": ms * 1e3 / (reps * n_layers),
            "what": "torch index_copy_ tail write + Inductor-compiled flex_attention with the cache's BlockMask, "
                    "CUDA-graph replay over the same 24 caches (frozen step: one index_copy_ per layer)",
            "torch": torch.__version__}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from world_engine_b200 import B200StaticKVCache, SessionSlab, ops, _lib, shard_sessions
    from world_engine_b200.synthetic import CONFIGS, scaled

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback "
                         "(use --impl reference for the CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    if args.workload == "cfg4":
        # 64 independent sessions (32-frame rings at random wrap offsets), session i on rank i mod world; the
        # sessions of a rank are batched in one launch per layer-step
        mine = shard_sessions(64, world, rank)
        cfg = scaled(CONFIGS["cfg4_session"], B=len(mine))
        n_layers = 2
        layers = []
        for _ in range(n_layers):
            slab = SessionSlab(cfg.B, cfg.Hkv, cfg.L, cfg.Dh, torch.bfloat16, cfg.T, device=dev)
            slab._slab.normal_(generator=g)
            slab._written.fill_(True)
            slab.frame_t.copy_(32 + torch.randint(0, 10000, (cfg.B,), device=dev, generator=g))
            layers.append((slab.kv, slab._written, slab.frame_t, 1))
        cache = None
    else:
        cfg = CONFIGS["cfg3_layer" if args.workload == "cfg3" else args.workload]
        n_layers = N_LAYERS if args.workload in ("cfg2", "cfg3") else 4

        class ModelCfg:   # the reference's config keys that size the cache (src/model/kv_cache.py:161-179)
            tokens_per_frame = cfg.T
            local_window = cfg.ring_frames
            global_window = cfg.ring_frames
            global_attn_period = 1 << 30
            global_attn_offset = 1
            global_pinned_dilation = 1
            n_heads = cfg.Hq
            n_kv_heads = cfg.Hkv
            d_model = cfg.Hq * cfg.Dh

        ModelCfg.n_layers = n_layers
        cache = B200StaticKVCache(ModelCfg, batch_size=cfg.B, dtype=torch.bfloat16).to(dev)
        t_pos = torch.full((cfg.B, cfg.T), cfg.frame_t, dtype=torch.long, device=dev)
        layers = []
        for layer in cache.layers:
            layer.kv.normal_(generator=g)
            layer.written.fill_(True)
            layer.validate = False
            layers.append((layer.kv, layer.written, t_pos, 0))
        cache.set_frozen(True)
        pos = {"t_pos": t_pos}
    shape_q = (n_layers, cfg.B, cfg.Hq, cfg.T, cfg.Dh)
    shape_kv = (n_layers, cfg.B, cfg.Hkv, cfg.T, cfg.Dh)
    q = torch.randn(shape_q, device=dev, dtype=torch.bfloat16, generator=g)
    k = torch.randn(shape_kv, device=dev, dtype=torch.bfloat16, generator=g)
    v = torch.randn(shape_kv, device=dev, dtype=torch.bfloat16, generator=g)
    out = torch.empty_like(q)

    # frozen flag of each pass over the layers within one graph (src/world_engine.py:139-152 for cfg3)
    passes = [True, True, True, True, False] if args.workload == "cfg3" else [True]

    def forward_layers():
        for frozen in passes:
            for li, (kv, wr, ft, fts) in enumerate(layers):
                ops.append_attend(q[li], k[li], v[li], kv, wr, ft, cfg.T, 1, frozen, 0.0, out=out[li],
                                  frame_t_stride=fts)
        if args.workload == "cfg3":
            t_pos.add_(1)        # next frame: the device-resident frame counter all layers read

    def attention_only():
        for li, (kv, wr, ft, fts) in enumerate(layers):
            ops.frame_attn(q[li], kv, wr, ft, cfg.T, 1, 0.0, out=out[li], frame_t_stride=fts)

    # warm-up outside graphs (allocates the workspace, sets function attributes)
    forward_layers()
    attention_only()
    torch.cuda.synchronize()
    # host cost of one eager call of the public entry point (tensor-map encodes, argument checks, launch)
    host_us = None
    if rank == 0:
        kv0, wr0, ft0, fts0 = layers[0]
        t0 = time.perf_counter()
        for _ in range(200):
            ops.append_attend(q[0], k[0], v[0], kv0, wr0, ft0, cfg.T, 1, True, 0.0, out=out[0], frame_t_stride=fts0)
        host_us = (time.perf_counter() - t0) / 200 * 1e6
        torch.cuda.synchronize()
    side = torch.cuda.Stream(device=dev)
    graph_step, graph_attn = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        n0 = lib.we_b200_launch_count()
        with torch.cuda.graph(graph_step, stream=side):
            forward_layers()
        launches_per_graph = lib.we_b200_launch_count() - n0
        with torch.cuda.graph(graph_attn, stream=side):
            attention_only()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream(dev)
    for _ in range(3):
        graph_step.replay()
    torch.cuda.synchronize()
    # size of a bench step: as many graph replays as last about STEP_TARGET_MS (the same number on every rank)
    probe_ms = time_graph(torch, graph_step, stream, 5) / 5
    want = args.inner if args.inner > 0 else max(1, math.ceil(STEP_TARGET_MS / max(probe_ms, 1e-3)))
    inner_t = torch.tensor([want], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(inner_t, op=dist.ReduceOp.MAX)
    inner = int(inner_t.item())
    layer_steps_per_graph = n_layers * len(passes)
    layer_steps_per_step = layer_steps_per_graph * inner

    def step():
        for _ in range(inner):
            graph_step.replay()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    with ClockSampler(local_rank) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)

        # the dominant kernel alone (attention, no append), same caches, same stream, same number of launches
        for _ in range(3):
            graph_attn.replay()
        torch.cuda.synchronize()
        attn_reps = args.steps * inner
        attn_us = time_graph(torch, graph_attn, stream, attn_reps) * 1e3 / (attn_reps * n_layers)
        ops.check_status(dev)

        # The one-pass q/k/v prologue (value residual + QK-norm + RoPE) that feeds the layer-step: timed on its own,
        # one launch per layer on the layers' q/k/v, reported beside the headline (it is not part of `value`).
        prologue = None
        if args.workload in ("cfg2", "cfg3") and rank == 0:
            side_hw = int(round(cfg.T ** 0.5))
            if side_hw * side_hw == cfg.T:
                ang = torch.rand(4 * cfg.T, cfg.Dh // 2, device=dev, generator=g) * 6.28 - 3.14
                cos_t, sin_t = ang.cos().contiguous(), ang.sin().contiguous()
                yy, xx = torch.meshgrid(torch.arange(side_hw, device=dev), torch.arange(side_hw, device=dev),
                                        indexing="ij")
                tp = torch.full((cfg.B, cfg.T), 2, dtype=torch.long, device=dev)
                yp = yy.reshape(1, cfg.T).expand(cfg.B, cfg.T).contiguous()
                xp = xx.reshape(1, cfg.T).expand(cfg.B, cfg.T).contiguous()
                lamb = torch.tensor(0.5, dtype=torch.bfloat16, device=dev)
                v1 = torch.randn((cfg.B, cfg.Hkv, cfg.T, cfg.Dh), device=dev, dtype=torch.bfloat16, generator=g)

                def prologue_layers():
                    for li in range(n_layers):
                        ops.qkv_prologue(q[li], k[li], v[li], v1, lamb, cos_t, sin_t, tp, yp, xp, side_hw, side_hw)

                prologue_layers()
                torch.cuda.synchronize()
                graph_pro = torch.cuda.CUDAGraph()
                with torch.cuda.stream(side):
                    with torch.cuda.graph(graph_pro, stream=side):
                        prologue_layers()
                torch.cuda.synchronize()
                for _ in range(3):
                    graph_pro.replay()
                pro_reps = max(args.steps * inner // 4, 20)
                pro_us = time_graph(torch, graph_pro, stream, pro_reps) * 1e3 / (pro_reps * n_layers)
                pro_bytes = (2 * cfg.B * cfg.T * cfg.Dh * (2 * (cfg.Hq + 2 * cfg.Hkv) + cfg.Hkv)
                             + 2 * 4 * cfg.B * cfg.T * (cfg.Dh // 2))
                prologue = {"kernel": "qkv_prologue_kernel<bf16>", "us_per_launch": pro_us,
                            "algorithmic_bytes_per_launch": pro_bytes, "gbs": pro_bytes / (pro_us * 1e-6) / 1e9,
                            "note": "inputs and outputs of 24 layers = 180 MB > L2"}
                ops.check_status(dev)

        gpu_baseline = None
        if args.gpu_baseline and rank == 0 and cache is not None and args.workload == "cfg2":
            try:
                gpu_baseline = gpu_baseline_leg(torch, cfg, cache, q, k, v, t_pos, args.steps * inner, dev)
            except Exception as e:      # the compiled flex path is third-party code: report, do not fail the bench
                gpu_baseline = {"kind": "torch-inductor-flex", "unavailable": f"{type(e).__name__}: {e}"[:300]}

        if args.profile:
            if rank == 0:
                per = ms * 1e3 / (layer_steps_per_step * args.steps)
                print(json.dumps({"profile_run": True, "workload": args.workload, "us_per_layer_step": per,
                                  "attn_us_per_launch": attn_us, "prologue": prologue, "gpu_baseline": gpu_baseline,
                                  "host_us_per_eager_call": host_us,
                                  "layer_steps_per_step": layer_steps_per_step,
                                  "tflops": cfg.flops() / (per * 1e-6) / 1e12}))
            if world > 1:
                dist.destroy_process_group()
            return 0

        # end to end through the public API: inputs from pinned host memory, output read back, every pass
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        hout = torch.empty(shape_q, dtype=torch.bfloat16).pin_memory()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)

        # Copies in, compute and copies out run on three streams, chained by events per group of layers, the way a
        # host that feeds the layers from pinned memory would pipeline them: the step's time tends to the slowest of
        # the three (the host-to-device copy here).  Groups rather than single layers keep the host's call count low.
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        group = n_layers if len(passes) > 1 else (6 if n_layers % 6 == 0 else 1)
        dq_bufs = [dq, torch.empty_like(dq)] if len(passes) > 1 else [dq]   # queries of consecutive passes alternate
        n_groups = n_layers // group
        ev_in = [[torch.cuda.Event() for _ in range(n_groups)] for _ in passes]
        ev_c = [[torch.cuda.Event() for _ in range(n_groups)] for _ in passes]

        # A device buffer is refilled only after the last launch that read it has completed: the event of that
        # launch group is remembered per buffer slice, so consecutive passes (and consecutive replays within a step)
        # pipeline without draining; the host waits once per step, for the step's last output.
        last_read = {}
        keep = []                              # outputs stay referenced until the step's synchronize

        def refill(dst, src, key):
            ev = last_read.get(key)
            if ev is not None:
                s_in.wait_event(ev)
            dst.copy_(src, non_blocking=True)

        def e2e_pass():
            cur = torch.cuda.current_stream(dev)
            for pi, frozen in enumerate(passes):
                if cache is not None:
                    cache.set_frozen(frozen)
                for gi in range(n_groups):
                    lo, hi = gi * group, (gi + 1) * group
                    qi = pi % len(dq_bufs)
                    dqb = dq_bufs[qi]
                    with torch.cuda.stream(s_in):
                        refill(dqb[lo:hi], hq[lo:hi], ("q", qi, gi))       # every denoise pass brings new queries
                        if pi == 0:
                            refill(dk[lo:hi], hk[lo:hi], ("k", gi))
                            refill(dv[lo:hi], hv[lo:hi], ("v", gi))
                        ev_in[pi][gi].record(s_in)
                    cur.wait_event(ev_in[pi][gi])
                    ys = []
                    for li in range(lo, hi):
                        if cache is not None:     # public API of the layer caches
                            y = cache.append_and_attend(dqb[li], dk[li], dv[li], pos, li)
                        else:                     # public API of the session slab
                            kv, wr, ft, fts = layers[li]
                            y = ops.append_attend(dqb[li], dk[li], dv[li], kv, wr, ft, cfg.T, 1, frozen, 0.0,
                                                  frame_t_stride=fts)
                        ys.append(y)
                    ev_c[pi][gi].record(cur)
                    last_read[("q", qi, gi)] = ev_c[pi][gi]
                    last_read[("k", gi)] = last_read[("v", gi)] = ev_c[pi][gi]
                    keep.append(ys)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(ev_c[pi][gi])
                        for li, y in zip(range(lo, hi), ys):
                            hout[li].copy_(y, non_blocking=True)
            if args.workload == "cfg3":
                t_pos.add_(1)

        def e2e_step():
            cur = torch.cuda.current_stream(dev)
            s_in.wait_stream(cur)
            s_out.wait_stream(cur)
            for _ in range(inner):
                e2e_pass()
            torch.cuda.synchronize()
            keep.clear()
            return float(hout[0, 0, 0, 0, 0])     # the step's result, read on the host

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        barrier()
        e2e_s = time.perf_counter() - t0
        if args.workload != "cfg3":      # (frozen passes: what came back equals what the device-timed legs produced)
            torch.cuda.synchronize()
            if not torch.equal(hout, out.cpu()):
                raise RuntimeError("bench: the end-to-end leg's outputs differ from the device-resident leg's")
        h2d = inner * (len(passes) * hq.numel() + hk.numel() + hv.numel()) * 2
        d2h = inner * len(passes) * hout.numel() * 2

        # the copies alone (pinned host <-> device, this rank's share of the PCIe / host-memory path), all ranks at once
        barrier()
        t0 = time.perf_counter()
        for _ in range(8):
            dq.copy_(hq, non_blocking=True)
        torch.cuda.synchronize()
        barrier()
        h2d_gbs = 8 * hq.numel() * 2 / (time.perf_counter() - t0) / 1e9
        t0 = time.perf_counter()
        for _ in range(8):
            hout.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        barrier()
        d2h_gbs = 8 * hout.numel() * 2 / (time.perf_counter() - t0) / 1e9

    # max over ranks (copy rates: min over ranks)
    times = torch.tensor([ms, e2e_s * 1e3, attn_us, -h2d_gbs, -d2h_gbs], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, attn_us, h2d_gbs, d2h_gbs = (float(x) for x in times.tolist())
    h2d_gbs, d2h_gbs = -h2d_gbs, -d2h_gbs
    sessions_total = torch.tensor([cfg.B], device=dev, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(sessions_total)
    sessions_total = int(sessions_total.item())

    if rank == 0:
        hbm_peak, tc_peak, peak_kind = measured_peaks()
        # cfg2 / cfg3 / cfg5: every rank runs a replica of the workload.  cfg4: one layer-step is a layer-step of
        # all 64 sessions, of which a rank holds its shard, so the ranks together complete one per launch round.
        if args.workload == "cfg4":
            total_layer_steps = layer_steps_per_step * args.steps * sessions_total / 64.0
        else:
            total_layer_steps = world * layer_steps_per_step * args.steps
        value = total_layer_steps / (ms * 1e-3)
        us_per_layer_step = ms * 1e3 / (layer_steps_per_step * args.steps)
        elem = 2
        attn_bytes = cfg.B * (2 * cfg.Hkv * cfg.visible_keys() * cfg.Dh * elem + 2 * cfg.Hq * cfg.T * cfg.Dh * elem)
        # the slower of HBM time and tensor time bounds the kernel (measured peaks)
        t_hbm = attn_bytes / (hbm_peak * 1e9)
        t_tc = cfg.flops() / (tc_peak * 1e12)
        if t_tc > t_hbm:
            roof = {"bound": "tensor", "achieved": cfg.flops() / (attn_us * 1e-6) / 1e12, "peak": tc_peak,
                    "unit": "TFLOP/s"}
        else:
            roof = {"bound": "hbm", "achieved": attn_bytes / (attn_us * 1e-6) / 1e9, "peak": hbm_peak, "unit": "GB/s"}
        traffic = NCU_TRAFFIC.get(args.workload)
        roof.update({"frac": roof["achieved"] / roof["peak"], "traffic": traffic["bytes"] if traffic else None,
                     "traffic_source": traffic["source"] if traffic else None,
                     "peak_kind": peak_kind, "kernel": "frame_attn_kernel<128,bf16>", "us_per_launch": attn_us,
                     "algorithmic_bytes_per_launch": attn_bytes, "flop_per_launch": cfg.flops()})
        # whole-job figures against the slower of the two peaks, over all ranks (the throughput half of the metric)
        step_bytes = cfg.algorithmic_bytes(True)
        bound_s = max(step_bytes / (hbm_peak * 1e9), cfg.flops() / (tc_peak * 1e12))
        frames_per_s = value * cfg.B / (24 * 5)            # session-frames of a 24-layer, 5-pass model
        cpu = None
        if world == 1:   # reported baseline: rank 0 at N=1 only
            import warnings
            warnings.filterwarnings("ignore")
            c2 = CONFIGS["cfg2"]
            cores = use_host_threads(host_threads())
            leg = TorchEagerLeg(c2)
            leg.run(3)
            n_torch = 0
            t_torch = 0.0
            while t_torch < 8.0 and n_torch < 200:
                t_torch += leg.run(2)
                n_torch += 2
            use_host_threads(1)
            one = TorchEagerLeg(c2)
            one.run(1)
            t_one = one.run(1)
            use_host_threads(cores)
            np_med, np_times = cpu_numpy_layer_step_seconds(c2, 20)
            cpu = {"value": n_torch / t_torch, "unit": "layer-steps/s", "cores": cores, "kind": "port",
                   "sample": f"{n_torch} layer-steps of the cfg2 shape (bf16 tensors), mean",
                   "what": "the reference's CPU code path restated with the same torch operators "
                           "(oracle/torch_eager_path.py): index_copy_ cache update, make_block_mask tables, torch's "
                           "un-compiled flex_attention",
                   "one_thread_value": 1.0 / t_one,
                   "numpy_oracle_value": 1.0 / np_med,
                   "numpy_oracle_sample": f"{len(np_times)} layer-steps, median (fp32 math on bf16-rounded inputs)"}
        line = {
            "metric": METRIC, "value": value, "unit": "layer-steps/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak" if args.workload != "cfg4" else "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": config_dict(args.workload, layer_steps_per_step, cfg.B),
            "us_per_layer_step": us_per_layer_step,
            "tflops": cfg.flops() / (us_per_layer_step * 1e-6) / 1e12,
            "sessions_total": sessions_total,
            "sessions_frames_per_s": frames_per_s if args.workload != "cfg4" else value * 64 / (24 * 5),
            "frac_of_slower_peak": bound_s / (us_per_layer_step * 1e-6),
            "us_per_frame": (ms * 1e3 / (args.steps * inner)) if args.workload == "cfg3" else None,
            "roofline": roof,
            "prologue": prologue,
            "gpu_baseline": gpu_baseline,
            "cpu_baseline": cpu,
            "e2e": {"value": total_layer_steps / (e2e_ms * 1e-3), "unit": "layer-steps/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "copy_only_h2d_gbs_per_gpu": h2d_gbs, "copy_only_d2h_gbs_per_gpu": d2h_gbs},
            "host_us_per_eager_call": host_us,
            "gpu_launches": int(launches_per_graph) * inner * args.steps,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["cfg2", "cfg3", "cfg4", "cfg5"], default="cfg2",
                    help="cfg2 (default, the headline layer-step); cfg3 = whole frames of a 24-layer model (4 frozen "
                         "passes + 1 persisting pass, frame counter advancing on the device); cfg4 = 64 sessions with "
                         "32-frame rings sharded over the ranks, a rank's sessions batched in one launch per "
                         "layer-step; cfg5 = B=4, 1024 tokens per frame, 16384 keys")
    ap.add_argument("--gpu-baseline", action="store_true",
                    help="also time torch's Inductor-compiled flex_attention + index_copy_ append on the same caches "
                         "(cfg2 workload, rank 0); adds the Triton compile time to the run")
    ap.add_argument("--inner", type=int, default=0,
                    help="graph replays per step (default 0: as many as last about 6 ms); 1 keeps a run under a "
                         "profiler short")
    ap.add_argument("--profile", action="store_true",
                    help="device-timed legs only (skips the end-to-end and CPU-baseline legs): for runs under ncu")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
