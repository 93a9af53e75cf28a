#!/usr/bin/env python
"""Benchmark of the frame-causal attention + KV ring-buffer append on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1 and per rank for N > 1): the single frame step at small-model
scale -- B=1, H=16, head_dim=128, 256 tokens per frame, 16-frame ring that has
wrapped (write pointer at slot 11), bf16, K/V append included.  One bench STEP
is that layer-step run over 24 distinct layer caches (the 24 layers of one DiT
forward; 24 x 35.65 MB of cache = 855 MB, far larger than L2, so every
layer-step reads its K/V from HBM).  Sessions are independent, so N GPUs run N
replicas of the workload with no collective on the data path (weak scaling);
the only communication is the barrier and the max-over-ranks of the timing.

Printed JSON line (rank 0): `value` = layer-steps per second over all ranks
with inputs resident in HBM (CUDA-graph replay, CUDA events); `e2e` = the same
through the public Python API with q/k/v coming from pinned HOST memory and
the output read back every step; `roofline` = the attention kernel's
algorithmic bytes per launch over its measured average launch duration against
the measured HBM copy peak; `cpu_baseline` = the numpy oracle (a port of the
reference's algorithm) timed on this box's host cores on a bounded sample.

`--impl reference` times that CPU port alone (the reference itself is
PyTorch code whose only implementation of this path on CPU is torch's eager
flex_attention; its tree is not present on the GPU box).
"""
from __future__ import annotations

import argparse
import json
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the attention kernel, from the ncu captures
# summarised under profiles/ (bytes); None where no capture exists for that workload.
NCU_TRAFFIC_BYTES = {"cfg2": 34.71e6, "cfg3": 34.71e6, "cfg4": None, "cfg5": None}
WORKLOAD = ("cfg2: B=1 H=16 Dh=128 T=256, 16-frame ring wrapped (frame_t=27, slot 11), bf16, append included; "
            "one step = 24 distinct layer caches (855 MB > L2, no flush needed)")


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
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
            self._stop.wait(0.1)

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


# --------------------------------------------------------------------------- CPU port
def cpu_layer_step_seconds(cfg, repeats: int):
    """Times the oracle's layer-step (upsert + attention) on host cores.  Returns median seconds per layer-step."""
    import numpy as np
    from oracle import ring_attn_oracle as oracle   # CPU baseline leg: the one place bench.py may use oracle/
    use_all_host_threads()
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


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def use_all_host_threads() -> int:
    """The CPU legs use every host core the process may run on, whatever OMP_NUM_THREADS the launcher set
    (torchrun exports OMP_NUM_THREADS=1).  Returns the thread count in effect."""
    n = host_threads()
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=n)
    except Exception:
        pass
    return n


def run_reference(args):
    """`--impl reference`: the CPU port of the reference's path on this box's host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from world_engine_b200.synthetic import CONFIGS
    cfg = CONFIGS["cfg2"]
    cpu_layer_step_seconds(cfg, 2)                        # first calls pay page faults / BLAS thread start
    probe, _ = cpu_layer_step_seconds(cfg, 2)
    budget = 150.0                                        # seconds for the whole run
    per_step = max(1, min(N_LAYERS, int(budget / max(probe, 1e-3) / max(1, args.steps + args.warmup))))
    for _ in range(args.warmup):
        cpu_layer_step_seconds(cfg, per_step)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_layer_step_seconds(cfg, per_step)
    dt = time.perf_counter() - t0
    value = per_step * args.steps / dt
    cores = host_threads()
    sample = f"{per_step} layer-step(s) of the cfg2 shape per step (numpy, fp32 math on bf16-rounded inputs)"
    line = {
        "impl": "reference", "metric": "frame-attn layer-steps/s (append + attention)", "value": value,
        "unit": "layer-steps/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "layer_steps_per_step": per_step},
        "us_per_layer_step": 1e6 / value,
        "cpu_baseline": {"value": value, "unit": "layer-steps/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "layer-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


# --------------------------------------------------------------------------- ours
def run_ours(args):
    import torch
    import torch.distributed as dist
    from world_engine_b200 import B200StaticKVCache, ops, _lib
    from world_engine_b200.synthetic import CONFIGS

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback "
                         "(use --impl reference for the CPU port)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    from world_engine_b200 import SessionSlab
    from world_engine_b200.synthetic import scaled
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    if args.workload == "cfg4":
        # 64 independent sessions (32-frame rings at random wrap offsets) batched in one launch per layer-step
        cfg = scaled(CONFIGS["cfg4_session"], B=64)
        n_layers = 2
        workload = ("cfg4: 64 sessions x (H=16 Dh=128 T=256, 32-frame ring = 8192 keys), random wrap offsets, bf16, "
                    "append included; one step = 2 distinct session slabs (2 x 4.4 GB > L2)")
        layers = []
        for _ in range(n_layers):
            slab = SessionSlab(cfg.B, cfg.Hkv, cfg.L, cfg.Dh, torch.bfloat16, cfg.T, device=dev)
            slab._slab.normal_(generator=g)
            slab._written.fill_(True)
            slab.frame_t.copy_(32 + torch.randint(0, 10000, (cfg.B,), device=dev, generator=g))
            layers.append((slab.kv, slab._written.view(torch.uint8), slab.frame_t, 1))
        cache = None
    else:
        cfg = CONFIGS["cfg3_layer" if args.workload == "cfg3" else args.workload]
        n_layers = N_LAYERS if args.workload in ("cfg2", "cfg3") else 4
        workload = WORKLOAD if args.workload == "cfg2" else (
            "cfg5: B=4 H=16 Dh=128 T=1024, 16-frame ring wrapped (16384 keys), bf16, append included; "
            "one step = 4 distinct layer caches (4 x 570 MB > L2)")
        if args.workload == "cfg3":
            workload = ("cfg3: one step = one generated frame of a 24-layer model at the cfg2 layer shape: 4 frozen "
                        "denoise passes + 1 unfrozen pass that persists the frame = 120 layer-steps; the frame "
                        "counter advances on the device after every frame, so the ring slot moves and wraps")

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
            layers.append((layer.kv, layer.written.view(torch.uint8), t_pos, 0))
        cache.set_frozen(True)
        pos = {"t_pos": t_pos}
    shape_q = (n_layers, cfg.B, cfg.Hq, cfg.T, cfg.Dh)
    shape_kv = (n_layers, cfg.B, cfg.Hkv, cfg.T, cfg.Dh)
    q = torch.randn(shape_q, device=dev, dtype=torch.bfloat16, generator=g)
    k = torch.randn(shape_kv, device=dev, dtype=torch.bfloat16, generator=g)
    v = torch.randn(shape_kv, device=dev, dtype=torch.bfloat16, generator=g)
    out = torch.empty_like(q)

    # frozen flag of each pass over the layers within one step (src/world_engine.py:139-152 for cfg3)
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
    side = torch.cuda.Stream(device=dev)
    graph_step, graph_attn = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        n0 = lib.we_b200_launch_count()
        with torch.cuda.graph(graph_step, stream=side):
            forward_layers()
        launches_per_step = lib.we_b200_launch_count() - n0
        with torch.cuda.graph(graph_attn, stream=side):
            attention_only()
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream(dev)
    for _ in range(max(args.warmup, 3)):
        graph_step.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        e0.record(stream)
        for _ in range(args.steps):
            graph_step.replay()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)

        # the dominant kernel alone (attention, no append), same caches, same stream
        for _ in range(3):
            graph_attn.replay()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for _ in range(args.steps):
            graph_attn.replay()
        a1.record(stream)
        torch.cuda.synchronize()
        attn_us = a0.elapsed_time(a1) * 1e3 / (args.steps * n_layers)
    ops.check_status(dev)

    # The one-pass q/k/v prologue (value residual + QK-norm + RoPE) that feeds the layer-step: timed on its own,
    # one launch per layer on the layers' q/k/v, reported beside the headline (it is not part of `value`).
    prologue = None
    if args.workload in ("cfg2", "cfg3") and rank == 0:
        side_hw = int(round(cfg.T ** 0.5))
        if side_hw * side_hw == cfg.T:
            ang = torch.rand(4 * cfg.T, cfg.Dh // 2, device=dev, generator=g) * 6.28 - 3.14
            cos_t, sin_t = ang.cos().contiguous(), ang.sin().contiguous()
            yy, xx = torch.meshgrid(torch.arange(side_hw, device=dev), torch.arange(side_hw, device=dev), indexing="ij")
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
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record(stream)
            for _ in range(args.steps):
                graph_pro.replay()
            p1.record(stream)
            torch.cuda.synchronize()
            pro_us = p0.elapsed_time(p1) * 1e3 / (args.steps * n_layers)
            pro_bytes = 2 * cfg.B * cfg.T * cfg.Dh * (2 * (cfg.Hq + 2 * cfg.Hkv) + cfg.Hkv) + 2 * 4 * cfg.B * cfg.T * (cfg.Dh // 2)
            prologue = {"kernel": "qkv_prologue_kernel<bf16>", "us_per_launch": pro_us,
                        "algorithmic_bytes_per_launch": pro_bytes, "gbs": pro_bytes / (pro_us * 1e-6) / 1e9,
                        "note": "inputs and outputs of 24 layers = 180 MB > L2"}
            ops.check_status(dev)

    if args.profile:
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": args.workload,
                              "us_per_layer_step": ms * 1e3 / (n_layers * len(passes) * args.steps),
                              "attn_us_per_launch": attn_us, "prologue": prologue,
                              "tflops": cfg.flops() / (ms * 1e-3 / (n_layers * len(passes) * args.steps)) / 1e12}))
        if world > 1:
            dist.destroy_process_group()
        return 0

    # end to end through the public API: inputs from pinned host memory, output read back, every step
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

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        keep = []                          # outputs stay referenced until the final synchronize
        for pi, frozen in enumerate(passes):
            if cache is not None:
                cache.set_frozen(frozen)
            for gi in range(n_groups):
                lo, hi = gi * group, (gi + 1) * group
                dqb = dq_bufs[pi % len(dq_bufs)]
                with torch.cuda.stream(s_in):
                    if pi >= 2:
                        s_in.wait_event(ev_c[pi - 2][gi])     # the pass before last read this buffer
                    dqb[lo:hi].copy_(hq[lo:hi], non_blocking=True)   # every denoise pass brings new queries
                    if pi == 0:
                        dk[lo:hi].copy_(hk[lo:hi], non_blocking=True)
                        dv[lo:hi].copy_(hv[lo:hi], non_blocking=True)
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
                keep.append(ys)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_c[pi][gi])
                    for li, y in zip(range(lo, hi), ys):
                        hout[li].copy_(y, non_blocking=True)
        if args.workload == "cfg3":
            t_pos.add_(1)
        torch.cuda.synchronize()
        return float(hout[0, 0, 0, 0, 0])

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_s = time.perf_counter() - t0
    h2d = (len(passes) * hq.numel() + hk.numel() + hv.numel()) * 2
    d2h = len(passes) * hout.numel() * 2

    # max over ranks
    times = torch.tensor([ms, e2e_s * 1e3, attn_us], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms, attn_us = (float(x) for x in times.tolist())

    if rank == 0:
        hbm_peak, tc_peak, peak_kind = measured_peaks()
        total_layer_steps = world * n_layers * len(passes) * args.steps
        value = total_layer_steps / (ms * 1e-3)
        us_per_layer_step = ms * 1e3 / (n_layers * len(passes) * args.steps)
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
        roof.update({"frac": roof["achieved"] / roof["peak"], "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
                     "peak_kind": peak_kind, "kernel": "frame_attn_kernel<128,bf16>", "us_per_launch": attn_us,
                     "algorithmic_bytes_per_launch": attn_bytes, "flop_per_launch": cfg.flops()})
        cpu = None
        if world == 1:   # reported baseline: rank 0 at N=1 only
            cpu_med, cpu_times = cpu_layer_step_seconds(CONFIGS["cfg2"], 40)
            cpu = {"value": 1.0 / cpu_med, "unit": "layer-steps/s", "cores": host_threads(), "kind": "port",
                   "sample": f"{len(cpu_times)} layer-steps of the cfg2 shape, median (numpy oracle)"}
        line = {
            "metric": "frame-attn layer-steps/s (append + attention)", "value": value, "unit": "layer-steps/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload, "layer_steps_per_step": n_layers * len(passes), "sessions_per_gpu": cfg.B,
                       "l2": "inputs larger than L2 (distinct caches cycled within a step)"},
            "us_per_layer_step": us_per_layer_step,
            "tflops": cfg.flops() / (us_per_layer_step * 1e-6) / 1e12,
            "sessions_frames_per_s": value * cfg.B / (24 * 5) if args.workload == "cfg4" else value / (24 * 5),
            "us_per_frame": (ms * 1e3 / args.steps) if args.workload == "cfg3" else None,
            "roofline": roof,
            "prologue": prologue,
            "cpu_baseline": cpu,
            "e2e": {"value": total_layer_steps / (e2e_ms * 1e-3), "unit": "layer-steps/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches_per_step) * args.steps,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["cfg2", "cfg3", "cfg4", "cfg5"], default="cfg2",
                    help="cfg2 (default, the headline layer-step); cfg3 = whole frames of a 24-layer model (4 frozen passes + 1 "
                         "persisting pass, frame counter advancing on the device); cfg4 = 64 sessions with 32-frame rings batched in "
                         "one launch per layer-step; cfg5 = B=4, 1024 tokens per frame, 16384 keys")
    ap.add_argument("--profile", action="store_true",
                    help="device-timed legs only (skips the end-to-end and CPU-baseline legs): for runs under ncu")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
