"""Benchmark of the convolution hot path through the C ABI of libAvocadoCudaBackend.so.

    python bench.py --gpus N --steps K --warmup W [--config 2|3|4|5] [--matrices float16|float32] [--impl reference]

One "step" is one pass of the configured convolution over one batch of synthetic input.  The default workload is
configuration 2 of the baseline: a ResNet-style 3x3 layer, NHWC float16, N=64, 56x56, C=K=64, run as the non-fused
Winograd F(4x4,3x3) pipeline (weight, input and output transforms around the transform-domain batched GEMM).
With N > 1 GPUs (one process per GPU, launched by torch.distributed.run) every rank processes its own batch of the
same size (weak scaling, no data-path collective); only configuration 5 all-reduces the weight gradient.

Prints ONE JSON line (rank 0).  `value` is the device-timed throughput with inputs resident in HBM, `e2e` the
same metric through the same calls with pinned HOST buffers and the copies inside the timed region.
`--impl reference` times the CPU restatement of the reference's own naive convolution on the host cores instead.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CONFIGS = {
    2: dict(name="cfg2: 3x3 conv NHWC float16, N=64 56x56 C=K=64, non-fused Winograd F(4x4,3x3)", n=64, h=56, w=56, c=64, k=64, dtype="float16",
            kind="winograd_nonfused"),
    3: dict(name="cfg3: 3x3 conv NHWC bfloat16 + bias + ReLU, N=128 28x28 C=K=128, fused Winograd", n=128, h=28, w=28, c=128, k=128,
            dtype="bfloat16", kind="winograd_fused"),
    4: dict(name="cfg4: int8 3x3 implicit-GEMM conv with requantisation, N=256 14x14 C=K=256", n=256, h=14, w=14, c=256, k=256, dtype="int8",
            kind="implicit_gemm"),
    5: dict(name="cfg5: training step (fwd + dX + dW) NHWC float32, 56x56 C=K=64, non-fused Winograd F(4x4,3x3)", n=256, h=56, w=56, c=64, k=64,
            dtype="float32", kind="training"),
}


# dram__bytes_read.sum + dram__bytes_write.sum of one GEMM launch (profiles/winograd_nonfused_f43_fp16_cfg2.txt)
NCU_GEMM_TRAFFIC = {(2, "float16"): 58.124e6 + 10.220e6}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, window=None):
        """Stops sampling; `window` = (t0, t1) in time.time() keeps only the samples taken inside the timed region."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        in_window = [(t, l) for t, l in self.lines if window is None or window[0] <= t <= window[1] + 0.05]
        # a timed region shorter than the sampling period may hold no sample: then the samples of the whole run
        # (warm-up included, same kernels) stand in, and "window" says so
        self.window_used = "timed region" if in_window else "whole run (timed region shorter than the sampling period)"
        for stamp, line in (in_window or self.lines):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None, "reasons": sorted(reasons),
                "samples": len(sm), "window": self.window_used}


def synthetic(cfg, seed_offset=0):
    """Seeded synthetic tensors with the distributions the baseline configuration names."""
    r = np.random.default_rng(0x1001 + seed_offset)
    n, h, w, c, k = cfg["n"], cfg["h"], cfg["w"], cfg["c"], cfg["k"]
    data = {}
    if cfg["dtype"] == "int8":
        data["x"] = r.integers(-127, 128, (n, h, w, c), dtype=np.int8)
        data["w"] = np.random.default_rng(0x1002).integers(-127, 128, (k, 3, 3, c), dtype=np.int8)
        data["b"] = np.random.default_rng(0x1003).integers(-1000, 1001, k, dtype=np.int32)
        data["scales"] = np.random.default_rng(0x1005).uniform(1e-3, 1e-2, k).astype(np.float32)
    else:
        data["x"] = r.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
        data["w"] = np.random.default_rng(0x1002).normal(0, np.sqrt(2.0 / (9 * c)), (k, 3, 3, c)).astype(np.float32)
        data["b"] = np.random.default_rng(0x1003).uniform(-0.1, 0.1, k).astype(np.float32)
        data["dy"] = np.random.default_rng(0x1004 + seed_offset).uniform(-1, 1, (n, h, w, k)).astype(np.float32)
    return data


def direct_flops(cfg):
    f = 2.0 * cfg["n"] * cfg["h"] * cfg["w"] * cfg["k"] * cfg["c"] * 9
    return 3.0 * f if cfg["kind"] == "training" else f


def elem_size(dtype):
    return {"float16": 2, "bfloat16": 2, "float32": 4, "float64": 8, "int8": 1}[dtype]


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the restatement of the reference's naive convolution, timed on the host cores
# ------------------------------------------------------------------------------------------------------------
def cpu_sample(cfg, images):
    """Runs the naive CPU convolution on `images` images of the workload; returns (seconds, flops done)."""
    from oracle import oracle as o
    o.use_all_host_threads()  # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use the whole host
    sub = dict(cfg, n=images)
    data = synthetic(sub)
    t0 = time.perf_counter()
    if cfg["dtype"] == "int8":
        o.conv2d_forward_int8(data["x"], data["w"], data["b"], data["scales"])
        passes = 1.0
    else:
        o.conv2d_forward_f32_naive(data["x"], data["w"], data["b"] if cfg["kind"] == "winograd_fused" else None, relu=cfg["kind"] == "winograd_fused")
        passes = 1.0
        if cfg["kind"] == "training":
            # dX and dW cost the same as the forward pass; the naive float64 adjoints stand in for them
            o.conv2d_backward_data(data["dy"], data["w"], (cfg["h"], cfg["w"]))
            o.conv2d_backward_weights(data["x"], data["dy"])
            passes = 3.0
    seconds = time.perf_counter() - t0
    return seconds, passes * 2.0 * images * cfg["h"] * cfg["w"] * cfg["k"] * cfg["c"] * 9


def cpu_baseline(cfg, sample_images, target_seconds=12.0, max_passes=60):
    """Times the CPU port on `sample_images` images of the workload, pass after pass, until about target_seconds of CPU work."""
    from oracle import oracle as o
    cpu_sample(cfg, max(1, sample_images // 8))  # page the library and the data in
    seconds = flops = 0.0
    passes = 0
    while passes < max_passes and (seconds < target_seconds or passes == 0):
        s, f = cpu_sample(cfg, sample_images)
        seconds += s
        flops += f
        passes += 1
    return {"value": flops / seconds / 1e12, "unit": "TFLOP/s (effective, direct-conv FLOP count)", "cores": o.max_threads(), "kind": "port",
            "sample": "%d passes over %d of %d images of the workload, naive direct convolution (OpenMP over image x output row), %.1f s of CPU work"
                      % (passes, sample_images, cfg["n"], seconds),
            "images_per_s": passes * sample_images / seconds}


def run_reference_arm(args, cfg, rank):
    if rank != 0:
        return
    images = {2: 16, 3: 16, 4: 16, 5: 4}[args.config]
    for _ in range(args.warmup):
        cpu_sample(cfg, max(1, images // 4))
    total_s, total_flops = 0.0, 0.0
    for _ in range(args.steps):
        s, f = cpu_sample(cfg, images)
        total_s += s
        total_flops += f
    from oracle import oracle as o
    value = total_flops / total_s / 1e12
    sample = "each step = %d of %d images of the workload through the naive CPU convolution" % (images, cfg["n"])
    line = {"impl": "reference", "metric": "conv effective TFLOP/s (direct-convolution FLOP count)", "value": value, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_s / args.steps * cfg["n"] / images,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32" if cfg["dtype"] != "int8" else "s8->s32",
            "data": "synthetic", "config": {"workload": cfg["name"], "sample": sample},
            "images_per_s": images * args.steps / total_s,
            "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": o.max_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------
class Workload:
    """One buffer set (context + tensors) of the configured convolution; several are rotated so that a step never
    finds its inputs in L2 from the step before."""

    def __init__(self, cfg, device, matrices_dtype, data, side_stream=False):
        from cudabackend_b200 import api, pipeline
        self.api = api
        self.cfg = cfg
        self.ctx = api.Context(device)
        # a second context for the weight transform, which depends on nothing the input transform touches
        self.side_ctx = api.Context(device) if (side_stream and cfg["kind"] == "winograd_nonfused") else None
        n, h, w, c, k = cfg["n"], cfg["h"], cfg["w"], cfg["c"], cfg["k"]
        kind = cfg["kind"]
        if kind in ("winograd_nonfused", "training"):
            self.p = pipeline.WinogradNonFused(self.ctx, n, h, w, c, k, cfg["dtype"], matrices_dtype, 4, 3, device=device, training=(kind == "training"),
                                               side_ctx=self.side_ctx)
            self.p.x.upload(self.ctx, data["x"])
            self.p.wt.upload(self.ctx, data["w"])
            if kind == "training":
                self.p.dy.upload(self.ctx, data["dy"])
            self.x_tensor, self.y_tensor = self.p.x, (self.p.dw if kind == "training" else self.p.y)
        else:
            out_dtype = "int8" if cfg["dtype"] == "int8" else None
            self.p = pipeline.DirectConvolution(self.ctx, n, h, w, c, k, cfg["dtype"], out_dtype=out_dtype, device=device)
            self.p.x.upload(self.ctx, data["x"])
            self.p.wt.upload(self.ctx, data["w"])
            self.p.set_bias(data["b"])
            if cfg["dtype"] == "int8":
                self.p.set_scales(data["scales"])
            self.x_tensor, self.y_tensor = self.p.x, self.p.y
        self.ctx.synchronize()
        self.host_x = None
        self.host_y = None

    def launches_per_step(self):
        # kernels of this library launched per step: forward chain 4; dX chain 5 (its (N,N) contraction transposes U first);
        # dW chain 5 (split contraction + fixed-order reduction); one-call Winograd 3 (weight, input, contraction + output)
        return {"winograd_nonfused": 4, "training": 4 + 5 + 5, "winograd_fused": 3, "implicit_gemm": 1}[self.cfg["kind"]]

    def stages(self):
        """(name, callable) pairs making up one step, in issue order."""
        kind = self.cfg["kind"]
        p = self.p
        if kind == "winograd_nonfused":
            return [("weight_transform", p.weight_transform), ("input_transform", p.input_transform),
                    ("gemm", lambda: p.gemm(p.v, p.u, p.m, False, True)), ("output_transform", p.output_transform)]
        if kind == "training":
            return [("forward", p.forward), ("backward_data", p.backward_data), ("backward_weights", p.backward_weights)]
        if kind == "winograd_fused":
            return [("winograd_fused", lambda: p.winograd_fused(activation="relu"))]
        return [("implicit_gemm", p.implicit_gemm)]

    def step(self):
        if self.cfg["kind"] == "winograd_nonfused":
            self.p.forward()  # the four calls of stages(); the weight transform goes to the side context when there is one
            return
        for _, fn in self.stages():
            fn()

    def pin_host_buffers(self, data):
        api = self.api
        stored, _ = api.to_storage(data["x"], self.cfg["dtype"])
        self.host_x = np.array(stored, copy=True, order="C")
        self.host_y = api.host_buffer(self.y_tensor.shape, self.y_tensor.dtype)
        api.call("cudaPageLock", self.host_x.ctypes.data_as(api._VP), self.host_x.nbytes)
        api.call("cudaPageLock", self.host_y.ctypes.data_as(api._VP), self.host_y.nbytes)

    def unpin(self):
        api = self.api
        if self.host_x is not None:
            api.call("cudaPageUnlock", self.host_x.ctypes.data_as(api._VP))
            api.call("cudaPageUnlock", self.host_y.ctypes.data_as(api._VP))

    def step_e2e(self):
        """host x -> device, the step, device result -> host; all enqueued on this buffer set's stream"""
        self.x_tensor.mem.from_host(self.ctx, self.host_x)
        self.step()
        self.y_tensor.mem.to_host(self.ctx, self.host_y)


def stage_bytes(cfg, matrices_dtype):
    """Algorithmic bytes of each stage of the non-fused pipeline (inputs read once, outputs written once)."""
    n, h, w, c, k = cfg["n"], cfg["h"], cfg["w"], cfg["c"], cfg["k"]
    b = elem_size(cfg["dtype"])
    mb = elem_size(matrices_dtype)
    t = n * ((h + 3) // 4) * ((w + 3) // 4)
    return {"weight_transform": 9 * k * c * b + 36 * k * c * mb, "input_transform": n * h * w * c * b + 36 * t * c * mb,
            "gemm": 36 * t * c * mb + 36 * k * c * mb + 36 * t * k * mb, "output_transform": 36 * t * k * mb + n * h * w * k * b,
            "gemm_flops": 2.0 * 36 * t * c * k}


def run_gpu_arm(args, cfg, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from cudabackend_b200 import api

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = load_peaks()
    matrices_dtype = args.matrices or cfg["dtype"]
    data = synthetic(cfg, seed_offset=rank)

    rotation = args.rotation
    sets = [Workload(cfg, local_rank, matrices_dtype if cfg["kind"] in ("winograd_nonfused", "training") else None, data, side_stream=args.side_stream)
            for _ in range(rotation)]
    streams = [torch.cuda.ExternalStream(ws.ctx.stream(), device=local_rank) for ws in sets]

    grad_views = None
    if cfg["kind"] == "training" and world > 1:
        # dW lives in library memory; wrap it for the NCCL all-reduce without copying
        grad_views = []
        for ws in sets:
            class _Cai:
                pass
            holder = _Cai()
            holder.__cuda_array_interface__ = {"shape": ws.p.dw.shape, "typestr": "<f4", "data": (ws.p.dw.mem.pointer(), False), "version": 3}
            grad_views.append(torch.as_tensor(holder, device=torch.device("cuda", local_rank)))

    def full_step(i):
        ws = sets[i % rotation]
        ws.step()
        if grad_views is not None:
            with torch.cuda.stream(streams[0]):
                dist.all_reduce(grad_views[i % rotation])

    def sync_all():
        for ws in sets:
            ws.ctx.synchronize()
        torch.cuda.synchronize()

    def barrier():
        sync_all()
        if world > 1:
            dist.barrier()
        sync_all()

    use_graph = (not args.no_graph) and grad_views is None

    # ---- device-timed region ------------------------------------------------------------------------------
    # every buffer set is driven through ONE context (one stream) here, so steps run back to back on the device;
    # a step is replayed from a captured graph (one launch per step instead of one per kernel)
    shared_ctx = sets[0].ctx
    own_ctx = [ws.ctx for ws in sets]
    for ws in sets:
        ws.ctx = shared_ctx
        ws.p.ctx = shared_ctx
    s0 = streams[0]
    graphs = [shared_ctx.capture(ws.step) for ws in sets] if use_graph else None

    def timed_step(i):
        if graphs is not None:
            graphs[i % rotation].launch()
        else:
            full_step(i)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for i in range(args.warmup):
        timed_step(i)
    barrier()
    first = torch.cuda.Event(enable_timing=True)
    last = torch.cuda.Event(enable_timing=True)
    t_wall0 = time.perf_counter()
    window0 = time.time()
    first.record(s0)
    for i in range(args.steps):
        timed_step(i)
    last.record(s0)
    sync_all()
    window1 = time.time()
    elapsed_ms = first.elapsed_time(last)
    wall_ms = (time.perf_counter() - t_wall0) * 1e3
    clocks = sampler.stop((window0, window1)) if rank == 0 else None
    if world > 1:
        t = torch.tensor([elapsed_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())

    # ---- per-kernel durations: each stage launched back to back over the rotating buffer sets, CUDA events around ---
    stage_names = [name for name, _ in sets[0].stages()]
    stage_ms = {}
    stage_reps = max(20, min(args.steps, 200))
    for j, name in enumerate(stage_names):
        fns = [ws.stages()[j][1] for ws in sets]
        for i in range(rotation):
            fns[i]()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        shared_ctx.synchronize()
        e0.record(s0)
        for i in range(stage_reps):
            fns[i % rotation]()
        e1.record(s0)
        sync_all()
        stage_ms[name] = e0.elapsed_time(e1) / stage_reps

    # the practical ceiling for a transfer of this size: a plain device copy moving as many bytes (read + write) as the
    # dominant kernel, timed the same way (back to back over rotating cold buffers)
    copy_reference = None
    if cfg["kind"] == "winograd_nonfused":
        nbytes = stage_bytes(cfg, matrices_dtype)["gemm"] // 2 // 256 * 256
        pairs = [(api.Memory(nbytes, local_rank), api.Memory(nbytes, local_rank)) for _ in range(rotation)]
        for a, b in pairs:
            a.zero(shared_ctx)
            b.zero(shared_ctx)

        def copy_step(i):
            a, b = pairs[i % rotation]
            api.call("cudaCopyMemory", shared_ctx.handle, b.handle, 0, a.handle, 0, nbytes)

        for i in range(2 * rotation):
            copy_step(i)
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        shared_ctx.synchronize()
        e0.record(s0)
        for i in range(stage_reps):
            copy_step(i)
        e1.record(s0)
        sync_all()
        copy_ms = e0.elapsed_time(e1) / stage_reps
        copy_reference = {"bytes": 2 * nbytes, "us": copy_ms * 1e3, "gbs": 2 * nbytes / (copy_ms * 1e-3) / 1e9}
        del pairs

    status = sum(ctx.last_device_status() for ctx in own_ctx)
    if status != 0:
        raise RuntimeError("a tensor-core kernel reported a bounded wait that ran out (status %d)" % status)

    # ---- end-to-end region: pinned host buffers, copies inside; one stream per buffer set so copies overlap kernels --
    for ws, ctx in zip(sets, own_ctx):
        ws.ctx = ctx
        ws.p.ctx = ctx
        ws.pin_host_buffers(data)
    e2e_graphs = [ws.ctx.capture(ws.step_e2e) for ws in sets] if use_graph else None

    def e2e_step(i):
        if e2e_graphs is not None:
            e2e_graphs[i % rotation].launch()
        else:
            sets[i % rotation].step_e2e()
            if grad_views is not None:
                with torch.cuda.stream(streams[i % rotation]):
                    dist.all_reduce(grad_views[i % rotation])

    for i in range(min(args.warmup, 2 * rotation)):
        e2e_step(i)
    barrier()
    e2e_steps = max(rotation, min(args.steps, 400))
    # timed on the device: a start event on every stream of the region (all idle after the barrier), an end event on every
    # stream after its last step; the region lasts from the earliest start to the latest end.  The host clock is kept
    # beside it as a cross-check.
    starts = [torch.cuda.Event(enable_timing=True) for _ in streams]
    ends = [torch.cuda.Event(enable_timing=True) for _ in streams]
    t0 = time.perf_counter()
    for ev, st in zip(starts, streams):
        ev.record(st)
    for i in range(e2e_steps):
        e2e_step(i)
    for ev, st in zip(ends, streams):
        ev.record(st)
    sync_all()
    e2e_wall_s = (time.perf_counter() - t0) * args.steps / e2e_steps
    e2e_device_ms = max(starts[0].elapsed_time(ev) for ev in ends)  # the start events are recorded back to back on idle streams
    e2e_s = e2e_device_ms * 1e-3 * args.steps / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    h2d = sets[0].host_x.nbytes
    d2h = sets[0].host_y.nbytes
    sync_all()
    if e2e_graphs is not None:
        for gr in e2e_graphs:
            gr.destroy()
    if graphs is not None:
        for gr in graphs:
            gr.destroy()
    for ws in sets:
        ws.unpin()

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    flops = direct_flops(cfg)
    value = flops * args.steps * world / (elapsed_ms * 1e-3) / 1e12
    e2e_value = flops * args.steps * world / e2e_s / 1e12
    line = {"metric": "conv effective TFLOP/s (direct-convolution FLOP count)", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": {"float16": "f16 (f32 accumulate)", "bfloat16": "bf16 (f32 accumulate)", "float32": "f32",
                                           "int8": "s8 (s32 accumulate)"}[cfg["dtype"]],
            "data": "synthetic",
            "config": {"workload": cfg["name"], "per_gpu_batch": cfg["n"], "global_batch": cfg["n"] * world, "matrices_dtype": matrices_dtype,
                       "l2": "rotating %d buffer sets; each set's working set is re-read only after %d other steps" % (rotation, rotation - 1),
                       "parallelism": "batch sharded, dp%d" % world},
            "images_per_s": cfg["n"] * args.steps * world / (elapsed_ms * 1e-3),
            "host_wall_ms_per_step": wall_ms / args.steps,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "images_per_s": cfg["n"] * args.steps * world / e2e_s, "ms_per_step": 1e3 * e2e_s / args.steps,
                    "timing": "CUDA events over all streams of the region", "host_clock_ms_per_step": 1e3 * e2e_wall_s / args.steps},
            "gpu_launches": sets[0].launches_per_step() * args.steps, "launch_mode": ("cuda graph, one launch per step" if use_graph else "kernel by kernel")
            + ("; weight transform on a second context (parallel graph branch)" if sets[0].side_ctx is not None else ""),
            "stage_ms": stage_ms, "clocks": clocks}

    # roofline of the dominant kernel
    if cfg["kind"] == "winograd_nonfused":
        sb = stage_bytes(cfg, matrices_dtype)
        gemm_s = stage_ms["gemm"] * 1e-3
        achieved = sb["gemm"] / gemm_s / 1e9
        # DRAM bytes of one launch of this kernel from the committed ncu capture (cold caches); only known for the default workload
        traffic = NCU_GEMM_TRAFFIC.get((args.config, matrices_dtype))
        line["roofline"] = {"kernel": "kernel_gemm_nt_tc (transform-domain batched GEMM)" if matrices_dtype != "float32" else
                            "kernel_gemm_nt_tf32x3 (transform-domain batched GEMM)", "bound": "hbm", "achieved": achieved,
                            "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "traffic": traffic,
                            "algorithmic_bytes": sb["gemm"], "device_copy_of_same_bytes": copy_reference,
                            "peak_source": peaks["source"], "tensor_tflops": sb["gemm_flops"] / gemm_s / 1e12,
                            "tensor_frac": sb["gemm_flops"] / gemm_s / 1e12 / peaks["bf16_tflops"]}
        line["stage_gbs"] = {name: sb[name] / (stage_ms[name] * 1e-3) / 1e9 for name in stage_names}
        line["stage_hbm_frac"] = {name: line["stage_gbs"][name] / peaks["hbm_gbs"] for name in stage_names}
        total_bytes = sum(sb[name] for name in stage_names)
        line["pipeline_hbm_frac"] = total_bytes / (elapsed_ms / args.steps * 1e-3) / 1e9 / peaks["hbm_gbs"]
    elif cfg["kind"] in ("winograd_fused", "training"):
        # pipelines of HBM-bound kernels: the bytes every kernel of the step must move (inputs read once, outputs written
        # once, transform-domain tensors written by one kernel and read by the next), against the measured copy bandwidth
        n, h, w, c, k = cfg["n"], cfg["h"], cfg["w"], cfg["c"], cfg["k"]
        b = elem_size(cfg["dtype"])
        step_s = elapsed_ms / args.steps * 1e-3
        if cfg["kind"] == "winograd_fused":
            t = n * ((h + 1) // 2) * ((w + 1) // 2)
            u = 16 * k * c * 2
            algorithmic = (9 * k * c * b + u) + (n * h * w * c * b + 16 * t * c * 2) + (16 * t * c * 2 + u + n * h * w * k * b)
            kernels = "weight transform, input transform, kernel_f23_contract_output (contraction + output transform; M stays in TMEM)"
        else:
            t = n * ((h + 3) // 4) * ((w + 3) // 4)
            m = 4
            u = 36 * k * c * m
            transform_in = n * h * w * c * b + 36 * t * c * m
            transform_out = 36 * t * k * m + n * h * w * k * b
            gemm = 36 * t * (c + k) * m + u
            algorithmic = (transform_in + gemm + transform_out) * 2 + (transform_in + transform_out + gemm) + 3 * (9 * k * c * b + u)
            kernels = "12 kernels: forward, dX and dW chains (transforms + 3xTF32 tcgen05 contractions)"
        achieved = algorithmic / step_s / 1e9
        line["roofline"] = {"kernel": kernels, "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": achieved / peaks["hbm_gbs"], "traffic": None, "algorithmic_bytes": algorithmic, "peak_source": peaks["source"],
                            "tensor_tflops_effective": flops / step_s / 1e12}
    else:
        n, h, w, c, k = cfg["n"], cfg["h"], cfg["w"], cfg["c"], cfg["k"]
        b = elem_size(cfg["dtype"])
        algorithmic = n * h * w * c * b + 9 * k * c * b + n * h * w * k * b
        step_s = elapsed_ms / args.steps * 1e-3
        tensor_peak = peaks["bf16_tflops"] * (2.0 if cfg["dtype"] == "int8" else 1.0)
        ops = flops / step_s / 1e12
        line["roofline"] = {"kernel": cfg["kind"], "bound": "tensor", "achieved": ops, "peak": tensor_peak, "unit": "TFLOP/s",
                            "frac": ops / tensor_peak, "traffic": None, "peak_source": peaks["source"] + (" bf16 x2 (nominal int8 ratio)" if cfg["dtype"] == "int8" else ""),
                            "hbm_gbs": algorithmic / step_s / 1e9}

    if world == 1 and not args.no_cpu:
        images = {2: 64, 3: 64, 4: 64, 5: 16}[args.config]
        line["cpu_baseline"] = cpu_baseline(cfg, images)
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10000)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS))
    parser.add_argument("--matrices", default=None, choices=["float16", "bfloat16", "float32"], help="dtype of the transform-domain tensors")
    parser.add_argument("--rotation", type=int, default=4, help="buffer sets rotated between steps")
    parser.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    parser.add_argument("--no-graph", action="store_true", help="launch kernel by kernel instead of replaying a captured graph")
    parser.add_argument("--side-stream", action="store_true",
                        help="issue the weight transform on a second context (a parallel branch of the captured graph); measured slower, off by default")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = dict(CONFIGS[args.config])
    if cfg["kind"] == "training" and world > 1:
        cfg["n"] = cfg["n"] // 8  # 32 images per GPU, the share of one of 8 GPUs
    if args.impl == "reference":
        run_reference_arm(args, cfg, rank)
        return
    run_gpu_arm(args, cfg, rank, world, local_rank)


if __name__ == "__main__":
    main()
