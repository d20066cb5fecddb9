#!/usr/bin/env python
"""Headline benchmark: ResNet-50 v1.5 conv stack, forward, fp16 in / fp32 accumulate, NHWC,
batch 256 per GPU, through the C ABI of libportdnn_b200.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line on rank 0.  `value` is conv TFLOP/s (2*N*Ho*Wo*R*S*C*K summed over the 53
convolutions, the reference's forward counter, bench/conv2d/base_convolution_fixture.h:85-88)
over the whole job with inputs resident in HBM; `e2e` is the same metric with the step's input
copied from pinned host memory and the pooled result copied back inside the timed region.
The line also carries, from the same run:
  roofline      the 53 tensor-core convolution launches, timed INSIDE the replayed step (step time
                minus the time of a graph holding only the other kernels of the step)
  sustained     the same step replayed back to back for at least two seconds
  train         a training step of the same stack (forward, both backprops of every layer, filter
                gradients all-reduced stage by stage while the backward pass continues)
  hbm           the HBM-bound operators of the path on the benchmark networks' shapes (GB/s)
  parity_check  two images of the batch-256 run checked layer by layer against the CPU oracle
  cpu_baseline  the CPU restatement of portDNN's direct kernel timed on the host cores
With --impl reference the same network is timed on the host cores with that CPU restatement
(portDNN itself is SYCL and cannot be built with this toolchain).

Other modes (they print their own tables, not the JSON line):
    python bench.py --layer N H W C K WINDOW STRIDE [--dtype f16|bf16|f32] [--reps R]   one conv layer
    python bench.py --hbm-table          every HBM-bound operator, one line each
    python bench.py --layers             the JSON line, then per-layer times of the forward stack
    python bench.py --workload vgg16 | mobilenet | layer0     the other benchmark configurations
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "conv_tflops_resnet50_fp16_b256_forward"
# DRAM bytes per launch of the 53 forward convolutions (dram__bytes_read.sum + dram__bytes_write.sum):
# 8489 MB per step in a one-off ncu capture of the batch-256 stack, against 11.76 GB of algorithmic
# bytes (input + filter + output of every layer once) - the small feature maps are still in L2 when
# the next layer reads them.
FORWARD_DRAM_BYTES_PER_LAUNCH = int(8489e6 / 53)
UNIT = "TFLOP/s"
BATCH = 256


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(tflops_burst=d["bf16_tflops"], tflops_sustained=d["bf16_tflops_sustained"], hbm_gbs=d["hbm_gbs"],
                    source="measured")
    return dict(tflops_burst=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


def host_threads():
    """All host cores for the CPU legs, whatever OMP_NUM_THREADS the launcher exported (torchrun sets
    it to 1): the environment is fixed before the OpenMP runtime loads and the runtime is told as well."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(n)
    try:
        import ctypes
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(n)
    except OSError:
        pass
    return n


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                                          "-lms", "25", "-i", str(self.gpu_index)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# CPU legs
# ------------------------------------------------------------------------------------------------
def cpu_baseline_sample(seconds_target=12.0):
    """Times the CPU oracle's float forward conv on one ResNet stage-1 3x3 layer at a batch sized
    for ~10-20 s of CPU work; returns the cpu_baseline object."""
    threads = host_threads()
    from oracle import oracle as orc
    p = orc.conv_params(1, 56, 56, 64, 64, 3, 1, True)
    rng = np.random.default_rng(0)
    x = rng.standard_normal(56 * 56 * 64).astype(np.float32)
    w = (rng.standard_normal(9 * 64 * 64) * (2.0 / 576) ** 0.5).astype(np.float32)
    orc.conv2d_forward_f32(x, w, p)  # warm-up, also loads the library
    t0 = time.perf_counter()
    orc.conv2d_forward_f32(x, w, p)
    per_image = max(time.perf_counter() - t0, 1e-4)
    batch = int(max(1, min(64, seconds_target / per_image)))
    p = orc.conv_params(batch, 56, 56, 64, 64, 3, 1, True)
    x = rng.standard_normal(batch * 56 * 56 * 64).astype(np.float32)
    reps = int(max(1, seconds_target / (per_image * batch)))
    t0 = time.perf_counter()
    for _ in range(reps):
        orc.conv2d_forward_f32(x, w, p)
    dt = time.perf_counter() - t0
    flops = 2.0 * reps * batch * 56 * 56 * 9 * 64 * 64
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": "3x3 s1 56x56x64->64 fp32 forward (ResNet-50 stage 1), batch %d x %d passes, %.1f s, OpenMP "
                      "direct convolution restating portDNN's direct kernel, %d threads" % (batch, reps, dt, threads)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    from oracle import oracle as orc
    from portdnn_b200 import workloads
    layers = [l for l in workloads.resnet50_v15(1) if isinstance(l, workloads.ConvLayer)]
    rng = np.random.default_rng(0)
    tensors = []
    for l in layers:
        p = l.params
        po = orc.ConvParams(*[getattr(p, f) for f, _ in p._fields_])
        x = rng.standard_normal(p.in_rows * p.in_cols * p.channels).astype(np.float32)
        w = (rng.standard_normal(p.window_rows * p.window_cols * p.channels * p.features) *
             (2.0 / (p.window_rows * p.window_cols * p.channels)) ** 0.5).astype(np.float32)
        tensors.append((po, x, w))
    flops = sum(l.flops for l in layers)

    def step():
        for po, x, w in tensors:
            orc.conv2d_forward_f32(x, w, po)

    for _ in range(max(1, min(args.warmup, 2))):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    value = flops * args.steps / dt / 1e12
    sample = ("one image (batch 1 of the batch-256 workload: all 53 convolutions, fp32, OpenMP direct convolution "
              "restating portDNN's direct kernel, %d threads) per step" % threads)
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 5), "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "ResNet-50 v1.5 conv stack forward, NHWC, bounded sample of the batch-256 job",
                       "sample": sample, "host_threads": threads},
            "cpu_baseline": {"value": round(value, 5), "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": round(value, 5), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# GPU arm: helpers
# ------------------------------------------------------------------------------------------------
def capture_graph(torch, fn):
    """One eager run on a side stream (so that nothing is allocated during capture), then the capture."""
    stream = torch.cuda.current_stream()
    side = torch.cuda.Stream()
    side.wait_stream(stream)
    with torch.cuda.stream(side):
        fn()
    stream.wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


def timed(torch, fn, reps, barrier=None):
    """Milliseconds per call of fn over `reps` back-to-back calls, CUDA events on the current stream."""
    if barrier:
        barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    if barrier:
        barrier()
    else:
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def hbm_operators(torch, pd, workloads, peak_gbs, full=False):
    """GB/s of the HBM-bound operators on the benchmark networks' shapes: CUDA events over three replays
    of a CUDA graph of 20 launches, after warm-ups, algorithmic bytes (every tensor once; the max-pool gradient reads x, y, dy and writes
    dx; counters of bench/depthwise_conv2d/base_depthwise_convolution_fixture.h:77-79 and
    bench/pooling/base_pooling_fixture.h:72-73) / time.  Tensors are larger than the 126 MB L2 except
    where the name says so."""
    rows = []

    def add(name, fn, nbytes):
        for _ in range(3):
            fn()
        # 20 launches replayed as one CUDA graph: a host loop cannot issue the short kernels (5-15 us) as
        # fast as they run, and its time would be the host's
        graph = capture_graph(torch, lambda: [fn() for _ in range(20)])
        graph.replay()
        ms = timed(torch, graph.replay, 3) / 20
        rows.append({"op": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 0),
                     "frac": round(nbytes / ms / 1e6 / peak_gbs, 3)})
        return ms

    dev, f16 = "cuda", torch.float16
    # MobileNet-v2 depthwise 3x3 forward, batch 128 (the 17 layers, and the four larger than L2 by name)
    tot_b = tot_ms = 0.0
    for idx, p in enumerate(workloads.mobilenet_v2_depthwise(128)):
        x = torch.randn(p.batch * p.in_rows * p.in_cols * p.channels, device=dev).half()
        w = torch.randn(9 * p.channels, device=dev).half()
        y = torch.empty(p.batch * p.out_rows * p.out_cols * p.channels, device=dev, dtype=f16)
        nb = 2 * (x.numel() + w.numel() + y.numel())
        name = "depthwise fwd %dx%dx%d s%d f16 b128" % (p.in_rows, p.in_cols, p.channels, p.stride_rows)
        keep = len(rows)
        ms = add(name, lambda: pd.depthwise_conv2d(pd.FORWARD, x, w, p, out=y), nb)
        if idx >= 4 and not full:
            del rows[keep:]
        tot_b, tot_ms = tot_b + nb, tot_ms + ms
    rows.append({"op": "depthwise fwd, MobileNet-v2, all 17 layers f16 b128 (13 of them L2-resident)", "ms": round(tot_ms, 4),
                 "gbs": round(tot_b / tot_ms / 1e6, 0), "frac": round(tot_b / tot_ms / 1e6 / peak_gbs, 3)})
    for (s, c, st) in ((112, 96, 2), (56, 144, 1)) + (((14, 384, 1),) if full else ()):
        p = pd.depthwise_params(128, s, s, c, 1, 3, st)
        x = torch.randn(p.batch * s * s * c, device=dev).half()
        w = torch.randn(9 * c, device=dev).half()
        dy = torch.randn(p.batch * p.out_rows * p.out_cols * c, device=dev).half()
        dx, dw = torch.empty_like(x), torch.empty_like(w)
        nb = 2 * (x.numel() + w.numel() + dy.numel())
        add("depthwise input backprop %dx%dx%d s%d f16 b128" % (s, s, c, st),
            lambda: pd.depthwise_conv2d(pd.INPUT_BACKPROP, dy, w, p, out=dx), nb)
        add("depthwise filter backprop %dx%dx%d s%d f16 b128" % (s, s, c, st),
            lambda: pd.depthwise_conv2d(pd.FILTER_BACKPROP, x, dy, p, out=dw), nb)
    pools = [("max pool 3x3/2 SAME 256x112x112x64 f16 (ResNet stem)", 256, 112, 64, 3, 2, True, f16, pd.POOL_MAX),
             ("max pool 2x2/2 64x224x224x64 f32 (VGG)", 64, 224, 64, 2, 2, False, torch.float32, pd.POOL_MAX),
             ("average pool 7x7 256x7x7x2048 f16 (26 MB, L2-resident)", 256, 7, 2048, 7, 1, False, f16, pd.POOL_AVERAGE)]
    for name, n, h, c, win, st, same, dt, op in pools:
        p = pd.pool_params(n, h, h, c, win, st, same)
        x = torch.randn(n * h * h * c, device=dev).to(dt)
        y = torch.empty(n * p.out_rows * p.out_cols * c, device=dev, dtype=dt)
        es = x.element_size()
        add(name, lambda: pd.pooling(op, 0, x, p, out=y), es * (x.numel() + y.numel()))
        dy, dx = torch.randn_like(y), torch.empty_like(x)
        if op == pd.POOL_MAX:
            add(name.replace("max pool", "max-pool gradient"), lambda: pd.pooling_max_grad(op, x, y, dy, p, out=dx),
                es * (2 * x.numel() + 2 * y.numel()))
        elif full:
            add(name.replace("average pool", "average-pool gradient"), lambda: pd.pooling(op, 1, dy, p, out=dx),
                es * (x.numel() + y.numel()))
    n = 256 * 56 * 56 * 256
    x = torch.randn(n, device=dev).half()
    y, b = torch.empty_like(x), torch.randn(256, device=dev).half()
    add("bias + ReLU 256x56x56x256 f16", lambda: pd.bias_add(x, b, 256, activation=pd.ACT_RELU, out=y), 4 * n)
    add("ReLU gradient 256x56x56x256 f16", lambda: pd.pointwise_grad(pd.ACT_RELU, x, y, out=y), 6 * n)
    if full:
        add("ReLU forward f16", lambda: pd.pointwise(pd.ACT_RELU, x, out=y), 4 * n)
        add("tanh forward f16", lambda: pd.pointwise(pd.ACT_TANH, x, out=y), 4 * n)
        z = torch.randn(n, device=dev).half()
        add("binary add, equal shapes f16", lambda: pd.binaryop(pd.BINARY_ADD, x, [256, 56, 56, 256], z, [256, 56, 56, 256], out=y), 6 * n)
        add("binary mul, [rows,C] x [1,C] f16", lambda: pd.binaryop(pd.BINARY_MUL, x, [256 * 56 * 56, 256], b, [1, 256], out=y), 4 * n)
        del z
        beta, gamma, mean = (torch.randn(256, device=dev).half() for _ in range(3))
        var = (torch.rand(256, device=dev) + 0.5).half()
        dyb = torch.randn_like(x)
        for training in (False, True):
            pb = pd.batchnorm_params(256, 56, 56, 256, training)
            tag = "training" if training else "frozen"
            add("batchnorm forward %s f16" % tag, lambda: pd.batchnorm_forward(x, beta, gamma, mean, var, pb, out=y),
                (8 if training else 4) * n)
            add("batchnorm gradient %s f16" % tag,
                lambda: pd.batchnorm_gradient(x, dyb, gamma, pb, pop_mean=mean, pop_variance=var, out=y), (10 if training else 8) * n)
        xs = torch.randn(64 * 56 * 56 * 256, device=dev).half()
        ys = torch.empty_like(xs)
        add("softmax forward 64x56x56x256 f16", lambda: pd.softmax(xs, 64, 56, 56, 256, out=ys), 4 * xs.numel())
    return rows


def parity_check(torch, pd, workloads, net, images=(0, BATCH - 1), tol=2e-2):
    """Layer-by-layer check of the batch-256 run against the CPU oracle on a few images: every layer of
    the runner (a training-mode one, which keeps all activations) is recomputed by the oracle from the
    GPU's own input of that layer for the sampled images, as tests/test_gpu_workloads.py does at batch 2."""
    from oracle import oracle as orc
    host_threads()
    worst, worst_name, checked = 0.0, "", 0
    batch = net.layers[0].params.batch

    def rows(t, i_img):
        per = t.numel() // batch
        return t[i_img * per:(i_img + 1) * per].float().cpu().numpy()

    for i, l in enumerate(net.layers):
        p, j = l.params, net.src_idx[i]
        src = net.input if j < 0 else net.acts[j]
        for img in images:
            x, got = rows(src, img), rows(net.acts[i], img)
            if isinstance(l, workloads.ConvLayer):
                po = orc.ConvParams(*[getattr(p, f) for f, _ in p._fields_])
                po.batch = 1
                y = orc.conv2d(orc.FORWARD, x, net.weights[i].float().cpu().numpy(), po)
                y = torch.from_numpy(y).half().float().numpy().reshape(-1, p.features)
                y = torch.from_numpy(y + net.biases[i].float().cpu().numpy()[None, :]).half().float().numpy().ravel()
                ref = np.maximum(y, 0) if l.activation == pd.ACT_RELU else y
            else:
                po = orc.PoolParams(*[getattr(p, f) for f, _ in p._fields_])
                po.batch = 1
                ref = orc.pool_forward(l.op, x, po)
            diff = np.abs(got.astype(np.float64) - ref)
            rms = max(float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))), 1e-30)
            e = max(float(diff.max()) / max(float(np.abs(ref).max()), 1e-30), float((diff / (np.abs(ref) + rms)).max()))
            checked += got.size
            if e > worst:
                worst, worst_name = e, l.name
    return {"max_rel": float("%.3g" % worst), "tolerance": tol, "ok": bool(worst <= tol), "worst_layer": worst_name,
            "checked_values": int(checked),
            "what": "every layer's output for images %s of the batch-%d run against the CPU oracle fed the GPU's own "
                    "input of that layer; max over layers of max(max-norm, element-wise) relative error" % (list(images), batch)}


def run_layer_mode(args):
    import torch
    import portdnn_b200 as pd
    n, h, w, c, k, win, st = args.layer
    dt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[args.dtype]
    p = pd.conv_params(n, h, w, c, k, win, st)
    x = torch.randn(n * h * w * c, device="cuda").to(dt)
    wt = (torch.randn(win * win * c * k, device="cuda") * (2.0 / (win * win * c)) ** 0.5).to(dt)
    b = torch.zeros(k, device="cuda").to(dt)
    y = torch.empty(n * p.out_rows * p.out_cols * k, device="cuda", dtype=dt)
    flops = 2 * n * p.out_rows * p.out_cols * win * win * c * k
    ws = None
    if args.algorithm not in (pd.ALGO_TILED, pd.ALGO_IM2COL):
        ws = torch.empty(max(pd.conv2d_workspace_size(pd.FORWARD, {"f16": 1, "bf16": 2, "f32": 0}[args.dtype], p,
                                                      args.algorithm)[1], 1), device="cuda", dtype=dt)
    if args.conv_pass == "forward":
        run = lambda: pd.conv2d(pd.FORWARD, x, wt, p, algorithm=args.algorithm, out=y, bias=b, activation=pd.ACT_RELU,
                                workspace=ws)
    elif args.conv_pass == "input_backprop":  # with the ReLU-gradient mask of the producing layer fused in
        dx = torch.empty_like(x)
        mask = torch.relu(x) if dt != torch.float32 else None
        run = lambda: pd.conv2d(pd.INPUT_BACKPROP, y, wt, p, algorithm=args.algorithm, out=dx, workspace=ws,
                                relu_forward_output=mask)
        y.copy_(torch.randn(y.numel(), device="cuda").to(dt))
    else:  # filter backprop into fp32 gradients, as the training step asks for them
        dw = torch.empty(wt.numel(), device="cuda", dtype=torch.float32)
        y.copy_(torch.randn(y.numel(), device="cuda").to(dt))
        f32_out = dt != torch.float32
        run = lambda: pd.conv2d(pd.FILTER_BACKPROP, x, y, p, algorithm=args.algorithm, out=dw if f32_out else None,
                                workspace=ws, output_f32=f32_out)
    evs = []
    for _ in range(args.reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        evs.append((e0, e1))
    torch.cuda.synchronize()
    for e0, e1 in evs:
        ms = e0.elapsed_time(e1)
        print("ms %.4f  TFLOP/s %.1f" % (ms, flops / ms / 1e9))
    # a single launch bracketed by events includes the launch latency of an idle device (tens of microseconds
    # for the short layers); 20 launches replayed as a CUDA graph give the time of the kernel itself
    graph = capture_graph(torch, lambda: [run() for _ in range(20)])
    graph.replay()
    ms = timed(torch, graph.replay, 3) / 20
    print("graph replay of 20 launches: ms %.4f  TFLOP/s %.1f" % (ms, flops / ms / 1e9))
    print("device error record", pd.device_error_record())


def run_other_workload(args):
    """The other benchmark configurations, one JSON line each (not the headline): --workload vgg16 is the
    VGG-16 conv stack in fp32 (3xTF32), batch 64, forward and training step; --workload mobilenet is the
    dense convolutions of MobileNet-v2 in fp16, batch 128 (its depthwise layers are in the `hbm` block of the
    default run); --workload layer0 is the single 3x3 56x56x256->256 fp32 layer at batch 1."""
    import torch
    import portdnn_b200 as pd
    from portdnn_b200 import workloads
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    peaks = load_peaks()
    out = {"workload": args.workload, "unit": UNIT, "steps": args.steps}
    if args.workload == "layer0":
        p = pd.conv_params(1, 56, 56, 256, 256, 3, 1)
        g = torch.Generator(device=device).manual_seed(0)
        x = (torch.rand(56 * 56 * 256, device=device, generator=g) * 2 - 1)
        w = (torch.rand(9 * 256 * 256, device=device, generator=g) * 2 - 1) * (1.0 / 2304) ** 0.5
        y = torch.empty(56 * 56 * 256, device=device)
        flops = 2 * 56 * 56 * 9 * 256 * 256
        for algo, name in ((pd.ALGO_IM2COL, "implicit_gemm_3xtf32"), (pd.ALGO_WINOGRAD, "winograd_f2x2_unfused")):
            _, rec = pd.conv2d_workspace_size(pd.FORWARD, pd.F32, p, algo)
            ws = torch.empty(max(rec, 1), device=device)
            fn = lambda: pd.conv2d(pd.FORWARD, x, w, p, algorithm=algo, out=y, workspace=ws)
            for _ in range(5):
                fn()
            ms = timed(torch, fn, max(args.steps, 50))
            out[name] = {"us": round(ms * 1e3, 2), "value": round(flops / (ms * 1e-3) / 1e12, 2)}
        print(json.dumps(out))
        return
    if args.workload == "vgg16":
        layers, dtype, batch = workloads.vgg16(64), torch.float32, 64
    else:
        layers, dtype, batch = workloads.mobilenet_v2_convs(128), torch.float16, 128
    net = workloads.ConvStackRunner(layers, device, seed=7, dtype=dtype)
    for _ in range(3):
        net.forward()
    step = capture_graph(torch, net.forward).replay
    for _ in range(3):
        step()
    ms = timed(torch, step, args.steps)
    out.update({"dtype": "f32 (3xTF32)" if dtype == torch.float32 else "f16", "batch": batch,
                "forward": {"ms_per_step": round(ms, 4), "value": round(net.flops_forward / (ms * 1e-3) / 1e12, 2),
                            "flops_per_step": net.flops_forward}})
    if args.workload == "vgg16":
        del net
        tnet = workloads.ConvStackRunner(layers, device, seed=7, dtype=dtype, training=True)
        for _ in range(2):
            tnet.forward()
            tnet.backward()
        ms_t = timed(torch, lambda: (tnet.forward(), tnet.backward()), max(3, args.steps // 4))
        out["train"] = {"ms_per_step": round(ms_t, 4), "value": round(tnet.flops_train / (ms_t * 1e-3) / 1e12, 2),
                        "flops_per_step": tnet.flops_train}
        # fp32 is credited at direct FLOPs against a third of the TF32 peak (half the bf16 peak)
        out["frac_of_tf32_peak_over_3"] = round(out["forward"]["value"] / (peaks["tflops_burst"] / 2 / 3), 3)
    err = pd.device_error_record()
    if err[0] != 0:
        raise SystemExit("bench.py: tensor-core kernel reported %s" % err)
    print(json.dumps(out))


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from portdnn_b200 import build
    if rank == 0:
        build.build()
    if world > 1:
        dist.barrier()
    import portdnn_b200 as pd
    from portdnn_b200 import dist as pdist
    from portdnn_b200 import workloads
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(*vals):
        t = torch.tensor(list(vals), dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    if args.hbm_table:
        for r in hbm_operators(torch, pd, workloads, peaks["hbm_gbs"], full=True):
            print("%-78s %8.4f ms %6.0f GB/s  %.2f of %s peak" % (r["op"], r["ms"], r["gbs"], r["frac"], peaks["source"]))
        return

    train_only = args.workload == "train"
    stream = torch.cuda.current_stream()
    warmup = max(args.warmup, 3)
    # each rank holds its own 256-image shard of the global batch (weak scaling)
    net = workloads.ConvStackRunner(workloads.resnet50_v15(BATCH), device, seed=1234 + rank)
    result = net.forward()  # what a step hands back to the host: the pooled features
    host_in = torch.empty(net.input.numel(), dtype=torch.float16).pin_memory()
    host_in.copy_(net.input.cpu())
    host_out = torch.empty(result.numel(), dtype=result.dtype).pin_memory()
    for _ in range(warmup):
        net.forward()
    barrier()
    err = pd.device_error_record()
    if err[0] != 0:
        raise SystemExit("bench.py: tensor-core kernel reported %s" % err)

    # ---- timed region: inputs resident in HBM ----
    # One step = the 55 launches of the stack, captured once into a CUDA graph and replayed per step,
    # so that host-side launch cost (tensor-map encoding, ctypes) does not sit between kernels;
    # --no-graph times plain stream launches instead.
    l0 = pd.launch_count()
    net.forward()
    launches_per_step = pd.launch_count() - l0
    if args.no_graph:
        step = net.forward
    else:
        graph = capture_graph(torch, net.forward)
        step = graph.replay
    for _ in range(warmup):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms = timed(torch, step, args.steps, barrier)
    clocks = sampler.stop() if rank == 0 else None

    # ---- the convolutions inside the step: step time minus a graph of the step's other kernels ----
    other_ids = [i for i, l in enumerate(net.layers) if not isinstance(l, workloads.ConvLayer)]

    def others():
        for i in other_ids:
            net.run_layer(i)
    other_step = others if args.no_graph else capture_graph(torch, others).replay
    for _ in range(warmup):
        other_step()
    ms_other = timed(torch, other_step, args.steps, barrier)

    # ---- end to end: host buffers in, result out, every copy inside the timed region ----
    # Each step's input crosses PCIe from pinned host memory and its result is read back.  The
    # upload of step i+1 runs on a second stream into a staging buffer while step i computes; a
    # device-to-device copy moves it into the network's input just before the step runs.
    copy_stream = torch.cuda.Stream()
    staging = torch.empty_like(net.input)
    uploaded = [torch.cuda.Event() for _ in range(args.steps + 1)]
    consumed = [torch.cuda.Event() for _ in range(args.steps + 1)]
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    copy_stream.wait_stream(stream)
    with torch.cuda.stream(copy_stream):
        staging.copy_(host_in, non_blocking=True)
        uploaded[0].record(copy_stream)
    for i in range(args.steps):
        stream.wait_event(uploaded[i])
        net.input.copy_(staging, non_blocking=True)
        consumed[i].record(stream)
        if i + 1 < args.steps:
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[i])
                staging.copy_(host_in, non_blocking=True)
                uploaded[i + 1].record(copy_stream)
        step()
        host_out.copy_(result, non_blocking=True)
    e1.record(stream)
    barrier()
    ms_e2e = e0.elapsed_time(e1) / args.steps
    del staging

    # ---- sustained: the same step back to back for at least two seconds ----
    sustained = None
    if not args.quick:
        reps = int(max(args.steps, 2200.0 / ms))
        s2 = ClockSampler(local_rank)
        if rank == 0:
            s2.start()
        ms_sus = timed(torch, step, reps, barrier)
        c2 = s2.stop() if rank == 0 else None
        (ms_sus,) = max_over_ranks(ms_sus)
        if rank == 0:
            v = net.flops_forward * world / (ms_sus * 1e-3) / 1e12
            sustained = {"ms_per_step": round(ms_sus, 4), "value": round(v, 2), "unit": UNIT, "steps": reps,
                         "seconds": round(ms_sus * reps / 1e3, 2), "clocks": c2,
                         "ms_x_median_sm_mhz": round(ms_sus * c2["sm_mhz"], 1) if c2 and c2.get("sm_mhz") else None,
                         "frac_of_sustained_peak_per_gpu": round(v / world / peaks["tflops_sustained"], 4)}

    # ---- per-layer times (plain launches with events between them; --layers only) ----
    per_layer = None
    if args.layers and rank == 0:
        conv_ids = [i for i, l in enumerate(net.layers) if isinstance(l, workloads.ConvLayer)]
        evs = {i: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for i in conv_ids}
        acc = {i: 0.0 for i in conv_ids}
        for _ in range(5):
            for i in range(len(net.layers)):
                if i in evs:
                    evs[i][0].record(stream)
                net.run_layer(i)
                if i in evs:
                    evs[i][1].record(stream)
            torch.cuda.synchronize()
            for i in conv_ids:
                acc[i] += evs[i][0].elapsed_time(evs[i][1]) / 5
        per_layer = [{"layer": net.layers[i].name, "ms": round(acc[i], 4),
                      "tflops": round(net.layers[i].flops / (acc[i] * 1e-3) / 1e12, 1),
                      "gbs": round(net.layers[i].ideal_bytes / (acc[i] * 1e-3) / 1e9, 0)} for i in conv_ids]

    final_forward = result.clone()

    # ---- training step: forward, both backprops, filter gradients all-reduced stage by stage ----
    train = None
    tnet = None
    if not args.quick or train_only:
        tnet = workloads.ConvStackRunner(workloads.resnet50_v15(BATCH), device, seed=1234 + rank, training=True)
        for _ in range(2):
            tnet.forward()
            tnet.backward()
        torch.cuda.synchronize()
        l0 = pd.launch_count()
        tnet.forward()
        tnet.backward()
        train_launches = pd.launch_count() - l0
        side = torch.cuda.Stream()
        # the gradient sum goes through the library's own C-ABI collective (pdnn_allreduce_filter_grads)
        comm = pdist.GradientComm(rank, world) if world > 1 else None
        if args.no_graph:
            fwd_step, seg_steps = tnet.forward, [(lambda s=s: tnet.backward_segment(s)) for s in tnet.segments]
        else:
            fwd_step = capture_graph(torch, tnet.forward).replay
            tnet.backward_begin()
            seg_steps = []
            for seg in tnet.segments:  # captured in the order they run: the routing state carries over
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    tnet.backward_segment(seg)
                seg_steps.append(g.replay)
        ready = [torch.cuda.Event() for _ in tnet.segments]

        def train_step(reduce=True):
            fwd_step()
            if args.no_graph:
                tnet.backward_begin()
            for k, (seg, run) in enumerate(zip(tnet.segments, seg_steps)):
                run()
                if reduce and world > 1 and seg["bucket"] is not None:
                    # this stage's filter gradients are complete: sum them over ranks on the side
                    # stream while the backward pass of the earlier stages continues
                    ready[k].record(stream)
                    side.wait_event(ready[k])
                    with torch.cuda.stream(side):
                        tnet.bucket.all_reduce(span=seg["bucket"], comm=comm)
            stream.wait_stream(side)

        tsteps = max(5, min(args.steps, 20))
        for _ in range(3):
            train_step()
        ms_train = timed(torch, train_step, tsteps, barrier)
        ms_train_local = timed(torch, lambda: train_step(False), tsteps, barrier) if world > 1 else ms_train
        ms_train, ms_train_local = max_over_ranks(ms_train, ms_train_local)
        err = pd.device_error_record()
        if err[0] != 0:
            raise SystemExit("bench.py: tensor-core kernel reported %s in the training step" % err)
        train = {"ms_per_step": round(ms_train, 4), "value": round(tnet.flops_train * world / (ms_train * 1e-3) / 1e12, 2),
                 "unit": UNIT, "steps": tsteps, "launches": int(train_launches),
                 "allreduce_ms": round(max(ms_train - ms_train_local, 0.0), 4),
                 "allreduce": "fp32 filter gradients, %d floats, one pdnn_allreduce_filter_grads (ncclAllReduce) per stage "
                              "(5 per step) on a second stream, started when that stage's filter backprop is done"
                              % tnet.bucket.total,
                 "flops_per_step_per_gpu": tnet.flops_train,
                 "frac_of_sustained_peak_per_gpu": round(tnet.flops_train / (ms_train * 1e-3) / 1e12 / peaks["tflops_sustained"], 4)}

    ms, ms_e2e, ms_other = max_over_ranks(ms, ms_e2e, ms_other)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- single-GPU extras on rank 0 ----
    parity = hbm = None
    if not args.quick:
        if tnet is not None:
            tnet.forward()
            torch.cuda.synchronize()
            parity = parity_check(torch, pd, workloads, tnet)
            same = bool(torch.equal(tnet.acts[len(tnet.layers) - 1], final_forward))
            parity["timed_forward_equals_checked_run"] = same
            parity["ok"] = bool(parity["ok"] and same)
        del tnet
        torch.cuda.empty_cache()
        if world == 1:
            hbm = hbm_operators(torch, pd, workloads, peaks["hbm_gbs"])

    flops = net.flops_forward
    value = flops * world / (ms * 1e-3) / 1e12
    e2e_value = flops * world / (ms_e2e * 1e-3) / 1e12
    conv_ms = ms - ms_other
    achieved = flops / (conv_ms * 1e-3) / 1e12
    region_s = ms * args.steps / 1e3
    peak_kind = "burst" if region_s < 1.0 else "sustained"
    peak = peaks["tflops_burst"] if peak_kind == "burst" else peaks["tflops_sustained"]
    if train_only and train is not None:
        value, ms, flops = train["value"], train["ms_per_step"], train["flops_per_step_per_gpu"]
    line = {
        "metric": METRIC if not train_only else METRIC.replace("forward", "train_step"), "value": round(value, 2),
        "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": "ResNet-50 v1.5 conv stack forward, NHWC fp16, batch 256 per GPU, 53 convs with fused "
                               "bias (+ReLU on all but the 4 projection shortcuts), 3x3/2 max pool, global 7x7 average pool" if not train_only else
                               "ResNet-50 v1.5 training-step convs, NHWC fp16, batch 256 per GPU (the `train` object)",
                   "batch_per_gpu": BATCH, "global_batch": BATCH * world, "sharding": "batch, no forward collective",
                   "l2": "activations (103-411 MB per layer) exceed the 126 MB L2; no explicit flush",
                   "flops_per_step_per_gpu": flops,
                   "launch": "plain stream launches" if args.no_graph else "CUDA graph replay of one step"},
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": host_in.numel() * 2,
                "d2h_bytes_per_step": host_out.numel() * host_out.element_size(), "ms_per_step": round(ms_e2e, 4)},
        "gpu_launches": int(launches_per_step * args.steps),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "umma_gemm_kernel (the 53 forward implicit-GEMM conv launches of a step, "
                                                  "timed inside the replayed step: step minus its other kernels)",
                     "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                     "traffic": FORWARD_DRAM_BYTES_PER_LAUNCH,
                     "peak_source": "%s (%s bf16 matmul; the timed region lasts %.2f s)" % (peaks["source"], peak_kind, region_s),
                     "avg_launch_ms": round(conv_ms / 53, 4), "conv_ms_per_step": round(conv_ms, 4),
                     "other_kernels_ms_per_step": round(ms_other, 4),
                     "frac_of_burst_peak": round(achieved / peaks["tflops_burst"], 4),
                     "frac_of_sustained_peak": round(achieved / peaks["tflops_sustained"], 4)},
    }
    if sustained is not None:
        line["sustained"] = sustained
    if train is not None:
        line["train"] = train
    if hbm is not None:
        line["hbm"] = hbm
    if parity is not None:
        line["parity_check"] = parity
    if world == 1 and not args.quick:
        line["cpu_baseline"] = cpu_baseline_sample()
    print(json.dumps(line))
    if per_layer is not None:
        print(json.dumps(per_layer, indent=1))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="forward", choices=["forward", "train", "vgg16", "mobilenet", "layer0"],
                    help="forward: the headline conv stack; train: report the training step as the headline value; "
                         "vgg16 / mobilenet / layer0: the other benchmark configurations, one line each")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of replaying a CUDA graph")
    ap.add_argument("--quick", action="store_true", help="only the headline measurement (no sustained / train / hbm / parity / cpu legs)")
    ap.add_argument("--layers", action="store_true", help="after the JSON line, print per-layer times of the forward stack")
    ap.add_argument("--hbm-table", action="store_true", help="print every HBM-bound operator's bandwidth and exit")
    ap.add_argument("--layer", type=int, nargs=7, metavar=("N", "H", "W", "C", "K", "WINDOW", "STRIDE"),
                    help="time one forward convolution layer (fused bias + ReLU) and exit")
    ap.add_argument("--pass", dest="conv_pass", default="forward", choices=["forward", "input_backprop", "filter_backprop"],
                    help="which convolution pass --layer runs")
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16", "f32"])
    ap.add_argument("--algorithm", type=int, default=3, help="PdnnAlgorithm for --layer (3 im2col tag = implicit GEMM, 4 Winograd)")
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.layer:
        run_layer_mode(args)
    elif args.workload in ("vgg16", "mobilenet", "layer0"):
        run_other_workload(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
