#!/usr/bin/env python
"""Headline benchmark: ResNet-50 v1.5 conv stack, forward, fp16 in / fp32 accumulate, NHWC,
batch 256 per GPU, through the C ABI of libportdnn_b200.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line on rank 0.  `value` is conv TFLOP/s (2*N*Ho*Wo*R*S*C*K summed over the 53
convolutions, the reference's forward counter, bench/conv2d/base_convolution_fixture.h:85-88)
over the whole job with inputs resident in HBM; `e2e` is the same metric with the step's input
copied from pinned host memory and the pooled result copied back inside the timed region.
With --impl reference the same network is timed on the host cores with the CPU restatement of
portDNN's direct kernel (portDNN itself is SYCL and cannot be built with this toolchain).
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
# dram__bytes_read.sum + dram__bytes_write.sum of the 53 conv launches of one forward step, from an
# ncu capture of this script (profiles/bench_resnet50_forward_dram_traffic.md): 5003 MB read +
# 3486 MB written = 8489 MB per step, against 11.76 GB of algorithmic bytes (input + filter + output
# of every layer once) - the small feature maps are still in L2 when the next layer reads them.
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
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def cpu_baseline_sample(seconds_target=12.0):
    """Times the CPU oracle's float forward conv on one ResNet stage-1 3x3 layer at a batch sized
    for ~10-20 s of CPU work; returns the cpu_baseline object."""
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
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
            "sample": "3x3 s1 56x56x64->64 fp32 forward (ResNet-50 stage 1), batch %d x %d passes, %.1f s, OpenMP "
                      "direct convolution restating portDNN's direct kernel" % (batch, reps, dt)}


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
    from portdnn_b200 import workloads

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    train = args.workload == "train"
    # each rank holds its own 256-image shard of the global batch (weak scaling)
    net = workloads.ConvStackRunner(workloads.resnet50_v15(BATCH), device, seed=1234 + rank, training=train)
    step = net.train_step if train else net.forward
    step_flops = net.flops_train if train else net.flops_forward
    stream = torch.cuda.current_stream()
    result = net.bucket.buffer if train else net.forward()  # what a step hands back to the host
    host_in = torch.empty(net.input.numel(), dtype=torch.float16).pin_memory()
    host_in.copy_(net.input.cpu())
    host_out = torch.empty(result.numel(), dtype=result.dtype).pin_memory()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    err = pd.device_error_record()
    if err[0] != 0:
        raise SystemExit("bench.py: tensor-core kernel reported %s" % err)

    # ---- timed region: inputs resident in HBM ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    # One step = the 55 launches of the stack.  They are captured once into a CUDA graph and the
    # graph is replayed per step, so that host-side launch cost (tensor-map encoding, ctypes) does
    # not sit between kernels; --no-graph times plain stream launches instead.
    graph = None

    def compute():  # the kernels of one step; the filter-gradient all-reduce of a training step stays outside the graph
        net.forward()
        if train:
            net.backward()

    def replay():
        graph.replay()
        if train:
            net.bucket.all_reduce()

    if not args.no_graph:
        side = torch.cuda.Stream()
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            compute()
        stream.wait_stream(side)
        torch.cuda.synchronize()
        l0 = pd.launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            compute()
        launches_per_step = pd.launch_count() - l0
        replay()
        barrier()
    else:
        l0 = pd.launch_count()
        step()
        launches_per_step = pd.launch_count() - l0
        barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        if graph is not None:
            replay()
        else:
            step()
    ev1.record(stream)
    barrier()
    ms = ev0.elapsed_time(ev1)
    launches = launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None

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
        if graph is not None:
            replay()
        else:
            step()
        host_out.copy_(result, non_blocking=True)
    e1.record(stream)
    barrier()
    ms_e2e = e0.elapsed_time(e1)

    # ---- per-launch durations of the dominant kernel (the implicit-GEMM convolutions) ----
    conv_ids = [i for i, l in enumerate(net.layers) if isinstance(l, workloads.ConvLayer)]
    conv_layers = [net.layers[i] for i in conv_ids]
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in conv_layers]
    prof_steps = min(args.steps, 5)
    conv_ms = [0.0] * len(conv_layers)
    for _ in range(prof_steps):
        k = 0
        for i in range(len(net.layers)):
            if i in conv_ids:
                evs[k][0].record(stream)
                net.run_layer(i)
                evs[k][1].record(stream)
                k += 1
            else:
                net.run_layer(i)
        torch.cuda.synchronize()
        for j, (a, b) in enumerate(evs):
            conv_ms[j] += a.elapsed_time(b) / prof_steps

    times = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, ms_e2e = times.tolist()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    total_flops = step_flops * world * args.steps
    value = total_flops / (ms * 1e-3) / 1e12
    e2e_value = total_flops / (ms_e2e * 1e-3) / 1e12
    # forward convolutions, one umma_gemm_kernel launch each (the stem's interval also holds its
    # two small packing kernels)
    tc = list(zip(conv_layers, conv_ms))
    tc_flops = sum(l.flops for l, _ in tc)
    tc_ms = sum(t for _, t in tc)
    achieved = tc_flops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0
    per_layer = [{"layer": l.name, "ms": round(t, 4), "tflops": round(l.flops / (t * 1e-3) / 1e12, 1),
                  "gbs": round(l.ideal_bytes / (t * 1e-3) / 1e9, 0)} for l, t in zip(conv_layers, conv_ms)]
    os.makedirs(os.path.join(ROOT, "gpurun_out"), exist_ok=True)
    with open(os.path.join(ROOT, "gpurun_out", "bench_layers.json"), "w") as f:
        json.dump(per_layer, f, indent=1)

    line = {
        "metric": METRIC if not train else METRIC.replace("forward", "train_step"), "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": ("ResNet-50 v1.5 conv stack forward, NHWC fp16, batch 256 per GPU, 53 convs with fused "
                                "bias+ReLU, 3x3/2 max pool, global 7x7 average pool") if not train else
                               ("ResNet-50 v1.5 training-step convs, NHWC fp16, batch 256 per GPU: forward, ReLU/pool "
                                "gradients, filter backprop and input backprop of all 53 convs, one fp32 all-reduce "
                                "of the filter gradients"),
                   "batch_per_gpu": BATCH, "global_batch": BATCH * world,
                   "sharding": "batch, no forward collective" if not train else "batch, one NCCL all-reduce per step",
                   "l2": "activations (103-411 MB per layer) exceed the 126 MB L2; no explicit flush",
                   "flops_per_step_per_gpu": step_flops,
                   "launch": "plain stream launches" if graph is None else "CUDA graph replay of one step"},
        "e2e": {"value": round(e2e_value, 2), "unit": UNIT, "h2d_bytes_per_step": host_in.numel() * 2,
                "d2h_bytes_per_step": host_out.numel() * host_out.element_size(), "ms_per_step": round(ms_e2e / args.steps, 4)},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "umma_gemm_kernel (the 53 forward implicit-GEMM conv launches of a step)",
                     "achieved": round(achieved, 1), "peak": peaks["tflops_sustained"], "unit": "TFLOP/s",
                     "frac": round(achieved / peaks["tflops_sustained"], 4),
                     "traffic": None if train else FORWARD_DRAM_BYTES_PER_LAUNCH,
                     "peak_source": "%s (sustained bf16 matmul)" % peaks["source"],
                     "avg_launch_ms": round(tc_ms / max(len(tc), 1), 4)},
        "cpu_baseline": cpu_baseline_sample(),
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# reference arm: the CPU restatement on the host cores
# ------------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
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
              "restating portDNN's direct kernel) per step")
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 5), "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt / args.steps * 1e3, 2),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "ResNet-50 v1.5 conv stack forward, NHWC, bounded sample of the batch-256 job",
                       "sample": sample},
            "cpu_baseline": {"value": round(value, 5), "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": round(value, 5), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="forward", choices=["forward", "train"],
                    help="forward: the headline conv stack; train: forward + both backprops + gradient all-reduce")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from the host instead of replaying a CUDA graph")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
