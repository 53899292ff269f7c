#!/usr/bin/env python
"""Benchmark of the int8 quantized-convolution path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One step = one pass of the hot path (quantize -> conv2d_quantized + add_bias + ReLU, fp32 NCHW output) over the
batch-32 shape sweep (five layers; see tennis_b200/workloads.py CONFIG1) on synthetic seeded inputs.  With
N > 1 every rank owns one GPU and runs the same sweep on its own shard (per-rank seed); there is no
data-path collective, only the barrier and the max-over-ranks of the device time.

The ten launches of a step are captured once in a CUDA graph and replayed inside the timed region (--eager times the
plain launches); every step is preceded by a 256 MiB write that flushes L2 and is timed with its own pair of CUDA events.

Prints ONE JSON line (rank 0):
  value        int8 TOPS of the whole job, inputs resident in HBM, device time from CUDA events
  e2e          the same metric through the host-buffer C-ABI call (H2D of the fp32 input and D2H of the fp32
               output inside the timed region, pinned host memory)
  roofline     the dominant kernel (tcgen05 implicit-GEMM convolution): algorithmic ops / measured launch time
  cpu_baseline the reference's own CPU operators (oracle/_ref) or the C port, timed on this box's host cores
               on a bounded sample
  config0, resnet50, cspdarknet53
               secondary figures: latency of the batch-1 layer of configuration 0 beside the reference's CPU time,
               images/s of the ResNet-50-shaped (configuration 2) and CSPDarknet53-shaped (configuration 3) networks
--impl reference times that CPU path alone and prints the same line shape.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TRAFFIC_RECORD = os.path.join(ROOT, "profiles", "conv_i8_tc_kernel_config1.md")


def ncu_traffic_record():
    """DRAM bytes per convolution launch from the ncu capture summarised under profiles/, valid only for the kernel source
    it was captured with: the summary carries the SHA-256 of tennis_b200/csrc/conv_tc.cu at capture time.  Returns
    (bytes or None, stale flag, note)."""
    import hashlib
    import re
    try:
        text = open(TRAFFIC_RECORD).read()
        m_bytes = re.search(r"dram_bytes_per_launch\s*=\s*([0-9.eE+]+)", text)
        m_hash = re.search(r"conv_tc_sha256\s*=\s*([0-9a-f]{64})", text)
        if not m_bytes or not m_hash:
            return None, True, "no traffic record in %s" % os.path.relpath(TRAFFIC_RECORD, ROOT)
        now = hashlib.sha256(open(os.path.join(ROOT, "tennis_b200", "csrc", "conv_tc.cu"), "rb").read()).hexdigest()
        if now != m_hash.group(1):
            return None, True, "the kernel source changed since the ncu capture in %s" % os.path.relpath(TRAFFIC_RECORD, ROOT)
        return float(m_bytes.group(1)), False, "ncu capture summarised in %s" % os.path.relpath(TRAFFIC_RECORD, ROOT)
    except OSError as e:
        return None, True, repr(e)

METRIC = "int8_conv_tops"
UNIT = "TOPS"
WORKLOAD = "config1: int8 conv2d shape sweep, batch 32 (1x1 256->1024@14, 3x3 128->128@28, 3x3/2 256->512@28, 1x1 2048->512@7, 7x7/2 3->64@224), fp32 NCHW out, bias+ReLU"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--eager", action="store_true", help="time plain launches instead of a CUDA-graph replay of the step")
    ap.add_argument("--no-resnet", action="store_true", help="skip the secondary ResNet-50-shaped network measurement")
    ap.add_argument("--no-csp", action="store_true", help="skip the secondary CSPDarknet53-shaped backbone measurement")
    ap.add_argument("--cpu-budget-s", type=float, default=20.0, help="host seconds the cpu_baseline sample may take")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_tflops=p["bf16_tflops"], bf16_tflops_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


# -------------------------------------------------------------------------------------------------------
# CPU arm (the reference's own operators where oracle/_ref exists, else the C port)
# -------------------------------------------------------------------------------------------------------
def cpu_sample(layers, images, workers, checker):
    """Seconds for one pass of `images` samples of every layer on `workers` host threads."""
    import numpy as np
    from tennis_b200 import workloads
    total = 0.0
    for layer in layers:
        small = dict(layer, n=images)
        d = workloads.make_layer_data(small, seed=0)
        pad = (layer["pad"],) * 4
        if checker.kind == "reference":
            sec, _ = checker.time_layer(d["x"], d["w"], pad, (layer["stride"],) * 2, (layer["dilation"],) * 2,
                                        float(d["qscale"]), d["dq"], d["bias"], act=1, workers=workers, repeats=1)
        else:
            t0 = time.perf_counter()
            xq = checker.quantize(d["x"], [float(d["qscale"])] * images)
            checker.conv_block(xq, d["w"], pad, (layer["stride"],) * 2, (layer["dilation"],) * 2, d["dq"], d["bias"], act="relu")
            sec = time.perf_counter() - t0
        total += sec
    return total


def cpu_arm(layers):
    from oracle import oracle as orc
    from tennis_b200 import workloads
    orc.build() if not os.path.exists(os.path.join(ROOT, "oracle", "liboracle.so")) else None
    checker = orc.best()
    cores = orc.usable_cpus()
    # the reference's int8 GEMM is serial inside one Workbench; all host cores are used by running one
    # Workbench per core on its own samples.  The C port parallelises inside one call with OpenMP.
    workers = cores if checker.kind == "reference" else 1
    images = 4       # of each layer on each worker: about a second of wall clock, 10-20 core-seconds of CPU work
    ops_per_pass = sum(workloads.layer_ops(dict(l, n=images)) for l in layers) * workers
    return checker, cores, workers, images, ops_per_pass


def run_reference(args):
    from tennis_b200 import workloads
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    layers = workloads.CONFIG1
    checker, cores, workers, images, ops_per_pass = cpu_arm(layers)
    budget = 150.0
    for _ in range(min(args.warmup, 1)):
        cpu_sample(layers, images, workers, checker)
    times = []
    t_begin = time.perf_counter()
    for _ in range(args.steps):
        times.append(cpu_sample(layers, images, workers, checker))
        if time.perf_counter() - t_begin > budget:
            break
    sec = sum(times) / len(times)
    value = ops_per_pass / sec / 1e12
    sample = "%d image(s) of each of the 5 layers per worker, %d worker(s) (%s), %d of %d steps timed" % (
        images, workers, "one Workbench with 1 computing thread per host core" if checker.kind == "reference" else "OpenMP inside the port",
        len(times), args.steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "steps_timed": len(times), "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores if checker.kind == "reference" else cores,
                         "kind": checker.kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# -------------------------------------------------------------------------------------------------------
# GPU arm
# -------------------------------------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.error = None

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            names = {
                getattr(pynvml, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
                getattr(pynvml, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                getattr(pynvml, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                getattr(pynvml, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            }
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self.stop_flag.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                mask = get_reasons(h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                time.sleep(0.01)
        except Exception as e:  # NVML missing: report it, do not fail the benchmark
            self.error = repr(e)

    def summary(self):
        d = {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
             "reasons": sorted(self.reasons), "samples": len(self.samples)}
        if self.error:
            d["error"] = self.error
        return d



def layer_table(times, peaks):
    """Per-convolution figures of one network pass: time, TOPS, GB/s, which roofline binds the layer and the fraction of it."""
    int8_peak = 2.0 * peaks["bf16_tflops"]
    out = []
    for t in times:
        tops, gbs = t["ops"] / t["us"] / 1e6, t["bytes"] / t["us"] / 1e3
        floor_tensor, floor_hbm = t["ops"] / (int8_peak * 1e6), t["bytes"] / (peaks["hbm_gbs"] * 1e3)
        bound = "hbm" if floor_hbm >= floor_tensor else "tensor"
        out.append({"name": t["name"], "shape": "%dx%d%s %d->%d @%d" % (t["k"], t["k"], "/2" if t["stride"] == 2 else "", t["c"], t["o"], t["size"]),
                    "outputs": "+".join(x for x, on in (("residual", t["residual"]), ("f32", t["fp32_out"]), ("i8", t["int8_out"])) if on),
                    "us": round(t["us"], 2), "tops": round(tops, 1), "gbs": round(gbs, 1), "bound": bound,
                    "frac": round(max(floor_tensor, floor_hbm) / t["us"], 4)})
    return out


def pass_roofline(times, ms_pass, peaks, extra_bytes=0):
    """The whole pass against both rooflines: algorithmic ops and bytes of its convolutions (plus the glue kernels' bytes)."""
    int8_peak = 2.0 * peaks["bf16_tflops"]
    ops = sum(t["ops"] for t in times)
    nbytes = sum(t["bytes"] for t in times) + extra_bytes
    floor_tensor_ms, floor_hbm_ms = ops / (int8_peak * 1e9), nbytes / (peaks["hbm_gbs"] * 1e6)
    # a pass is a sequence of kernels, each bound by its own roofline: the floor is the sum of the per-layer floors
    floor_sum_ms = sum(max(t["ops"] / (int8_peak * 1e9), t["bytes"] / (peaks["hbm_gbs"] * 1e6)) for t in times) + extra_bytes / (peaks["hbm_gbs"] * 1e6)
    return {"algorithmic_gop": ops / 1e9, "algorithmic_mb": nbytes / 1e6, "min_ms_tensor": floor_tensor_ms, "min_ms_hbm": floor_hbm_ms,
            "min_ms_per_layer_bounds": floor_sum_ms, "measured_ms": ms_pass, "frac": floor_sum_ms / ms_pass,
            "sum_of_layer_times_ms": sum(t["us"] for t in times) / 1e3,
            "peaks": "int8 tensor = 2 x %s bf16 (%.0f TOPS), HBM %s %.0f GB/s" % (peaks["source"], int8_peak, peaks["source"], peaks["hbm_gbs"])}


def resnet_parity(net, spec, params, scales, x, logits):
    """First and last image of the batch against the reference operator chain run on those two images (the C port of the
    reference's arithmetic, OpenMP).  Test infrastructure used as the checker; returns the parity object of the bench line."""
    from oracle import chains, oracle as orc
    chk = orc.Port()
    picks = [0, x.shape[0] - 1]
    t0 = time.perf_counter()
    outs, last_f32, want = chains.resnet_forward(spec, params, scales, x[picks].cpu().numpy(), chk)
    bad = chains.resnet_mismatches(spec, net.buffers, logits, picks, outs, last_f32, want)
    return {"images_checked": len(picks), "mismatches": bad, "checker": "C port of the reference operators, block outputs int8 bit-exact, last fp32 tensor bit-exact up to the sign of zero, logits 1e-5",
            "host_s": round(time.perf_counter() - t0, 2)}


def csp_parity(net, spec, params, scales, x, out):
    from oracle import chains, oracle as orc
    from tennis_b200 import nets
    chk = orc.Port()
    picks = [0, x.shape[0] - 1]
    t0 = time.perf_counter()
    outs, last = chains.cspdarknet_forward(spec, params, scales, x[picks].cpu().numpy(), chk, leaky=nets.LEAKY)
    bad = chains.cspdarknet_mismatches(spec, net.buffers, out, picks, outs, last)
    return {"images_checked": len(picks), "mismatches": bad, "checker": "C port of the reference operators, every block / stage output int8 bit-exact",
            "host_s": round(time.perf_counter() - t0, 2)}

def run_workbench_resnet(reps):
    """The same ResNet-50 shape as a TenniS graph inside the reference's own runtime (Workbench::Load / Workbench::run on
    its "gpu" device, with this repo's operators and graph rewrite registered there): what the runtime around the
    kernels costs.  Needs tennis_b200/libtennis_b200_workbench.so, which is built against the reference's sources and
    its CUDA host library; without them the object says so."""
    import ctypes
    path = os.path.join(ROOT, "tennis_b200", "libtennis_b200_workbench.so")
    if not os.path.exists(path):
        return {"unavailable": "libtennis_b200_workbench.so was not built (needs the reference's sources at build time)"}
    lib = ctypes.CDLL(path)
    lib.tsb_workbench_resnet50.argtypes = [ctypes.c_int] * 4 + [ctypes.c_uint, ctypes.POINTER(ctypes.c_double), ctypes.c_char_p,
                                           ctypes.c_int]
    res = {"graph": "53 quantize -> conv2d_quantized -> add_bias [-> add] -> relu layers, pooling2d, global_pooling2d, flatten, "
                    "inner_prod; built with the reference's graph API, compiled by Workbench::Load for device gpu",
           "timing": "wall clock around reps x (Workbench::input, Workbench::run, output view on the host), device idle at both ends"}
    for key, batch, mode in (("batch64_host_input", 64, 0), ("batch64_resident_input", 64, -1), ("batch1_resident_input", 1, -1)):
        out = (ctypes.c_double * 8)()
        msg = ctypes.create_string_buffer(512)
        rc = lib.tsb_workbench_resnet50(batch, 224, reps, mode, 3, out, msg, 512)
        if rc != 0:
            res[key] = {"error": msg.value.decode(errors="replace")[:300]}
            continue
        res[key] = {"ms_per_pass": out[0], "images_per_sec": batch / (out[0] / 1e3), "library_kernel_launches_per_pass": out[1],
                    "fused_nodes_per_pass": out[2], "int8_handovers_per_pass": out[3], "shortcuts_in_epilogue_per_pass": out[4],
                    "host_ms_inside_fused_operators": out[6]}
    one = res.get("batch1_resident_input", {})
    if "ms_per_pass" in one:
        # 53 fused nodes + pooling2d + global_pooling2d + flatten + inner_prod = 57 operator instructions per pass
        res["host_us_per_operator_upper_bound"] = one["ms_per_pass"] * 1e3 / 57
        res["host_us_per_fused_operator_inside_plugin"] = one["host_ms_inside_fused_operators"] * 1e3 / 53
    return res


def run_resnet50(args, dev, rank, world, sharding, peaks):
    """Images/s of the ResNet-50-shaped int8 network (53 convolutions with folded BN, fused ReLU / residual / requantize,
    int8 max pool, fp32 average pool and inner product), batch 64 per GPU, synthetic N(0,1) input, whole forward pass
    captured once in a CUDA graph and replayed.  The pass touches ~3 GB, far more than L2, so no flush is needed."""
    import torch
    from tennis_b200 import nets
    batch = 64
    spec = nets.resnet_spec()
    params = nets.make_params(spec, seed=0)
    net = nets.QuantResNet(spec, params, batch, dev)
    g = torch.Generator(device=dev).manual_seed(0 if world == 1 else sharding.shard_seed(rank))
    x = torch.randn((batch, 3, 224, 224), device=dev, generator=g)
    scales = net.calibrate(x)
    parity = None
    if rank == 0:
        try:
            first = net.forward(x).clone()
            net.status()
            torch.cuda.synchronize()
            parity = resnet_parity(net, spec, params, scales, x, first)
        except Exception as e:
            parity = {"images_checked": 0, "mismatches": None, "error": repr(e)[:200]}
    layer_times = net.layer_times(x) if rank == 0 else []
    stream = torch.cuda.Stream(device=dev)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            net.forward(x)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            logits = net.forward(x)
    torch.cuda.current_stream().wait_stream(stream)
    net.status()
    reps = max(5, min(args.steps, 30))
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / reps
    # end to end: pinned host input -> device, replay, logits -> pinned host
    # Every batch is uploaded from pinned host memory and its logits are downloaded; uploads are double-buffered on a
    # copy stream, so the upload of batch i+1 runs under the kernels of batch i.
    hx = x.cpu().pin_memory()
    e_reps = 32     # as many batches as a shard of configuration 4 has: the first upload, which nothing hides, weighs 1/32
    houts = [torch.empty(logits.shape, dtype=torch.float32).pin_memory() for _ in range(e_reps)]
    stage = [torch.empty_like(x) for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream()

    def upload(i):
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(consumed[i % 2])
            stage[i % 2].copy_(hx, non_blocking=True)
            copied[i % 2].record(copy_stream)

    torch.cuda.synchronize()
    t0 = time.perf_counter()
    upload(0)
    for i in range(e_reps):
        if i + 1 < e_reps:
            upload(i + 1)
        main.wait_event(copied[i % 2])
        x.copy_(stage[i % 2], non_blocking=True)
        consumed[i % 2].record(main)
        graph.replay()
        houts[i].copy_(logits, non_blocking=True)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e_reps
    hout = houts[-1]
    ms_max, images = sharding.aggregate(ms, batch, dev)
    e2e_max, _ = sharding.aggregate(e2e_ms, batch, dev)
    ops_batch = nets.conv_ops(spec, batch)
    # bytes of the four glue kernels: stem quantize (5 B per input element), max pool (int8 in + out), average pool, inner product
    c0 = spec["convs"][0]
    glue_bytes = (5 * x.numel() + batch * c0["oh"] * c0["oh"] * 64 + batch * spec["stem_pooled"] ** 2 * 64
                  + 4 * batch * spec["final_size"] ** 2 * spec["features"] + 4 * spec["classes"] * spec["features"])
    config4 = None
    try:
        config4 = run_config4(args, dev, rank, world, sharding, net, graph, x, logits, spec, params, scales)
    except Exception as e:
        config4 = {"error": repr(e)[:300]}
    workbench = None
    if rank == 0:
        try:
            workbench = run_workbench_resnet(max(5, min(args.steps, 20)))
        except Exception as e:
            workbench = {"error": repr(e)[:300]}
    return {"workload": "config2: ResNet-50-shaped int8 network, batch 64 per GPU, CUDA graph replay", "batch_per_gpu": batch,
            "images_per_sec": images / (ms_max / 1e3), "ms_per_batch": ms_max, "int8_conv_tops": ops_batch * world / (ms_max / 1e3) / 1e12,
            "e2e_images_per_sec": images / (e2e_max / 1e3), "e2e_ms_per_batch": e2e_max,
            "h2d_bytes_per_batch": hx.numel() * 4 * world, "d2h_bytes_per_batch": hout.numel() * 4 * world,
            "kernels_per_pass": 49 + 4, "projections_inside_conv3": 4, "parity": parity,
            "pass_roofline": pass_roofline(layer_times, ms_max, peaks, extra_bytes=glue_bytes) if layer_times else None,
            "layers": layer_table(layer_times, peaks),
            "config4": config4, "workbench": workbench}



def run_config4(args, dev, rank, world, sharding, net, graph, x_static, logits, spec, params, scales):
    """Configuration 4: the ResNet-50-shaped network over a global batch of 2048 images split evenly over the replicas
    (shard_range), each replica working through its shard in micro-batches of 64 with inputs drawn from its own seed
    1000 + rank.  Device figure: shard resident in HBM, events around the shard's micro-batches.  End to end: the shard in
    pinned host memory, every micro-batch uploaded (double-buffered on a copy stream) and its logits read back, all inside
    the timed region.  Replica 0 also checks two images of its first micro-batch against the operator chain."""
    import torch
    start, count = sharding.shard_range(2048, world, rank)
    sizes = sharding.micro_batches(count, 64)
    full = [n for n in sizes if n == 64]          # the network is planned for micro-batches of 64 (2048 / N is a multiple for N <= 32)
    g = torch.Generator(device=dev).manual_seed(sharding.shard_seed(rank))
    shard = torch.randn((len(full) * 64, 3, 224, 224), device=dev, generator=g)
    # parity of this seed's inputs: first micro-batch, first and last image (replica 0)
    parity = None
    if rank == 0:
        x_static.copy_(shard[:64])
        graph.replay()
        torch.cuda.synchronize()
        parity = resnet_parity(net, spec, params, scales, x_static, logits)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(min(2, len(full))):
        x_static.copy_(shard[i * 64:(i + 1) * 64]); graph.replay()
    torch.cuda.synchronize()
    a.record()
    for i in range(len(full)):
        x_static.copy_(shard[i * 64:(i + 1) * 64], non_blocking=True)
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    dev_ms = a.elapsed_time(b)
    # end to end from pinned host memory
    host = shard.cpu().pin_memory()
    del shard
    houts = torch.empty((len(full), 64, logits.shape[1]), dtype=torch.float32).pin_memory()
    stage = [torch.empty_like(x_static) for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream()

    def upload(i):
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(consumed[i % 2])
            stage[i % 2].copy_(host[i * 64:(i + 1) * 64], non_blocking=True)
            copied[i % 2].record(copy_stream)

    torch.cuda.synchronize()
    t0 = time.perf_counter()
    upload(0)
    for i in range(len(full)):
        if i + 1 < len(full):
            upload(i + 1)
        main.wait_event(copied[i % 2])
        x_static.copy_(stage[i % 2], non_blocking=True)
        consumed[i % 2].record(main)
        graph.replay()
        houts[i].copy_(logits, non_blocking=True)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    images = len(full) * 64
    dev_max, images_all = sharding.aggregate(dev_ms, images, dev)
    e2e_max, _ = sharding.aggregate(e2e_ms, images, dev)
    return {"workload": "config4: ResNet-50-shaped int8 network, global batch 2048 split over %d replica(s), micro-batches of 64, inputs N(0,1) from seed 1000 + rank" % world,
            "global_batch": int(images_all), "images_per_replica": images, "micro_batches_per_replica": len(full), "shard_of_rank0": [start, count],
            "images_per_sec": images_all / (dev_max / 1e3), "ms_per_shard": dev_max,
            "e2e_images_per_sec": images_all / (e2e_max / 1e3), "e2e_ms_per_shard": e2e_max,
            "h2d_bytes": int(host.numel() * 4 * world), "d2h_bytes": int(houts.numel() * 4 * world), "parity": parity}

def run_cspdarknet(args, dev, rank, world, sharding, peaks):
    """Images/s of the CSPDarknet53-shaped int8 backbone (72 convolutions, LeakyReLU(0.1), Darknet shortcuts added in fp32
    after the activation, cross-stage routes joined by an int8 concatenation), batch 16 per GPU at 3x608x608, synthetic
    U(0,1) input, whole forward pass captured in a CUDA graph and replayed."""
    import torch
    from tennis_b200 import nets
    batch = 16
    spec = nets.cspdarknet_spec()
    params = nets.make_conv_params(spec, seed=0)
    net = nets.QuantCSPDarknet(spec, params, batch, dev)
    g = torch.Generator(device=dev).manual_seed(0 if world == 1 else sharding.shard_seed(rank))
    x = torch.rand((batch, 3, 608, 608), device=dev, generator=g)
    t0 = time.perf_counter()
    scales = net.calibrate(x)
    net.status()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    first_out = net.forward(x)
    torch.cuda.synchronize()
    first = time.perf_counter() - t1
    parity = None
    if rank == 0:
        try:
            parity = csp_parity(net, spec, params, scales, x, first_out.clone())
        except Exception as e:
            parity = {"images_checked": 0, "mismatches": None, "error": repr(e)[:200]}
    layer_times = net.layer_times(x) if rank == 0 else []
    if first > 1.0 or t1 - t0 > 60.0:   # a secondary figure must never stall the benchmark
        return {"error": "skipped: calibration took %.1f s, one eager pass %.3f s" % (t1 - t0, first)}
    stream = torch.cuda.Stream(device=dev)
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            net.forward(x)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            out = net.forward(x)
    torch.cuda.current_stream().wait_stream(stream)
    net.status()
    reps = max(5, min(args.steps, 20))
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / reps
    # end to end: every batch uploaded from pinned host memory (double-buffered on a copy stream, so the upload of batch
    # i+1 runs under the kernels of batch i) and the backbone's output downloaded
    hx = x.cpu().pin_memory()
    e_reps = 16     # the first upload, which nothing hides, weighs 1/16
    houts = [torch.empty(out.shape, dtype=out.dtype).pin_memory() for _ in range(e_reps)]
    stage = [torch.empty_like(x) for _ in range(2)]
    copied = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream()

    def upload(i):
        with torch.cuda.stream(copy_stream):
            if i >= 2:
                copy_stream.wait_event(consumed[i % 2])
            stage[i % 2].copy_(hx, non_blocking=True)
            copied[i % 2].record(copy_stream)

    # the 5.9 MB output leaves through a download stream: a device copy of it (two, used in turn) is what the download reads,
    # so the next batch's kernels do not wait for the PCIe transfer
    outs = [torch.empty_like(out) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    drained = [torch.cuda.Event() for _ in range(2)]
    down_stream = torch.cuda.Stream(device=dev)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    upload(0)
    for i in range(e_reps):
        if i + 1 < e_reps:
            upload(i + 1)
        main.wait_event(copied[i % 2])
        x.copy_(stage[i % 2], non_blocking=True)
        consumed[i % 2].record(main)
        graph.replay()
        if i >= 2:
            main.wait_event(drained[i % 2])
        outs[i % 2].copy_(out, non_blocking=True)
        ready[i % 2].record(main)
        with torch.cuda.stream(down_stream):
            down_stream.wait_event(ready[i % 2])
            houts[i].copy_(outs[i % 2], non_blocking=True)
            drained[i % 2].record(down_stream)
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e_reps
    ms_max, images = sharding.aggregate(ms, batch, dev)
    e2e_max, _ = sharding.aggregate(e2e_ms, batch, dev)
    ops_batch = nets.conv_ops(spec, batch)
    return {"workload": "config3: CSPDarknet53-shaped int8 backbone, batch 16 per GPU at 608x608, CUDA graph replay",
            "batch_per_gpu": batch, "images_per_sec": images / (ms_max / 1e3), "ms_per_batch": ms_max,
            "e2e_images_per_sec": images / (e2e_max / 1e3), "e2e_ms_per_batch": e2e_max,
            "h2d_bytes_per_batch": hx.numel() * 4 * world, "d2h_bytes_per_batch": houts[0].numel() * houts[0].element_size() * world,
            "int8_conv_tops": ops_batch * world / (ms_max / 1e3) / 1e12, "kernels_per_pass": 72 + 1, "concatenations_inside_transition": 5,
            "parity": parity, "pass_roofline": pass_roofline(layer_times, ms_max, peaks) if layer_times else None,
            "layers": layer_table(layer_times, peaks)}



def run_elementwise(dev, peaks):
    """Achieved HBM bandwidth of the standalone elementwise operators on tensors far larger than L2 (CUDA events around
    a run of eight launches, best of five runs): the operator-visible quantize with 1 and 64 scales on 64 Mi fp32 elements,
    the staging quantize on the two network inputs (four input tensors in rotation), add_bias and relu on 64 Mi elements,
    the int8 max pool of the ResNet stem.  Algorithmic bytes: 5 per element for quantize (4 read + 1 written), 8 for
    add_bias / relu, input + output for the pool."""
    import torch
    from tennis_b200 import _lib, ops
    lib = _lib.load()
    out = []

    def timed(fns, nbytes, name):
        """fns: the same call on different buffers (together larger than L2 where one alone is not); one event pair around
        a run of launches, so that the few microseconds an event pair costs do not count against a short kernel."""
        fns = fns if isinstance(fns, list) else [fns]
        rounds = max(1, 8 // len(fns))
        for fn in fns:
            fn()
        best = None
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(rounds):
                for fn in fns:
                    fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / (rounds * len(fns))
            best = ms if best is None or ms < best else best
        gbs = nbytes / best / 1e6
        out.append({"kernel": name, "mb": round(nbytes / 1e6, 1), "us": round(best * 1e3, 1), "gbs": round(gbs, 1),
                    "frac_of_hbm": round(gbs / peaks["hbm_gbs"], 4), "launches_per_timing": rounds * len(fns)})

    n = 64 * 1024 * 1024
    x = torch.randn(n, device=dev)
    y8 = torch.empty(n, dtype=torch.int8, device=dev)
    yf = torch.empty(n, device=dev)
    sp = ops._stream_ptr
    one, many = _lib.float_array([31.0]), _lib.float_array([31.0] * 64)
    timed(lambda: _lib.check(lib.tsb_quantize_f32_i8(x.data_ptr(), y8.data_ptr(), n, one, 1, sp())), 5 * n, "tsb_quantize_f32_i8, 1 scale, 64 Mi elements")
    timed(lambda: _lib.check(lib.tsb_quantize_f32_i8(x.data_ptr(), y8.data_ptr(), n, many, 64, sp())), 5 * n, "tsb_quantize_f32_i8, 64 scales, 64 Mi elements")
    bias = torch.randn(64, device=dev)
    timed(lambda: _lib.check(lib.tsb_add_bias_f32_nchw(x.data_ptr(), yf.data_ptr(), 1024, 64, 1024, bias.data_ptr(), sp())), 8 * n, "tsb_add_bias_f32_nchw, 1024x64x1024")
    timed(lambda: _lib.check(lib.tsb_relu_f32(x.data_ptr(), yf.data_ptr(), n, sp())), 8 * n, "tsb_relu_f32, 64 Mi elements")
    del y8, yf
    for (nb, hw, o, k, st, pad, label) in ((64, 224, 64, 7, 2, 3, "ResNet stem input 64x3x224x224"), (16, 608, 32, 3, 1, 1, "CSPDarknet stem input 16x3x608x608")):
        xs = [torch.randn((nb, 3, hw, hw), device=dev) for _ in range(4)]      # 4 inputs: more than L2 together
        plan = ops.ConvPlan(xs[0].shape, (o, 3, k, k), (pad,) * 4, (st, st), (1, 1), 0.0, _lib.KERNEL_TCGEN05, dev)
        sc = _lib.float_array([31.0] * nb)
        text = plan.describe()
        cpix = 16 if "cpix=16" in text else 8
        timed([(lambda xi=xi: plan.quantize_input(xi, sc)) for xi in xs], 5 * xs[0].numel(),
              "tsb_conv2d_i8_quantize_input (staging quantize), " + label)
        # what the kernel really moves: 12 bytes read and one staged pixel (8 or 16 bytes: the layout the convolution's
        # sliding-window descriptor needs) written per pixel, against 15 algorithmic bytes
        out[-1]["staged_bytes_per_pixel"] = cpix
        out[-1]["moved_gbs"] = round(xs[0].numel() // 3 * (12 + cpix) / out[-1]["us"] / 1e3, 1)
        out[-1]["moved_frac_of_hbm"] = round(out[-1]["moved_gbs"] / peaks["hbm_gbs"], 4)
        del plan, xs
    # the ResNet stem pool: int8 [64][112][112][64] -> [64][56][56][64], 3x3 / 2
    xs = [torch.randint(-128, 128, (64, 112, 112, 64), dtype=torch.int8, device=dev) for _ in range(4)]
    yp = torch.empty((64, 56, 56, 64), dtype=torch.int8, device=dev)
    timed([(lambda xi=xi: _lib.check(lib.tsb_maxpool_i8_nhwc(xi.data_ptr(), yp.data_ptr(), 64, 112, 112, 64, 3, 2, 1, 0, 1, 0, sp())))
           for xi in xs], xs[0].numel() + yp.numel(), "tsb_maxpool_i8_nhwc, 64x112x112x64, 3x3 / 2")
    del xs, yp
    return out

def copy_rates(dev, barrier, megabytes=256, reps=4):
    """Plain pinned-memory copies on this rank while every other rank does the same: GB/s of uploads alone, downloads alone,
    and both directions at once on two streams.  The ceiling any end-to-end figure of this run sits under."""
    import torch
    n = megabytes << 20
    h_up, h_down = torch.empty(n, dtype=torch.uint8).pin_memory(), torch.empty(n, dtype=torch.uint8).pin_memory()
    h_up.zero_(); h_down.zero_()
    d_up, d_down = torch.empty(n, dtype=torch.uint8, device=dev), torch.zeros(n, dtype=torch.uint8, device=dev)
    s_up, s_down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def timed(up, down):
        torch.cuda.synchronize()
        barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            if up:
                with torch.cuda.stream(s_up):
                    d_up.copy_(h_up, non_blocking=True)
            if down:
                with torch.cuda.stream(s_down):
                    h_down.copy_(d_down, non_blocking=True)
        s_up.synchronize(); s_down.synchronize()
        return reps * n / (time.perf_counter() - t0) / 1e9

    timed(True, True)
    up, down, both = timed(True, False), timed(False, True), timed(True, True)
    return [up, down, both, both]      # with both on, each direction moved reps * n bytes in the same time


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from tennis_b200 import _lib, ops, sharding, workloads

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # Before any pinned buffer exists: keep this rank on the CPUs next to its GPU, so that the host side of every
    # upload and download (first touch) lies on the GPU's NUMA node.  Reads sysfs, changes this process's mask only.
    props = torch.cuda.get_device_properties(dev)
    try:
        bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        locality = sharding.bind_to_gpu(bus)
    except Exception as e:
        locality = {"error": repr(e)[:100]}
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    warmup = max(args.warmup, 3)
    layers = workloads.CONFIG1
    peaks = measured_peaks()

    # ---- resident state: inputs, weights, plans, outputs ----
    state = []
    for layer in layers:
        d = workloads.make_layer_data(layer, seed=0 if world == 1 else sharding.shard_seed(rank))  # seed 0 alone, 1000 + rank per shard
        x = torch.from_numpy(d["x"]).to(dev)
        w = torch.from_numpy(d["w"]).to(dev)
        pad = (layer["pad"],) * 4
        plan = ops.ConvPlan(x.shape, w.shape, pad, (layer["stride"],) * 2, (layer["dilation"],) * 2, 0.0, _lib.KERNEL_AUTO, dev)
        plan.set_weights(w)
        tc = plan.kernel == _lib.KERNEL_TCGEN05
        state.append(dict(layer=layer, d=d, x=x, w=w, plan=plan, tc=tc,
                          scales=_lib.float_array([float(d["qscale"])] * layer["n"]),
                          dq=torch.from_numpy(d["dq"]).to(dev), bias=torch.from_numpy(d["bias"]).to(dev),
                          out=torch.empty(plan.out_shape, dtype=torch.float32, device=dev)))

    def sptr():
        return ops._stream_ptr()

    def quantize(s):
        # fp32 NCHW -> the int8 layout the plan's kernel reads, inside the plan's workspace
        s["plan"].quantize_input(s["x"], s["scales"])

    def conv(s):
        s["plan"].run(None, _lib.LAYOUT_STAGED, s["dq"], bias=s["bias"], activation=_lib.ACT_RELU, out_f32=s["out"])

    def step():
        for s in state:
            quantize(s)
            conv(s)

    flush_buf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)  # > 126 MB of L2

    def flush_l2():
        flush_buf.fill_(1)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    for s in state:
        s["plan"].status()
    barrier()

    # The ten launches of a step are captured once in a CUDA graph and replayed: the host then issues one call per step
    # instead of ten, so the timed region measures the device and not the Python launch path.  --eager times the
    # plain launches instead.
    run_step, launch_mode = step, "eager launches"
    if not args.eager:
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize()
            for s in state:
                s["plan"].status()
            run_step, launch_mode = graph.replay, "CUDA graph replay of the step (10 kernels)"
        except Exception as e:   # capture unavailable: time the eager launches
            launch_mode = "eager launches (graph capture failed: %r)" % (e,)
    launches_per_step = 2 * len(state)

    sampler = ClockSampler(local_rank)
    sampler.start()

    # ---- timed region: exactly K steps, device time by CUDA events around each step, L2 flushed in between ----
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    launches0 = lib.tsb_kernel_launch_count()
    barrier()
    wall0 = time.perf_counter()
    for k in range(args.steps):
        flush_l2()
        starts[k].record()
        run_step()
        ends[k].record()
    barrier()
    wall = time.perf_counter() - wall0
    launches = lib.tsb_kernel_launch_count() - launches0
    if run_step is not step:
        launches = launches_per_step * args.steps   # replayed launches do not pass through the library's counter
    step_ms = [a.elapsed_time(b) for a, b in zip(starts, ends)]
    total_ms = sum(step_ms)

    # ---- the same steps back to back WITHOUT the L2 flush (inputs and weights of the small layers then stay in the 126 MB L2):
    # stated beside the cold figure, not used for `value` ----
    warm_steps = max(5, min(args.steps, 50))
    wa, wb = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    run_step()
    wa.record()
    for _ in range(warm_steps):
        run_step()
    wb.record()
    torch.cuda.synchronize()
    warm_ms = wa.elapsed_time(wb) / warm_steps

    # ---- the same step with its five independent layers on five streams (one graph, fork / join): what a host that
    # serves independent requests gets; a secondary figure, `value` stays the one-stream step ----
    concurrent = None
    try:
        lanes = [torch.cuda.Stream(device=dev) for _ in state]
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())

        def forked_step():
            cur = torch.cuda.current_stream()
            for lane, st in zip(lanes, state):
                lane.wait_stream(cur)
                with torch.cuda.stream(lane):
                    quantize(st)
                    conv(st)
            for lane in lanes:
                cur.wait_stream(lane)

        with torch.cuda.stream(side):
            forked_step()
            cgraph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cgraph, stream=side):
                forked_step()
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            cgraph.replay()
        torch.cuda.synchronize()
        for st in state:
            st["plan"].status()
        csteps = max(5, min(args.steps, 30))
        cev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(csteps)]
        for a, b in cev:
            flush_l2()
            a.record()
            cgraph.replay()
            b.record()
        torch.cuda.synchronize()
        cms = sum(a.elapsed_time(b) for a, b in cev) / csteps
        concurrent = {"launch": "the five layers on five streams inside one CUDA graph", "ms_per_step": cms,
                      "tops": sum(workloads.layer_ops(l) for l in layers) / cms / 1e9, "steps": csteps}
    except Exception as e:
        concurrent = {"error": repr(e)[:200]}

    # ---- per-kernel launch times (conv kernels only), for the roofline ----
    reps = max(10, min(args.steps, 50))
    per_layer = []
    for s in state:
        quantize(s)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        qevs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
        for a, b in evs:
            flush_l2()
            a.record()
            conv(s)
            b.record()
        for a, b in qevs:
            flush_l2()
            a.record()
            quantize(s)
            b.record()
        torch.cuda.synchronize()
        ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
        qms = statistics.mean(a.elapsed_time(b) for a, b in qevs)
        l = s["layer"]
        n_in = l["n"] * l["c"] * l["h"] * l["w"]
        per_layer.append(dict(name=l["name"], kernel="tcgen05" if s["tc"] else "direct", conv_ms=ms, quantize_ms=qms,
                              ops=workloads.layer_ops(l), tops=workloads.layer_ops(l) / ms / 1e9,
                              conv_bytes=workloads.layer_bytes(l), conv_gbs=workloads.layer_bytes(l) / ms / 1e6,
                              written_bytes=4 * l["n"] * l["o"] * workloads.out_hw(l)[0] * workloads.out_hw(l)[1],
                              quantize_gbs=5 * n_in / qms / 1e6))

    # ---- what this GPU takes as writes alone and reads alone (the copy bandwidth of the roofline is a half-and-half mix):
    # a fill and a sum over 1 GiB, best of three ----
    mem_rates = None
    try:
        big = torch.empty(1 << 30, dtype=torch.uint8, device=dev)

        def rate(fn):
            fn()
            best = None
            for _ in range(3):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); fn(); b.record()
                torch.cuda.synchronize()
                t = a.elapsed_time(b)
                best = t if best is None or t < best else best
            return big.numel() / best / 1e6
        mem_rates = {"write_only_gbs": rate(lambda: big.fill_(3)), "read_only_gbs": rate(lambda: big.view(torch.float32).sum())}
        del big
    except Exception as e:
        mem_rates = {"error": repr(e)[:200]}

    # ---- configuration 0: the single batch-1 layer the reference runs on its CPU today; latency of quantize + conv ----
    config0 = None
    try:
        l0 = workloads.CONFIG0[0]
        d0 = workloads.make_layer_data(l0, seed=0)
        x0 = torch.from_numpy(d0["x"]).to(dev)
        plan0 = ops.ConvPlan(x0.shape, d0["w"].shape, (l0["pad"],) * 4, (l0["stride"],) * 2, (l0["dilation"],) * 2, 0.0, _lib.KERNEL_AUTO, dev)
        plan0.set_weights(torch.from_numpy(d0["w"]).to(dev))
        dq0, b0 = torch.from_numpy(d0["dq"]).to(dev), torch.from_numpy(d0["bias"]).to(dev)
        out0 = torch.empty(plan0.out_shape, dtype=torch.float32, device=dev)
        s0 = _lib.float_array([float(d0["qscale"])])

        def run0():
            plan0.quantize_input(x0, s0)
            plan0.run(None, _lib.LAYOUT_STAGED, dq0, bias=b0, activation=_lib.ACT_RELU, out_f32=out0)
        for _ in range(5):
            run0()
        ev0 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(20)]
        for a, b in ev0:
            flush_l2()
            a.record()
            run0()
            b.record()
        torch.cuda.synchronize()
        plan0.status()
        us0 = statistics.median(a.elapsed_time(b) for a, b in ev0) * 1e3
        config0 = {"workload": "config0: 1x64x56x56, 3x3 64->64, quantize + conv + bias + ReLU, fp32 NCHW out",
                   "gpu_us": us0, "gpu_tops": workloads.layer_ops(l0) / us0 / 1e6,
                   "note": "two launches, event-timed after an L2 flush (an event pair around an empty kernel reads ~6 us)"}
        if world == 1 and rank == 0:
            try:
                from oracle import oracle as orc
                chk0 = orc.best()
                if chk0.kind == "reference":
                    sec0, _ = chk0.time_layer(d0["x"], d0["w"], (l0["pad"],) * 4, (l0["stride"],) * 2, (l0["dilation"],) * 2,
                                              float(d0["qscale"]), d0["dq"], d0["bias"], act=1, workers=1, repeats=3)
                    config0["cpu_reference_us"] = sec0 * 1e6
                    config0["cpu_reference_note"] = "the reference's operators, one Workbench with 1 computing thread (its correct setting)"
            except Exception as e:
                config0["cpu_reference_error"] = repr(e)[:200]
    except Exception as e:
        config0 = {"error": repr(e)[:200]}

    # ---- how fast this kernel's main loop runs when nothing else binds: a GEMM-shaped layer with int8 output ----
    probe = None
    try:
        pn, pc, phw, po = 32, 2048, 32, 2048
        px = torch.randint(-128, 128, (pn, phw, phw, pc), dtype=torch.int8, device=dev)
        pw = torch.randint(-127, 128, (po, pc, 1, 1), dtype=torch.int8, device=dev)
        pplan = ops.ConvPlan((pn, pc, phw, phw), (po, pc, 1, 1), (0,) * 4, (1, 1), (1, 1), 0.0, _lib.KERNEL_TCGEN05, dev)
        pplan.set_weights(pw)
        pdq = torch.full((po,), 1e-4, device=dev)
        pout = torch.empty((pn, phw, phw, po), dtype=torch.int8, device=dev)

        def probe_run():
            pplan.run(px, _lib.LAYOUT_NHWC_PAD, pdq, activation=_lib.ACT_RELU, out_i8=pout, out_i8_layout=_lib.LAYOUT_NHWC_PAD,
                      requant_scales=[1.0] * pn)
        for _ in range(3):
            probe_run()
        pe = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(10)]
        for a, b in pe:
            flush_l2()
            a.record()
            probe_run()
            b.record()
        torch.cuda.synchronize()
        pplan.status()
        pms = statistics.mean(a.elapsed_time(b) for a, b in pe)
        pops = 2.0 * pn * phw * phw * pc * po
        probe = {"layer": "1x1 2048->2048 at 32x32, batch 32, int8 NHWC out", "ms": pms, "tops": pops / pms / 1e9}
        del px, pw, pout, pplan
    except Exception as e:
        probe = {"error": repr(e)[:200]}

    # ---- end to end through the host-buffer C-ABI call ----
    host = []
    for s in state:
        l = s["layer"]
        nbytes = lib.tsb_conv2d_host_scratch_bytes(s["plan"].handle)
        host.append(dict(scratch=torch.empty(nbytes, dtype=torch.uint8, device=dev), nbytes=nbytes,
                         x=torch.from_numpy(s["d"]["x"]).pin_memory(), out=torch.empty(s["plan"].out_shape, dtype=torch.float32).pin_memory(),
                         w=s["d"]["w"], dq=s["d"]["dq"], bias=s["d"]["bias"]))

    # The five layers of a step are independent, so they go out through the non-waiting host call on three streams:
    # one layer's upload runs under another's kernels and a third's download.  The step ends when all three
    # streams are synchronised, i.e. when every result is in host memory.
    e2e_streams = [torch.cuda.Stream(device=dev) for _ in range(3)]

    def e2e_step(resident):
        for i, (s, h) in enumerate(zip(state, host)):
            l = s["layer"]
            _lib.check(lib.tsb_conv2d_quantized_host_async(
                s["plan"].handle, h["x"].data_ptr(), s["scales"], l["n"], h["w"].ctypes.data, h["dq"].ctypes.data,
                h["bias"].ctypes.data, _lib.ACT_RELU, 0.0, h["out"].data_ptr(), h["scratch"].data_ptr(), h["nbytes"],
                resident, e2e_streams[i % 3].cuda_stream))
        for st in e2e_streams:
            st.synchronize()

    e2e_step(0)
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):
        e2e_step(1)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step(1)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    # restore the plans' weights/workspaces used by the resident path (the host call rebinds them)
    for s in state:
        s["plan"].set_weights(s["w"])
    h2d = sum(h["x"].numel() * 4 for h in host)
    d2h = sum(h["out"].numel() * 4 for h in host)
    # what the host side of this machine gives every rank at this N: plain pinned copies, all ranks at once
    try:
        rates = sharding.gather_values(copy_rates(dev, barrier), dev)
    except Exception as e:
        rates = None
    localities = sharding.gather_values([locality.get("numa_node", -1), locality.get("bound_cpus", 0),
                                         locality.get("local_cpus", 0), locality.get("allowed_cpus", 0)], dev)
    e2e_all = sharding.gather_values([e2e_s * 1e3], dev)

    # ---- secondary workload: the ResNet-50-shaped int8 network (configuration 2), batch 64 per GPU, one CUDA graph ----
    resnet = None
    if not args.no_resnet:
        try:
            resnet = run_resnet50(args, dev, rank, world, sharding, peaks)
        except Exception as e:  # reported, never fatal for the primary metric
            resnet = {"error": repr(e)[:300]}

    csp = None
    if not args.no_csp:
        try:
            if resnet is not None:
                torch.cuda.empty_cache()
            csp = run_cspdarknet(args, dev, rank, world, sharding, peaks)
        except Exception as e:
            csp = {"error": repr(e)[:300]}

    elementwise = None
    if rank == 0:
        try:
            torch.cuda.empty_cache()
            elementwise = run_elementwise(dev, peaks)
        except Exception as e:
            elementwise = {"error": repr(e)[:300]}

    sampler.stop_flag.set()
    sampler.join(timeout=2)

    # ---- reduce over ranks: max of the device time, sum of the work ----
    ops_per_step = sum(workloads.layer_ops(l) for l in layers)
    total_ms_max, ops_all = sharding.aggregate(total_ms, ops_per_step * args.steps, dev)
    e2e_ms_max, e2e_ops_all = sharding.aggregate(e2e_s * 1e3, ops_per_step, dev)
    e2e_s_max = e2e_ms_max / 1e3
    value = ops_all / (total_ms_max / 1e3) / 1e12
    e2e_value = e2e_ops_all / e2e_s_max / 1e12

    if rank == 0:
        tc_layers = [p for p in per_layer if p["kernel"] == "tcgen05"]
        tc_ops = sum(p["ops"] for p in tc_layers)
        tc_ms = sum(p["conv_ms"] for p in tc_layers)
        int8_peak = 2.0 * peaks["bf16_tflops"]
        tc_bytes = sum(p["conv_bytes"] for p in tc_layers)
        tops = tc_ops / tc_ms / 1e9 if tc_layers else 0.0
        gbs = tc_bytes / tc_ms / 1e6 if tc_layers else 0.0
        # which roofline binds this workload: the one whose minimum time for the five launches is the larger
        floor_tensor_ms = tc_ops / (int8_peak * 1e9)
        floor_hbm_ms = tc_bytes / (peaks["hbm_gbs"] * 1e6)
        n_tc = max(1, len(tc_layers))
        tensor_view = {"achieved": tops, "peak": int8_peak, "unit": "TOPS", "frac": tops / int8_peak, "min_ms": floor_tensor_ms,
                       "peak_source": "2 x %s burst bf16 TFLOP/s (the driver's file has no int8 figure; dense int8 is nominally twice bf16)" % peaks["source"]}
        hbm_view = {"achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"], "min_ms": floor_hbm_ms,
                    "peak_source": "%s copy bandwidth" % peaks["source"]}
        bound = "hbm" if floor_hbm_ms >= floor_tensor_ms else "tensor"
        traffic, traffic_stale, traffic_note = ncu_traffic_record()
        main_view = hbm_view if bound == "hbm" else tensor_view
        roofline = {"kernel": "conv_i8_tc_kernel", "bound": bound, "achieved": main_view["achieved"], "peak": main_view["peak"],
                    "unit": main_view["unit"], "frac": main_view["frac"], "peak_source": main_view["peak_source"],
                    "why_this_bound": "minimum time of the step's conv launches: %.1f us on the HBM roofline, %.1f us on the tensor roofline; measured %.1f us"
                                      % (floor_hbm_ms * 1e3, floor_tensor_ms * 1e3, tc_ms * 1e3),
                    # dram__bytes_read.sum + dram__bytes_write.sum per conv launch, averaged over the launches of one
                    # step, from the ncu capture summarised under profiles/ (null when the kernel changed since)
                    "traffic": traffic, "traffic_stale": traffic_stale, "traffic_source": traffic_note,
                    "traffic_unit": "bytes per launch (part of the fp32 output is still in L2 when the kernel ends)",
                    "algorithmic_bytes_per_launch": tc_bytes / n_tc, "algorithmic_ops_per_launch": tc_ops / n_tc,
                    "avg_launch_ms": tc_ms / n_tc,
                    "tensor_view": tensor_view, "hbm_view": hbm_view, "int8_gemm_probe": probe}
        if mem_rates and "write_only_gbs" in mem_rates:
            # the fp32 outputs are 92 % of the step's bytes and all of them are writes: against what this GPU takes as
            # writes alone (measured just now), not against the half-read half-write copy figure
            written = sum(p["written_bytes"] for p in tc_layers)
            roofline["write_view"] = {"written_bytes_per_launch": written / n_tc, "achieved": written / tc_ms / 1e6,
                                      "peak": mem_rates["write_only_gbs"], "unit": "GB/s", "frac": written / tc_ms / 1e6 / mem_rates["write_only_gbs"],
                                      "min_ms": written / (mem_rates["write_only_gbs"] * 1e6), "read_only_gbs": mem_rates["read_only_gbs"],
                                      "peak_source": "torch fill of 1 GiB timed in this run (reads alone: a sum over the same buffer)"}
        if probe and "tops" in probe:
            probe["frac_of_peak"] = probe["tops"] / int8_peak
            probe["frac_of_nominal_dense_int8"] = probe["tops"] / 4500.0   # NVIDIA's dense int8 figure for B200
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": total_ms_max / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "step_ms": {"l2": "flushed before every step", "median": statistics.median(step_ms), "min": min(step_ms), "max": max(step_ms),
                        "rank": 0},
            "l2_warm": {"ms_per_step": warm_ms, "tops": ops_per_step / warm_ms / 1e9, "steps": warm_steps,
                        "note": "rank 0, no flush between steps: the steps' small inputs and weights stay in L2"},
            "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "256 MiB buffer written between timed steps", "launch": launch_mode, "global_batch": 32 * world,
                       "parallelism": "replicas x%d, batch-sharded, no collective" % world},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s_max * 1e3, "steps": e2e_steps},
            "gpu_launches": int(launches), "wall_s_timed_region": wall,
            "clocks": sampler.summary(), "roofline": roofline, "layers": per_layer,
        }
        if concurrent is not None:
            line["layers_concurrent"] = concurrent
        if config0 is not None:
            line["config0"] = config0
        if resnet is not None:
            line["resnet50"] = resnet
        if csp is not None:
            line["cspdarknet53"] = csp
        if elementwise is not None:
            line["elementwise"] = elementwise
        line["e2e"]["h2d_bytes_per_step"] = h2d * world
        line["e2e"]["d2h_bytes_per_step"] = d2h * world
        # per rank: the step's own transfer rates, the plain-copy rates of the same run, and the time the slower
        # direction alone needs at the both-directions rate -- the floor the end-to-end step cannot go under
        line["e2e"]["per_rank"] = []
        for r in range(world):
            ms_r = e2e_all[r][0]
            rec = {"rank": r, "ms_per_step": ms_r, "h2d_gbs": h2d / ms_r / 1e6, "d2h_gbs": d2h / ms_r / 1e6,
                   "numa_node": int(localities[r][0]), "cpus_bound": int(localities[r][1]), "cpus_local": int(localities[r][2]),
                   "cpus_allowed": int(localities[r][3])}
            if rates is not None:
                up, down, both = rates[r][0], rates[r][1], rates[r][2]
                rec.update({"copy_h2d_gbs": up, "copy_d2h_gbs": down, "copy_both_each_gbs": both,
                            "transfer_floor_ms": max(h2d, d2h) / (both * 1e6)})
            line["e2e"]["per_rank"].append(rec)
        if rates is not None:
            floor = max(rec["transfer_floor_ms"] for rec in line["e2e"]["per_rank"])
            line["e2e"]["transfer_floor_ms"] = floor
            line["e2e"]["frac_of_transfer_floor"] = floor / (e2e_s_max * 1e3)
            line["e2e"]["transfer_floor_note"] = ("the larger of a step's upload and download bytes at the rate of plain pinned copies in "
                                                  "both directions, measured on every rank at once in this run")
        if world == 1:
            try:
                checker, cores, workers, images, ops_pass = cpu_arm(layers)
                t0 = time.perf_counter()
                sec = cpu_sample(layers, images, workers, checker)
                line["cpu_baseline"] = {
                    "value": ops_pass / sec / 1e12, "unit": UNIT, "cores": cores, "kind": checker.kind,
                    "sample": "%d images of each of the 5 layers on each of %d worker(s); %.1f s" % (images, workers, time.perf_counter() - t0)}
            except Exception as e:
                line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": 0, "kind": "port", "sample": "failed: %r" % (e,)}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
