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

NCU_TRAFFIC_BYTES_PER_LAUNCH = 15.7e6
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
    images = 1
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


def run_resnet50(args, dev, rank, world, sharding):
    """Images/s of the ResNet-50-shaped int8 network (53 convolutions with folded BN, fused ReLU / residual / requantize,
    int8 max pool, fp32 average pool and inner product), batch 64 per GPU, synthetic N(0,1) input, whole forward pass
    captured once in a CUDA graph and replayed.  The pass touches ~3 GB, far more than L2, so no flush is needed."""
    import torch
    from tennis_b200 import nets
    batch = 64
    spec = nets.resnet_spec()
    params = nets.make_params(spec, seed=0)
    net = nets.QuantResNet(spec, params, batch, dev)
    g = torch.Generator(device=dev).manual_seed(sharding.shard_seed(0, rank))
    x = torch.randn((batch, 3, 224, 224), device=dev, generator=g)
    net.calibrate(x)
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
    e_reps = max(4, min(args.steps, 12))
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
    return {"workload": "config2: ResNet-50-shaped int8 network, batch 64 per GPU, CUDA graph replay", "batch_per_gpu": batch,
            "images_per_sec": images / (ms_max / 1e3), "ms_per_batch": ms_max, "int8_conv_tops": ops_batch * world / (ms_max / 1e3) / 1e12,
            "e2e_images_per_sec": images / (e2e_max / 1e3), "e2e_ms_per_batch": e2e_max,
            "h2d_bytes_per_batch": hx.numel() * 4 * world, "d2h_bytes_per_batch": hout.numel() * 4 * world,
            "kernels_per_pass": 53 + 4, "logits_checksum": float(logits.double().abs().sum())}


def run_cspdarknet(args, dev, rank, world, sharding):
    """Images/s of the CSPDarknet53-shaped int8 backbone (72 convolutions, LeakyReLU(0.1), Darknet shortcuts added in fp32
    after the activation, cross-stage routes joined by an int8 concatenation), batch 16 per GPU at 3x608x608, synthetic
    U(0,1) input, whole forward pass captured in a CUDA graph and replayed."""
    import torch
    from tennis_b200 import nets
    batch = 16
    spec = nets.cspdarknet_spec()
    params = nets.make_conv_params(spec, seed=0)
    net = nets.QuantCSPDarknet(spec, params, batch, dev)
    g = torch.Generator(device=dev).manual_seed(sharding.shard_seed(0, rank))
    x = torch.rand((batch, 3, 608, 608), device=dev, generator=g)
    t0 = time.perf_counter()
    net.calibrate(x)
    net.status()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    net.forward(x)
    torch.cuda.synchronize()
    first = time.perf_counter() - t1
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
    ms_max, images = sharding.aggregate(ms, batch, dev)
    ops_batch = nets.conv_ops(spec, batch)
    return {"workload": "config3: CSPDarknet53-shaped int8 backbone, batch 16 per GPU at 608x608, CUDA graph replay",
            "batch_per_gpu": batch, "images_per_sec": images / (ms_max / 1e3), "ms_per_batch": ms_max,
            "int8_conv_tops": ops_batch * world / (ms_max / 1e3) / 1e12, "kernels_per_pass": 72 + 1 + 5,
            "features_checksum": int(out.to(torch.int64).abs().sum())}


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
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    warmup = max(args.warmup, 3)
    layers = workloads.CONFIG1
    peaks = measured_peaks()

    # ---- resident state: inputs, weights, plans, outputs ----
    state = []
    for layer in layers:
        d = workloads.make_layer_data(layer, seed=sharding.shard_seed(0, rank))  # per-shard seed
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
                              quantize_gbs=5 * n_in / qms / 1e6))

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

    # ---- secondary workload: the ResNet-50-shaped int8 network (configuration 2), batch 64 per GPU, one CUDA graph ----
    resnet = None
    if not args.no_resnet:
        try:
            resnet = run_resnet50(args, dev, rank, world, sharding)
        except Exception as e:  # reported, never fatal for the primary metric
            resnet = {"error": repr(e)[:300]}

    csp = None
    if not args.no_csp:
        try:
            if resnet is not None:
                torch.cuda.empty_cache()
            csp = run_cspdarknet(args, dev, rank, world, sharding)
        except Exception as e:
            csp = {"error": repr(e)[:300]}

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
        main_view = hbm_view if bound == "hbm" else tensor_view
        roofline = {"kernel": "conv_i8_tc_kernel", "bound": bound, "achieved": main_view["achieved"], "peak": main_view["peak"],
                    "unit": main_view["unit"], "frac": main_view["frac"], "peak_source": main_view["peak_source"],
                    "why_this_bound": "minimum time of the step's conv launches: %.1f us on the HBM roofline, %.1f us on the tensor roofline; measured %.1f us"
                                      % (floor_hbm_ms * 1e3, floor_tensor_ms * 1e3, tc_ms * 1e3),
                    # dram__bytes_read.sum + dram__bytes_write.sum per conv launch, averaged over the launches of one
                    # step, from the ncu capture summarised in profiles/conv_i8_tc_kernel_config1.md
                    "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                    "traffic_unit": "bytes per launch (ncu capture of this workload; part of the fp32 output is still in L2 when the kernel ends)",
                    "algorithmic_bytes_per_launch": tc_bytes / n_tc, "algorithmic_ops_per_launch": tc_ops / n_tc,
                    "avg_launch_ms": tc_ms / n_tc,
                    "tensor_view": tensor_view, "hbm_view": hbm_view, "int8_gemm_probe": probe}
        if probe and "tops" in probe:
            probe["frac_of_peak"] = probe["tops"] / int8_peak
            probe["frac_of_nominal_dense_int8"] = probe["tops"] / 4500.0   # NVIDIA's dense int8 figure for B200
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": total_ms_max / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "int8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "l2": "256 MiB buffer written between timed steps", "launch": launch_mode, "global_batch": 32 * world,
                       "parallelism": "replicas x%d, batch-sharded, no collective" % world},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s_max * 1e3, "steps": e2e_steps},
            "gpu_launches": int(launches), "wall_s_timed_region": wall,
            "clocks": sampler.summary(), "roofline": roofline, "layers": per_layer,
        }
        if config0 is not None:
            line["config0"] = config0
        if resnet is not None:
            line["resnet50"] = resnet
        if csp is not None:
            line["cspdarknet53"] = csp
        line["e2e"]["h2d_bytes_per_step"] = h2d * world
        line["e2e"]["d2h_bytes_per_step"] = d2h * world
        if world == 1:
            try:
                checker, cores, workers, images, ops_pass = cpu_arm(layers)
                t0 = time.perf_counter()
                sec = cpu_sample(layers, images, workers, checker)
                line["cpu_baseline"] = {
                    "value": ops_pass / sec / 1e12, "unit": UNIT, "cores": cores, "kind": checker.kind,
                    "sample": "%d image of each of the 5 layers on each of %d worker(s); %.1f s" % (images, workers, time.perf_counter() - t0)}
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
