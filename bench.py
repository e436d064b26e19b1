#!/usr/bin/env python
"""Headline benchmark: ResNet-50 fp32 inference, global batch 256, images/s on 1/2/4/8 B200.

A step is one forward pass of the whole network over a global batch of 256 synthetic images, split by
batch over the ranks (replicated weights, no communication during the pass, outputs gathered to rank 0
with NCCL).  Rank 0 prints ONE JSON line.

  python bench.py [--gpus N] [--steps K] [--warmup W]          this library on the GPU(s)
  python bench.py --impl reference [...]                        the reference's own CPU Net on the host cores

Launched under torch.distributed.run for N > 1 (one rank per GPU).
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

GLOBAL_BATCH = 256
METRIC = "resnet50_fp32_inference_images_per_sec"
WORKLOAD = "resnet50_v1.5_fp32_inference_b256_3x224x224_bn_folded"


def measured_peaks():
    """Driver-measured peaks; the stated fallback when the file is absent."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def committed_traffic():
    """DRAM bytes per contraction launch from the committed profiler summary, or None when it has no such line."""
    path = os.path.join(ROOT, "profiles", "contraction_tf32x3_forward_dram_traffic.md")
    try:
        with open(path) as f:
            for line in f:
                if line.startswith("traffic_bytes_per_launch_batch256:"):
                    return float(line.split(":", 1)[1])
    except OSError:
        pass
    return None


def shard(total, world, rank):
    """Images [begin, end) of the global batch that belong to `rank`."""
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, devices):
        self.devices = set(devices)
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
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
        self.file.flush()
        self.file.seek(0)
        sm, smax, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not f[0].isdigit() or int(f[0]) not in self.devices:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.file.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load: the upper half by power draw
        cut = statistics.median(power)
        loaded = [s for s, p in zip(sm, power) if p >= cut] or sm
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm),
                "power_w_max": max(power)}


# ------------------------------------------------------------------------------------------------ reference arm
def cpu_reference_run(steps, warmup, sample_images=2):
    """The reference's own CPU Net (oracle/_ref, built from the reference sources) on a bounded sample of
    the workload: `sample_images` images of the 256 per step.  Falls back to the C restatement."""
    from dlprimitives_b200 import resnet50
    from oracle import bindings as ob
    net_json = resnet50.make_json(sample_images)
    params = resnet50.make_params(net_json, seed=0)
    x = resnet50.make_input(resnet50.make_json(GLOBAL_BATCH), seed=1)[:sample_images]
    times = []
    if ob.ref_available():
        kind, cores = "reference", 1      # the reference has no threading of its own (internal BLAS)
        net = ob.RefNet(net_json)
        for name in net.param_names():
            net.set_param(name, params[name])
        net.set_tensor("data", x)
        for i in range(warmup + steps):
            net.forward()
            if i >= warmup:
                times.append(net.seconds)
        out = net.get_tensor("prob")
    else:
        from oracle import netrun
        kind, cores = "port", os.cpu_count() or 1
        ob.set_threads(cores)
        for i in range(warmup + steps):
            res, sec = netrun.run(net_json, params, {"data": x})
            if i >= warmup:
                times.append(sec)
        out = res["prob"]
    sec = statistics.median(times)
    return {"value": sample_images / sec, "unit": "images/s", "cores": cores, "kind": kind,
            "sample": "%d of the %d images of one step through the full-size network, %d timed passes" % (sample_images, GLOBAL_BATCH, len(times)),
            "seconds_per_pass": sec}, out, x, params


def _reference_worker(net_json, params, x, passes, warmup, barrier, queue):
    """One process of the parallel reference run: the reference's CPU Net on its own images."""
    from oracle import bindings as ob
    net = ob.RefNet(net_json)
    for name in net.param_names():
        net.set_param(name, params[name])
    net.set_tensor("data", x)
    for _ in range(warmup):
        net.forward()
    barrier.wait()
    t0 = time.time()
    for _ in range(passes):
        net.forward()
    queue.put(time.time() - t0)


def cpu_reference_run_all_cores(steps, warmup, images_per_worker=1):
    """The reference's CPU Net has no threading of its own, so the way to use every host core with it is one
    process per core, each taking images of the batch (they are independent).  All workers start their timed
    passes together; the rate is the images they finished over the slowest worker's time."""
    import multiprocessing as mp
    from dlprimitives_b200 import resnet50
    workers = max(1, min(os.cpu_count() or 1, 64, GLOBAL_BATCH // images_per_worker))
    net_json = resnet50.make_json(images_per_worker)
    params = resnet50.make_params(net_json, seed=0)
    x_all = resnet50.make_input(resnet50.make_json(GLOBAL_BATCH), seed=1)
    ctx = mp.get_context("fork")            # no CUDA in this process: the workers share the weights copy-on-write
    barrier, queue = ctx.Barrier(workers), ctx.Queue()
    procs = [ctx.Process(target=_reference_worker,
                         args=(net_json, params, x_all[i * images_per_worker:(i + 1) * images_per_worker], steps, warmup, barrier, queue))
             for i in range(workers)]
    for pr in procs:
        pr.start()
    import queue as queue_mod
    times, deadline = [], time.time() + 1800
    while len(times) < workers:
        try:
            times.append(queue.get(timeout=2))
        except queue_mod.Empty:
            if time.time() > deadline or any(pr.exitcode not in (None, 0) for pr in procs):
                for pr in procs:
                    if pr.is_alive():
                        pr.terminate()
                raise RuntimeError("a worker of the parallel reference run failed")
    for pr in procs:
        pr.join()
    sec = max(times)
    return {"value": workers * images_per_worker * steps / sec, "unit": "images/s", "cores": workers, "kind": "reference",
            "sample": "%d processes x %d image(s) x %d passes of the full-size network, started together; slowest worker %.1f s"
                      % (workers, images_per_worker, steps, sec)}


def run_reference_arm(args, rank):
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 1))
    from oracle import bindings as ob
    base = None
    if ob.ref_available():
        try:
            base = cpu_reference_run_all_cores(steps, warmup)
        except (RuntimeError, OSError) as e:
            sys.stderr.write("parallel reference run failed (%s); timing one process instead\n" % e)
    if base is None:
        base, _, _, _ = cpu_reference_run(steps, warmup)
    line = {"metric": METRIC, "value": base["value"], "unit": "images/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": 1000.0 * GLOBAL_BATCH / base["value"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "note": "CPU path timed on a bounded sample; ms_per_step extrapolated to 256 images"},
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm
def layer_table(net_json, plan, step_ms, batch, peaks):
    """Per-step algorithmic work and achieved rate.  FLOP = 2*N*Cout*OH*OW*(Cin/g)*KH*KW and
    bytes = 4*(x + y + w + bias), the formulas of the reference's own tool (tools/flops.cpp:660-661)."""
    shapes = {i["name"]: list(i["shape"]) for i in net_json["inputs"]}
    shapes[net_json["inputs"][0]["name"]][0] = batch
    ops = {op["name"]: op for op in net_json["operators"]}
    info = {}
    for op in net_json["operators"]:
        o = op.get("options", {})
        s = shapes[op["inputs"][0]]
        flops, wbytes = 0, 0
        if op["type"] == "Convolution2D":
            k, st, pd = o["kernel"], o["stride"], o["pad"]
            oh, ow = (s[2] + 2 * pd[0] - k[0]) // st[0] + 1, (s[3] + 2 * pd[1] - k[1]) // st[1] + 1
            out = [s[0], o["channels_out"], oh, ow]
            kk = (o["channels_in"] // o.get("groups", 1)) * k[0] * k[1]
            flops = 2 * int(np.prod(out)) * kk
            wbytes = 4 * (o["channels_out"] * kk + (o["channels_out"] if o.get("bias", True) else 0))
        elif op["type"] == "Pooling2D":
            k, st, pd = o["kernel"], o.get("stride", 1), o.get("pad", 0)
            out = [s[0], s[1], (s[2] + 2 * pd - k) // st + 1, (s[3] + 2 * pd - k) // st + 1]
        elif op["type"] == "GlobalPooling":
            out = [s[0], s[1], 1, 1]
        elif op["type"] == "InnerProduct":
            out = [s[0], o["outputs"]]
            flops = 2 * s[0] * o["inputs"] * o["outputs"]
            wbytes = 4 * (o["inputs"] * o["outputs"] + o["outputs"])
        else:
            out = list(s)
        for name in op["outputs"]:
            shapes[name] = out
        in_bytes = 4 * sum(int(np.prod(shapes[n])) for n in op["inputs"])
        info[op["name"]] = {"flops": flops, "bytes": in_bytes + 4 * int(np.prod(out)) + wbytes, "out": out}
    rows = []
    tensor_peak = peaks["bf16_tflops_sustained"] / 2.0 / 3.0      # TF32 = bf16/2, three products per term
    ridge = tensor_peak * 1e3 / peaks["hbm_gbs"]                  # FLOP per byte above which the tensor roof is the lower one
    for line, ms in zip(plan, step_ms):
        name = line.split(" ")[0]
        i = dict(info[name])
        fused = None
        if "absorbs" in line:
            fused = line.rsplit(" ", 1)[-1]
            i["bytes"] += 4 * int(np.prod(i["out"]))             # the residual operand is read as well
        tflops = i["flops"] / ms / 1e9 if ms > 0 else 0.0
        gbs = i["bytes"] / ms / 1e6 if ms > 0 else 0.0
        # the applicable roof: the lower of the two for this step's arithmetic intensity
        intensity = i["flops"] / i["bytes"] if i["bytes"] else 0.0
        tensor_bound = "tf32x3" in line and intensity > ridge
        rows.append({"step": name, "type": ops[name]["type"], "kernel": " ".join(line.split(" ")[2:4]), "fused": fused, "ms": ms,
                     "gflop": i["flops"] / 1e9, "mbytes": i["bytes"] / 1e6, "tflops": tflops, "gbs": gbs, "flop_per_byte": intensity,
                     "tensor_core": "tf32x3" in line, "bound": "tensor" if tensor_bound else "hbm",
                     "frac": (tflops / tensor_peak) if tensor_bound else (gbs / peaks["hbm_gbs"])})
    return rows, tensor_peak


def run_gpu_arm(args, rank, world, local_rank):
    import torch
    import torch.distributed as dist
    from dlprimitives_b200 import capi, hostapi, resnet50

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if GLOBAL_BATCH % world != 0:
        raise SystemExit("the global batch of %d must divide by the number of GPUs (the gather needs equal shards)" % GLOBAL_BATCH)
    begin, end = shard(GLOBAL_BATCH, world, rank)
    local_batch = end - begin
    peaks = measured_peaks()

    net_json = resnet50.make_json(local_batch)
    params = resnet50.make_params(net_json, seed=0)           # every rank holds the full weights
    x_all = resnet50.make_input(resnet50.make_json(GLOBAL_BATCH), seed=1)
    # the projection shortcuts of the four stage-opening blocks run on a second stream (a Net option, bit-identical results)
    net = hostapi.Net(net_json, device=local_rank, flags=hostapi.Net.CONCURRENT_BRANCHES)
    for name, value in params.items():
        net.set_param(name, value)
    net.upload_params()
    plan = net.plan()

    stream = torch.cuda.Stream(device=dev)
    x_host = torch.from_numpy(np.ascontiguousarray(x_all[begin:end])).pin_memory()
    probs_local = torch.empty(local_batch, 1000, device=dev)
    counts = [shard(GLOBAL_BATCH, world, r)[1] - shard(GLOBAL_BATCH, world, r)[0] for r in range(world)]
    gathered = [torch.empty(c, 1000, device=dev) for c in counts] if rank == 0 and world > 1 else None
    probs_host = torch.empty(GLOBAL_BATCH, 1000).pin_memory() if rank == 0 else None

    def barrier():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize(dev)

    # End-to-end steps are pipelined the way a serving loop would be: the host-to-device copy of step i+1's
    # input (pinned memory -> one of two staging buffers, on a copy stream) runs while step i computes;
    # step i starts with a device-to-device move of its staged input into the network's input tensor.
    copy_stream = torch.cuda.Stream(device=dev)
    staged = [torch.empty(x_host.shape, device=dev) for _ in range(2)]
    staged_ready = [torch.cuda.Event() for _ in range(2)]
    staged_free = [torch.cuda.Event() for _ in range(2)]

    def prefetch(i):
        slot = i % 2
        copy_stream.wait_event(staged_free[slot])
        with torch.cuda.stream(copy_stream):
            staged[slot].copy_(x_host, non_blocking=True)
        staged_ready[slot].record(copy_stream)

    def step(end_to_end, index=0, more=False):
        """One forward pass over this rank's shard; with end_to_end the shard comes from pinned host memory
        (copied during the step before) and rank 0 reads the gathered probabilities back to the host."""
        if end_to_end:
            slot = index % 2
            stream.wait_event(staged_ready[slot])
            net.copy_tensor_from("data", staged[slot], stream)
            staged_free[slot].record(stream)
            if more:
                prefetch(index + 2)
        net.forward(stream)
        net.copy_tensor_to("prob", probs_local, stream)
        if world > 1:
            dist.gather(probs_local, gathered, dst=0)
        if end_to_end and rank == 0:
            if world > 1:
                off = 0
                for g, c in zip(gathered, counts):
                    probs_host[off:off + c].copy_(g, non_blocking=True)
                    off += c
            else:
                probs_host.copy_(probs_local, non_blocking=True)

    def timed(steps, end_to_end, sampler=None):
        barrier()
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        if end_to_end:
            # every host-to-device copy of the timed steps starts after e0
            copy_stream.wait_event(e0)
            for slot in range(2):
                staged_free[slot].record(stream)
            for i in range(min(2, steps)):
                prefetch(i)
        for i in range(steps):
            step(end_to_end, i, i + 2 < steps)
        e1.record(stream)
        barrier()
        clocks = sampler.stop() if sampler else None
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), clocks

    with torch.cuda.stream(stream):
        net.set_tensor("data", x_host, stream)          # inputs resident in HBM before the timed region
        launches0 = capi.launch_count()
        net.forward(stream)                             # first pass: eager, packs the weights
        stream.synchronize()
        launches_first = capi.launch_count() - launches0
        launches0 = capi.launch_count()
        net.forward(stream)                             # second pass: recorded into the CUDA graph
        stream.synchronize()
        launches_per_forward = capi.launch_count() - launches0
        for _ in range(max(args.warmup, 3)):
            step(False)
        sampler = ClockSampler(range(world)) if rank == 0 else None
        ms_total, clocks = timed(args.steps, False, sampler)
        timed(2, True)                                  # warm the end-to-end path
        ms_e2e, _ = timed(args.steps, True)
        # per-operator pass for the roofline: operator by operator with an event pair around each
        reps = [net.forward_timed(stream) for _ in range(5)]
        step_ms = [statistics.median(v) for v in zip(*reps)]
        status = capi.device_status(stream)
        if rank == 0:
            net.copy_tensor_to("prob", probs_local, stream)
            stream.synchronize()
            probs0 = probs_local.cpu().numpy()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    if status != 0:
        raise RuntimeError("a bounded device-side wait gave up during the benchmark, code %d" % status)

    ms_per_step = ms_total / args.steps
    value = GLOBAL_BATCH / (ms_per_step / 1000.0)
    e2e_value = GLOBAL_BATCH / (ms_e2e / args.steps / 1000.0)
    rows, tensor_peak = layer_table(net_json, plan, step_ms, local_batch, peaks)
    tc = [r for r in rows if r["tensor_core"]]
    tc_ms, tc_flops = sum(r["ms"] for r in tc), sum(r["gflop"] for r in tc)
    achieved = tc_flops / tc_ms if tc_ms > 0 else 0.0      # GFLOP / ms = TFLOP/s
    # Every launch against its own applicable roof (tensor or HBM, by arithmetic intensity): the time the roofs allow over the time taken.
    roof_ms = sum(max(r["gflop"] / tensor_peak, r["mbytes"] / peaks["hbm_gbs"]) for r in tc)
    # DRAM bytes per contraction launch come from a committed profiler summary (a line "traffic_bytes_per_launch_batch256: N");
    # measured at 256 images on one GPU only
    traffic = committed_traffic() if local_batch == 256 else None
    with torch.cuda.stream(stream):
        tf32_rate = capi.tf32_mma_rate(stream)              # the tensor pipe's own dense TF32 rate on this GPU, now
    roofline = {"bound": "tensor", "kernel": "contraction_tf32x3_kernel + pointwise_tf32x3_kernel", "achieved": achieved, "peak": tensor_peak,
                "unit": "TFLOP/s", "frac": achieved / tensor_peak, "traffic": traffic,
                "traffic_unit": "DRAM bytes per launch, average over the forward's launches",
                "algorithmic_bytes_per_launch": 1e6 * sum(r["mbytes"] for r in tc) / max(len(tc), 1), "launches": len(tc), "avg_launch_ms": tc_ms / max(len(tc), 1),
                "peak_source": "%s bf16 sustained %.1f TFLOP/s / 2 (TF32) / 3 (products per term)" % (peaks["source"], peaks["bf16_tflops_sustained"]),
                "share_of_forward": tc_ms / sum(r["ms"] for r in rows),
                "frac_applicable": roof_ms / tc_ms if tc_ms > 0 else 0.0,
                "frac_applicable_note": "sum over the launches of max(FLOP / tensor peak, bytes / HBM peak) over their measured time",
                "launches_below_0.6": [r["step"] for r in tc if r["frac"] < 0.6],
                "tf32_measured": tf32_rate, "tf32x3_measured": tf32_rate / 3.0,
                "tf32_measured_note": "dense TF32 TFLOP/s of an MMA-only kernel on this GPU in this run; a 3xTF32 kernel can reach a third of it",
                "frac_of_tf32x3_measured": achieved / (tf32_rate / 3.0) if tf32_rate > 0 else None}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu, ref_out, _, _ = cpu_reference_run(2, 1)
        err = float(np.abs(probs0[:ref_out.shape[0]] - ref_out).max())
        cpu = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        cpu["max_abs_prob_diff_vs_gpu"] = err

    if args.layers_out:
        with open(args.layers_out, "w") as f:
            json.dump({"local_batch": local_batch, "tensor_peak_tflops": tensor_peak, "hbm_peak_gbs": peaks["hbm_gbs"], "rows": rows}, f, indent=1)

    line = {"metric": METRIC, "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "per_gpu_batch": local_batch, "parallelism": "batch-split x%d, replicated weights, NCCL gather of outputs" % world,
                       "math": "3xTF32 tensor cores, fp32 accumulate", "l2": "working set per step (activations > 1 GB, input %d MB) exceeds the 126 MB L2" % (x_host.numel() * 4 // 2**20),
                       "tflops": value * resnet50.flops_per_image(net_json) / 1e12},
            "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": GLOBAL_BATCH * 3 * 224 * 224 * 4, "d2h_bytes_per_step": GLOBAL_BATCH * 1000 * 4},
            "gpu_launches": launches_per_forward * args.steps * world,
            "launches_per_forward": launches_per_forward,
            "clocks": clocks, "roofline": roofline}
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_single_conv(args):
    """One convolution through the C ABI, repeated: the small case profiler captures are taken on.
    --conv N,Cin,H,Cout,K,stride,pad[,groups[,residual]]   (residual = 1: the fused "+ residual, ReLU" form)"""
    import torch
    from dlprimitives_b200 import capi
    v = [int(t) for t in args.conv.split(",")]
    n, cin, hw, cout, k, stride, pad = v[:7]
    groups = v[7] if len(v) > 7 else 1
    with_res = len(v) > 8 and v[8] != 0
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(1)
    x = torch.randn(n, cin, hw, hw, device=dev, generator=g)
    w = torch.randn(cout, cin // groups, k, k, device=dev, generator=g) * (2.0 / (cin // groups * k * k)) ** 0.5
    b = torch.rand(cout, device=dev, generator=g) * 0.2 - 0.1
    plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=k, stride=stride, pad=pad, groups=groups, batch=n, height=hw, width=hw,
                              bias=True, activation="relu", algo=args.conv_algo)
    y = torch.empty(plan.output_shape(n), device=dev)
    res = torch.randn(plan.output_shape(n), device=dev, generator=g) if with_res else None
    extra = dict(residual=res, post_activation="relu") if with_res else {}
    packed = plan.prepack(w)
    extra["ws"] = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=dev)
    for _ in range(max(args.warmup, 3)):
        plan.enqueue_packed(x, packed, b, y, **extra)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        plan.enqueue_packed(x, packed, b, y, **extra)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 2.0 * y.numel() * (cin // groups) * k * k
    byts = 4.0 * (x.numel() + y.numel() * (2 if with_res else 1) + w.numel() + b.numel())
    print(json.dumps({"conv": args.conv, "algo": plan.algo(), "kernel": plan.kernel(), "ms": ms, "tflops": flops / ms / 1e9, "gbs": byts / ms / 1e6,
                      "gflop": flops / 1e9, "mbytes": byts / 1e6, "status": capi.device_status()}), flush=True)


def run_issue_probe(args):
    """What an MMA issuing scheme costs (dlp_tf32_issue_probe): clock cycles per k-block of twelve TF32 MMAs with every barrier
    already complete, for 64- and 128-column MMAs.  Prints a markdown table."""
    import torch
    from dlprimitives_b200 import capi
    torch.cuda.set_device(0)
    torch.zeros(1, device="cuda")
    names = ["one thread, no waits", "lanes 0..2 each wait on one barrier, vote", "every lane tests the same barriers (uniform)",
             "two issuer warps, pairs of k-blocks in turn"]
    print("| scheme | N = 64 | N = 128 |\n|---|---:|---:|")
    for scheme, name in enumerate(names):
        print("| %d: %s | %.0f | %.0f |" % (scheme, name, capi.tf32_issue_probe(scheme, 64), capi.tf32_issue_probe(scheme, 128)))
    print("\nfloor: twelve MMAs of 32 (N = 64) or 64 (N = 128) cycles = 384 / 768; device status %s" % (capi.device_status(),))


def run_config_table(args):
    """The shapes of the benchmark configurations 1-4, one row each: GPU time through the C ABI (packed weights, CUDA events,
    median of a few bursts), TFLOP/s, GB/s, the applicable roof and the fraction reached, and beside it the reference's own
    CPU operator (oracle/_ref, one core; the C restatement when that build is absent) timed on one or two images of the row
    and scaled to its batch.  Prints a markdown table."""
    import torch
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    peaks = measured_peaks()
    tensor_peak = peaks["bf16_tflops_sustained"] / 6.0
    ridge = tensor_peak * 1e3 / peaks["hbm_gbs"]
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev)
    gen.manual_seed(7)
    rows = []

    def gpu_time(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(10):
                fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / 10)
        return statistics.median(times)

    def cpu_conv_seconds(x, w, b, opts, images):
        """Seconds per image of the reference CPU operator (its own code when built here, else the C restatement)."""
        xs = x[:images].cpu().numpy()
        if ob.ref_available():
            op = ob.RefOperator("Convolution2D", opts, [xs.shape])
            op.forward([xs], [w.cpu().numpy()] + ([b.cpu().numpy()] if b is not None else []))
            return op.seconds / images, "reference"
        t0 = time.time()
        ob.conv2d(xs, w.cpu().numpy(), None if b is None else b.cpu().numpy(), stride=opts["stride"][0], pad=opts["pad"][0], groups=opts["groups"],
                  activation=opts.get("activation", "identity"))
        return (time.time() - t0) / images, "port"

    def conv_row(cfg, n, cin, hw, cout, k, stride, pad, groups=1, act="identity", bias=False, algo=""):
        x = torch.randn(n, cin, hw, hw, device=dev, generator=gen)
        w = torch.randn(cout, cin // groups, k, k, device=dev, generator=gen) * (2.0 / (cin // groups * k * k)) ** 0.5
        b = (torch.rand(cout, device=dev, generator=gen) * 0.2 - 0.1) if bias else None
        plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=k, stride=stride, pad=pad, groups=groups, batch=n, height=hw,
                                  width=hw, bias=bias, activation=act, algo=algo)
        y = torch.empty(plan.output_shape(n), device=dev)
        ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=dev)
        packed = plan.prepack(w)
        ms = gpu_time(lambda: plan.enqueue_packed(x, packed, b, y, ws=ws))
        flops = 2.0 * y.numel() * (cin // groups) * k * k
        byts = 4.0 * (x.numel() + y.numel() + w.numel() + (cout if bias else 0))
        opts = {"channels_in": cin, "channels_out": cout, "kernel": [k, k], "stride": [stride, stride], "pad": [pad, pad], "dilate": [1, 1],
                "groups": groups, "bias": bias, "activation": act}
        sec, kind = cpu_conv_seconds(x, w, b, opts, 1 if flops / n > 2e8 else 2)
        rows.append((cfg, "conv %dx%d/%d g%d %d->%d @%d N=%d %s" % (k, k, stride, groups, cin, cout, hw, n, act), plan.algo() + " " + plan.kernel(), ms, flops, byts,
                     sec * n * 1e3, kind))

    conv_row("1", 16, 64, 56, 64, 3, 1, 1, act="relu", bias=True)
    # configuration 2: InnerProduct 256 x 2048 -> 1000 and the three 1x1 convolutions
    x = torch.randn(256, 2048, device=dev, generator=gen)
    w = torch.randn(1000, 2048, device=dev, generator=gen) * (2.0 / 2048) ** 0.5
    b = torch.zeros(1000, device=dev)
    ip = capi.IPForward(2048, 1000, 256, bias=True)
    y = torch.empty(256, 1000, device=dev)
    ws = torch.empty(max(ip.workspace(), 16), dtype=torch.uint8, device=dev)
    packed = ip.prepack(w)
    ms = gpu_time(lambda: ip.enqueue_packed(x, packed, b, y, ws=ws))
    t0 = time.time()
    ob.inner_product(x[:16].cpu().numpy(), w.cpu().numpy(), b.cpu().numpy())
    rows.append(("2", "InnerProduct 2048->1000 M=256", ip.kernel(), ms, 2.0 * 256 * 1000 * 2048, 4.0 * (x.numel() + y.numel() + w.numel() + 1000),
                 (time.time() - t0) / 16 * 256 * 1e3, "port"))
    for cin, cout in ((256, 1024), (1024, 256), (512, 2048)):
        conv_row("2", 64, cin, 14, cout, 1, 1, 0, bias=True)
    for c, hw, stride, cout in ((32, 112, 1, 16), (96, 112, 2, 24), (144, 56, 1, 24), (144, 56, 2, 32), (192, 28, 1, 32), (192, 28, 2, 64), (384, 14, 1, 64),
                                (384, 14, 1, 96), (576, 14, 1, 96), (576, 14, 2, 160), (960, 7, 1, 160), (960, 7, 1, 320)):
        conv_row("3 dw", 128, c, hw, c, 3, stride, 1, groups=c)
        conv_row("3 pw", 128, c, (hw + 2 - 3) // stride + 1, cout, 1, 1, 0, act="relu6")
    for c, hw in ((64, 56), (128, 28), (256, 14), (512, 7)):
        for algo in ("gemm", "winograd"):
            conv_row("4 " + algo, 64, c, hw, c, 3, 1, 1, algo=algo)
    print("| cfg | shape | algorithm / kernel | GPU ms | TFLOP/s | GB/s | FLOP/B | roof | frac | CPU ms (1 core, scaled) | CPU code | GPU/CPU |")
    print("|---|---|---|---:|---:|---:|---:|---|---:|---:|---|---:|")
    for cfg, shape, kernel, ms, flops, byts, cpu_ms, kind in rows:
        tf, gbs, ai = flops / ms / 1e9, byts / ms / 1e6, flops / byts
        tensor = "tf32x3" in kernel and ai > ridge
        frac = tf / tensor_peak if tensor else gbs / peaks["hbm_gbs"]
        print("| %s | %s | %s | %.4f | %.1f | %.0f | %.0f | %s | %.2f | %.0f | %s | %.0fx |"
              % (cfg, shape, kernel, ms, tf, gbs, ai, "tensor" if tensor else "hbm", frac, cpu_ms, kind, cpu_ms / ms))
    print()
    print("roofs: tensor %.1f TFLOP/s (3xTF32 = bf16 sustained / 6), HBM %.1f GB/s (%s); tensor roof applies above %.0f FLOP/B"
          % (tensor_peak, peaks["hbm_gbs"], peaks["source"], ridge))


def main():
    global GLOBAL_BATCH
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--conv-algo", default="", help="algorithm request for --conv: '', gemm, winograd, depthwise_separable")
    ap.add_argument("--batch", type=int, default=GLOBAL_BATCH, help="global batch; the benchmark configuration is 256 -- other values are for "
                    "profiler captures on a small case only, and the line then says so in config.global_batch")
    ap.add_argument("--layers-out", default=None, help="write the per-layer table (time, FLOP, bytes, applicable roof, fraction) to this JSON file")
    ap.add_argument("--configs", action="store_true", help="print the per-shape table of benchmark configurations 1-4 (GPU, with the reference CPU time beside it)")
    ap.add_argument("--issue-probe", action="store_true", help="print what the MMA issuing schemes cost (cycles per k-block, MMA-only kernels)")
    ap.add_argument("--conv", default=None, help="profile one convolution instead: N,Cin,H,Cout,K,stride,pad[,groups[,residual]]")
    args = ap.parse_args()
    GLOBAL_BATCH = args.batch
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.conv:
        run_single_conv(args)
        return
    if args.configs:
        run_config_table(args)
        return
    if args.issue_probe:
        run_issue_probe(args)
        return
    if world != args.gpus:
        raise SystemExit("--gpus %d needs %d ranks (launch with torch.distributed.run --nproc-per-node %d), got WORLD_SIZE=%d"
                         % (args.gpus, args.gpus, args.gpus, world))
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
