"""Per-layer throughput sweep: GFLOP/s and GB/s of convolution and GEMM shapes through the C ABI.

The counterpart of the reference's ``dlprim_flops`` tool (tools/flops.cpp:594-671 for the convolution
loop, :343-388 for GEMM, :678-760 for the table of layer shapes it sweeps by default): the same default
layer shapes at batch 64, the same work and byte counts (flops = 2 * |Y| * Cin/g * k * k,
bytes = 4 * (|X| + |Y| + |W|)), timed with CUDA events over repeated launches after a warm-up, reported
against the measured tensor-core and HBM peaks.  Forward only.

    python -m dlprimitives_b200.flops [--batch 64] [--full] [--csv report.csv] [--gemm] [--algo winograd]
"""
import argparse
import json
import os
import sys

# (kernel, pad, stride, groups, channels in, channels out, height = width, network): the reference tool's default sweep
CONV_SHAPES = [
    (3, 1, 1, 480, 480, 480, 14, "effnet"),
    (11, 2, 4, 1, 3, 64, 224, "alexnet"),
    (5, 2, 1, 2, 96, 192, 27, "alexnet"),
    (5, 2, 1, 1, 64, 192, 27, "alexnet"),
    (3, 1, 1, 1, 384, 256, 13, "alexnet"),
    (7, 3, 2, 1, 3, 64, 224, "resnet"),
    (1, 0, 1, 1, 64, 256, 56, "resnet"),
    (1, 0, 1, 1, 64, 64, 56, "resnet"),
    (3, 1, 1, 1, 64, 64, 56, "resnet"),
    (1, 0, 2, 1, 1024, 2048, 14, "resnet"),
    (1, 0, 1, 1, 1024, 256, 14, "resnet"),
    (3, 1, 1, 1, 256, 256, 14, "resnet"),
    (3, 1, 1, 1, 3, 64, 224, "vgg"),
    (3, 1, 1, 1, 64, 64, 224, "vgg"),
    (3, 1, 1, 1, 512, 512, 28, "vgg"),
    (3, 1, 2, 1, 3, 32, 224, "mobile"),
    (3, 1, 1, 144, 144, 144, 56, "mobile"),
    (3, 1, 2, 144, 144, 144, 56, "mobile"),
    (1, 0, 1, 1, 144, 24, 56, "mobile"),
    (1, 0, 1, 1, 24, 144, 56, "mobile"),
    (1, 0, 1, 1, 960, 160, 7, "mobile"),
    (1, 0, 1, 1, 960, 320, 7, "mobile"),
    (3, 1, 1, 960, 960, 960, 7, "mobile"),
    (1, 0, 1, 256, 256, 256, 56, "scale"),
    (1, 0, 1, 1024, 1024, 1024, 7, "scale"),
]
# The further layer shapes the reference tool adds when it is built with FULL_TEST (tools/flops.cpp:709-760), which then
# also runs batches 16, 64 and 128: --full here.
FULL_CONV_SHAPES = [
    (3, 1, 1, 1, 192, 384, 13, "alexnet"), (3, 1, 1, 1, 256, 256, 13, "alexnet"), (3, 1, 1, 2, 384, 256, 13, "alexnet"),
    (11, 2, 4, 1, 3, 96, 224, "alexnet"),
    (1, 0, 1, 1, 1024, 512, 14, "resnet"), (3, 1, 1, 1, 128, 128, 28, "resnet"), (3, 1, 2, 1, 128, 128, 56, "resnet"),
    (1, 0, 1, 1, 128, 512, 28, "resnet"), (1, 0, 1, 1, 2048, 512, 7, "resnet"), (1, 0, 1, 1, 256, 1024, 14, "resnet"),
    (1, 0, 1, 1, 256, 128, 56, "resnet"), (3, 1, 2, 1, 256, 256, 28, "resnet"), (1, 0, 2, 1, 256, 512, 56, "resnet"),
    (1, 0, 1, 1, 256, 64, 56, "resnet"), (1, 0, 2, 1, 512, 1024, 28, "resnet"), (1, 0, 1, 1, 512, 128, 28, "resnet"),
    (1, 0, 1, 1, 512, 2048, 7, "resnet"), (1, 0, 1, 1, 512, 256, 28, "resnet"), (3, 1, 1, 1, 512, 512, 7, "resnet"),
    (3, 1, 2, 1, 512, 512, 14, "resnet"),
    (3, 1, 1, 1, 128, 128, 112, "vgg"), (3, 1, 1, 1, 128, 256, 56, "vgg"), (3, 1, 1, 1, 256, 256, 56, "vgg"),
    (3, 1, 1, 1, 256, 512, 28, "vgg"), (3, 1, 1, 1, 512, 512, 14, "vgg"), (3, 1, 1, 1, 64, 128, 112, "vgg"),
    (1, 0, 1, 1, 144, 32, 28, "mobile"), (1, 0, 1, 1, 160, 960, 7, "mobile"), (1, 0, 1, 1, 16, 96, 112, "mobile"),
    (3, 1, 1, 192, 192, 192, 28, "mobile"), (3, 1, 2, 192, 192, 192, 28, "mobile"), (1, 0, 1, 1, 192, 32, 28, "mobile"),
    (1, 0, 1, 1, 192, 64, 14, "mobile"), (1, 0, 1, 1, 320, 1280, 7, "mobile"), (1, 0, 1, 1, 32, 16, 112, "mobile"),
    (1, 0, 1, 1, 32, 192, 28, "mobile"), (3, 1, 1, 32, 32, 32, 112, "mobile"), (3, 1, 1, 384, 384, 384, 14, "mobile"),
    (1, 0, 1, 1, 384, 64, 14, "mobile"), (1, 0, 1, 1, 384, 96, 14, "mobile"), (1, 0, 1, 1, 576, 160, 7, "mobile"),
    (3, 1, 1, 576, 576, 576, 14, "mobile"), (3, 1, 2, 576, 576, 576, 14, "mobile"), (1, 0, 1, 1, 576, 96, 14, "mobile"),
    (1, 0, 1, 1, 64, 384, 14, "mobile"), (1, 0, 1, 1, 96, 24, 56, "mobile"), (1, 0, 1, 1, 96, 576, 14, "mobile"),
    (3, 1, 2, 96, 96, 96, 112, "mobile"),
]
FULL_BATCHES = (16, 64, 128)
# (M, N, K): square and skinny products, and the InnerProduct shapes of the classifier heads
GEMM_SHAPES = [(512, 512, 512), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (64, 1000, 2048), (256, 1000, 2048),
               (64, 4096, 9216), (8192, 256, 1024), (12544, 64, 147)]


def peaks():
    """HBM GB/s and 3xTF32 TFLOP/s roofs: from MEASURED_PEAKS.json at the repository root when that file exists (a copy
    bandwidth and a bf16 GEMM rate measured on the target GPUs), else from an earlier measurement of the same kind."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    hbm, bf16 = 6650.0, 1400.0
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        hbm = float(d.get("hbm_gbs", hbm))
        bf16 = float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", bf16)))
    return hbm, bf16 / 2.0 / 3.0          # 3xTF32: half the bf16 rate, three products per term


def time_launches(fn, warmup, reps):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def run_conv(batch, algo, reps, rows, shapes=None):
    import torch
    from . import capi
    hbm, tensor = peaks()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(3)
    print("%-8s %-30s %9s %7s %8s %7s  %s" % ("net", "convolution", "GFLOP/s", "% roof", "GB/s", "% HBM", "algorithm / kernel"))
    for k, pad, stride, groups, cin, cout, dim, net in (shapes or CONV_SHAPES):
        plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=k, stride=stride, pad=pad, groups=groups, batch=batch,
                                  height=dim, width=dim, bias=False, activation="identity", algo=algo)
        x = torch.randn(batch, cin, dim, dim, device=dev, generator=g)
        w = torch.randn(cout, cin // groups, k, k, device=dev, generator=g)
        y = torch.empty(plan.output_shape(batch), device=dev)
        packed = plan.prepack(w)                                     # inference weights are constant: packed once
        ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=dev)
        ms = time_launches(lambda: plan.enqueue_packed(x, packed, None, y, ws=ws), 3, reps)
        flops = 2.0 * y.numel() * (cin // groups) * k * k
        byts = 4.0 * (x.numel() + y.numel() + w.numel())
        gflops, gbs = flops / ms / 1e6, byts / ms / 1e6
        name = "k%d p%d s%d g%d %d->%d @%d" % (k, pad, stride, groups, cin, cout, dim)
        print("%-8s %-30s %9.0f %6.1f%% %8.0f %6.1f%%  %s / %s" % (net, name, gflops, gflops / 10.0 / tensor, gbs, gbs / hbm * 100.0,
                                                                 plan.algo(), plan.kernel()))
        rows.append(["conv", net, batch, k, pad, stride, cin, cout, groups, dim, "%.1f" % gflops, "%.1f" % (gflops / 10.0 / tensor),
                     "%.1f" % gbs, "%.1f" % (gbs / hbm * 100.0), plan.algo(), plan.kernel()])
    if capi.device_status() != 0:
        raise RuntimeError("a bounded device-side wait gave up during the sweep, code %d" % capi.device_status())


def run_gemm(reps, rows):
    import torch
    from . import capi
    hbm, tensor = peaks()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev)
    g.manual_seed(4)
    print("%-24s %9s %7s %8s  %s" % ("GEMM  C = A * B^T", "GFLOP/s", "% roof", "GB/s", "kernel"))
    for m, n, k in GEMM_SHAPES:
        gm = capi.Gemm(False, True, m, n, k)
        a = torch.randn(m, k, device=dev, generator=g)
        b = torch.randn(n, k, device=dev, generator=g)
        c = torch.empty(m, n, device=dev)
        ws = torch.empty(max(gm.workspace(), 16), dtype=torch.uint8, device=dev)
        ms = time_launches(lambda: gm.gemm(m, n, k, a, k, b, k, c, n, ws=ws), 3, reps)     # packs B on every call, as the interface implies
        flops = 2.0 * m * n * k
        byts = 4.0 * (m * k + n * k + m * n)
        gflops, gbs = flops / ms / 1e6, byts / ms / 1e6
        print("%-24s %9.0f %6.1f%% %8.0f  %s" % ("%d x %d x %d" % (m, n, k), gflops, gflops / 10.0 / tensor, gbs, gm.kernel()))
        rows.append(["gemm", "", "", "", "", "", k, n, "", m, "%.1f" % gflops, "%.1f" % (gflops / 10.0 / tensor), "%.1f" % gbs,
                     "%.1f" % (gbs / hbm * 100.0), "gemm", gm.kernel()])


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--algo", default="", help="convolution algorithm request: '', gemm, winograd, depthwise_separable")
    ap.add_argument("--gemm", action="store_true", help="sweep the GEMM shapes as well")
    ap.add_argument("--csv", default=None, help="also write the table as CSV")
    ap.add_argument("--full", action="store_true", help="the reference tool's FULL_TEST sweep: 48 more layer shapes, batches 16, 64 and 128")
    args = ap.parse_args()
    rows = []
    if args.full:
        for batch in FULL_BATCHES:
            print("batch %d" % batch)
            run_conv(batch, args.algo, args.reps, rows, CONV_SHAPES + FULL_CONV_SHAPES)
    else:
        run_conv(args.batch, args.algo, args.reps, rows)
    if args.gemm:
        run_gemm(args.reps, rows)
    if args.csv:
        import csv
        with open(args.csv, "w", newline="") as f:
            wr = csv.writer(f)
            wr.writerow(["op", "network", "batch", "kernel", "pad", "stride", "channels_in_or_K", "channels_out_or_N", "groups", "size_or_M",
                         "gflops", "gflops_pct_of_roof", "gbs", "gbs_pct_of_hbm", "algorithm", "kernel_name"])
            wr.writerows(rows)
    return 0


if __name__ == "__main__":
    sys.exit(main())
