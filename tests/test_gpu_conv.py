"""GPU parity of the convolution forward path, through the C ABI and through the factory-made
Convolution2D operator, against the golden vectors and the CPU checker."""
import numpy as np
import pytest
import torch

from conftest import reference_tolerance, small_frac
from gpu_util import DEV, REL_TOL, kaiming, pair, rel_err, to_dev

pytestmark = pytest.mark.gpu


def oracle_conv(opt, x, w, b):
    from oracle import bindings as ob
    return ob.conv2d(x, w, b, stride=opt.get("stride", 1), pad=opt.get("pad", 0), dilate=opt.get("dilate", 1),
                     groups=opt.get("groups", 1), activation=opt.get("activation", "identity"))


def run_operator(opt, x, params):
    from dlprimitives_b200 import hostapi
    op = hostapi.Operator("Convolution2D", opt, [x.shape])
    out, = op.forward([to_dev(x)], [to_dev(p) for p in params])
    torch.cuda.synchronize()
    return op, out.cpu().numpy()


@pytest.mark.parametrize("algo", ["", "gemm", "winograd", "depthwise_separable"])
def test_golden_conv2d_cases(golden, algo):
    """The reference's conv2d / conv2d_gemm / conv2d_win / conv2d_dsc sweeps: every embedded case."""
    n = 0
    worst = 0.0
    for opt, params, ins, outs, eps in golden.embedded("conv2d"):
        opt = dict(opt)
        if algo:
            opt["fwd_algo"] = algo
        op, y = run_operator(opt, ins[0], params)
        assert y.shape == outs[0].shape
        err = rel_err(y, outs[0])
        worst = max(worst, err)
        assert err <= REL_TOL, (opt, op.kernel, err)
        # the reference's own bound, eps * max(1, sigma), loosened by the 3xTF32 rounding headroom
        assert np.abs(y - outs[0]).max() <= 4 * reference_tolerance(outs[0], eps), (opt, op.kernel)
        n += 1
    assert n >= 100
    print("worst normalised error", worst)


def test_reference_sweep_large_shapes_bit_exact_on_small_frac(golden):
    """The cases the reference checks against its CPU operator ("use_cpu_reference"), with its
    "small_frac" inputs (multiples of 0.5): every product and partial sum is exact in fp32, so the
    GPU result must equal the CPU checker's bit for bit whatever the summation order."""
    from oracle import bindings as ob
    ob.set_threads(16)
    rng = np.random.default_rng(21)
    seen = 0
    for opt, param_shapes, in_shapes, out_shapes, params in golden.checker_only("conv2d"):
        shape = list(in_shapes[0])
        if shape[0] * shape[1] * shape[2] * shape[3] > 3_000_000:
            shape[0] = max(1, 3_000_000 // (shape[1] * shape[2] * shape[3]))    # bound the CPU checker's time
        x = small_frac(rng, shape)
        ps = [small_frac(rng, s) for s in param_shapes]
        b = ps[1] if opt.get("bias", True) else None
        want = oracle_conv(opt, x, ps[0], b)
        op, got = run_operator(opt, x, ps)
        assert got.shape == want.shape
        assert np.array_equal(got, want), (opt, shape, op.kernel, np.abs(got - want).max())
        seen += 1
    assert seen >= 100


CONFIG_SHAPES = [
    # (name, N, Cin, H, Cout, k, stride, pad, groups, bias, act)
    ("cfg1_3x3_64_56", 16, 64, 56, 64, 3, 1, 1, 1, True, "relu"),
    ("cfg2_1x1_256_1024", 64, 256, 14, 1024, 1, 1, 0, 1, True, "identity"),
    ("cfg2_1x1_1024_256", 64, 1024, 14, 256, 1, 1, 0, 1, True, "identity"),
    ("cfg2_1x1_512_2048", 64, 512, 14, 2048, 1, 1, 0, 1, True, "identity"),
    ("cfg4_3x3_64_56", 64, 64, 56, 64, 3, 1, 1, 1, False, "identity"),
    ("cfg4_3x3_128_28", 64, 128, 28, 128, 3, 1, 1, 1, False, "identity"),
    ("cfg4_3x3_256_14", 64, 256, 14, 256, 3, 1, 1, 1, False, "identity"),
    ("cfg4_3x3_512_7", 64, 512, 7, 512, 3, 1, 1, 1, False, "identity"),
    ("resnet_stem_7x7", 8, 3, 224, 64, 7, 2, 3, 1, True, "relu"),
    ("resnet_3x3_s2", 16, 128, 56, 128, 3, 2, 1, 1, True, "relu"),
    ("resnet_1x1_s2", 16, 256, 56, 512, 1, 2, 0, 1, True, "identity"),
]


@pytest.mark.parametrize("cfg", CONFIG_SHAPES, ids=[c[0] for c in CONFIG_SHAPES])
def test_config_shapes_full_size(cfg):
    """The benchmark configurations at their full sizes against the CPU checker; the batch the CPU
    side computes is capped (images are independent) so each case stays within seconds."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    ob.set_threads(16)
    name, N, cin, H, cout, k, stride, pad, groups, bias, act = cfg
    rng = np.random.default_rng(hash(name) % 2**31)
    x = rng.standard_normal((N, cin, H, H), dtype=np.float32)
    w = kaiming(rng, (cout, cin // groups, k, k))
    b = (rng.uniform(-0.1, 0.1, cout).astype(np.float32) if name.startswith("cfg1") else np.zeros(cout, np.float32)) if bias else None
    plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=k, stride=stride, pad=pad, groups=groups, batch=N, height=H,
                              width=H, bias=bias, activation=act)
    xd, wd, bd = to_dev(x), to_dev(w), to_dev(b)
    y = torch.full(plan.output_shape(N), float("nan"), device=DEV)
    ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=DEV)
    plan.enqueue(xd, wd, bd, y, ws)
    assert capi.device_status() == 0
    got = y.cpu().numpy()
    assert not np.isnan(got).any()
    cpu_images = min(N, 8)
    sel = np.linspace(0, N - 1, cpu_images).astype(int)          # first, last and some in between
    want = ob.conv2d(x[sel], w, b, stride=stride, pad=pad, groups=groups, activation=act)
    err = rel_err(got[sel], want)
    assert err <= REL_TOL, (plan.kernel(), err)
    # a cheap whole-batch property: every image of the batch gives the same result as when it runs alone,
    # up to the order of the fp32 sum over K (a batch with few output tiles is cut along K)
    y1 = torch.empty(plan.output_shape(1), device=DEV)
    for i in (0, N - 1):
        plan.enqueue(xd[i:i + 1].contiguous(), wd, bd, y1, ws)
        assert rel_err(y1[0].cpu().numpy(), y[i].cpu().numpy()) <= 2e-6


def test_depthwise_mobilenet_rows():
    """Config 3: the depthwise layers of MobileNetV2 (stride 1 and 2) followed by their pointwise
    1x1 convolution with ReLU6, N = 128, compared on a subset of the images."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    ob.set_threads(16)
    rows = [(32, 112, 1, 16), (96, 112, 2, 24), (144, 56, 1, 24), (144, 56, 2, 32), (192, 28, 1, 32), (192, 28, 2, 64),
            (384, 14, 1, 64), (384, 14, 1, 96), (576, 14, 1, 96), (576, 14, 2, 160), (960, 7, 1, 160), (960, 7, 1, 320)]
    rng = np.random.default_rng(33)
    for C, H, stride, cout in rows:
        N = 128                                           # the configuration's batch; the CPU side checks three of the images
        x = rng.standard_normal((N, C, H, H), dtype=np.float32)
        wd_ = (rng.standard_normal((C, 1, 3, 3)) * np.sqrt(2.0 / 9)).astype(np.float32)
        wp = kaiming(rng, (cout, C, 1, 1))
        dw = capi.Conv2DForward(channels_in=C, channels_out=C, kernel=3, stride=stride, pad=1, groups=C, batch=N, height=H, width=H,
                                bias=False, activation="identity")
        assert dw.algo() == "depthwise_separable" and dw.kernel() == "depthwise_k3_s%d" % stride
        mid = torch.empty(dw.output_shape(N), device=DEV)
        dw.enqueue(to_dev(x), to_dev(wd_), None, mid, None)
        OH = mid.shape[2]
        pw = capi.Conv2DForward(channels_in=C, channels_out=cout, kernel=1, batch=N, height=OH, width=OH, bias=False, activation="relu6")
        out = torch.empty(pw.output_shape(N), device=DEV)
        ws = torch.empty(max(pw.workspace(), 16), dtype=torch.uint8, device=DEV)
        pw.enqueue(mid, to_dev(wp), None, out, ws)
        assert capi.device_status() == 0
        sel = [0, N // 2, N - 1]
        want_mid = ob.conv2d(x[sel], wd_, None, stride=stride, pad=1, groups=C)
        want = ob.conv2d(want_mid, wp, None, activation="relu6")
        assert rel_err(mid.cpu().numpy()[sel], want_mid) <= 1e-5, (C, H, stride)     # plain fp32 FMA path
        assert rel_err(out.cpu().numpy()[sel], want) <= REL_TOL, (C, H, stride, cout)


def test_enqueue_contract():
    """y = factor*y + act(conv + bias); y is not read when factor == 0; a smaller batch than planned
    is accepted; every activation; all three kernel families."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    rng = np.random.default_rng(5)
    cases = [dict(groups=1, math_mode=capi.MATH_AUTO), dict(groups=1, math_mode=capi.MATH_FP32_FFMA), dict(groups=2, math_mode=capi.MATH_AUTO),
             dict(groups=12, math_mode=capi.MATH_AUTO)]
    for case in cases:
        g = case["groups"]
        for act in ("identity", "relu", "tanh", "sigmoid", "relu6"):
            x = rng.standard_normal((3, 12, 10, 9), dtype=np.float32)
            w = kaiming(rng, (12, 12 // g, 3, 3)) * 3
            b = rng.uniform(-1, 1, 12).astype(np.float32)
            plan = capi.Conv2DForward(channels_in=12, channels_out=12, kernel=3, pad=1, groups=g, batch=5, height=10, width=9, bias=True,
                                      activation=act, math_mode=case["math_mode"])
            ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=DEV)
            want = ob.conv2d(x, w, b, pad=1, groups=g, activation=act)
            y = torch.full(plan.output_shape(3), float("nan"), device=DEV)
            plan.enqueue(to_dev(x), to_dev(w), to_dev(b), y, ws, factor=0.0)
            assert rel_err(y.cpu().numpy(), want) <= REL_TOL, (case, act, plan.kernel())
            y0 = rng.standard_normal(want.shape).astype(np.float32)
            y = to_dev(y0)
            plan.enqueue(to_dev(x), to_dev(w), to_dev(b), y, ws, factor=0.5)
            assert rel_err(y.cpu().numpy(), 0.5 * y0 + want) <= REL_TOL, (case, act, plan.kernel())
    assert capi.device_status() == 0


def test_fused_residual_matches_conv_then_elementwise():
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    rng = np.random.default_rng(6)
    x = rng.standard_normal((4, 64, 14, 14), dtype=np.float32)
    w = kaiming(rng, (256, 64, 1, 1))
    b = rng.uniform(-0.1, 0.1, 256).astype(np.float32)
    res = rng.standard_normal((4, 256, 14, 14), dtype=np.float32)
    plan = capi.Conv2DForward(channels_in=64, channels_out=256, kernel=1, batch=4, height=14, width=14, bias=True, activation="identity")
    packed = plan.prepack(to_dev(w))
    y = torch.empty(plan.output_shape(4), device=DEV)
    plan.enqueue_packed(to_dev(x), packed, to_dev(b), y, residual=to_dev(res), residual_scale=1.0, post_activation="relu")
    want = ob.elementwise(ob.conv2d(x, w, b), res, "sum", 1.0, 1.0, "relu")
    assert rel_err(y.cpu().numpy(), want) <= REL_TOL
    # in place: the residual buffer is also the output
    r = to_dev(res)
    plan.enqueue_packed(to_dev(x), packed, to_dev(b), r, residual=r, residual_scale=0.5, post_activation="identity")
    want = ob.elementwise(ob.conv2d(x, w, b), res, "sum", 1.0, 0.5, "identity")
    assert rel_err(r.cpu().numpy(), want) <= REL_TOL


def test_algorithm_selection_follows_the_reference_rules():
    """src/core/conv.cpp:672-729: "depthwise_separable" and "winograd" requests that are not
    eligible fall back to "gemm"; the selection strings are the reference's."""
    from dlprimitives_b200 import capi
    mk = lambda **kw: capi.Conv2DForward(batch=2, height=16, width=16, **kw)
    assert mk(channels_in=16, channels_out=16, kernel=3, pad=1, groups=16).algo() == "depthwise_separable"
    assert mk(channels_in=16, channels_out=16, kernel=3, pad=1, groups=16, algo="gemm").algo() == "gemm"
    assert mk(channels_in=16, channels_out=16, kernel=3, pad=1, groups=16, stride=2).algo() == "depthwise_separable"   # native stride 2
    assert mk(channels_in=16, channels_out=16, kernel=3, pad=1, groups=16, stride=2, algo="depthwise_separable").algo() == "gemm"
    assert mk(channels_in=16, channels_out=32, kernel=3, pad=1, groups=16).algo() == "gemm"     # channel multiplier: not handled as depthwise
    assert mk(channels_in=16, channels_out=16, kernel=3, pad=0, algo="winograd").algo() == "gemm"
    assert mk(channels_in=16, channels_out=16, kernel=3, pad=1, stride=2, algo="winograd").algo() == "gemm"
    win = mk(channels_in=16, channels_out=16, kernel=3, pad=1, algo="winograd")
    assert win.algo() == "winograd" and win.kernel() == "winograd_f23_tf32x3"         # the sixteen products on the tensor cores
    win = mk(channels_in=16, channels_out=16, kernel=3, pad=1, algo="winograd", math_mode=capi.MATH_FP32_FFMA)
    assert win.algo() == "winograd" and win.kernel() == "winograd_f23_ffma"
    assert win.workspace() >= 16 * 16 * 16 * 4          # the reference's 16*Cin*Cout floats (src/core/conv.cpp:229-232)
    assert mk(channels_in=16, channels_out=16, kernel=3, pad=1).algo() == "gemm"    # "auto" keeps the tensor-core kernel here
    assert mk(channels_in=16, channels_out=16, kernel=1).algo() == "gemm"
    assert mk(channels_in=16, channels_out=16, kernel=1).kernel().startswith("igemm_tf32x3")
    assert mk(channels_in=16, channels_out=16, kernel=3, groups=2).kernel().startswith("igemm_ffma")


def test_errors_are_reported_not_swallowed():
    from dlprimitives_b200 import capi, hostapi
    plan = capi.Conv2DForward(channels_in=8, channels_out=8, kernel=3, pad=1, batch=2, height=8, width=8, bias=True)
    x = torch.zeros(2, 8, 8, 8, device=DEV)
    w = torch.zeros(8, 8, 3, 3, device=DEV)
    y = torch.zeros(2, 8, 8, 8, device=DEV)
    ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=DEV)
    with pytest.raises(capi.ValidationError):
        plan.enqueue(x, w, None, y, ws)                            # the plan has a bias, none given
    with pytest.raises(capi.ValidationError):
        plan.enqueue(torch.zeros(2, 8, 9, 8, device=DEV), w, torch.zeros(8, device=DEV), y, ws)   # height differs from the plan
    if plan.workspace() > 0:
        with pytest.raises(capi.ValidationError):
            plan.enqueue(x, w, torch.zeros(8, device=DEV), y, None)    # workspace missing
    with pytest.raises(hostapi.HostError) as e:
        hostapi.Operator("Convolution2D", {"channels_in": 4, "channels_out": 8, "kernel": 3}, [(1, 5, 8, 8)])   # channel mismatch
    assert e.value.kind == "ValidationError"
    with pytest.raises(hostapi.HostError) as e:
        hostapi.Operator("NoSuchOperator", {}, [(1, 5, 8, 8)])
    assert e.value.kind == "ValidationError"
    # empty batch: nothing to do, no launch, no error
    plan.enqueue(torch.zeros(0, 8, 8, 8, device=DEV), w, torch.zeros(8, device=DEV), torch.zeros(0, 8, 8, 8, device=DEV), ws)


@pytest.mark.parametrize("math_mode", [0, 1], ids=["tensor_cores", "ffma"])
@pytest.mark.parametrize("cin,hw,cout,batch", [(64, 56, 64, 4), (128, 28, 128, 8), (256, 14, 256, 8), (512, 7, 512, 16), (24, 13, 40, 3)])
def test_winograd_config_shapes(cin, hw, cout, batch, math_mode):
    """The Winograd benchmark configuration's shapes (and one with odd sizes and ragged channel counts)
    against the CPU checker: plain call with factor, packed call with the fused residual."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    ob.set_threads(16)
    rng = np.random.default_rng(cin * 1000 + hw)
    x = rng.standard_normal((batch, cin, hw, hw), dtype=np.float32)
    w = kaiming(rng, (cout, cin, 3, 3))
    b = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=3, stride=1, pad=1, batch=batch, height=hw, width=hw,
                              bias=True, activation="relu", algo="winograd", math_mode=math_mode)
    assert plan.algo() == "winograd" and plan.kernel() == ("winograd_f23_ffma" if math_mode else "winograd_f23_tf32x3")
    xd, wd, bd = to_dev(x), to_dev(w), to_dev(b)
    want = ob.conv2d(x, w, b, stride=1, pad=1, activation="relu")
    y0 = rng.standard_normal(want.shape, dtype=np.float32)
    y = to_dev(y0)
    ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=DEV)
    plan.enqueue(xd, wd, bd, y, ws, factor=0.5)
    assert rel_err(y.cpu().numpy(), want + 0.5 * y0) <= REL_TOL
    res = rng.standard_normal(want.shape, dtype=np.float32)
    packed = plan.prepack(wd)
    y2 = torch.full(plan.output_shape(batch), float("nan"), device=DEV)
    plan.enqueue_packed(xd, packed, bd, y2, residual=to_dev(res), residual_scale=1.0, post_activation="relu", ws=ws)
    assert rel_err(y2.cpu().numpy(), np.maximum(want + res, 0.0)) <= REL_TOL
    # a smaller batch than planned runs in the same workspace
    y3 = torch.empty(plan.output_shape(1), device=DEV)
    plan.enqueue_packed(xd[:1].contiguous(), packed, bd, y3, ws=ws)
    assert rel_err(y3.cpu().numpy(), want[:1]) <= REL_TOL
    assert capi.device_status() == 0


def test_split_k_small_batch_matches_checker_and_is_deterministic():
    """A problem with few output tiles (layer-4 shapes at a small batch) is cut along K when the caller
    provides the workspace: same result as the checker, run-to-run identical, and within rounding of the
    uncut kernel (a different but fixed summation order)."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    ob.set_threads(16)
    rng = np.random.default_rng(404)
    for cin, cout, k, pad in ((512, 512, 3, 1), (1024, 512, 1, 0)):
        batch, hw = 4, 7
        x = rng.standard_normal((batch, cin, hw, hw), dtype=np.float32)
        w = kaiming(rng, (cout, cin, k, k))
        b = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
        res = rng.standard_normal((batch, cout, hw, hw), dtype=np.float32)
        plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=k, stride=1, pad=pad, batch=batch, height=hw, width=hw,
                                  bias=True, activation="identity")
        assert plan.workspace() > plan.packed_bytes()        # room for the partial sums is part of the workspace
        xd, wd, bd, rd = to_dev(x), to_dev(w), to_dev(b), to_dev(res)
        packed = plan.prepack(wd)
        ws = torch.empty(plan.workspace(), dtype=torch.uint8, device=DEV)
        want = np.maximum(ob.conv2d(x, w, b, stride=1, pad=pad) + res, 0.0)
        outs = []
        for use_ws in (ws, ws, None):
            y = torch.full(plan.output_shape(batch), float("nan"), device=DEV)
            plan.enqueue_packed(xd, packed, bd, y, residual=rd, post_activation="relu", ws=use_ws)
            torch.cuda.synchronize()
            outs.append(y.cpu().numpy())
        assert rel_err(outs[0], want) <= REL_TOL and rel_err(outs[2], want) <= REL_TOL
        assert np.array_equal(outs[0], outs[1])
        # the plain call packs into the same workspace and cuts K as well
        y = torch.full(plan.output_shape(batch), float("nan"), device=DEV)
        plan.enqueue(xd, wd, bd, y, ws)
        assert rel_err(y.cpu().numpy(), ob.conv2d(x, w, b, stride=1, pad=pad)) <= REL_TOL
    assert capi.device_status() == 0


@pytest.mark.parametrize("cin,cout,hw,batch", [(40, 200, 13, 3), (64, 256, 28, 5), (96, 384, 13, 7), (128, 512, 14, 9), (256, 130, 9, 4)])
def test_one_by_one_expansions_with_fused_residual_ragged(cin, cout, hw, batch):
    """1x1 convolutions with the fused residual at sizes that leave partial row and column tiles and planes
    that are not a multiple of anything: covers the short-K mode (one or two k-blocks per tile, second set of
    epilogue warps) and the residual prefetcher (3 to 8 k-blocks)."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    ob.set_threads(16)
    rng = np.random.default_rng(cin * 7 + cout)
    x = rng.standard_normal((batch, cin, hw, hw), dtype=np.float32)
    w = kaiming(rng, (cout, cin, 1, 1))
    b = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    res = rng.standard_normal((batch, cout, hw, hw), dtype=np.float32)
    plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=1, batch=batch, height=hw, width=hw, bias=True, activation="identity")
    assert plan.kernel().startswith("igemm_tf32x3_bn128")
    xd, wd, bd, rd = to_dev(x), to_dev(w), to_dev(b), to_dev(res)
    packed = plan.prepack(wd)
    want = np.maximum(ob.conv2d(x, w, b) + 0.5 * res, 0.0)
    for _ in range(2):
        y = torch.full(plan.output_shape(batch), float("nan"), device=DEV)
        plan.enqueue_packed(xd, packed, bd, y, residual=rd, residual_scale=0.5, post_activation="relu")
        got = y.cpu().numpy()
        assert not np.isnan(got).any()
        assert rel_err(got, want) <= REL_TOL
    # residual aliasing the output, as the reference's in-place Elementwise allows
    y = rd.clone()
    plan.enqueue_packed(xd, packed, bd, y, residual=y, residual_scale=0.5, post_activation="relu")
    assert rel_err(y.cpu().numpy(), want) <= REL_TOL
    assert capi.device_status() == 0


@pytest.mark.parametrize("cin,cout,groups,k,hw", [(96, 192, 2, 5, 27), (64, 128, 4, 3, 14), (128, 64, 2, 1, 9)])
def test_grouped_convolution_on_the_tensor_core_path(cin, cout, groups, k, hw):
    """Groups that are wide enough run group by group through the tensor-core kernel (one packed operand
    and one launch per group): checked against the CPU checker, plain and with the fused residual."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    ob.set_threads(16)
    rng = np.random.default_rng(cin + cout + groups)
    batch, pad = 3, k // 2
    x = rng.standard_normal((batch, cin, hw, hw), dtype=np.float32)
    w = kaiming(rng, (cout, cin // groups, k, k))
    b = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=k, pad=pad, groups=groups, batch=batch, height=hw, width=hw,
                              bias=True, activation="relu")
    assert plan.kernel().startswith("igemm_tf32x3")
    xd, wd, bd = to_dev(x), to_dev(w), to_dev(b)
    want = ob.conv2d(x, w, b, stride=1, pad=pad, groups=groups, activation="relu")
    y = torch.full(plan.output_shape(batch), float("nan"), device=DEV)
    ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=DEV)
    plan.enqueue(xd, wd, bd, y, ws)
    assert rel_err(y.cpu().numpy(), want) <= REL_TOL
    res = rng.standard_normal(want.shape, dtype=np.float32)
    y2 = torch.full(plan.output_shape(batch), float("nan"), device=DEV)
    plan.enqueue_packed(xd, plan.prepack(wd), bd, y2, residual=to_dev(res), post_activation="relu")
    assert rel_err(y2.cpu().numpy(), np.maximum(want + res, 0.0)) <= REL_TOL
    assert capi.device_status() == 0


def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_device_usable():
    """Failure detection without a fault: a kernel whose wait can never be satisfied runs into the time limit of the
    library's bounded waits, the status word reports it as DLP_TIMEOUT with the waiter's code, the role that was only
    waiting for the first is released by the abort flag, and the next real convolution is computed as usual."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    assert capi.device_status() == 0
    first_ok, first_ms, second_ok, second_ms = capi.selftest_wait_expiry()
    assert first_ok == 0 and 300 <= first_ms <= 2000, (first_ok, first_ms)            # gave up at the 0.4 s limit
    assert second_ok == 0 and second_ms <= first_ms - 100, (second_ok, second_ms)     # it began later and was released by the abort flag
    import ctypes
    code = ctypes.c_int(0)
    st = capi.lib().dlp_device_status(None, ctypes.byref(code))
    assert st == capi.TIMEOUT and code.value == capi.SELFTEST_WAIT_CODE
    assert "gave up" in capi.lib().dlp_last_error().decode()
    assert capi.device_status() == 0                                                   # reading the word cleared it
    rng = np.random.default_rng(44)
    x = rng.standard_normal((2, 32, 14, 14), dtype=np.float32)
    w = kaiming(rng, (48, 32, 3, 3))
    plan = capi.Conv2DForward(channels_in=32, channels_out=48, kernel=3, pad=1, batch=2, height=14, width=14, bias=False, activation="relu")
    y = torch.empty(plan.output_shape(2), device=DEV)
    ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=DEV)
    plan.enqueue(to_dev(x), to_dev(w), None, y, ws)
    assert rel_err(y.cpu().numpy(), ob.conv2d(x, w, None, pad=1, activation="relu")) <= REL_TOL
    assert capi.device_status() == 0


ROWTAPS_CASES = [
    # N, Cin, H, W, Cout, kernel, stride, pad, groups
    (3, 3, 37, 45, 64, 7, 2, 3, 1),            # the stem's geometry on an odd-sized image
    (2, 5, 19, 23, 40, 5, 1, 2, 1),            # 5 columns padded to 8, ragged column tile
    (2, 3, 21, 21, 130, (3, 8), (1, 2), (1, 0), 1),   # 8 columns exactly, non-square, two column tiles
    (4, 1, 30, 30, 16, (7, 6), 1, (0, 5), 1),  # one channel: fewer row groups than a k-block; padding wider than the image edge
    (2, 48, 12, 12, 32, 5, 1, 2, 2),           # groups of 24 channels: 120 row groups
    (1, 200, 9, 9, 24, 7, 1, 3, 1),            # 1400 row groups: beyond the table, falls back to the gather loaders
]


@pytest.mark.parametrize("case", ROWTAPS_CASES, ids=[str(i) for i in range(len(ROWTAPS_CASES))])
def test_row_taps_loader(case):
    """Wide kernels over channel counts that are not blocks of 32: the reduction runs (channel, kernel row, column
    padded to 8).  Compared with the CPU checker; every case names the kernel it expects."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    N, cin, H, W, cout, k, stride, pad, groups = case
    rng = np.random.default_rng(cin * 1000 + H)
    kh, kw = (k, k) if isinstance(k, int) else k
    x = rng.standard_normal((N, cin, H, W), dtype=np.float32)
    w = kaiming(rng, (cout, cin // groups, kh, kw))
    b = rng.uniform(-0.1, 0.1, cout).astype(np.float32)
    plan = capi.Conv2DForward(channels_in=cin, channels_out=cout, kernel=k, stride=stride, pad=pad, groups=groups, batch=N, height=H,
                              width=W, bias=True, activation="relu")
    expect = "_gather" if cin // groups * kh > 1024 else "_rowtaps"
    assert plan.kernel().endswith(expect), plan.kernel()
    y = torch.full(plan.output_shape(N), float("nan"), device=DEV)
    ws = torch.empty(max(plan.workspace(), 16), dtype=torch.uint8, device=DEV)
    plan.enqueue(to_dev(x), to_dev(w), to_dev(b), y, ws)
    assert capi.device_status() == 0
    want = ob.conv2d(x, w, b, stride=stride, pad=pad, groups=groups, activation="relu")
    got = y.cpu().numpy()
    assert got.shape == want.shape and not np.isnan(got).any()
    assert rel_err(got, want) <= REL_TOL, (plan.kernel(), rel_err(got, want))


@pytest.mark.parametrize("case", [(2, 5, 9, 12, 1), (3, 7, 15, 14, 2), (1, 3, 6, 8, 2), (2, 4, 5, 6, 1), (1, 33, 7, 10, 2), (2, 40, 20, 36, 1),
                                  (1, 6, 7, 7, 1), (2, 8, 14, 14, 1), (1, 4, 12, 12, 1), (2, 5, 14, 14, 2), (1, 3, 13, 9, 1), (2, 9, 30, 11, 1),
                                  (1, 5, 9, 7, 2)],
                         ids=lambda c: "x".join(str(v) for v in c))
def test_depthwise_3x3_register_kernel(case):
    """Depthwise 3x3 / pad 1 at stride 1 and 2 over even widths (16- and 8-byte loads, halo by shuffle), odd heights, lane
    counts that do not fill the last warp, stride-2 planes that are one strip, bias + ReLU6, and y = factor*y + ...; the odd
    widths take the staged kernel."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    N, C, H, W, stride = case
    rng = np.random.default_rng(N * 100 + C)
    x = rng.standard_normal((N, C, H, W), dtype=np.float32)
    w = kaiming(rng, (C, 1, 3, 3))
    b = rng.uniform(-0.5, 0.5, C).astype(np.float32)
    plan = capi.Conv2DForward(channels_in=C, channels_out=C, kernel=3, stride=stride, pad=1, groups=C, batch=N, height=H, width=W,
                              bias=True, activation="relu6")
    assert plan.algo() == "depthwise_separable"
    want = ob.conv2d(x, w, b, stride=stride, pad=1, groups=C, activation="relu6")
    y0 = rng.standard_normal(want.shape).astype(np.float32)
    for factor in (0.0, 0.5):
        y = to_dev(y0) if factor else torch.full(plan.output_shape(N), float("nan"), device=DEV)
        plan.enqueue(to_dev(x), to_dev(w), to_dev(b), y, None, factor=factor)
        got = y.cpu().numpy()
        assert got.shape == want.shape
        assert rel_err(got, want + factor * y0) <= REL_TOL, (case, factor)


@pytest.mark.parametrize("shape", [(2, 6, 8, 8), (1, 5, 7, 7), (3, 16, 13, 4), (1, 2, 1, 3)], ids=lambda c: "x".join(str(v) for v in c))
def test_depthwise_1x1_scale(shape):
    """A 1x1 depthwise convolution is a per-channel scale: planes of a multiple of 4 elements (16-byte path) and not,
    bias + ReLU6, y = factor*y + ..."""
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    N, C, H, W = shape
    rng = np.random.default_rng(N + 10 * C + H)
    x = rng.standard_normal(shape, dtype=np.float32) * 3
    w = rng.standard_normal((C, 1, 1, 1), dtype=np.float32)
    b = rng.uniform(-0.5, 0.5, C).astype(np.float32)
    plan = capi.Conv2DForward(channels_in=C, channels_out=C, kernel=1, groups=C, batch=N, height=H, width=W, bias=True, activation="relu6")
    want = ob.conv2d(x, w, b, groups=C, activation="relu6")
    y0 = rng.standard_normal(want.shape).astype(np.float32)
    for factor in (0.0, -1.5):
        y = to_dev(y0) if factor else torch.full(plan.output_shape(N), float("nan"), device=DEV)
        plan.enqueue(to_dev(x), to_dev(w), to_dev(b), y, None, factor=factor)
        assert rel_err(y.cpu().numpy(), want + factor * y0) <= 1e-6, (plan.algo(), plan.kernel(), factor)


def test_issue_probe_orders_the_schemes():
    """The MMA-only probe behind the pointwise kernel's issue loop: uniform barrier tests cost less than a lane per barrier,
    two issuer warps reach the 64-column MMA's own rate, and nothing runs faster than the tensor pipe (12 x 32 or 64 cycles)."""
    from dlprimitives_b200 import capi
    bare, divergent, uniform, two = [capi.tf32_issue_probe(s, 64) for s in range(4)]
    assert capi.device_status() == 0
    assert 380 <= two < bare and uniform < divergent
    bare128, divergent128, uniform128, two128 = [capi.tf32_issue_probe(s, 128) for s in range(4)]
    assert capi.device_status() == 0
    assert 760 <= min(bare128, uniform128, two128) and uniform128 < divergent128 and two128 < 900
