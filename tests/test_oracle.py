"""CPU-only checks that pin the checker (oracle/) itself.

1. Against the golden vectors: PyTorch-made inputs/outputs that the reference's own operator tests
   embed (InnerProduct, Pooling2D, GlobalPooling, Softmax, Activation) or that its generator
   produces (Convolution2D, Elementwise), at the reference's tolerance.
2. Bit-for-bit against the reference's own CPU context compiled from its sources (oracle/_ref),
   when that build is present.
"""
import numpy as np
import pytest

from oracle import bindings as ob
from conftest import reference_tolerance, small_frac


def _pair(v):
    return [v, v] if np.isscalar(v) else list(v)


def oracle_conv_from_options(opt, params, x):
    w = params[0]
    b = params[1] if opt.get("bias", True) else None
    return ob.conv2d(x, w, b, stride=opt.get("stride", 1), pad=opt.get("pad", 0), dilate=opt.get("dilate", 1),
                     groups=opt.get("groups", 1), activation=opt.get("activation", "identity"))


def test_conv2d_golden(golden):
    n = 0
    for opt, params, ins, outs, eps in golden.embedded("conv2d"):
        y = oracle_conv_from_options(opt, params, ins[0])
        assert y.shape == outs[0].shape
        assert np.abs(y - outs[0]).max() <= reference_tolerance(outs[0], eps), opt
        n += 1
    assert n >= 100


def test_conv2d_winograd_restatement_golden(golden):
    n = 0
    for opt, params, ins, outs, eps in golden.embedded("conv2d"):
        if _pair(opt["kernel"]) != [3, 3] or _pair(opt["stride"]) != [1, 1] or _pair(opt["pad"]) != [1, 1] \
                or _pair(opt["dilate"]) != [1, 1] or opt["groups"] != 1:
            continue
        y = ob.conv2d(ins[0], params[0], params[1] if opt["bias"] else None, pad=1,
                      activation=opt.get("activation", "identity"), winograd=True)
        assert np.abs(y - outs[0]).max() <= reference_tolerance(outs[0], eps), opt
        n += 1
    assert n >= 30


def test_inner_product_golden(golden):
    n = 0
    for opt, params, ins, outs, eps in golden.embedded("inner_product"):
        y = ob.inner_product(ins[0], params[0], params[1] if opt.get("bias", True) else None, opt.get("activation", "identity"))
        assert np.abs(y - outs[0]).max() <= reference_tolerance(outs[0], eps), opt
        n += 1
    assert n == 28


def test_glue_golden(golden):
    for opt, params, ins, outs, eps in golden.embedded("pooling2d"):
        y = ob.pooling2d(ins[0], opt["kernel"], opt.get("stride", 1), opt.get("pad", 0), opt.get("mode", "max"),
                         opt.get("ceil_mode", False), opt.get("count_include_pad", False))
        assert y.shape == outs[0].shape, opt
        assert np.abs(y - outs[0]).max() <= reference_tolerance(outs[0], eps), opt
    for opt, params, ins, outs, eps in golden.embedded("global_pooling"):
        y = ob.global_pooling(ins[0], opt.get("mode", "max"))
        assert np.abs(y - outs[0]).max() <= reference_tolerance(outs[0], eps), opt
    for opt, params, ins, outs, eps in golden.embedded("softmax"):
        y = ob.softmax(ins[0], opt.get("log", False))
        assert np.abs(y - outs[0]).max() <= reference_tolerance(outs[0], eps), opt
    for opt, params, ins, outs, eps in golden.embedded("activation"):
        y = ob.activation(ins[0], opt["activation"])
        assert np.abs(y - outs[0]).max() <= reference_tolerance(outs[0], eps), opt
    n = 0
    for opt, params, ins, outs, eps in golden.embedded("elementwise"):
        if ins[0].shape != ins[1].shape:
            continue  # broadcasting is outside the hot path (the residual add is same-shape)
        y = ob.elementwise(ins[0], ins[1], opt.get("operation", "sum"), opt.get("coef1", 1.0), opt.get("coef2", 1.0),
                           opt.get("activation", "identity"))
        assert np.abs(y - outs[0]).max() <= reference_tolerance(outs[0], eps), opt
        n += 1
    assert n > 10


def test_gemm_integer_exact():
    """The reference GEMM test's trick (tests/test_gemm.cpp:19-25): integer-valued inputs make every
    fp32 sum exact, so all four loop orders must agree bit for bit with an integer product."""
    rng = np.random.default_rng(5)
    for M, N, K in [(1, 1, 1), (31, 7, 5), (64, 65, 129), (5, 1025, 3)]:
        for ta in (False, True):
            for tb in (False, True):
                a = np.round(rng.normal(-5, 5, size=(K, M) if ta else (M, K))).astype(np.float32)
                b = np.round(rng.normal(-5, 5, size=(N, K) if tb else (K, N))).astype(np.float32)
                c0 = np.round(rng.normal(-5, 5, size=(M, N))).astype(np.float32)
                want = (a.T if ta else a).astype(np.int64) @ (b.T if tb else b).astype(np.int64) + 2 * c0.astype(np.int64)
                got = ob.sgemm(a, b, ta, tb, beta=2.0, c=c0)
                assert np.array_equal(got.astype(np.int64), want)


def test_bn_fold_matches_unfolded():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 5, 9, 9), dtype=np.float32)
    w = rng.standard_normal((7, 5, 3, 3), dtype=np.float32)
    mean, var = rng.standard_normal(7).astype(np.float32), rng.uniform(0.5, 2, 7).astype(np.float32)
    gamma, beta = rng.uniform(0.5, 1.5, 7).astype(np.float32), rng.uniform(-0.1, 0.1, 7).astype(np.float32)
    want = ob.batchnorm_inference(ob.conv2d(x, w, None, pad=1), mean, var, gamma, beta)
    w2, b2 = ob.fold_batchnorm(w, None, mean, var, gamma, beta)
    got = ob.conv2d(x, w2, b2, pad=1)
    assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max()


needs_ref = pytest.mark.skipif(not ob.ref_available(), reason="reference CPU build (oracle/_ref) not present")


@needs_ref
def test_conv2d_bit_exact_vs_reference_cpu(golden):
    """Every option set of the reference's conv sweep, on small_frac and on normal inputs."""
    rng = np.random.default_rng(11)
    seen = 0
    for test in golden.index["conv2d"]["tests"]:
        opt = dict(test["options"])
        cin, cout = opt["channels_in"], opt["channels_out"]
        k = _pair(opt["kernel"])
        shape = (2, cin, 10, 12) if cin * cout < 50000 else (1, cin, 7, 7)
        if shape[2] + _pair(opt["pad"])[0] < k[0] * _pair(opt["dilate"])[0]:
            shape = (1, cin, 40, 40)
        op = ob.RefOperator("Convolution2D", opt, [shape])
        for init in (small_frac, lambda r, s: r.standard_normal(s, dtype=np.float32)):
            x = init(rng, shape)
            params = [init(rng, s) for s in op.param_shapes]
            want, = op.forward([x], params)
            got = oracle_conv_from_options(opt, params, x)
            assert got.shape == want.shape
            assert np.array_equal(got, want), opt
        seen += 1
    assert seen == 22


@needs_ref
def test_inner_product_and_glue_bit_exact_vs_reference_cpu():
    rng = np.random.default_rng(12)
    for act in ("identity", "relu", "tanh", "sigmoid", "relu6"):
        for bias in (True, False):
            opt = {"inputs": 37, "outputs": 19, "bias": bias, "activation": act}
            op = ob.RefOperator("InnerProduct", opt, [(6, 37)])
            x = rng.standard_normal((6, 37), dtype=np.float32)
            params = [rng.standard_normal(s, dtype=np.float32) for s in op.param_shapes]
            want, = op.forward([x], params)
            got = ob.inner_product(x, params[0], params[1] if bias else None, act)
            assert np.array_equal(got, want), opt
    x = rng.standard_normal((2, 3, 13, 11), dtype=np.float32)
    for opt in ({"mode": "max", "kernel": 3, "stride": 2, "pad": 1}, {"mode": "avg", "kernel": [2, 3], "stride": 2},
                {"mode": "avg", "kernel": 3, "stride": 2, "pad": 1, "count_include_pad": True},
                {"mode": "max", "kernel": 3, "stride": 2, "ceil_mode": True}):
        want, = ob.RefOperator("Pooling2D", opt, [x.shape]).forward([x])
        got = ob.pooling2d(x, opt["kernel"], opt.get("stride", 1), opt.get("pad", 0), opt["mode"], opt.get("ceil_mode", False),
                           opt.get("count_include_pad", False))
        assert got.shape == want.shape and np.array_equal(got, want), opt
    for mode in ("max", "avg"):
        want, = ob.RefOperator("GlobalPooling", {"mode": mode}, [x.shape]).forward([x])
        assert np.array_equal(ob.global_pooling(x, mode), want)
    y = rng.standard_normal(x.shape, dtype=np.float32)
    for opt in ({"operation": "sum", "activation": "relu"}, {"operation": "prod", "coef1": 0.5, "coef2": 3.0}, {"operation": "max", "coef2": -1.0}):
        want, = ob.RefOperator("Elementwise", opt, [x.shape, y.shape]).forward([x, y])
        got = ob.elementwise(x, y, opt["operation"], opt.get("coef1", 1.0), opt.get("coef2", 1.0), opt.get("activation", "identity"))
        assert np.array_equal(got, want), opt
    z = rng.standard_normal((5, 1000), dtype=np.float32)
    for log in (False, True):
        want, = ob.RefOperator("Softmax", {"log": log}, [z.shape]).forward([z])
        assert np.array_equal(ob.softmax(z, log), want)
    mean, var = rng.standard_normal(3).astype(np.float32), rng.uniform(0.5, 2, 3).astype(np.float32)
    gamma, beta = rng.uniform(0.5, 1.5, 3).astype(np.float32), rng.uniform(-0.1, 0.1, 3).astype(np.float32)
    op = ob.RefOperator("BatchNorm", {"features": 3}, [x.shape])
    want, = op.forward([x], [mean, var, gamma, beta])
    assert np.array_equal(ob.batchnorm_inference(x, mean, var, gamma, beta), want)
