"""GPU parity of the bandwidth-bound operators between convolutions, on the golden vectors of the
reference's own operator tests (Pooling2D, GlobalPooling, Softmax, Activation, Elementwise) and
against the CPU checker (BatchNorm, large shapes)."""
import numpy as np
import pytest
import torch

from conftest import reference_tolerance
from gpu_util import DEV, rel_err, to_dev

pytestmark = pytest.mark.gpu


def run(op_type, opt, ins, params=()):
    from dlprimitives_b200 import hostapi
    op = hostapi.Operator(op_type, opt, [a.shape for a in ins])
    outs = op.forward([to_dev(a) for a in ins], [to_dev(p) for p in params])
    return [o.cpu().numpy() for o in outs]


@pytest.mark.parametrize("name,op_type", [("pooling2d", "Pooling2D"), ("global_pooling", "GlobalPooling"), ("softmax", "Softmax"),
                                          ("activation", "Activation"), ("elementwise", "Elementwise")])
def test_golden_cases(golden, name, op_type):
    n = 0
    for opt, params, ins, outs, eps in golden.embedded(name):
        if name == "elementwise" and ins[0].shape != ins[1].shape:
            continue   # broadcasting is outside the inference hot path (NotImplementedError, checked below)
        got, = run(op_type, opt, ins)
        assert got.shape == outs[0].shape, opt
        assert np.abs(got - outs[0]).max() <= reference_tolerance(outs[0], eps), (name, opt)
        n += 1
    assert n >= 5


def test_elementwise_broadcast_is_refused():
    from dlprimitives_b200 import hostapi
    with pytest.raises(hostapi.HostError) as e:
        hostapi.Operator("Elementwise", {"operation": "sum"}, [(2, 3, 4, 4), (2, 3, 1, 1)])
    assert e.value.kind == "NotImplementedError"


def test_large_shapes_against_checker():
    from oracle import bindings as ob
    rng = np.random.default_rng(41)
    x = rng.standard_normal((8, 64, 112, 112), dtype=np.float32)
    got, = run("Pooling2D", {"mode": "max", "kernel": 3, "stride": 2, "pad": 1}, [x])
    assert np.array_equal(got, ob.pooling2d(x, 3, 2, 1, "max"))
    got, = run("Pooling2D", {"mode": "avg", "kernel": [3, 2], "stride": [2, 1], "pad": [1, 0], "count_include_pad": True}, [x[:2]])
    assert rel_err(got, ob.pooling2d(x[:2], [3, 2], [2, 1], [1, 0], "avg", False, True)) <= 1e-6
    z = rng.standard_normal((16, 2048, 7, 7), dtype=np.float32)
    for mode in ("avg", "max"):
        got, = run("GlobalPooling", {"mode": mode}, [z])
        assert rel_err(got, ob.global_pooling(z, mode)) <= 1e-6
    a, b = x[:4], rng.standard_normal((4, 64, 112, 112), dtype=np.float32)
    got, = run("Elementwise", {"operation": "sum", "activation": "relu"}, [a, b])
    assert np.array_equal(got, ob.elementwise(a, b, "sum", 1.0, 1.0, "relu"))
    got, = run("Elementwise", {"operation": "max", "coef1": 0.5, "coef2": -2.0}, [a, b])
    assert np.array_equal(got, ob.elementwise(a, b, "max", 0.5, -2.0))
    logits = (rng.standard_normal((256, 1000)) * 5).astype(np.float32)
    for log in (False, True):
        got, = run("Softmax", {"log": log}, [logits])
        assert np.abs(got - ob.softmax(logits, log)).max() <= 1e-5
    mean, var = rng.standard_normal(64).astype(np.float32), rng.uniform(0.5, 2, 64).astype(np.float32)
    gamma, beta = rng.uniform(0.5, 1.5, 64).astype(np.float32), rng.uniform(-0.1, 0.1, 64).astype(np.float32)
    got, = run("BatchNorm", {"features": 64}, [a], [mean, var, gamma, beta])
    assert rel_err(got, ob.batchnorm_inference(a, mean, var, gamma, beta)) <= 1e-6
    got, = run("BatchNorm", {"features": 64, "affine": False}, [a], [mean, var])
    assert rel_err(got, ob.batchnorm_inference(a, mean, var)) <= 1e-6


@pytest.mark.parametrize("shape", [(3, 5, 30, 70), (1, 2, 7, 6), (2, 3, 113, 200), (1, 1, 2, 2)])
def test_max_pool_3x3_stride2_ragged_shapes(shape):
    """The register kernel for max 3x3 / stride 2 / pad 1 over even widths: strips and column blocks that end inside
    the plane, odd heights, a single window.  Bit-exact against the checker."""
    from oracle import bindings as ob
    x = np.random.default_rng(sum(shape)).standard_normal(shape, dtype=np.float32)
    got, = run("Pooling2D", {"mode": "max", "kernel": 3, "stride": 2, "pad": 1}, [x])
    assert np.array_equal(got, ob.pooling2d(x, 3, 2, 1, "max"))


@pytest.mark.parametrize("shape", [(3, 50, 5, 5), (1, 7, 3, 3), (2, 129, 7, 7), (1, 3, 9, 9), (2, 5, 4, 4)])
def test_global_pooling_plane_counts(shape):
    """Plane counts that do not fill the last CTA of the tiled kernel (odd plane sizes) and an even plane size (the
    warp-per-plane kernel)."""
    from oracle import bindings as ob
    x = np.random.default_rng(sum(shape)).standard_normal(shape, dtype=np.float32)
    for mode in ("avg", "max"):
        got, = run("GlobalPooling", {"mode": mode}, [x])
        assert rel_err(got, ob.global_pooling(x, mode)) <= 1e-6
