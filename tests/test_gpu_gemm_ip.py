"""GPU parity of the GEMM interface and the InnerProduct path."""
import numpy as np
import pytest
import torch

from conftest import reference_tolerance, small_frac
from gpu_util import DEV, REL_TOL, kaiming, rel_err, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("math_mode", [0, 1], ids=["auto", "ffma"])
def test_gemm_integer_exact_sweep(math_mode):
    """The reference's GEMM test (tests/test_gemm.cpp:10-144): integer-valued inputs, so the result
    must be bit-exact whatever the order of summation; shapes with 1, 31, 1025, 2049 and skinny
    ones; all four transpositions; beta 0 and 2."""
    from dlprimitives_b200 import capi
    rng = np.random.default_rng(9)
    shapes = [(1, 1, 1), (31, 31, 31), (64, 64, 64), (128, 128, 128), (129, 65, 33), (1025, 31, 65), (31, 1025, 129), (64, 2049, 64),
              (2049, 64, 31), (5, 1000, 2048), (256, 1000, 512), (1, 513, 700), (300, 1, 257)]
    for M, N, K in shapes:
        for ta in (False, True):
            for tb in (False, True):
                for beta in (0.0, 2.0):
                    a = np.round(rng.normal(-5, 5, size=(K, M) if ta else (M, K))).astype(np.float32)
                    b = np.round(rng.normal(-5, 5, size=(N, K) if tb else (K, N))).astype(np.float32)
                    c0 = np.round(rng.normal(-5, 5, size=(M, N))).astype(np.float32)
                    want = (a.T if ta else a).astype(np.int64) @ (b.T if tb else b).astype(np.int64) + int(beta) * c0.astype(np.int64)
                    g = capi.Gemm(ta, tb, M, N, K, math_mode=math_mode)
                    c = to_dev(c0)
                    ws = torch.empty(max(g.workspace(), 16), dtype=torch.uint8, device=DEV)
                    g.gemm(M, N, K, to_dev(a), a.shape[1], to_dev(b), b.shape[1], c, N, beta=beta, ws=ws)
                    got = c.cpu().numpy()
                    assert np.array_equal(got.astype(np.int64), want), (M, N, K, ta, tb, beta, g.kernel())
    assert capi.device_status() == 0


def test_gemm_bias_activation_leading_dimensions_and_batches():
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    rng = np.random.default_rng(10)
    M, N, K = 70, 200, 150
    for bias_mode in (capi.GEMM_NO_BIAS, capi.GEMM_BIAS_M, capi.GEMM_BIAS_N):
        for act in ("identity", "relu", "sigmoid"):
            a = rng.standard_normal((M, K + 7), dtype=np.float32)      # lda > K
            b = rng.standard_normal((K, N + 3), dtype=np.float32)      # ldb > N
            c0 = rng.standard_normal((M, N + 5), dtype=np.float32)     # ldc > N
            bias = None if bias_mode == 0 else rng.standard_normal(M if bias_mode == 1 else N).astype(np.float32)
            g = capi.Gemm(False, False, M, N, K, bias_mode=bias_mode, activation=act, math_mode=capi.MATH_TF32X3)
            ws = torch.empty(max(g.workspace(), 16), dtype=torch.uint8, device=DEV)
            c = to_dev(c0)
            g.gemm(M, N, K, to_dev(a), K + 7, to_dev(b), N + 3, c, N + 5, bias=to_dev(bias), beta=0.5, ws=ws)
            want = ob.gemm_bias_act(a[:, :K], b[:, :N], beta=0.5, c=c0[:, :N], bias=bias, bias_mode=bias_mode, activation=act)
            got = c.cpu().numpy()
            assert rel_err(got[:, :N], want) <= REL_TOL, (bias_mode, act)
            assert np.array_equal(got[:, N:], c0[:, N:])               # padding columns untouched
    # batched product (GEMM::batch_sgemm)
    B = 5
    a = rng.standard_normal((B, M, K), dtype=np.float32)
    b = rng.standard_normal((B, K, N), dtype=np.float32)
    g = capi.Gemm(False, False, M, N, K)
    ws = torch.empty(max(g.workspace(), 16), dtype=torch.uint8, device=DEV)
    c = torch.zeros(B, M, N, device=DEV)
    g.batch_gemm(B, M, N, K, to_dev(a), M * K, K, to_dev(b), K * N, N, c, M * N, N, ws=ws)
    want = np.stack([ob.sgemm(a[i], b[i]) for i in range(B)])
    assert rel_err(c.cpu().numpy(), want) <= REL_TOL
    assert capi.device_status() == 0


def test_inner_product_golden_cases(golden):
    from dlprimitives_b200 import hostapi
    n = 0
    for opt, params, ins, outs, eps in golden.embedded("inner_product"):
        op = hostapi.Operator("InnerProduct", opt, [ins[0].shape])
        y, = op.forward([to_dev(ins[0])], [to_dev(p) for p in params])
        got = y.cpu().numpy()
        assert got.shape == outs[0].shape
        assert np.abs(got - outs[0]).max() <= 4 * reference_tolerance(outs[0], eps), (opt, op.kernel)
        n += 1
    assert n == 28


def test_inner_product_reference_sweep_bit_exact_on_small_frac(golden):
    """The reference's large InnerProduct cases (batch up to 512, 4096 x 4096) on "small_frac" inputs,
    where fp32 arithmetic is exact: the GPU must match the CPU checker bit for bit."""
    from dlprimitives_b200 import hostapi
    from oracle import bindings as ob
    rng = np.random.default_rng(13)
    seen = 0
    for opt, param_shapes, in_shapes, out_shapes, _ in golden.checker_only("inner_product"):
        batch, inputs = in_shapes[0][0], int(np.prod(in_shapes[0][1:]))
        if batch * inputs * opt["outputs"] > 2**29 and seen % 4:
            continue                                   # one in four of the very large ones: CPU time
        x = small_frac(rng, in_shapes[0])
        ps = [small_frac(rng, s) for s in param_shapes]
        b = ps[1] if opt.get("bias", True) else None
        want = ob.inner_product(x, ps[0], b, opt.get("activation", "identity"))
        op = hostapi.Operator("InnerProduct", opt, [x.shape])
        y, = op.forward([to_dev(x)], [to_dev(p) for p in ps])
        assert np.array_equal(y.cpu().numpy(), want), (opt, in_shapes, op.kernel)
        seen += 1
    assert seen >= 50


def test_config2_inner_product_full_size():
    from dlprimitives_b200 import capi
    from oracle import bindings as ob
    rng = np.random.default_rng(14)
    x = rng.standard_normal((256, 2048), dtype=np.float32)
    w = kaiming(rng, (1000, 2048))
    b = np.zeros(1000, np.float32)
    ip = capi.IPForward(2048, 1000, 256, bias=True)
    y = torch.empty(256, 1000, device=DEV)
    ws = torch.empty(max(ip.workspace(), 16), dtype=torch.uint8, device=DEV)
    ip.enqueue(to_dev(x), to_dev(w), to_dev(b), y, ws)
    want = ob.inner_product(x, w, b)
    assert rel_err(y.cpu().numpy(), want) <= REL_TOL, ip.kernel()
    # packed weights, smaller batch than planned
    packed = ip.prepack(to_dev(w))
    y2 = torch.empty(32, 1000, device=DEV)
    ip.enqueue_packed(to_dev(x[:32]), packed, to_dev(b), y2)
    assert torch.equal(y2, y[:32])
    assert capi.device_status() == 0
