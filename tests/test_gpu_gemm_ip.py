"""GPU parity of the GEMM interface and the InnerProduct path."""
import numpy as np
import pytest
import torch

from conftest import reference_tolerance, small_frac
from gpu_util import DEV, REL_TOL, kaiming, rel_err, to_dev

pytestmark = pytest.mark.gpu


# the reference's GEMM test shapes (tests/test_gemm.cpp:104-123) and a few ragged ones of our own
REFERENCE_GEMM_SHAPES = [(1, 1, 1), (8, 1, 8), (1, 8, 8), (8, 8, 1), (31, 16, 31), (16, 31, 31), (31, 31, 16), (512, 512, 512),
                         (1024, 1024, 1024), (1025, 1025, 1025), (2048, 2048, 2048), (2049, 2049, 2049), (64, 2048, 64), (2048, 64, 2048),
                         (2048, 2048, 64), (2048, 64, 64), (64, 2048, 2048), (64, 64, 2048)]
OWN_GEMM_SHAPES = [(129, 65, 33), (1025, 31, 65), (31, 1025, 129), (64, 2049, 64), (2049, 64, 31), (5, 1000, 2048), (256, 1000, 512),
                   (1, 513, 700), (300, 1, 257)]


def _integer_matrices(gen, count, rows, cols):
    """Integer-valued fp32 matrices (N(-5, 5) rounded, as in tests/test_gemm.cpp:35-38): every product and sum of the
    test is an integer far below 2^24, so any order of summation gives the same fp32 result and equality is exact."""
    return torch.round(torch.randn(count, rows, cols, device=DEV, generator=gen) * 5 - 5)


@pytest.mark.parametrize("math_mode", [0, 1], ids=["auto", "ffma"])
def test_gemm_integer_exact_sweep(math_mode):
    """The reference's GEMM test (tests/test_gemm.cpp:10-144): its 18 shapes plus ragged ones, all four transpositions,
    beta 0 and 2, batch none / 1 / 5 (batch_sgemm), integer-valued inputs, so the result must be bit-exact.  The
    expected product is computed in float64 (exact for these magnitudes) on the same device; a few small shapes are
    also checked against numpy's int64 product."""
    from dlprimitives_b200 import capi
    gen = torch.Generator(device=DEV)
    gen.manual_seed(9)
    cases = 0
    for M, N, K in REFERENCE_GEMM_SHAPES + OWN_GEMM_SHAPES:
        big = M * N * K > 2 ** 28
        if math_mode == 1 and M * N * K > 2 ** 31:
            continue                                # the plain-FMA kernel on 2048^3 and up: covered by the 1024/1025 cubes
        for batch in (0, 1, 5):
            if big and batch == 5 and (M, N, K) not in ((2048, 2048, 2048),):
                continue                            # one large batched case is enough GPU memory and time
            for ta in (False, True):
                for tb in (False, True):
                    for beta in (0.0, 2.0):
                        nb = max(batch, 1)
                        a = _integer_matrices(gen, nb, K if ta else M, M if ta else K)
                        b = _integer_matrices(gen, nb, N if tb else K, K if tb else N)
                        c = _integer_matrices(gen, nb, M, N)
                        opa = a.transpose(1, 2) if ta else a
                        opb = b.transpose(1, 2) if tb else b
                        c0 = c.clone()
                        want = torch.bmm(opa.double(), opb.double()) + beta * c0.double()
                        g = capi.Gemm(ta, tb, M, N, K, math_mode=math_mode)
                        if batch == 0:
                            ws = torch.empty(max(g.workspace(), 16), dtype=torch.uint8, device=DEV)
                            g.gemm(M, N, K, a[0], a.shape[2], b[0], b.shape[2], c[0], N, beta=beta, ws=ws)
                        else:
                            ws = torch.empty(max(g.batched_workspace(nb), 16), dtype=torch.uint8, device=DEV)
                            g.batch_gemm(nb, M, N, K, a, a.shape[1] * a.shape[2], a.shape[2], b, b.shape[1] * b.shape[2], b.shape[2], c, M * N, N,
                                         beta=beta, ws=ws)
                        assert torch.equal(c.double(), want), (M, N, K, batch, ta, tb, beta, g.kernel())
                        if M * N * K <= 31 ** 3:
                            ref = opa.cpu().numpy().astype(np.int64) @ opb.cpu().numpy().astype(np.int64) + int(beta) * c0.cpu().numpy().astype(np.int64)
                            assert np.array_equal(c.cpu().numpy().astype(np.int64), ref)
                        cases += 1
    assert cases >= 500
    assert capi.device_status() == 0


def test_host_gemm_interface():
    """The C++ gpu::GEMM class: an object made for small sizes called with larger ones (its scratch grows), batch_sgemm
    (asynchronous, scratch from the stream's pool) in all transpositions, and the convolution GEMM factory called the
    way the reference's Conv2DForwardGEMM calls it."""
    from dlprimitives_b200 import capi, hostapi
    from oracle import bindings as ob
    gen = torch.Generator(device=DEV)
    gen.manual_seed(21)
    M, N, K = 300, 520, 200
    a = _integer_matrices(gen, 1, M, K)[0]
    b = _integer_matrices(gen, 1, K, N)[0]
    c = torch.zeros(M, N, device=DEV)
    hostapi.gemm(False, False, M, N, K, a, K, b, N, c, N, planned=(64, 64, 64))
    assert torch.equal(c.double(), a.double() @ b.double())
    stream = torch.cuda.Stream()
    for ta in (False, True):
        for tb in (False, True):
            B, m, n, k = 5, 96, 200, 130
            a = _integer_matrices(gen, B, k if ta else m, m if ta else k)
            b = _integer_matrices(gen, B, n if tb else k, k if tb else n)
            c = _integer_matrices(gen, B, m, n)
            want = torch.bmm((a.transpose(1, 2) if ta else a).double(), (b.transpose(1, 2) if tb else b).double()) + 2.0 * c.double()
            torch.cuda.synchronize()
            with torch.cuda.stream(stream):
                hostapi.batch_sgemm(ta, tb, B, m, n, k, a, a.shape[1] * a.shape[2], a.shape[2], b, b.shape[1] * b.shape[2], b.shape[2], c,
                                    m * n, n, beta=2.0, stream=stream)
            stream.synchronize()
            assert torch.equal(c.double(), want), (ta, tb)
    rng = np.random.default_rng(22)
    for groups, k, stride, pad in ((1, 3, 1, 1), (2, 3, 2, 1), (1, 1, 1, 0)):
        x = rng.standard_normal((3, 16, 20, 18), dtype=np.float32)
        w = kaiming(rng, (24, 16 // groups, k, k))
        bias = rng.uniform(-1, 1, 24).astype(np.float32)
        want = ob.conv2d(x, w, bias, stride=stride, pad=pad, groups=groups, activation="relu")
        y0 = rng.standard_normal(want.shape).astype(np.float32)
        y = to_dev(y0)
        hostapi.conv_gemm(to_dev(x), to_dev(w), to_dev(bias), y, stride=stride, pad=pad, groups=groups, activation="relu", factor=0.5)
        assert rel_err(y.cpu().numpy(), 0.5 * y0 + want) <= REL_TOL, (groups, k, stride, pad)
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
    ws = torch.empty(max(g.batched_workspace(B), 16), dtype=torch.uint8, device=DEV)
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
