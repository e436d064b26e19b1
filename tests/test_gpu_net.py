"""GPU parity of whole-network inference: dlprim::Net on the CUDA context against the reference's
own Net on its CPU context (committed outputs, and live when the reference CPU build is present)."""
import importlib.util
import os

import numpy as np
import pytest
import torch

from conftest import ROOT
from gpu_util import DEV, REL_TOL, rel_err

pytestmark = pytest.mark.gpu

_spec = importlib.util.spec_from_file_location("make_net_golden", os.path.join(ROOT, "tests", "golden", "make_net_golden.py"))
net_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(net_golden)


def build_gpu_net(net_json, params, flags=0):
    from dlprimitives_b200 import hostapi
    net = hostapi.Net(net_json, flags=flags)
    assert set(net.param_names()) == set(params)
    for name, value in params.items():
        assert net.param_shape(name) == value.shape
        net.set_param(name, value)
    net.upload_params()
    return net


def run_gpu(net, x, outputs=("fc", "prob"), repeats=3):
    """Several forwards on a side stream: eager first, then graph capture, then replay."""
    stream = torch.cuda.Stream()
    results = []
    xh = torch.from_numpy(x).pin_memory()
    with torch.cuda.stream(stream):
        for _ in range(repeats):
            net.set_tensor("data", xh, stream)
            net.forward(stream)
            outs = {name: torch.empty(net.tensor_shape(name)).pin_memory() for name in outputs}
            for name, t in outs.items():
                net.get_tensor(name, t, stream)
            stream.synchronize()
            results.append({k: v.numpy().copy() for k, v in outs.items()})
    return results


@pytest.mark.parametrize("case", list(net_golden.CASES))
@pytest.mark.parametrize("flags", [0, 2, 1 | 4, 16, 16 | 4], ids=["fused+graph", "unfused+graph", "keep_intermediate+eager", "branches+graph",
                                                             "branches+eager"])
def test_small_resnet_against_reference_cpu_outputs(case, flags):
    from dlprimitives_b200 import capi, resnet50
    batch, h, w, folded, div, pseed, iseed = net_golden.CASES[case]
    net_json = resnet50.make_json(batch, h, w, folded=folded, width_div=div)
    params = resnet50.make_params(net_json, seed=pseed)
    x = resnet50.make_input(net_json, seed=iseed)
    golden = np.load(os.path.join(ROOT, "tests", "golden", "net_cases.npz"))
    net = build_gpu_net(net_json, params, flags)
    plan = net.plan()
    fused = [line for line in plan if "+residual" in line]
    if flags & 16:
        # the four projection shortcuts run on the second stream, from the block's input to the convolution that adds them
        side = [line for line in plan if "[second stream" in line]
        assert len(side) == 4 and all(".downsample" in line.split()[0] for line in side), plan
    if flags in (0, 16, 20) and folded:
        assert len(fused) == 16, plan             # every bottleneck's sum is folded into a convolution
        assert not any(" Elementwise" in line for line in plan)
    else:
        assert not fused or not folded
    results = run_gpu(net, x)
    for r in results:                               # eager, captured and replayed runs agree exactly
        assert np.array_equal(r["fc"], results[0]["fc"])
    assert rel_err(results[0]["fc"], golden[case + "_fc"]) <= REL_TOL
    assert np.abs(results[0]["prob"] - golden[case + "_prob"]).max() <= 1e-4     # the reference scripts' bar
    assert (results[0]["prob"].argmax(1) == golden[case + "_prob"].argmax(1)).all()
    assert capi.device_status() == 0
    if flags == 0:
        assert net.activation_bytes() < net.activation_bytes(without_reuse=True)


@pytest.mark.parametrize("batch,sel", [(256, [0, 100, 255]), (32, [0, 13, 31])], ids=["batch256", "batch32"])
def test_resnet50_full_size_rows_against_reference_cpu(batch, sel):
    """Config 5 at its real size on the GPU (3x224x224, full channel widths): the configuration's own batch of
    256 and the per-GPU batch of an 8-GPU run (tile scheduling and the cuts along K differ with the batch).
    The reference's CPU Net computes three of those images (it handles images independently), which keeps
    the CPU side to about half a minute per case."""
    from oracle import bindings as ob
    if not ob.ref_available():
        pytest.skip("reference CPU build (oracle/_ref) not present")
    from dlprimitives_b200 import capi, resnet50
    net_json = resnet50.make_json(batch)
    params = resnet50.make_params(net_json, seed=0)
    x = resnet50.make_input(net_json, seed=1)
    net = build_gpu_net(net_json, params)
    got = run_gpu(net, x, repeats=2)[-1]
    ref_json = resnet50.make_json(len(sel))
    ref = ob.RefNet(ref_json)
    for name in ref.param_names():
        ref.set_param(name, params[name])
    ref.set_tensor("data", x[sel])
    ref.forward()
    want_fc, want_prob = ref.get_tensor("fc"), ref.get_tensor("prob")
    assert rel_err(got["fc"][sel], want_fc) <= REL_TOL
    assert np.abs(got["prob"][sel] - want_prob).max() <= 1e-4
    assert (got["prob"][sel].argmax(1) == want_prob.argmax(1)).all()
    assert capi.device_status() == 0


def test_reshape_to_smaller_and_larger_batch():
    from dlprimitives_b200 import resnet50
    net_json = resnet50.make_json(4, 64, 64, width_div=8)
    params = resnet50.make_params(net_json, seed=3)
    net = build_gpu_net(net_json, params)
    x = np.random.default_rng(8).standard_normal((6, 3, 64, 64), dtype=np.float32)
    full = None
    for b in (4, 2, 6):
        net.reshape_input("data", (b, 3, 64, 64))
        net.reshape()
        assert net.tensor_shape("prob") == (b, 1000)
        out = run_gpu(net, np.ascontiguousarray(x[:b]), repeats=2)[-1]["fc"]
        if full is None:
            full = out
        n = min(b, 4)
        assert np.array_equal(out[:n], full[:n])    # per-image results do not depend on the batch


def test_parameter_file_round_trip(tmp_path):
    from dlprimitives_b200 import resnet50
    net_json = resnet50.make_json(2, 64, 64, width_div=8)
    params = resnet50.make_params(net_json, seed=3)
    x = resnet50.make_input(net_json, seed=4)
    a = build_gpu_net(net_json, params)
    path = str(tmp_path / "weights.dlp")
    a.save_params_file(path)
    assert open(path, "rb").read(4) == b"DLPW"
    from dlprimitives_b200 import hostapi
    b = hostapi.Net(net_json)
    b.load_params_file(path)
    assert np.array_equal(run_gpu(a, x, repeats=1)[0]["fc"], run_gpu(b, x, repeats=1)[0]["fc"])


def _in_place_sum_graph(side_reader_between):
    """conv_a(x) -> a; conv_b(a) -> t; [relu(x) -> z]; add(x, t) -> x (in place on the shortcut); [relu(x) -> z]."""
    conv = lambda name, src, dst: {"name": name, "type": "Convolution2D", "inputs": [src], "outputs": [dst],
                                   "options": {"channels_in": 16, "channels_out": 16, "kernel": [3, 3], "stride": [1, 1], "pad": [1, 1],
                                               "dilate": [1, 1], "groups": 1, "bias": True, "activation": "relu"}}
    side = {"name": "side", "type": "Activation", "inputs": ["x"], "outputs": ["z"], "options": {"activation": "relu"}}
    add = {"name": "add", "type": "Elementwise", "inputs": ["x", "t"], "outputs": ["x"], "options": {"operation": "sum", "activation": "relu"}}
    ops = [conv("stem", "data", "x"), conv("conv_a", "x", "a"), conv("conv_b", "a", "t")]
    ops += [side, add] if side_reader_between else [add, side]
    return {"inputs": [{"name": "data", "shape": [2, 16, 12, 12]}], "outputs": ["x", "z"], "operators": ops}


@pytest.mark.parametrize("side_reader_between", [True, False])
def test_in_place_sum_with_a_side_reader_of_the_shortcut(side_reader_between):
    """The residual fusion writes the sum at the convolution's step.  With the sum in place on the shortcut, an
    operator between the two that reads the shortcut must still see the shortcut: the fusion has to be refused."""
    from dlprimitives_b200 import resnet50
    from oracle import netrun
    net_json = _in_place_sum_graph(side_reader_between)
    params = resnet50.make_params(net_json, seed=11)
    x = resnet50.make_input(net_json, seed=12)
    net = build_gpu_net(net_json, params)
    fused = [line for line in net.plan() if "+residual" in line]
    assert bool(fused) == (not side_reader_between), net.plan()
    got = run_gpu(net, x, outputs=("x", "z"), repeats=3)
    want, _ = netrun.run(net_json, params, {"data": x}, ["x", "z"])
    for r in got:
        assert rel_err(r["x"], want["x"]) <= REL_TOL
        assert rel_err(r["z"], want["z"]) <= REL_TOL


_spec2 = importlib.util.spec_from_file_location("make_reference_graph_golden", os.path.join(ROOT, "tests", "golden", "make_reference_graph_golden.py"))
ref_graph = importlib.util.module_from_spec(_spec2)
_spec2.loader.exec_module(ref_graph)


@pytest.mark.parametrize("flags", [0, 2], ids=["fused+graph", "unfused+graph"])
def test_the_reference_shipped_resnet50_description_runs_as_it_is(flags):
    """docs/nets_for_benchmark/resnet50-b16.js of the reference, unchanged but for the batch in its input
    specification (Convolution2D -> BatchNorm -> Activation un-fused, named parameters, in-place activations, 158
    operators), loaded by dlprim::Net; its output against the reference's own Net on its CPU context for the same
    file and the same parameters (committed), and live when the reference CPU build is present."""
    import json
    from dlprimitives_b200 import capi, hostapi
    from oracle import bindings as ob
    graph = json.load(open(os.path.join(ROOT, "tests", "golden", "reference_resnet50_b16.json")))
    assert len(graph["operators"]) == 158 and graph["outputs"] == ["loss"]
    net = hostapi.Net(graph, flags=flags)
    params = {name: ref_graph.synthetic_parameter(name, net.param_shape(name)) for name in net.param_names()}
    assert "conv1.weight" in params and "bn1.running_var" in params and "fc.bias" in params     # the file's own parameter names
    for name, value in params.items():
        net.set_param(name, value)
    net.upload_params()
    x = ref_graph.synthetic_input(graph["inputs"][0]["shape"])
    results = run_gpu(net, x, outputs=("loss",), repeats=3)
    for r in results:
        assert np.array_equal(r["loss"], results[0]["loss"])
    want = np.load(os.path.join(ROOT, "tests", "golden", "reference_resnet50_b16.npz"))["loss"]
    assert rel_err(results[0]["loss"], want) <= REL_TOL
    assert (results[0]["loss"].argmax(1) == want.argmax(1)).all()
    if ob.ref_available() and flags == 0:
        ref = ob.RefNet(graph)
        assert set(ref.param_names()) == set(params)
        for name in ref.param_names():
            ref.set_param(name, params[name])
        ref.set_tensor("data", x)
        ref.forward()
        assert np.array_equal(ref.get_tensor("loss"), want)                # the committed output is the reference's
    assert capi.device_status() == 0


def _small_interchange_net():
    from dlprimitives_b200 import resnet50
    c = ref_graph.SMALL_NET
    return resnet50.make_json(c["batch"], c["height"], c["width"], folded=c["folded"], width_div=c["width_div"], classes=c["classes"])


def test_parameter_file_written_by_the_reference_is_read(tmp_path):
    """DLPW interchange, reference -> here: a file written by the reference's Net::save_parameters (src/net.cpp:63-101,
    committed) loaded by Net::load_parameters here gives bit for bit the results of setting the same values directly."""
    from dlprimitives_b200 import hostapi
    graph = _small_interchange_net()
    a = hostapi.Net(graph)
    params = {name: ref_graph.synthetic_parameter(name, a.param_shape(name)) for name in a.param_names()}
    for name, value in params.items():
        a.set_param(name, value)
    a.upload_params()
    b = hostapi.Net(graph)
    b.load_params_file(os.path.join(ROOT, "tests", "golden", "reference_written.dlp"))
    x = ref_graph.synthetic_input(graph["inputs"][0]["shape"], seed=5)
    ya, yb = run_gpu(a, x, repeats=1)[0], run_gpu(b, x, repeats=1)[0]
    assert np.array_equal(ya["fc"], yb["fc"]) and np.abs(ya["fc"]).max() > 0


def test_parameter_file_interchange_with_the_live_reference(tmp_path):
    """DLPW interchange both ways against the reference's own reader and writer (src/net.cpp:63-101, :227-305): the
    reference reads the file written here and finds every value bit for bit; the file it writes from those values is
    read back here with identical results."""
    from oracle import bindings as ob
    if not ob.ref_available():
        pytest.skip("reference CPU build (oracle/_ref) not present")
    from dlprimitives_b200 import hostapi
    graph = _small_interchange_net()
    ours = hostapi.Net(graph)
    params = {name: ref_graph.synthetic_parameter(name + "#2", ours.param_shape(name)) for name in ours.param_names()}
    for name, value in params.items():
        ours.set_param(name, value)
    ours.upload_params()
    ours_path, ref_path = str(tmp_path / "ours.dlp"), str(tmp_path / "reference.dlp")
    ours.save_params_file(ours_path)
    ref = ob.RefNet(graph)
    ref.load_params_file(ours_path)
    assert set(ref.param_names()) == set(params)
    for name in ref.param_names():
        assert np.array_equal(ref.get_param(name), params[name]), name
    ref.save_params_file(ref_path)
    back = hostapi.Net(graph)
    back.load_params_file(ref_path)
    x = ref_graph.synthetic_input(graph["inputs"][0]["shape"], seed=6)
    assert np.array_equal(run_gpu(ours, x, repeats=1)[0]["fc"], run_gpu(back, x, repeats=1)[0]["fc"])
    # and the reference computes the same network from the file written here
    ref.set_tensor("data", x)
    ref.forward()
    assert rel_err(run_gpu(ours, x, repeats=1)[0]["fc"], ref.get_tensor("fc")) <= REL_TOL


def test_activation_merge_keeps_the_results():
    """The description with its mergeable activations merged (flag bit 3) computes bit for bit what the unmerged one does."""
    from dlprimitives_b200 import hostapi, resnet50
    from test_host_logic import merge_cases_graph
    graph = merge_cases_graph()
    rng = np.random.default_rng(31)
    plain, merged = hostapi.Net(graph), hostapi.Net(graph, flags=8)
    assert len(merged.plan()) == len(plain.plan()) - 3
    for net in (plain, merged):
        r = np.random.default_rng(32)
        for name in sorted(net.param_names()):
            shape = net.param_shape(name)
            net.set_param(name, (r.standard_normal(shape) * 0.5).astype(np.float32))
        net.upload_params()
    x = rng.standard_normal((2, 8, 6, 6), dtype=np.float32)
    a = run_gpu(plain, x, outputs=("t11", "t15"), repeats=2)[-1]
    b = run_gpu(merged, x, outputs=("t11", "t15"), repeats=2)[-1]
    assert np.array_equal(a["t11"], b["t11"]) and np.array_equal(a["t15"], b["t15"])


def test_concurrent_branches_give_the_same_bits():
    """With the projection shortcuts on a second stream the same kernels run on the same data: the outputs are
    bit-identical to the one-stream run, eager, captured and replayed, and the activation pool only grows."""
    from dlprimitives_b200 import hostapi, resnet50
    net_json = resnet50.make_json(6, 64, 64, folded=True, width_div=4)
    params = resnet50.make_params(net_json, seed=3)
    x = resnet50.make_input(net_json, seed=4)
    one = build_gpu_net(net_json, params, 0)
    two = build_gpu_net(net_json, params, hostapi.Net.CONCURRENT_BRANCHES)
    a, b = run_gpu(one, x, repeats=4), run_gpu(two, x, repeats=4)
    for ra, rb in zip(a, b):
        assert np.array_equal(ra["fc"], rb["fc"]) and np.array_equal(ra["prob"], rb["prob"])
    assert two.activation_bytes() >= one.activation_bytes()
