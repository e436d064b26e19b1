"""CPU-only tests of host-side logic that needs no device."""
import json
import os

from conftest import ROOT


def _op(name, typ, ins, outs, **options):
    return {"name": name, "type": typ, "inputs": ins, "outputs": outs, "options": options}


def merge_cases_graph():
    """Every situation the activation merge of the reference's ONNX importer distinguishes (src/importers/onnx.cpp:531-579)."""
    conv = dict(channels_in=8, channels_out=8, kernel=[1, 1], bias=True)
    ops = [
        _op("c0", "Convolution2D", ["data"], ["t0"], **conv),
        _op("r0", "Activation", ["t0"], ["t1"], activation="relu"),                  # merged into c0
        _op("c1", "Convolution2D", ["t1"], ["t2"], **conv),
        _op("p1", "Pooling2D", ["t2"], ["t3"], kernel=1, stride=1, mode="max"),
        _op("r1", "Activation", ["t3"], ["t4"], activation="relu"),                  # follows a Pooling2D: stays
        _op("c2", "Convolution2D", ["t4"], ["t5"], **conv),
        _op("r2", "Activation", ["t5"], ["t6"], activation="tanh"),                  # t5 has a second consumer: stays
        _op("e2", "Elementwise", ["t5", "t6"], ["t7"], operation="sum"),
        _op("r3", "Activation", ["t7"], ["t8"], activation="relu6"),                 # merged into e2
        _op("c3", "Convolution2D", ["t8"], ["t9"], activation="relu", **conv),
        _op("r4", "Activation", ["t9"], ["t10"], activation="sigmoid"),              # c3 already has an activation: stays
        _op("c4", "Convolution2D", ["t10"], ["t11"], **conv),
        _op("r5", "Activation", ["t11"], ["t12"], activation="relu"),                # t11 is a network output: stays
        _op("g", "GlobalPooling", ["t12"], ["t13"], mode="avg"),
        _op("ip", "InnerProduct", ["t13"], ["t14"], inputs=8, outputs=5),
        _op("r6", "Activation", ["t14"], ["t15"], activation="sigmoid"),             # merged into ip
    ]
    return {"inputs": [{"name": "data", "shape": [2, 8, 6, 6]}], "outputs": ["t11", "t15"], "operators": ops}


def test_activation_merge_pass():
    from dlprimitives_b200 import hostapi
    graph = merge_cases_graph()
    merged, count = hostapi.merge_activations(graph)
    assert count == 3
    names = [op["name"] for op in merged["operators"]]
    assert names == ["c0", "c1", "p1", "r1", "c2", "r2", "e2", "c3", "r4", "c4", "r5", "g", "ip"]
    by_name = {op["name"]: op for op in merged["operators"]}
    assert by_name["c0"]["options"]["activation"] == "relu" and by_name["c0"]["outputs"] == ["t1"]
    assert by_name["e2"]["options"]["activation"] == "relu6" and by_name["e2"]["outputs"] == ["t8"]
    assert by_name["ip"]["options"]["activation"] == "sigmoid" and by_name["ip"]["outputs"] == ["t15"]
    assert by_name["c2"]["outputs"] == ["t5"] and by_name["c3"]["options"]["activation"] == "relu"
    assert merged["outputs"] == ["t11", "t15"] and merged["inputs"] == graph["inputs"]
    again, count = hostapi.merge_activations(merged)
    assert count == 0 and again == merged


def test_the_reference_shipped_description_has_nothing_left_to_merge():
    """Its activations follow BatchNorm operators, and the sums carry theirs already."""
    from dlprimitives_b200 import hostapi
    graph = json.load(open(os.path.join(ROOT, "tests", "golden", "reference_resnet50_b16.json")))
    merged, count = hostapi.merge_activations(graph)
    assert count == 0 and len(merged["operators"]) == 158
