"""ResNet-50 inference graph in the reference's network-JSON schema, with synthetic parameters.

The graph is the bottleneck [3, 4, 6, 3] network of the reference's own benchmark file
(docs/nets_for_benchmark/resnet50-b16.js: 7x7/2 stem, 3x3/2 max-pool with pad 1, stride 2 on the 3x3
convolution of the first block of stages 2-4, i.e. the torchvision layout), followed by global
average pooling, a 2048 -> 1000 InnerProduct and Softmax.

Two forms, both valid input for the reference's own Net as well:
  folded=True   BatchNorm folded into the convolutions (weight scale + bias), ReLU as the
                convolution's / Elementwise's "activation" option
  folded=False  Convolution2D(bias=false) -> BatchNorm -> Activation(relu) as separate operators,
                the form the reference ships

No dataset or checkpoint is involved: inputs are N(0,1) noise of ImageNet shape and the weights are
Kaiming-normal, from one integer seed.
"""
import numpy as np

STAGES = [(64, 256, 3, 1), (128, 512, 4, 2), (256, 1024, 6, 2), (512, 2048, 3, 2)]   # mid, out, blocks, stride


def _conv(ops, name, src, dst, cin, cout, k, stride, pad, relu, folded):
    opts = {"channels_in": cin, "channels_out": cout, "kernel": [k, k], "stride": [stride, stride], "pad": [pad, pad],
            "dilate": [1, 1], "groups": 1, "bias": bool(folded)}
    if folded:
        if relu:
            opts["activation"] = "relu"
        ops.append({"name": name, "type": "Convolution2D", "inputs": [src], "outputs": [dst], "options": opts})
        return
    ops.append({"name": name, "type": "Convolution2D", "inputs": [src], "outputs": [dst + "_c"], "options": opts})
    ops.append({"name": name + "_bn", "type": "BatchNorm", "inputs": [dst + "_c"], "outputs": [dst if not relu else dst + "_b"],
                "options": {"features": cout, "eps": 1e-5}})
    if relu:
        ops.append({"name": name + "_relu", "type": "Activation", "inputs": [dst + "_b"], "outputs": [dst], "options": {"activation": "relu"}})


def make_json(batch, height=224, width=224, folded=True, softmax=True, classes=1000, width_div=1):
    """Network description.  width_div > 1 shrinks every channel count (for quick tests)."""
    ch = lambda c: max(8, c // width_div)
    ops = []
    _conv(ops, "conv1", "data", "conv1", 3, ch(64), 7, 2, 3, True, folded)
    ops.append({"name": "pool1", "type": "Pooling2D", "inputs": ["conv1"], "outputs": ["pool1"],
                "options": {"mode": "max", "kernel": 3, "stride": 2, "pad": 1}})
    cur, cin = "pool1", ch(64)
    for si, (mid, out, blocks, stride) in enumerate(STAGES):
        mid, out = ch(mid), ch(out)
        for b in range(blocks):
            p = "layer%d.%d" % (si + 1, b)
            s = stride if b == 0 else 1
            _conv(ops, p + ".conv1", cur, p + ".c1", cin, mid, 1, 1, 0, True, folded)
            _conv(ops, p + ".conv2", p + ".c1", p + ".c2", mid, mid, 3, s, 1, True, folded)
            if b == 0:
                _conv(ops, p + ".downsample", cur, p + ".sc", cin, out, 1, s, 0, False, folded)
                shortcut = p + ".sc"
            else:
                shortcut = cur
            _conv(ops, p + ".conv3", p + ".c2", p + ".c3", mid, out, 1, 1, 0, False, folded)
            ops.append({"name": p + ".add", "type": "Elementwise", "inputs": [p + ".c3", shortcut], "outputs": [p + ".out"],
                        "options": {"operation": "sum", "activation": "relu"}})
            cur, cin = p + ".out", out
    ops.append({"name": "gap", "type": "GlobalPooling", "inputs": [cur], "outputs": ["gap"], "options": {"mode": "avg"}})
    ops.append({"name": "fc", "type": "InnerProduct", "inputs": ["gap"], "outputs": ["fc"],
                "options": {"inputs": cin, "outputs": classes, "bias": True}})
    last = "fc"
    if softmax:
        ops.append({"name": "prob", "type": "Softmax", "inputs": ["fc"], "outputs": ["prob"], "options": {}})
        last = "prob"
    return {"inputs": [{"name": "data", "shape": [batch, 3, height, width]}], "outputs": [last], "operators": ops}


def make_params(net_json, seed=0):
    """Synthetic parameters for a graph made by make_json: name -> float32 array.

    Convolution / InnerProduct weights are Kaiming-normal, std = sqrt(2 / fan_in).  Every convolution
    is followed by a BatchNorm with running mean 0, variance 1, gamma ~ U(0.5, 1.5), beta ~ U(-0.1, 0.1);
    in the folded form those are multiplied into the weights in float64 and rounded once
    (w' = A*w, b' = B with A = gamma / sqrt(var + eps), B = beta - mean*A)."""
    rng = np.random.default_rng(seed)
    params = {}
    bn_eps = 1e-5
    for op in net_json["operators"]:
        o = op.get("options", {})
        if op["type"] == "Convolution2D":
            cin, cout, k = o["channels_in"], o["channels_out"], o["kernel"]
            fan_in = cin // o.get("groups", 1) * k[0] * k[1]
            w = rng.standard_normal((cout, cin // o.get("groups", 1), k[0], k[1])) * np.sqrt(2.0 / fan_in)
            gamma, beta = rng.uniform(0.5, 1.5, cout), rng.uniform(-0.1, 0.1, cout)
            mean, var = np.zeros(cout), np.ones(cout)
            if o.get("bias", True):
                a = gamma / np.sqrt(var + bn_eps)
                params[op["name"] + ".0"] = (w * a[:, None, None, None]).astype(np.float32)
                params[op["name"] + ".1"] = (beta - mean * a).astype(np.float32)
            else:
                params[op["name"] + ".0"] = w.astype(np.float32)
                for i, v in enumerate((mean, var, gamma, beta)):
                    params[op["name"] + "_bn.%d" % i] = v.astype(np.float32)
        elif op["type"] == "InnerProduct":
            fin, fout = o["inputs"], o["outputs"]
            params[op["name"] + ".0"] = (rng.standard_normal((fout, fin)) * np.sqrt(2.0 / fin)).astype(np.float32)
            params[op["name"] + ".1"] = rng.uniform(-0.1, 0.1, fout).astype(np.float32)
    return params


def make_input(net_json, seed=1):
    shape = net_json["inputs"][0]["shape"]
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)


def flops_per_image(net_json):
    """2*MAC of the convolutions and the InnerProduct, per image, by propagating shapes."""
    shapes = {i["name"]: i["shape"] for i in net_json["inputs"]}
    total = 0
    for op in net_json["operators"]:
        o = op.get("options", {})
        s = shapes[op["inputs"][0]]
        if op["type"] == "Convolution2D":
            k, st, pd = o["kernel"], o["stride"], o["pad"]
            oh = (s[2] + 2 * pd[0] - k[0]) // st[0] + 1
            ow = (s[3] + 2 * pd[1] - k[1]) // st[1] + 1
            total += 2 * o["channels_out"] * oh * ow * (o["channels_in"] // o.get("groups", 1)) * k[0] * k[1]
            out = [s[0], o["channels_out"], oh, ow]
        elif op["type"] == "Pooling2D":
            k, st, pd = o["kernel"], o.get("stride", 1), o.get("pad", 0)
            out = [s[0], s[1], (s[2] + 2 * pd - k) // st + 1, (s[3] + 2 * pd - k) // st + 1]
        elif op["type"] == "GlobalPooling":
            out = [s[0], s[1], 1, 1]
        elif op["type"] == "InnerProduct":
            total += 2 * o["inputs"] * o["outputs"]
            out = [s[0], o["outputs"]]
        else:
            out = list(s)
        for name in op["outputs"]:
            shapes[name] = out
    return total
