"""Regenerate net_cases.npz: outputs of the reference's own Net, on its CPU context, for small
ResNet-style graphs made by dlprimitives_b200.resnet50 (same seeds as the tests use).

Needs the reference CPU build under oracle/_ref (make -C oracle ref), i.e. the reference tree.
Usage: python tests/golden/make_net_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from dlprimitives_b200 import resnet50   # noqa: E402
from oracle import bindings as ob        # noqa: E402

CASES = {
    # name: (batch, height, width, folded, width_div, param seed, input seed)
    "small_folded": (3, 64, 64, True, 8, 3, 4),
    "small_unfolded": (3, 64, 64, False, 8, 3, 4),
    "odd_size_folded": (2, 75, 53, True, 16, 5, 6),
}


def run_reference(case):
    batch, h, w, folded, div, pseed, iseed = CASES[case]
    net_json = resnet50.make_json(batch, h, w, folded=folded, width_div=div)
    params = resnet50.make_params(net_json, seed=pseed)
    x = resnet50.make_input(net_json, seed=iseed)
    net = ob.RefNet(net_json)
    for name in net.param_names():
        net.set_param(name, params[name])
    net.set_tensor("data", x)
    net.forward()
    return net.get_tensor("fc"), net.get_tensor("prob")


if __name__ == "__main__":
    if not ob.ref_available():
        ob.build()
    out = {}
    for case in CASES:
        fc, prob = run_reference(case)
        out[case + "_fc"] = fc
        out[case + "_prob"] = prob
        print(case, fc.shape, float(np.abs(fc).max()))
    np.savez_compressed(os.path.join(HERE, "net_cases.npz"), **out)
