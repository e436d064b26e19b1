"""Run a network JSON with the C restatement (liboracle.so), operator by operator.

TEST INFRASTRUCTURE ONLY.  The stand-in for the reference's CPU Net when the reference CPU build
(oracle/_ref) is not present: the smoke check and the bench's CPU-baseline leg use it as the checker
and as the timed "port" baseline.  Supports the operators of the inference graphs made by
dlprimitives_b200.resnet50.
"""
import time

import numpy as np

from . import bindings as ob


def run(net_json, params, inputs, outputs=None):
    """inputs: dict name -> array.  Returns (dict of requested tensors, seconds spent in the operators)."""
    tensors = dict(inputs)
    seconds = 0.0
    for op in net_json["operators"]:
        o = op.get("options", {})
        ins = [tensors[n] for n in op["inputs"]]
        name = op["name"]
        t0 = time.perf_counter()
        if op["type"] == "Convolution2D":
            bias = params[name + ".1"] if o.get("bias", True) else None
            y = ob.conv2d(ins[0], params[name + ".0"], bias, stride=o.get("stride", 1), pad=o.get("pad", 0), dilate=o.get("dilate", 1),
                          groups=o.get("groups", 1), activation=o.get("activation", "identity"))
        elif op["type"] == "InnerProduct":
            bias = params[name + ".1"] if o.get("bias", True) else None
            y = ob.inner_product(ins[0], params[name + ".0"], bias, o.get("activation", "identity"))
        elif op["type"] == "BatchNorm":
            affine = o.get("affine", True)
            y = ob.batchnorm_inference(ins[0], params[name + ".0"], params[name + ".1"], params[name + ".2"] if affine else None,
                                       params[name + ".3"] if affine else None, o.get("eps", 1e-5))
        elif op["type"] == "Activation":
            y = ob.activation(ins[0], o.get("activation", "identity"))
        elif op["type"] == "Elementwise":
            y = ob.elementwise(ins[0], ins[1], o.get("operation", "sum"), o.get("coef1", 1.0), o.get("coef2", 1.0), o.get("activation", "identity"))
        elif op["type"] == "Pooling2D":
            y = ob.pooling2d(ins[0], o["kernel"], o.get("stride", 1), o.get("pad", 0), o.get("mode", "max"), o.get("ceil_mode", False),
                             o.get("count_include_pad", False))
        elif op["type"] == "GlobalPooling":
            y = ob.global_pooling(ins[0], o.get("mode", "max"))
        elif op["type"] == "Softmax":
            y = ob.softmax(ins[0], o.get("log", False))
        elif op["type"] == "Flatten":
            y = ins[0].reshape(ins[0].shape[0], -1)
        else:
            raise NotImplementedError(op["type"])
        seconds += time.perf_counter() - t0
        tensors[op["outputs"][0]] = y
    wanted = outputs or net_json["outputs"]
    return {n: tensors[n] for n in wanted}, seconds
