"""Regenerate the golden fixtures in this directory.  Runs only where the reference tree is mounted.

Two sources, both belonging to the reference project:

* its committed operator test files (tests/test_case_<op>.json): the cases whose inputs and
  outputs were produced by PyTorch and embedded in the file are copied out, forward part only;
* its generator tests/make_test_cases_from_pt.py, imported from the reference tree and called with
  the seed it uses itself (123), for the operator files that are absent from the reference checkout
  (the convolution files and elementwise).

Every fixture keeps the operator's factory name, the JSON options, the parameter tensors and, per
case, the input and output tensors.  Cases the reference marks "use_cpu_reference" (too large to
embed) keep only their shapes: tests run those against the CPU checker instead.

Usage: python tests/golden/make_golden.py [--reference /path/to/reference]
"""
import argparse
import importlib.util
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def _flat(x):
    return np.asarray(x, dtype=np.float32).reshape(-1)


def convert(report, arrays, tag, max_case_elems):
    """Strip a reference test report down to its forward part; tensors go to `arrays` as float32."""
    out = {"operator": report["operator"], "tests": []}
    for ti, test in enumerate(report["tests"]):
        t = {"options": test["options"],
             "setup_shapes": [s["shape"] for s in test["setup_tensors"]],
             "param_shapes": [s["shape"] for s in test.get("param_specs", [])],
             "cases": []}
        if "param_tensors" in test:
            t["params"] = []
            for pi, p in enumerate(test["param_tensors"]):
                key = "%s_t%d_p%d" % (tag, ti, pi)
                arrays[key] = _flat(p)
                t["params"].append(key)
        for ci, case in enumerate(test["cases"]):
            c = {"in_shapes": case["in_shapes"], "out_shapes": case["out_shapes"]}
            if "eps" in case:
                c["eps"] = case["eps"]
            if "in_tensors" in case and "out_tensors" in case:
                n = sum(len(v) for v in case["in_tensors"]) + sum(len(v) for v in case["out_tensors"])
                if n > max_case_elems:
                    continue
                c["in"], c["out"] = [], []
                for k, v in enumerate(case["in_tensors"]):
                    key = "%s_t%d_c%d_i%d" % (tag, ti, ci, k)
                    arrays[key] = _flat(v)
                    c["in"].append(key)
                for k, v in enumerate(case["out_tensors"]):
                    key = "%s_t%d_c%d_o%d" % (tag, ti, ci, k)
                    arrays[key] = _flat(v)
                    c["out"].append(key)
            else:
                c["use_cpu_reference"] = True
            t["cases"].append(c)
        out["tests"].append(t)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--max-case-elems", type=int, default=6000)
    args = ap.parse_args()
    ref_tests = os.path.join(args.reference, "tests")

    arrays = {}
    index = {}
    for name in ["inner_product", "pooling2d", "global_pooling", "softmax", "activation"]:
        with open(os.path.join(ref_tests, "test_case_%s.json" % name)) as f:
            index[name] = convert(json.load(f), arrays, name, args.max_case_elems)
        index[name]["source"] = "tests/test_case_%s.json" % name

    spec = importlib.util.spec_from_file_location("ref_gen", os.path.join(ref_tests, "make_test_cases_from_pt.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    import torch
    # The reference's conv2d_gemm / conv2d_win / conv2d_dsc files differ from conv2d only in the
    # forced "fwd_algo" option (same seed, same tensors), so one copy of the tensors is kept and the
    # tests apply the four algorithm settings themselves.
    for name, fn in [("conv2d", gen.make_conv2d), ("elementwise", gen.make_eltwise)]:
        torch.random.manual_seed(123)
        sys.stdout = open(os.devnull, "w")
        try:
            report = fn()
        finally:
            sys.stdout = sys.__stdout__
        index[name] = convert(report, arrays, name, args.max_case_elems)
        index[name]["source"] = "tests/make_test_cases_from_pt.py --case %s (seed 123, torch %s)" % (name, torch.__version__)
    index["conv2d"]["fwd_algo_variants"] = ["", "gemm", "winograd", "depthwise_separable"]

    with open(os.path.join(HERE, "operator_cases.json"), "w") as f:
        json.dump(index, f, separators=(",", ":"))
    np.savez_compressed(os.path.join(HERE, "operator_cases.npz"), **arrays)
    for name, rep in index.items():
        cases = [c for t in rep["tests"] for c in t["cases"]]
        print("%-15s %3d option sets, %3d embedded cases, %3d checker-only cases"
              % (name, len(rep["tests"]), sum("in" in c for c in cases), sum("in" not in c for c in cases)))


if __name__ == "__main__":
    main()
