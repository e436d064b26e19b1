import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (the parity tests proper)")


class Golden:
    """Golden operator cases: PyTorch-made vectors taken from the reference's own test files or
    regenerated with its generator (tests/golden/make_golden.py)."""

    def __init__(self):
        here = os.path.join(ROOT, "tests", "golden")
        with open(os.path.join(here, "operator_cases.json")) as f:
            self.index = json.load(f)
        self.arrays = np.load(os.path.join(here, "operator_cases.npz"))

    def embedded(self, name):
        """Yield (options, params, case_inputs, case_outputs, eps) for every case with embedded tensors."""
        for test in self.index[name]["tests"]:
            if "params" in test:
                params = [self.arrays[k].reshape(s) for k, s in zip(test["params"], test["param_shapes"])]
            else:
                params = []
            for case in test["cases"]:
                if "in" not in case:
                    continue
                ins = [self.arrays[k].reshape(s) for k, s in zip(case["in"], case["in_shapes"])]
                outs = [self.arrays[k].reshape(s) for k, s in zip(case["out"], case["out_shapes"])]
                yield test["options"], params, ins, outs, case.get("eps", 1e-5)

    def checker_only(self, name):
        """Yield (options, param_shapes, in_shapes, out_shapes) of the cases too large to embed."""
        for test in self.index[name]["tests"]:
            for case in test["cases"]:
                if "in" not in case:
                    yield test["options"], test["param_shapes"], case["in_shapes"], case["out_shapes"], "params" in test and [
                        self.arrays[k].reshape(s) for k, s in zip(test["params"], test["param_shapes"])]


@pytest.fixture(scope="session")
def golden():
    return Golden()


def reference_tolerance(ref, eps=1e-5):
    """The reference test driver's bound: |d| <= eps * max(1, std(ref)) (tests/test_from_template.cpp:111-158)."""
    sigma = float(np.std(ref)) if ref.size else 0.0
    return eps * max(1.0, sigma)


def small_frac(rng, shape):
    """The reference driver's "small_frac" initialisation: multiples of 0.5 in [-1, 1]
    (tests/test_from_template.cpp:169-192), which keeps fp32 sums exact for moderate sizes."""
    return (rng.integers(-2, 3, size=shape) * 0.5).astype(np.float32)
