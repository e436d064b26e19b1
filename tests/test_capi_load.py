"""CPU-only: the shared libraries load and export every symbol their headers declare, and the
product path fails loudly (no fallback) when there is no CUDA device."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dlp_[a-z0-9_]+)\s*\(", text)))


def test_cuda_library_exports_every_declared_symbol():
    from dlprimitives_b200 import capi
    names = declared("dlp_cuda.h")
    assert len(names) >= 35
    lib = ctypes.CDLL(capi.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    # the binding's table and the header agree
    assert sorted(capi.SYMBOLS) == names
    assert capi.lib().dlp_version().decode().startswith("dlprim-b200")


def test_host_library_exports_every_declared_symbol():
    from dlprimitives_b200 import hostapi
    names = declared("dlp_host.h")
    lib = ctypes.CDLL(hostapi.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(hostapi.SYMBOLS) == names


def test_no_cpu_fallback_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from dlprimitives_b200 import capi, hostapi
    with pytest.raises(capi.DlpError):
        capi.Conv2DForward(channels_in=8, channels_out=8, kernel=3, pad=1, height=8, width=8, batch=1)
    with pytest.raises(hostapi.HostError) as e:
        hostapi.Operator("Convolution2D", {"channels_out": 8, "kernel": 3}, [(1, 8, 8, 8)])
    assert e.value.kind == "DeviceError"
    with pytest.raises(ValueError):
        capi._ptr(torch.zeros(4))   # host tensors are refused, nothing computes on the CPU


def test_argument_validation_needs_no_device():
    """Checks that run before any CUDA call behave like the reference's DLPRIM_CHECKs."""
    from dlprimitives_b200 import capi
    with pytest.raises(capi.ValidationError):
        capi.Conv2DForward(channels_in=6, channels_out=8, kernel=3, groups=4, height=8, width=8)      # groups must divide
    with pytest.raises(capi.ValidationError):
        capi.Conv2DForward(channels_in=8, channels_out=8, kernel=9, height=4, width=4)                 # output size <= 0
    with pytest.raises(capi.ValidationError):
        capi.Conv2DForward(channels_in=8, channels_out=8, kernel=3, height=8, width=8, algo="fft")     # unknown algorithm
    with pytest.raises(capi.ValidationError):
        capi.Gemm(False, False, 4, 4, 4, bias_mode=7)
    with pytest.raises(capi.ValidationError):
        capi.IPForward(0, 10)
    cycles = ctypes.c_double(0.0)
    with pytest.raises(capi.ValidationError):
        capi.check(capi.lib().dlp_tf32_issue_probe(4, 128, ctypes.byref(cycles), None))                # schemes are 0..3
    with pytest.raises(capi.ValidationError):
        capi.check(capi.lib().dlp_tf32_issue_probe(0, 96, ctypes.byref(cycles), None))                 # 64 or 128 columns
    assert capi.pooling2d_output_shape(112, 112, 3, 2, 1) == (56, 56)
    assert capi.pooling2d_output_shape(7, 7, 2, 2, 0, ceil_mode=True) == (4, 4)
    d = capi.make_conv_desc(channels_in=3, channels_out=64, kernel=7, stride=2, pad=3, height=224, width=224)
    oh, ow = ctypes.c_int(), ctypes.c_int()
    capi.check(capi.lib().dlp_conv2d_output_shape(ctypes.byref(d), 224, 224, ctypes.byref(oh), ctypes.byref(ow)))
    assert (oh.value, ow.value) == (112, 112)
