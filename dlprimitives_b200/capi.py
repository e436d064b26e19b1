"""ctypes binding of the C ABI in include/dlp_cuda.h.

Device memory, streams and process groups come from PyTorch (plumbing only); every computation goes
through the C entry points of ``lib/libdlprim_b200_cuda.so``.  There is no CPU or PyTorch fallback:
if the library is missing this module raises at import, and every call needs CUDA tensors.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libdlprim_b200_cuda.so")

ACTIVATIONS = {"identity": 0, "relu": 1, "tanh": 2, "sigmoid": 3, "relu6": 4}
MATH_AUTO, MATH_FP32_FFMA, MATH_TF32X3 = 0, 1, 2
GEMM_NO_BIAS, GEMM_BIAS_M, GEMM_BIAS_N = 0, 1, 2
OK, INVALID_ARGUMENT, NOT_IMPLEMENTED, CUDA_ERROR, TIMEOUT = 0, 1, 2, 3, 4


class DlpError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("dlp status %d: %s" % (status, message))
        self.status = status


class ValidationError(DlpError):
    """Mirrors dlprim::ValidationError."""


class NotImplementedDlpError(DlpError):
    """Mirrors dlprim::NotImplementedError."""


class ConvDesc(C.Structure):
    _fields_ = [("channels_in", C.c_int), ("channels_out", C.c_int), ("kernel", C.c_int * 2), ("stride", C.c_int * 2),
                ("dilate", C.c_int * 2), ("pad", C.c_int * 2), ("groups", C.c_int), ("batch", C.c_int), ("height", C.c_int),
                ("width", C.c_int), ("bias", C.c_int), ("activation", C.c_int), ("algo", C.c_char_p), ("math_mode", C.c_int)]


class GemmDesc(C.Structure):
    _fields_ = [("trans_a", C.c_int), ("trans_b", C.c_int), ("m", C.c_int), ("n", C.c_int), ("k", C.c_int),
                ("bias_mode", C.c_int), ("activation", C.c_int), ("math_mode", C.c_int)]


class IpDesc(C.Structure):
    _fields_ = [("inputs", C.c_int), ("outputs", C.c_int), ("optimal_batch_size", C.c_int), ("bias", C.c_int),
                ("activation", C.c_int), ("math_mode", C.c_int)]


# every symbol include/dlp_cuda.h declares: name -> (restype, argtypes)
_vp, _fp, _i, _f, _sz, _ll = C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_longlong
_ip = C.POINTER(C.c_int)
_i2 = C.c_int * 2
SYMBOLS = {
    "dlp_last_error": (C.c_char_p, []),
    "dlp_version": (C.c_char_p, []),
    "dlp_launch_count": (C.c_uint64, []),
    "dlp_device_status": (_i, [_vp, _ip]),
    "dlp_selftest_wait_expiry": (_i, [C.POINTER(C.c_int * 4), _vp]),
    "dlp_tf32_mma_rate": (_i, [C.POINTER(C.c_double), _vp]),
    "dlp_tf32_issue_probe": (_i, [C.c_int, C.c_int, C.POINTER(C.c_double), _vp]),
    "dlp_conv2d_output_shape": (_i, [C.POINTER(ConvDesc), _i, _i, _ip, _ip]),
    "dlp_conv2d_fwd_create": (_i, [C.POINTER(ConvDesc), C.POINTER(_vp)]),
    "dlp_conv2d_fwd_destroy": (None, [_vp]),
    "dlp_conv2d_fwd_algo": (C.c_char_p, [_vp]),
    "dlp_conv2d_fwd_kernel": (C.c_char_p, [_vp]),
    "dlp_conv2d_fwd_workspace": (_sz, [_vp]),
    "dlp_conv2d_fwd_packed_bytes": (_sz, [_vp]),
    "dlp_conv2d_fwd_prepack": (_i, [_vp, _fp, _vp, _vp]),
    "dlp_conv2d_fwd_enqueue": (_i, [_vp, _fp, _fp, _fp, _fp, _vp, _sz, _f, _i, _i, _i, _vp]),
    "dlp_conv2d_fwd_enqueue_packed": (_i, [_vp, _fp, _vp, _fp, _fp, _vp, _sz, _f, _fp, _f, _i, _i, _i, _i, _vp]),
    "dlp_gemm_create": (_i, [C.POINTER(GemmDesc), C.POINTER(_vp)]),
    "dlp_gemm_destroy": (None, [_vp]),
    "dlp_gemm_kernel": (C.c_char_p, [_vp]),
    "dlp_gemm_workspace": (_sz, [_vp]),
    "dlp_gemm_batched_workspace": (_sz, [_vp, _i]),
    "dlp_gemm_enqueue": (_i, [_vp, _i, _i, _i, _fp, _i, _fp, _i, _fp, _i, _fp, _f, _vp, _sz, _vp]),
    "dlp_gemm_batched_enqueue": (_i, [_vp, _i, _i, _i, _i, _fp, _ll, _i, _fp, _ll, _i, _fp, _ll, _i, _f, _vp, _sz, _vp]),
    "dlp_ip_fwd_create": (_i, [C.POINTER(IpDesc), C.POINTER(_vp)]),
    "dlp_ip_fwd_destroy": (None, [_vp]),
    "dlp_ip_fwd_kernel": (C.c_char_p, [_vp]),
    "dlp_ip_fwd_workspace": (_sz, [_vp]),
    "dlp_ip_fwd_packed_bytes": (_sz, [_vp]),
    "dlp_ip_fwd_prepack": (_i, [_vp, _fp, _vp, _vp]),
    "dlp_ip_fwd_enqueue": (_i, [_vp, _fp, _fp, _fp, _fp, _vp, _sz, _i, _vp]),
    "dlp_ip_fwd_enqueue_packed": (_i, [_vp, _fp, _vp, _fp, _fp, _vp, _sz, _i, _vp]),
    "dlp_ip_fwd_enqueue_static": (_i, [_vp, _fp, _fp, _fp, _fp, _i, _vp]),
    "dlp_pooling2d_output_shape": (_i, [_i, _i, _i2, _i2, _i2, _i, _ip, _ip]),
    "dlp_pooling2d_fwd": (_i, [_fp, _fp, _i, _i, _i, _i2, _i2, _i2, _i, _i, _i, _vp]),
    "dlp_global_pooling_fwd": (_i, [_fp, _fp, _i, _i, _i, _vp]),
    "dlp_elementwise_fwd": (_i, [_fp, _fp, _fp, _sz, _i, _f, _f, _i, _vp]),
    "dlp_activation_fwd": (_i, [_fp, _fp, _sz, _i, _vp]),
    "dlp_softmax_fwd": (_i, [_fp, _fp, _i, _i, _i, _i, _vp]),
    "dlp_batchnorm_inference_fwd": (_i, [_fp, _fp, _i, _i, _i, _f, _fp, _fp, _fp, _fp, _vp]),
}

_lib = None


def lib():
    """Load the CUDA library.  Fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: run `python -m dlprimitives_b200.build` (there is no fallback path)" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)   # AttributeError here means the header and the library disagree
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(status):
    if status == OK:
        return
    msg = lib().dlp_last_error().decode()
    if status == INVALID_ARGUMENT:
        raise ValidationError(status, msg)
    if status == NOT_IMPLEMENTED:
        raise NotImplementedDlpError(status, msg)
    raise DlpError(status, msg)


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _act(a):
    return ACTIVATIONS[a] if isinstance(a, str) else int(a)


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise ValueError("the CUDA library takes device tensors only")
    if not t.is_contiguous():
        raise ValueError("tensors must be contiguous")
    import torch
    if t.dtype not in (torch.float32, torch.uint8):
        raise ValueError("fp32 tensors expected")
    return t.data_ptr()


def _stream(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


def launch_count():
    return int(lib().dlp_launch_count())


def device_status(stream=None):
    """Synchronise the stream and return the device status word (0 = no bounded wait ever gave up)."""
    code = C.c_int(0)
    st = lib().dlp_device_status(_stream(stream), C.byref(code))
    if st not in (OK, TIMEOUT):
        check(st)
    return code.value


SELFTEST_WAIT_CODE = 900


def selftest_wait_expiry(stream=None):
    """Run the bounded-wait self-test kernel; returns (warp 0 succeeded, its wait in ms, warp 1 succeeded, its wait in ms)."""
    observed = (C.c_int * 4)()
    check(lib().dlp_selftest_wait_expiry(C.byref(observed), _stream(stream)))
    return tuple(observed)


def tf32_mma_rate(stream=None):
    """Measured dense TF32 rate of the tensor pipe on the current device, TFLOP/s (MMA-only kernel, about 2 ms)."""
    v = C.c_double(0.0)
    check(lib().dlp_tf32_mma_rate(C.byref(v), _stream(stream)))
    return v.value


def tf32_issue_probe(scheme, n, stream=None):
    """Clock cycles per k-block (twelve TF32 MMAs of N = n columns) of MMA issuing scheme 0..3 with every barrier already complete."""
    v = C.c_double(0.0)
    check(lib().dlp_tf32_issue_probe(int(scheme), int(n), C.byref(v), _stream(stream)))
    return v.value


def make_conv_desc(channels_in, channels_out, kernel, stride=1, dilate=1, pad=0, groups=1, batch=1, height=1, width=1,
                   bias=False, activation="identity", algo="", math_mode=MATH_AUTO):
    d = ConvDesc()
    d.channels_in, d.channels_out = int(channels_in), int(channels_out)
    for name, v in (("kernel", kernel), ("stride", stride), ("dilate", dilate), ("pad", pad)):
        a, b = _pair(v)
        getattr(d, name)[0], getattr(d, name)[1] = a, b
    d.groups, d.batch, d.height, d.width = int(groups), int(batch), int(height), int(width)
    d.bias, d.activation, d.math_mode = int(bool(bias)), _act(activation), int(math_mode)
    d.algo = algo.encode() if algo is not None else None
    return d


class Conv2DForward:
    """Plan object over dlp_conv2d_fwd_*: the C-ABI face of dlprim::core::Conv2DForward."""

    def __init__(self, **kw):
        self.desc = make_conv_desc(**kw)
        h = C.c_void_p()
        check(lib().dlp_conv2d_fwd_create(C.byref(self.desc), C.byref(h)))
        self.h = h
        self.packed = None

    def algo(self):
        return lib().dlp_conv2d_fwd_algo(self.h).decode()

    def kernel(self):
        return lib().dlp_conv2d_fwd_kernel(self.h).decode()

    def workspace(self):
        return int(lib().dlp_conv2d_fwd_workspace(self.h))

    def packed_bytes(self):
        return int(lib().dlp_conv2d_fwd_packed_bytes(self.h))

    def output_shape(self, batch, in_h=None, in_w=None):
        oh, ow = C.c_int(), C.c_int()
        check(lib().dlp_conv2d_output_shape(C.byref(self.desc), in_h or self.desc.height, in_w or self.desc.width, C.byref(oh), C.byref(ow)))
        return (batch, self.desc.channels_out, oh.value, ow.value)

    def enqueue(self, x, w, bias, y, ws=None, factor=0.0, stream=None):
        ws_bytes = ws.numel() * ws.element_size() if ws is not None else 0
        check(lib().dlp_conv2d_fwd_enqueue(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(y), _ptr(ws), ws_bytes, float(factor),
                                           x.shape[0], x.shape[2], x.shape[3], _stream(stream)))

    def prepack(self, w, stream=None):
        import torch
        n = self.packed_bytes()
        if n == 0:
            self.packed = w
            return w
        buf = torch.empty(n, dtype=torch.uint8, device=w.device)
        check(lib().dlp_conv2d_fwd_prepack(self.h, _ptr(w), _ptr(buf), _stream(stream)))
        self.packed = buf
        return buf

    def enqueue_packed(self, x, packed, bias, y, factor=0.0, residual=None, residual_scale=1.0, post_activation="identity", stream=None,
                       ws=None):
        ws_bytes = ws.numel() * ws.element_size() if ws is not None else 0
        check(lib().dlp_conv2d_fwd_enqueue_packed(self.h, _ptr(x), _ptr(packed), _ptr(bias), _ptr(y), _ptr(ws), ws_bytes, float(factor),
                                                  _ptr(residual), float(residual_scale), _act(post_activation),
                                                  x.shape[0], x.shape[2], x.shape[3], _stream(stream)))

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.dlp_conv2d_fwd_destroy(self.h)
            self.h = None


class Gemm:
    """Plan object over dlp_gemm_*: the C-ABI face of dlprim::gpu::GEMM."""

    def __init__(self, trans_a, trans_b, m, n, k, bias_mode=GEMM_NO_BIAS, activation="identity", math_mode=MATH_AUTO):
        d = GemmDesc(int(trans_a), int(trans_b), m, n, k, bias_mode, _act(activation), math_mode)
        self.desc = d
        h = C.c_void_p()
        check(lib().dlp_gemm_create(C.byref(d), C.byref(h)))
        self.h = h

    def kernel(self):
        return lib().dlp_gemm_kernel(self.h).decode()

    def workspace(self):
        return int(lib().dlp_gemm_workspace(self.h))

    def gemm(self, m, n, k, a, lda, b, ldb, c, ldc, bias=None, beta=0.0, ws=None, stream=None):
        ws_bytes = ws.numel() * ws.element_size() if ws is not None else 0
        check(lib().dlp_gemm_enqueue(self.h, m, n, k, _ptr(a), lda, _ptr(b), ldb, _ptr(c), ldc, _ptr(bias), float(beta), _ptr(ws),
                                     ws_bytes, _stream(stream)))

    def batched_workspace(self, batch):
        return int(lib().dlp_gemm_batched_workspace(self.h, batch))

    def batch_gemm(self, batch, m, n, k, a, stride_a, lda, b, stride_b, ldb, c, stride_c, ldc, beta=0.0, ws=None, stream=None):
        ws_bytes = ws.numel() * ws.element_size() if ws is not None else 0
        check(lib().dlp_gemm_batched_enqueue(self.h, batch, m, n, k, _ptr(a), stride_a, lda, _ptr(b), stride_b, ldb, _ptr(c), stride_c,
                                             ldc, float(beta), _ptr(ws), ws_bytes, _stream(stream)))

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.dlp_gemm_destroy(self.h)
            self.h = None


class IPForward:
    """Plan object over dlp_ip_fwd_*: the C-ABI face of dlprim::core::IPForward."""

    def __init__(self, inputs, outputs, optimal_batch_size=1, bias=True, activation="identity", math_mode=MATH_AUTO):
        d = IpDesc(inputs, outputs, optimal_batch_size, int(bool(bias)), _act(activation), math_mode)
        self.desc = d
        h = C.c_void_p()
        check(lib().dlp_ip_fwd_create(C.byref(d), C.byref(h)))
        self.h = h

    def kernel(self):
        return lib().dlp_ip_fwd_kernel(self.h).decode()

    def workspace(self):
        return int(lib().dlp_ip_fwd_workspace(self.h))

    def enqueue(self, x, w, bias, y, ws=None, stream=None):
        ws_bytes = ws.numel() * ws.element_size() if ws is not None else 0
        check(lib().dlp_ip_fwd_enqueue(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(y), _ptr(ws), ws_bytes, x.shape[0], _stream(stream)))

    def prepack(self, w, stream=None):
        import torch
        n = int(lib().dlp_ip_fwd_packed_bytes(self.h))
        if n == 0:
            return w
        buf = torch.empty(n, dtype=torch.uint8, device=w.device)
        check(lib().dlp_ip_fwd_prepack(self.h, _ptr(w), _ptr(buf), _stream(stream)))
        return buf

    def enqueue_packed(self, x, packed, bias, y, stream=None, ws=None):
        ws_bytes = ws.numel() * ws.element_size() if ws is not None else 0
        check(lib().dlp_ip_fwd_enqueue_packed(self.h, _ptr(x), _ptr(packed), _ptr(bias), _ptr(y), _ptr(ws), ws_bytes, x.shape[0],
                                              _stream(stream)))

    def enqueue_static(self, x, w, bias, y, stream=None):
        """The allocation-free variant: scratch is the library's own fixed device array (no workspace)."""
        check(lib().dlp_ip_fwd_enqueue_static(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(y), x.shape[0], _stream(stream)))

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.dlp_ip_fwd_destroy(self.h)
            self.h = None


# ---- stateless operators ---------------------------------------------------------------------------
def pooling2d_output_shape(in_h, in_w, kernel, stride=1, pad=0, ceil_mode=False):
    oh, ow = C.c_int(), C.c_int()
    check(lib().dlp_pooling2d_output_shape(in_h, in_w, _i2(*_pair(kernel)), _i2(*_pair(stride)), _i2(*_pair(pad)), int(ceil_mode),
                                           C.byref(oh), C.byref(ow)))
    return oh.value, ow.value


def pooling2d(x, y, kernel, stride=1, pad=0, mode="max", ceil_mode=False, count_include_pad=False, stream=None):
    check(lib().dlp_pooling2d_fwd(_ptr(x), _ptr(y), x.shape[0] * x.shape[1], x.shape[2], x.shape[3], _i2(*_pair(kernel)),
                                  _i2(*_pair(stride)), _i2(*_pair(pad)), int(ceil_mode), int(mode == "avg"), int(count_include_pad),
                                  _stream(stream)))


def global_pooling(x, y, mode="max", stream=None):
    check(lib().dlp_global_pooling_fwd(_ptr(x), _ptr(y), x.shape[0] * x.shape[1], x.shape[2] * x.shape[3], int(mode == "avg"), _stream(stream)))


def elementwise(a, b, c, operation="sum", coef1=1.0, coef2=1.0, activation="identity", stream=None):
    check(lib().dlp_elementwise_fwd(_ptr(a), _ptr(b), _ptr(c), a.numel(), {"sum": 0, "prod": 1, "max": 2}[operation], coef1, coef2,
                                    _act(activation), _stream(stream)))


def activation(x, y, name, stream=None):
    check(lib().dlp_activation_fwd(_ptr(x), _ptr(y), x.numel(), _act(name), _stream(stream)))


def softmax(x, y, log=False, stream=None):
    inner = 1
    for s in x.shape[2:]:
        inner *= s
    check(lib().dlp_softmax_fwd(_ptr(x), _ptr(y), x.shape[0], x.shape[1], inner, int(log), _stream(stream)))


def batchnorm_inference(x, y, mean, var, gamma=None, beta=None, eps=1e-5, stream=None):
    plane = 1
    for s in x.shape[2:]:
        plane *= s
    check(lib().dlp_batchnorm_inference_fwd(_ptr(x), _ptr(y), x.shape[0], x.shape[1], plane, eps, _ptr(mean), _ptr(var), _ptr(gamma),
                                            _ptr(beta), _stream(stream)))
