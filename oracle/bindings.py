"""numpy-facing ctypes bindings for the CPU checker libraries.

TEST INFRASTRUCTURE ONLY: imported by tests/, the smoke check and the bench's CPU-baseline leg.
Nothing in the product package imports this module.

* ``liboracle.so``      -- this repository's C restatement of the reference CPU path (oracle.c)
* ``_ref/libref_runner.so`` -- the reference library's own CPU context, built from the reference
  sources where the reference tree is mounted (see Makefile); optional.
"""
import ctypes as C
import json
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ACTIVATIONS = {"identity": 0, "relu": 1, "tanh": 2, "sigmoid": 3, "relu6": 4}
_f32p = C.POINTER(C.c_float)


def _ptr(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _pair(v):
    return [int(v), int(v)] if np.isscalar(v) else [int(v[0]), int(v[1])]


def build(reference=None):
    """Compile liboracle.so and, when the reference tree is present, the _ref libraries."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    reference = reference or os.environ.get("DLPRIM_REFERENCE", "/root/reference")
    if os.path.isdir(os.path.join(reference, "src", "ops")):
        subprocess.run(["make", "-s", "-j8", "-C", HERE, "ref", "REF=" + reference], check=True)


class ConvDesc(C.Structure):
    _fields_ = [("batch", C.c_int), ("channels_in", C.c_int), ("height", C.c_int), ("width", C.c_int),
                ("channels_out", C.c_int), ("kernel", C.c_int * 2), ("stride", C.c_int * 2),
                ("dilate", C.c_int * 2), ("pad", C.c_int * 2), ("groups", C.c_int), ("activation", C.c_int)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        L = C.CDLL(path)
        L.oracle_conv2d_forward.argtypes = [C.POINTER(ConvDesc), _f32p, _f32p, _f32p, _f32p]
        L.oracle_conv2d_winograd_forward.argtypes = [C.POINTER(ConvDesc), _f32p, _f32p, _f32p, _f32p]
        L.oracle_conv2d_output_hw.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_int), C.POINTER(C.c_int)]
        L.oracle_sgemm.argtypes = [C.c_int] * 5 + [C.c_float, _f32p, C.c_int, _f32p, C.c_int, C.c_float, _f32p, C.c_int]
        L.oracle_gemm_bias_act.argtypes = [C.c_int] * 5 + [_f32p, C.c_int, _f32p, C.c_int, C.c_float, _f32p, C.c_int, _f32p, C.c_int, C.c_int]
        L.oracle_inner_product_forward.argtypes = [C.c_int] * 3 + [_f32p, _f32p, _f32p, C.c_int, _f32p]
        L.oracle_activation.argtypes = [_f32p, C.c_size_t, C.c_int]
        L.oracle_pooling_output_size.argtypes = [C.c_int] * 5
        L.oracle_pooling2d_forward.argtypes = [C.c_int] * 3 + [C.POINTER(C.c_int)] * 3 + [C.c_int] * 3 + [_f32p, _f32p]
        L.oracle_global_pooling_forward.argtypes = [C.c_int] * 3 + [_f32p, _f32p]
        L.oracle_elementwise_forward.argtypes = [C.c_size_t, C.c_int, C.c_float, C.c_float, C.c_int, _f32p, _f32p, _f32p]
        L.oracle_softmax_forward.argtypes = [C.c_int] * 4 + [_f32p, _f32p]
        L.oracle_batchnorm_inference.argtypes = [C.c_int] * 3 + [C.c_float] + [_f32p] * 6
        L.oracle_fold_batchnorm.argtypes = [C.c_int, C.c_size_t, C.c_float] + [_f32p] * 8
        L.oracle_set_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def set_threads(n):
    lib().oracle_set_threads(int(n))


def conv_desc(x_shape, w_shape, stride=1, pad=0, dilate=1, groups=1, activation="identity"):
    d = ConvDesc()
    d.batch, d.channels_in, d.height, d.width = [int(v) for v in x_shape]
    d.channels_out = int(w_shape[0])
    d.kernel[0], d.kernel[1] = int(w_shape[2]), int(w_shape[3])
    for name, v in (("stride", stride), ("pad", pad), ("dilate", dilate)):
        p = _pair(v)
        getattr(d, name)[0], getattr(d, name)[1] = p
    d.groups = int(groups)
    d.activation = ACTIVATIONS[activation] if isinstance(activation, str) else int(activation)
    return d


def conv2d(x, w, bias=None, stride=1, pad=0, dilate=1, groups=1, activation="identity", winograd=False):
    x, w, bias = _f32(x), _f32(w), _f32(bias)
    d = conv_desc(x.shape, w.shape, stride, pad, dilate, groups, activation)
    oh, ow = C.c_int(), C.c_int()
    lib().oracle_conv2d_output_hw(C.byref(d), C.byref(oh), C.byref(ow))
    y = np.empty((x.shape[0], w.shape[0], oh.value, ow.value), dtype=np.float32)
    fn = lib().oracle_conv2d_winograd_forward if winograd else lib().oracle_conv2d_forward
    rc = fn(C.byref(d), _ptr(x), _ptr(w), _ptr(bias), _ptr(y))
    if rc != 0:
        raise ValueError("oracle conv2d rejected the configuration (%d)" % rc)
    return y


def sgemm(a, b, trans_a=False, trans_b=False, alpha=1.0, beta=0.0, c=None):
    a, b = _f32(a), _f32(b)
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    out = np.zeros((M, N), dtype=np.float32) if c is None else np.array(c, dtype=np.float32, order="C")
    lib().oracle_sgemm(int(trans_a), int(trans_b), M, N, K, alpha, _ptr(a), a.shape[1], _ptr(b), b.shape[1], beta, _ptr(out), N)
    return out


def gemm_bias_act(a, b, trans_a=False, trans_b=False, beta=0.0, c=None, bias=None, bias_mode=0, activation="identity"):
    a, b, bias = _f32(a), _f32(b), _f32(bias)
    M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
    N = b.shape[0] if trans_b else b.shape[1]
    out = np.zeros((M, N), dtype=np.float32) if c is None else np.array(c, dtype=np.float32, order="C")
    lib().oracle_gemm_bias_act(int(trans_a), int(trans_b), M, N, K, _ptr(a), a.shape[1], _ptr(b), b.shape[1], beta,
                               _ptr(out), N, _ptr(bias), bias_mode, ACTIVATIONS[activation])
    return out


def inner_product(x, w, bias=None, activation="identity"):
    x, w, bias = _f32(x), _f32(w), _f32(bias)
    x2 = x.reshape(x.shape[0], -1)
    y = np.empty((x2.shape[0], w.shape[0]), dtype=np.float32)
    lib().oracle_inner_product_forward(x2.shape[0], x2.shape[1], w.shape[0], _ptr(x2), _ptr(w), _ptr(bias), ACTIVATIONS[activation], _ptr(y))
    return y


def activation(x, name):
    y = np.array(x, dtype=np.float32, order="C")
    lib().oracle_activation(_ptr(y), y.size, ACTIVATIONS[name])
    return y


def pooling2d(x, kernel, stride=1, pad=0, mode="max", ceil_mode=False, count_include_pad=False):
    x = _f32(x)
    k, s, p = _pair(kernel), _pair(stride), _pair(pad)
    oh = lib().oracle_pooling_output_size(x.shape[2], k[0], p[0], s[0], int(ceil_mode))
    ow = lib().oracle_pooling_output_size(x.shape[3], k[1], p[1], s[1], int(ceil_mode))
    y = np.empty((x.shape[0], x.shape[1], oh, ow), dtype=np.float32)
    I2 = C.c_int * 2
    lib().oracle_pooling2d_forward(x.shape[0] * x.shape[1], x.shape[2], x.shape[3], I2(*k), I2(*s), I2(*p), int(ceil_mode),
                                   int(mode == "avg"), int(count_include_pad), _ptr(x), _ptr(y))
    return y


def global_pooling(x, mode="max"):
    x = _f32(x)
    y = np.empty((x.shape[0], x.shape[1], 1, 1), dtype=np.float32)
    lib().oracle_global_pooling_forward(x.shape[0] * x.shape[1], x.shape[2] * x.shape[3], int(mode == "avg"), _ptr(x), _ptr(y))
    return y


def elementwise(a, b, operation="sum", coef1=1.0, coef2=1.0, activation="identity"):
    a, b = _f32(a), _f32(b)
    assert a.shape == b.shape
    c = np.empty_like(a)
    lib().oracle_elementwise_forward(a.size, {"sum": 0, "prod": 1, "max": 2}[operation], coef1, coef2, ACTIVATIONS[activation], _ptr(a), _ptr(b), _ptr(c))
    return c


def softmax(x, log=False):
    x = _f32(x)
    inner = int(np.prod(x.shape[2:])) if x.ndim > 2 else 1
    y = np.empty_like(x)
    lib().oracle_softmax_forward(x.shape[0], x.shape[1], inner, int(log), _ptr(x), _ptr(y))
    return y


def batchnorm_inference(x, mean, var, gamma=None, beta=None, eps=1e-5):
    x, mean, var, gamma, beta = _f32(x), _f32(mean), _f32(var), _f32(gamma), _f32(beta)
    y = np.empty_like(x)
    lib().oracle_batchnorm_inference(x.shape[0], x.shape[1], int(np.prod(x.shape[2:])), eps, _ptr(mean), _ptr(var), _ptr(gamma), _ptr(beta), _ptr(x), _ptr(y))
    return y


def fold_batchnorm(w, bias, mean, var, gamma, beta, eps=1e-5):
    w, bias, mean, var, gamma, beta = _f32(w), _f32(bias), _f32(mean), _f32(var), _f32(gamma), _f32(beta)
    w2, b2 = np.empty_like(w), np.empty(w.shape[0], dtype=np.float32)
    lib().oracle_fold_batchnorm(w.shape[0], w[0].size, eps, _ptr(mean), _ptr(var), _ptr(gamma), _ptr(beta), _ptr(w), _ptr(bias), _ptr(w2), _ptr(b2))
    return w2, b2


# ---------------------------------------------------------------------------------------------
# The reference's own CPU context (optional)
# ---------------------------------------------------------------------------------------------
_ref = None


def ref_available():
    return os.path.exists(os.path.join(HERE, "_ref", "libref_runner.so"))


def ref():
    global _ref
    if _ref is None:
        R = C.CDLL(os.path.join(HERE, "_ref", "libref_runner.so"))
        R.ref_last_error.restype = C.c_char_p
        R.ref_op_create.restype = C.c_void_p
        R.ref_op_create.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        R.ref_op_destroy.argtypes = [C.c_void_p]
        for n in ("ref_op_num_outputs", "ref_op_num_params"):
            getattr(R, n).argtypes = [C.c_void_p]
        for n in ("ref_op_output_shape", "ref_op_param_shape"):
            getattr(R, n).argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
        R.ref_op_forward.restype = C.c_double
        R.ref_op_forward.argtypes = [C.c_void_p, C.POINTER(_f32p), C.POINTER(_f32p), C.POINTER(_f32p)]
        R.ref_net_create.restype = C.c_void_p
        R.ref_net_create.argtypes = [C.c_char_p]
        R.ref_net_destroy.argtypes = [C.c_void_p]
        R.ref_net_keep_intermediate.argtypes = [C.c_void_p, C.c_int]
        R.ref_net_num_params.argtypes = [C.c_void_p]
        R.ref_net_param_name.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_int]
        R.ref_net_param_shape.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int)]
        R.ref_net_tensor_shape.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_int)]
        for n in ("ref_net_set_param", "ref_net_set_tensor", "ref_net_get_tensor", "ref_net_get_param"):
            getattr(R, n).argtypes = [C.c_void_p, C.c_char_p, _f32p, C.c_ulonglong]
        for n in ("ref_net_save_params", "ref_net_load_params"):
            getattr(R, n).argtypes = [C.c_void_p, C.c_char_p]
        R.ref_net_forward.restype = C.c_double
        R.ref_net_forward.argtypes = [C.c_void_p]
        _ref = R
    return _ref


class RefError(RuntimeError):
    pass


def _ref_fail():
    raise RefError(ref().ref_last_error().decode())


class RefOperator:
    """One reference operator on the reference's CPU context (create_by_name + setup)."""

    def __init__(self, op_type, options, in_shapes):
        ranks = (C.c_int * len(in_shapes))(*[len(s) for s in in_shapes])
        flat = [int(v) for s in in_shapes for v in s]
        dims = (C.c_int * len(flat))(*flat)
        self.h = ref().ref_op_create(op_type.encode(), json.dumps(options).encode(), len(in_shapes), ranks, dims)
        if not self.h:
            _ref_fail()
        buf = (C.c_int * 8)()
        self.out_shapes = [tuple(buf[:ref().ref_op_output_shape(self.h, i, buf)]) for i in range(ref().ref_op_num_outputs(self.h))]
        self.param_shapes = [tuple(buf[:ref().ref_op_param_shape(self.h, i, buf)]) for i in range(ref().ref_op_num_params(self.h))]
        self.seconds = 0.0

    def forward(self, inputs, params=()):
        ins = [_f32(a) for a in inputs]
        pars = [_f32(a) for a in params]
        assert len(pars) == len(self.param_shapes)
        outs = [np.empty(s, dtype=np.float32) for s in self.out_shapes]
        mk = lambda arrs: (_f32p * max(1, len(arrs)))(*[_ptr(a) for a in arrs])
        t = ref().ref_op_forward(self.h, mk(ins), mk(pars), mk(outs))
        if t < 0:
            _ref_fail()
        self.seconds = t
        return outs

    def __del__(self):
        if getattr(self, "h", None):
            ref().ref_op_destroy(self.h)
            self.h = None


class RefNet:
    """A reference Net on its CPU context, built from the network JSON."""

    def __init__(self, net_json, keep_intermediate=False):
        text = net_json if isinstance(net_json, str) else json.dumps(net_json)
        self.h = ref().ref_net_create(text.encode())
        if not self.h:
            _ref_fail()
        if keep_intermediate:
            ref().ref_net_keep_intermediate(self.h, 1)
        self.seconds = 0.0

    def param_names(self):
        buf = C.create_string_buffer(512)
        names = []
        for i in range(ref().ref_net_num_params(self.h)):
            ref().ref_net_param_name(self.h, i, buf, 512)
            names.append(buf.value.decode())
        return names

    def _shape(self, fn, name):
        buf = (C.c_int * 8)()
        n = fn(self.h, name.encode(), buf)
        if n < 0:
            _ref_fail()
        return tuple(buf[:n])

    def param_shape(self, name):
        return self._shape(ref().ref_net_param_shape, name)

    def tensor_shape(self, name):
        return self._shape(ref().ref_net_tensor_shape, name)

    def set_param(self, name, value):
        a = _f32(value)
        if ref().ref_net_set_param(self.h, name.encode(), _ptr(a), a.size) != 0:
            _ref_fail()

    def set_tensor(self, name, value):
        a = _f32(value)
        if ref().ref_net_set_tensor(self.h, name.encode(), _ptr(a), a.size) != 0:
            _ref_fail()

    def get_tensor(self, name):
        out = np.empty(self.tensor_shape(name), dtype=np.float32)
        if ref().ref_net_get_tensor(self.h, name.encode(), _ptr(out), out.size) != 0:
            _ref_fail()
        return out

    def get_param(self, name):
        out = np.empty(self.param_shape(name), dtype=np.float32)
        if ref().ref_net_get_param(self.h, name.encode(), _ptr(out), out.size) != 0:
            _ref_fail()
        return out

    def save_params_file(self, path):
        """The reference's own Net::save_parameters (its DLPW writer)."""
        if ref().ref_net_save_params(self.h, str(path).encode()) != 0:
            _ref_fail()

    def load_params_file(self, path):
        """The reference's own Net::load_parameters (its DLPW reader)."""
        if ref().ref_net_load_params(self.h, str(path).encode()) != 0:
            _ref_fail()

    def forward(self):
        t = ref().ref_net_forward(self.h)
        if t < 0:
            _ref_fail()
        self.seconds = t

    def __del__(self):
        if getattr(self, "h", None):
            ref().ref_net_destroy(self.h)
            self.h = None
