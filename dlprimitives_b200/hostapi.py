"""ctypes binding of include/dlp_host.h: the factory-made operators and the Net of the C++ host
library (lib/libdlprim_b200.so), driven the way the reference's own test driver and benchmark tool
drive them.  PyTorch supplies device memory and streams only."""
import ctypes as C
import json
import os

from . import capi

LIB_PATH = os.path.join(capi.HERE, "lib", "libdlprim_b200.so")
_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_ip = C.POINTER(C.c_int)
_vpp = C.POINTER(C.c_void_p)

SYMBOLS = {
    "dlp_host_last_error": (C.c_char_p, []),
    "dlp_op_create": (_i, [C.c_char_p, C.c_char_p, _i, _i, _ip, _ip, _vpp]),
    "dlp_op_destroy": (None, [_vp]),
    "dlp_op_num_outputs": (_i, [_vp]),
    "dlp_op_num_params": (_i, [_vp]),
    "dlp_op_output_shape": (_i, [_vp, _i, _ip]),
    "dlp_op_param_shape": (_i, [_vp, _i, _ip]),
    "dlp_op_workspace": (_sz, [_vp]),
    "dlp_op_kernel": (C.c_char_p, [_vp]),
    "dlp_op_reshape": (_i, [_vp, _i, _ip, _ip]),
    "dlp_op_forward": (_i, [_vp, _vpp, _vpp, _vpp, _vp, _vp]),
    "dlp_net_create": (_i, [C.c_char_p, _i, _i, _vpp]),
    "dlp_net_destroy": (None, [_vp]),
    "dlp_net_num_params": (_i, [_vp]),
    "dlp_net_param_name": (_i, [_vp, _i, C.c_char_p, _i]),
    "dlp_net_param_shape": (_i, [_vp, C.c_char_p, _ip]),
    "dlp_net_tensor_shape": (_i, [_vp, C.c_char_p, _ip]),
    "dlp_net_set_param": (_i, [_vp, C.c_char_p, _vp, _sz]),
    "dlp_net_upload_params": (_i, [_vp]),
    "dlp_net_load_params_file": (_i, [_vp, C.c_char_p]),
    "dlp_net_save_params_file": (_i, [_vp, C.c_char_p]),
    "dlp_net_set_tensor": (_i, [_vp, C.c_char_p, _vp, _sz, _vp]),
    "dlp_net_get_tensor": (_i, [_vp, C.c_char_p, _vp, _sz, _vp]),
    "dlp_net_tensor_device_ptr": (_vp, [_vp, C.c_char_p]),
    "dlp_net_reshape_input": (_i, [_vp, C.c_char_p, _i, _ip]),
    "dlp_net_reshape": (_i, [_vp]),
    "dlp_net_forward": (_i, [_vp, _vp, _i]),
    "dlp_net_forward_timed": (_i, [_vp, _vp, C.POINTER(C.c_float), _i]),
    "dlp_net_copy_tensor_to_device": (_i, [_vp, C.c_char_p, _vp, _sz, _vp]),
    "dlp_net_copy_tensor_from_device": (_i, [_vp, C.c_char_p, _vp, _sz, _vp]),
    "dlp_net_num_steps": (_i, [_vp]),
    "dlp_net_step_description": (_i, [_vp, _i, C.c_char_p, _i]),
    "dlp_net_activation_bytes": (_sz, [_vp, _i]),
    "dlp_host_merge_activations": (_i, [C.c_char_p, C.c_char_p, _sz]),
    "dlp_host_gemm": (_i, [_i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _i, _vp, _i, _vp, _i, _vp, C.c_float, _vp]),
    "dlp_host_batch_sgemm": (_i, [_i, _i, _i, _i, _i, _i, _i, _vp, _i, _i, _vp, _i, _i, _vp, _i, _i, C.c_float, _vp]),
    "dlp_host_conv_gemm": (_i, [_i, _ip, _i, _i, _i, _i, _vp, _vp, _vp, _vp, C.c_float, _vp]),
}
_lib = None


class HostError(RuntimeError):
    """An exception thrown by the C++ host library; `kind` is its class name there."""

    def __init__(self, message):
        super().__init__(message)
        self.kind = message.split(":", 1)[0]


def lib():
    global _lib
    if _lib is None:
        capi.lib()   # the kernels' library first: fails loudly when it is missing
        if not os.path.exists(LIB_PATH):
            raise ImportError("%s is missing: run `python -m dlprimitives_b200.build`" % LIB_PATH)
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def _fail():
    raise HostError(lib().dlp_host_last_error().decode())


def _shapes(shapes):
    ranks = (C.c_int * max(1, len(shapes)))(*[len(s) for s in shapes])
    flat = [int(v) for s in shapes for v in s]
    dims = (C.c_int * max(1, len(flat)))(*flat)
    return ranks, dims


def _stream(stream):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return s.cuda_stream


class Operator:
    """create_by_name(type, options) + setup(input shapes) on a CUDA context."""

    def __init__(self, op_type, options, in_shapes, device=0):
        ranks, dims = _shapes(in_shapes)
        h = C.c_void_p()
        if lib().dlp_op_create(op_type.encode(), json.dumps(options).encode(), device, len(in_shapes), ranks, dims, C.byref(h)) != 0:
            _fail()
        self.h = h
        self.device = device
        self._refresh()

    def _refresh(self):
        buf = (C.c_int * 8)()
        L = lib()
        self.out_shapes = [tuple(buf[:L.dlp_op_output_shape(self.h, i, buf)]) for i in range(L.dlp_op_num_outputs(self.h))]
        self.param_shapes = [tuple(buf[:L.dlp_op_param_shape(self.h, i, buf)]) for i in range(L.dlp_op_num_params(self.h))]
        self.workspace = int(L.dlp_op_workspace(self.h))
        self.kernel = L.dlp_op_kernel(self.h).decode()

    def reshape(self, in_shapes):
        ranks, dims = _shapes(in_shapes)
        if lib().dlp_op_reshape(self.h, len(in_shapes), ranks, dims) != 0:
            _fail()
        self._refresh()

    def forward(self, inputs, params=(), outputs=None, stream=None):
        """inputs/params/outputs: CUDA fp32 tensors; outputs are allocated when not given."""
        import torch
        dev = inputs[0].device
        if outputs is None:
            outputs = [torch.empty(s, dtype=torch.float32, device=dev) for s in self.out_shapes]
        ws = torch.empty(max(self.workspace, 16), dtype=torch.uint8, device=dev)
        mk = lambda ts: (C.c_void_p * max(1, len(ts)))(*[capi._ptr(t) for t in ts])
        if lib().dlp_op_forward(self.h, mk(inputs), mk(params), mk(outputs), capi._ptr(ws), _stream(stream)) != 0:
            _fail()
        self._ws_keepalive = ws
        return outputs

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.dlp_op_destroy(self.h)
            self.h = None


class Net:
    """A dlprim::Net built from the network JSON (predict mode, setup done)."""
    KEEP_INTERMEDIATE, NO_FUSION, NO_GRAPH, MERGE_ACTIVATIONS, CONCURRENT_BRANCHES = 1, 2, 4, 8, 16

    def __init__(self, net_json, device=0, flags=0):
        text = net_json if isinstance(net_json, str) else json.dumps(net_json)
        h = C.c_void_p()
        if lib().dlp_net_create(text.encode(), device, flags, C.byref(h)) != 0:
            _fail()
        self.h = h
        self.device = device

    def param_names(self):
        buf = C.create_string_buffer(1024)
        names = []
        for i in range(lib().dlp_net_num_params(self.h)):
            lib().dlp_net_param_name(self.h, i, buf, 1024)
            names.append(buf.value.decode())
        return names

    def _shape(self, fn, name):
        buf = (C.c_int * 8)()
        n = fn(self.h, name.encode(), buf)
        if n < 0:
            _fail()
        return tuple(buf[:n])

    def param_shape(self, name):
        return self._shape(lib().dlp_net_param_shape, name)

    def tensor_shape(self, name):
        return self._shape(lib().dlp_net_tensor_shape, name)

    def set_param(self, name, array):
        import numpy as np
        a = np.ascontiguousarray(array, dtype=np.float32)
        if lib().dlp_net_set_param(self.h, name.encode(), a.ctypes.data, a.size) != 0:
            _fail()

    def upload_params(self):
        if lib().dlp_net_upload_params(self.h) != 0:
            _fail()

    def load_params_file(self, path):
        if lib().dlp_net_load_params_file(self.h, path.encode()) != 0:
            _fail()

    def save_params_file(self, path):
        if lib().dlp_net_save_params_file(self.h, path.encode()) != 0:
            _fail()

    def set_tensor(self, name, host_tensor, stream=None):
        """Asynchronous host->device copy of a (preferably pinned) torch CPU tensor or numpy array."""
        ptr, n = _host_ptr(host_tensor)
        if lib().dlp_net_set_tensor(self.h, name.encode(), ptr, n, _stream(stream)) != 0:
            _fail()

    def get_tensor(self, name, host_tensor, stream=None):
        ptr, n = _host_ptr(host_tensor)
        if lib().dlp_net_get_tensor(self.h, name.encode(), ptr, n, _stream(stream)) != 0:
            _fail()

    def tensor_device_ptr(self, name):
        p = lib().dlp_net_tensor_device_ptr(self.h, name.encode())
        if not p:
            _fail()
        return p

    def reshape_input(self, name, shape):
        dims = (C.c_int * len(shape))(*[int(v) for v in shape])
        if lib().dlp_net_reshape_input(self.h, name.encode(), len(shape), dims) != 0:
            _fail()

    def reshape(self):
        if lib().dlp_net_reshape(self.h) != 0:
            _fail()

    def forward(self, stream=None, sync=False):
        if lib().dlp_net_forward(self.h, _stream(stream), int(sync)) != 0:
            _fail()

    def forward_timed(self, stream=None):
        """One eager pass with an event pair around every plan step; returns milliseconds per step."""
        n = lib().dlp_net_num_steps(self.h)
        buf = (C.c_float * n)()
        if lib().dlp_net_forward_timed(self.h, _stream(stream), buf, n) != 0:
            _fail()
        return list(buf)

    def copy_tensor_to(self, name, device_tensor, stream=None):
        if lib().dlp_net_copy_tensor_to_device(self.h, name.encode(), capi._ptr(device_tensor), device_tensor.numel(), _stream(stream)) != 0:
            _fail()

    def copy_tensor_from(self, name, device_tensor, stream=None):
        if lib().dlp_net_copy_tensor_from_device(self.h, name.encode(), capi._ptr(device_tensor), device_tensor.numel(), _stream(stream)) != 0:
            _fail()

    def plan(self):
        buf = C.create_string_buffer(2048)
        out = []
        for i in range(lib().dlp_net_num_steps(self.h)):
            lib().dlp_net_step_description(self.h, i, buf, 2048)
            out.append(buf.value.decode())
        return out

    def activation_bytes(self, without_reuse=False):
        return int(lib().dlp_net_activation_bytes(self.h, int(without_reuse)))

    def __del__(self):
        if getattr(self, "h", None) and _lib is not None:
            _lib.dlp_net_destroy(self.h)
            self.h = None


def _host_ptr(t):
    import numpy as np
    if isinstance(t, np.ndarray):
        assert t.dtype == np.float32 and t.flags["C_CONTIGUOUS"]
        return t.ctypes.data, t.size
    assert not t.is_cuda and t.is_contiguous()
    return t.data_ptr(), t.numel()


def _dptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def gemm(trans_a, trans_b, m, n, k, a, lda, b, ldb, c, ldc, bias=None, bias_mode=0, activation="identity", beta=0.0, planned=None,
         stream=None, device=0):
    """gpu::GEMM::get_optimal_gemm(...)->gemm(...) on device tensors; planned = (M, N, K) the object is made for."""
    pm, pn, pk = planned or (m, n, k)
    if lib().dlp_host_gemm(device, int(trans_a), int(trans_b), pm, pn, pk, m, n, k, bias_mode, capi._act(activation), _dptr(a), lda, _dptr(b),
                           ldb, _dptr(c), ldc, _dptr(bias), float(beta), _stream(stream)):
        _fail()


def batch_sgemm(trans_a, trans_b, batch, m, n, k, a, stride_a, lda, b, stride_b, ldb, c, stride_c, ldc, beta=0.0, stream=None, device=0):
    """gpu::GEMM::batch_sgemm on device tensors (asynchronous on the stream)."""
    if lib().dlp_host_batch_sgemm(device, int(trans_a), int(trans_b), batch, m, n, k, _dptr(a), stride_a, lda, _dptr(b), stride_b, ldb,
                                  _dptr(c), stride_c, ldc, float(beta), _stream(stream)):
        _fail()


def conv_gemm(x, w, bias, y, stride=1, pad=0, dilate=1, groups=1, activation="identity", factor=0.0, stream=None, device=0):
    """gpu::GEMM::get_optimal_conv_gemm(forward)->gemm(filters, x, y) the way the reference's Conv2DForwardGEMM calls it."""
    pair = lambda v: [v, v] if isinstance(v, int) else list(v)
    n, cin, h, wd = x.shape
    cout, cin_g, kh, kw = w.shape
    geometry = [kh, kw] + pair(dilate) + pair(pad) + pair(stride) + [groups, cin_g, h, wd, y.shape[2], y.shape[3]]
    arr = (C.c_int * 14)(*geometry)
    if lib().dlp_host_conv_gemm(device, arr, cout // groups, n, int(bias is not None), capi._act(activation), _dptr(w), _dptr(x), _dptr(y),
                                _dptr(bias), float(factor), _stream(stream)):
        _fail()


def merge_activations(net_json):
    """Net::merge_activations on a network description (dict or JSON text); returns (merged description as a dict, count).
    Needs no device."""
    text = net_json if isinstance(net_json, str) else json.dumps(net_json)
    buf = C.create_string_buffer(len(text) + 1024)
    n = lib().dlp_host_merge_activations(text.encode(), buf, len(buf))
    if n < 0:
        _fail()
    return json.loads(buf.value.decode()), n
