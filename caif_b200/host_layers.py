"""ctypes doorway onto libcaif_host.so: the C++ layer classes that mirror the
reference's CAIF_DeviceFrozenLinear / CAIF_DeviceLoRAAdapter interface
(caif_b200/host/caif_host.hpp).  Used by the tests; holds no compute."""
import ctypes
import os

import torch

from . import native

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libcaif_host.so")
_lib = None

EXPORTS = ["caifh_last_error", "caifh_frozen_linear_create", "caifh_load_weight_from_device",
           "caifh_load_scales_from_host", "caifh_lora_wrap", "caifh_forward", "caifh_backward", "caifh_description",
           "caifh_parameter_names", "caifh_counts", "caifh_parameter_copy", "caifh_frozen_tensor_fp32",
           "caifh_moe_frozen_expert_create", "caifh_destroy"]


class HostLayerError(RuntimeError):
    pass


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise HostLayerError("%s is missing: run `python caif_b200/host/build.py`" % LIB_PATH)
        native.lib()  # libcaifq.so first: the host library links against it
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.caifh_last_error.restype = ctypes.c_char_p
    return _lib


def _check(rc):
    if rc != 0:
        raise HostLayerError(lib().caifh_last_error().decode())


_ELEM = {native.F32: 4, native.F16: 2, native.BF16: 2}


class Layer:
    """A frozen linear (optionally wrapped by a LoRA adapter) living in the C++ host library."""

    def __init__(self, in_dim, out_dim, storage, compute=native.F32, group_size=128, cache_fp32=True,
                 scheme=native.PER_TENSOR):
        self.in_dim, self.out_dim = in_dim, out_dim
        self.out_code = native.F32
        self.h = ctypes.c_void_p()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream) if torch.cuda.is_available() else None
        _check(lib().caifh_frozen_linear_create(ctypes.c_uint32(in_dim), ctypes.c_uint32(out_dim), int(storage),
                                                int(compute), ctypes.c_uint32(group_size), int(cache_fp32),
                                                int(scheme), stream, ctypes.byref(self.h)))

    def load_weight(self, codes, dtype_code):
        _check(lib().caifh_load_weight_from_device(self.h, ctypes.c_void_p(codes.data_ptr()), int(dtype_code),
                                                   ctypes.c_uint32(self.in_dim), ctypes.c_uint32(self.out_dim)))

    def load_scales_from_host(self, host_bytes):
        buf = ctypes.create_string_buffer(bytes(host_bytes), len(host_bytes))
        _check(lib().caifh_load_scales_from_host(self.h, buf, ctypes.c_size_t(len(host_bytes))))

    def wrap_lora(self, rank, alpha, storage, compute=native.F32, seed=1):
        new = ctypes.c_void_p()
        _check(lib().caifh_lora_wrap(self.h, ctypes.c_uint32(rank), ctypes.c_float(alpha), int(storage), int(compute),
                                     ctypes.c_uint32(seed), ctypes.byref(new)))
        self.h = new
        self.out_code = storage
        return self

    def _run(self, fn, x, last_in, last_out, *extra):
        last_in = x.shape[-1]  # what the caller really passes: the layer checks it against its own dims
        rows = x.numel() // last_in
        out = torch.empty((rows, last_out), dtype=native._CODE_TO_TORCH[self.out_code], device=x.device)
        _check(fn(self.h, ctypes.c_void_p(x.data_ptr()), native.dtype_code(x), ctypes.c_uint32(rows),
                  ctypes.c_uint32(last_in), ctypes.c_void_p(out.data_ptr()),
                  ctypes.c_size_t(out.numel() * _ELEM[self.out_code]), *extra))
        return out

    def forward(self, x, training=True):
        return self._run(lib().caifh_forward, x, self.in_dim, self.out_dim, int(training))

    def backward(self, dy):
        return self._run(lib().caifh_backward, dy, self.out_dim, self.in_dim)

    def description(self):
        buf = ctypes.create_string_buffer(512)
        _check(lib().caifh_description(self.h, buf, ctypes.c_size_t(512)))
        return buf.value.decode()

    def parameter_names(self, prefix=""):
        buf = ctypes.create_string_buffer(1024)
        _check(lib().caifh_parameter_names(self.h, prefix.encode(), buf, ctypes.c_size_t(1024)))
        return [n for n in buf.value.decode().split(";") if n]

    def counts(self):
        a, b, c = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        _check(lib().caifh_counts(self.h, ctypes.byref(a), ctypes.byref(b), ctypes.byref(c)))
        return a.value, b.value, c.value

    def parameter(self, index, like, gradient=False):
        out = torch.empty_like(like)
        _check(lib().caifh_parameter_copy(self.h, ctypes.c_uint64(index), int(gradient), 0,
                                          ctypes.c_void_p(out.data_ptr()),
                                          ctypes.c_size_t(out.numel() * out.element_size())))
        return out

    def set_parameter(self, index, value):
        _check(lib().caifh_parameter_copy(self.h, ctypes.c_uint64(index), 0, 1, ctypes.c_void_p(value.data_ptr()),
                                          ctypes.c_size_t(value.numel() * value.element_size())))

    def frozen_tensor_fp32(self):
        out = torch.empty((self.out_dim, self.in_dim), dtype=torch.float32, device="cuda")
        _check(lib().caifh_frozen_tensor_fp32(self.h, ctypes.c_void_p(out.data_ptr()), ctypes.c_size_t(out.numel() * 4)))
        return out

    def close(self):
        if self.h:
            lib().caifh_destroy(self.h)
            self.h = ctypes.c_void_p()


class FrozenExpert(Layer):
    """CAIF_DeviceMoEFrozenExpert over three frozen linears (gate may be None: the non-gated form).
    The expert takes the three layers over: their Python objects are emptied."""

    def __init__(self, gate, up, down, input_dim, hidden_dim, storage, compute=native.F32):
        self.in_dim, self.out_dim = input_dim, input_dim
        self.out_code = storage
        self.h = ctypes.c_void_p()
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream) if torch.cuda.is_available() else None
        _check(lib().caifh_moe_frozen_expert_create(gate.h if gate is not None else None, up.h, down.h,
                                                    ctypes.c_uint32(input_dim), ctypes.c_uint32(hidden_dim),
                                                    int(gate is not None), int(storage), int(compute), stream,
                                                    ctypes.byref(self.h)))
        for layer in (gate, up, down):
            if layer is not None:
                layer.h = ctypes.c_void_p()
