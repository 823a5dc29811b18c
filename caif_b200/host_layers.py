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
           "caifh_moe_frozen_expert_create", "caifh_destroy", "caifh_st_open", "caifh_st_open_directory",
           "caifh_st_close", "caifh_st_names", "caifh_st_info", "caifh_st_metadata", "caifh_st_read", "caifh_st_save",
           "caifh_st_save_device", "caifh_st_load_device", "caifh_load_frozen_linear", "caifh_mapper_create",
           "caifh_mapper_destroy", "caifh_mapper_add", "caifh_mapper_translate", "caifh_mapper_query",
           "caifh_save_parameters", "caifh_load_parameters"]


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

    def save_parameters(self, path, prefix=""):
        """The trainable tensors (LoRA A and B) as a SafeTensors file under parameter_names(prefix)."""
        _check(lib().caifh_save_parameters(self.h, prefix.encode(), path.encode()))

    def load_parameters(self, safetensors_file, prefix=""):
        _check(lib().caifh_load_parameters(self.h, prefix.encode(), safetensors_file.h))

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


# ---------------------------------------------------------------------------- SafeTensors files
_TEXT_CAP = 1 << 22


def _strings(items):
    arr = (ctypes.c_char_p * max(1, len(items)))()
    for i, s in enumerate(items):
        arr[i] = s.encode()
    return arr


def _flat_shapes(shapes):
    flat = [d for shape in shapes for d in shape]
    return ((ctypes.c_uint32 * max(1, len(shapes)))(*[len(s) for s in shapes]),
            (ctypes.c_uint32 * max(1, len(flat)))(*flat))


def save_safetensors(path, tensors, metadata=None):
    """tensors: list of (name, SafeTensors dtype name, shape, bytes-like) written back to back in this order
    (CAIF_SafeTensorsFormat::SaveHost)."""
    metadata = metadata or {}
    held = [bytes(t[3]) for t in tensors]
    data = (ctypes.c_void_p * max(1, len(tensors)))()
    for i, b in enumerate(held):
        data[i] = ctypes.cast(ctypes.c_char_p(b), ctypes.c_void_p)
    ranks, flat = _flat_shapes([t[2] for t in tensors])
    keys = sorted(metadata)
    _check(lib().caifh_st_save(path.encode(), ctypes.c_uint32(len(tensors)), _strings([t[0] for t in tensors]),
                               _strings([t[1] for t in tensors]), ranks, flat, data, ctypes.c_uint32(len(keys)),
                               _strings(keys), _strings([metadata[k] for k in keys])))


def save_safetensors_device(path, tensors):
    """tensors: list of (name, CAIF dtype code, shape, CUDA tensor holding the raw bytes); written through
    CAIF_SafeTensorsFormat::Save with {"framework": "CAIF"} as metadata."""
    data = (ctypes.c_void_p * max(1, len(tensors)))(*[t[3].data_ptr() for t in tensors])
    ranks, flat = _flat_shapes([t[2] for t in tensors])
    codes = (ctypes.c_int * max(1, len(tensors)))(*[int(t[1]) for t in tensors])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _check(lib().caifh_st_save_device(path.encode(), ctypes.c_uint32(len(tensors)), _strings([t[0] for t in tensors]),
                                      codes, ranks, flat, data, stream))


class SafeTensors:
    """One opened .safetensors file, or a checkpoint directory (index + shards)."""

    def __init__(self, path, directory=False):
        self.h = ctypes.c_void_p()
        fn = lib().caifh_st_open_directory if directory else lib().caifh_st_open
        _check(fn(path.encode(), ctypes.byref(self.h)))

    def _text(self, fn, *args):
        buf = ctypes.create_string_buffer(_TEXT_CAP)
        _check(fn(self.h, *args, buf, ctypes.c_size_t(_TEXT_CAP)))
        return buf.value.decode()

    def names(self):
        return [n for n in self._text(lib().caifh_st_names).split("\n") if n]

    def metadata(self):
        flat = self._text(lib().caifh_st_metadata).split("\n")[:-1]
        return dict(zip(flat[0::2], flat[1::2]))

    def info(self, name):
        dtype = ctypes.create_string_buffer(16)
        path = ctypes.create_string_buffer(4096)
        rank, begin, end, nbytes = ctypes.c_uint32(), ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
        shape = (ctypes.c_uint32 * 16)()
        _check(lib().caifh_st_info(self.h, name.encode(), dtype, ctypes.c_size_t(16), ctypes.byref(rank), shape,
                                   ctypes.c_uint32(16), ctypes.byref(begin), ctypes.byref(end), ctypes.byref(nbytes),
                                   path, ctypes.c_size_t(4096)))
        return {"dtype": dtype.value.decode(), "shape": list(shape[:rank.value]), "begin": begin.value,
                "end": end.value, "bytes": nbytes.value, "file": path.value.decode()}

    def read(self, name):
        n = self.info(name)["bytes"]
        buf = ctypes.create_string_buffer(max(1, n))
        _check(lib().caifh_st_read(self.h, name.encode(), buf, ctypes.c_size_t(n)))
        return buf.raw[:n]

    def load_device(self, name):
        n = self.info(name)["bytes"]
        out = torch.empty(max(1, n), dtype=torch.uint8, device="cuda")
        _check(lib().caifh_st_load_device(self.h, name.encode(), ctypes.c_void_p(out.data_ptr()), ctypes.c_size_t(n),
                                          ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        return out[:n]

    def load_frozen_linear(self, layer, weight_name, scales_name=""):
        _check(lib().caifh_load_frozen_linear(layer.h, self.h, weight_name.encode(), scales_name.encode()))

    def close(self):
        if self.h:
            lib().caifh_st_close(self.h)
            self.h = ctypes.c_void_p()


class WeightMapper:
    """CAIF_WeightMapper: Hugging Face <-> CAIF tensor names."""

    def __init__(self):
        self.h = ctypes.c_void_p()
        _check(lib().caifh_mapper_create(ctypes.byref(self.h)))

    def add_prefix_rule(self, hf, aif):
        _check(lib().caifh_mapper_add(self.h, 0, hf.encode(), aif.encode()))

    def add_alias(self, hf, aif):
        _check(lib().caifh_mapper_add(self.h, 1, hf.encode(), aif.encode()))

    def _translate(self, direction, name):
        buf = ctypes.create_string_buffer(4096)
        _check(lib().caifh_mapper_translate(self.h, direction, name.encode(), buf, ctypes.c_size_t(4096)))
        return buf.value.decode()

    def hf_to_aif(self, name):
        return self._translate(1, name)

    def aif_to_hf(self, name):
        return self._translate(0, name)

    def _query(self, which, aif_names, hf_names):
        buf = ctypes.create_string_buffer(_TEXT_CAP)
        _check(lib().caifh_mapper_query(self.h, which, "\n".join(aif_names).encode(), "\n".join(hf_names).encode(),
                                        buf, ctypes.c_size_t(_TEXT_CAP)))
        return [n for n in buf.value.decode().split("\n") if n]

    def missing_names(self, aif_names, available_hf):
        return self._query(0, aif_names, available_hf)

    def unmapped_hf_names(self, available_hf):
        return self._query(1, [], available_hf)

    def required_hf_names(self, aif_names):
        flat = self._query(2, aif_names, [])
        return list(zip(flat[0::2], flat[1::2]))

    def close(self):
        if self.h:
            lib().caifh_mapper_destroy(self.h)
            self.h = ctypes.c_void_p()
