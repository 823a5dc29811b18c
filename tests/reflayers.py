"""ctypes binding of oracle/_ref/libcaif_ref_layers.so: the reference's own layer classes
(CAIF_DeviceFrozenLinear, CAIF_DeviceLoRAAdapter, CAIF_DeviceMoEFrozenExpert), every translation unit
compiled unmodified by oracle/build_ref_layers.py.  Test infrastructure: used to capture golden vectors
from the executing reference and to time its device path as a comparator.  All buffers are numpy arrays
on the host; the reference uploads and downloads them itself."""
import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "oracle", "_ref", "libcaif_ref_layers.so")

# CAIF_DataType_e
F32, F16, BF16, I4, I8, U8 = 0, 2, 3, 4, 5, 9

_lib = None


def available():
    return os.path.exists(PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(PATH)
        _lib.refl_last_error.restype = ctypes.c_char_p
    return _lib


def _check(rc):
    if rc != 0:
        raise RuntimeError("reference layer call failed: %s" % lib().refl_last_error().decode())


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


def set_accuracy(on=True):
    _check(lib().refl_set_accuracy(int(on)))


def u8_code():
    """CAIF_DataType_e::UInt8, read from the enum's order in include/caif/caif_data_type.h."""
    return U8


_ELEM = {F32: 4, F16: 2, BF16: 2}


class Layer:
    def __init__(self, handle, in_dim, out_dim):
        self.h = handle
        self.in_dim, self.out_dim = in_dim, out_dim

    def _run(self, fn, x, dtype, last_dim, out_dim, *extra):
        x = np.ascontiguousarray(x)
        rows = x.size * x.itemsize // (_ELEM[dtype] * last_dim)
        cap = rows * out_dim * 4
        out = np.empty(cap, np.uint8)
        out_dtype, out_bytes = ctypes.c_int(), ctypes.c_size_t()
        _check(fn(self.h, _p(x), dtype, ctypes.c_uint32(rows), ctypes.c_uint32(last_dim), *extra, _p(out),
                  ctypes.c_size_t(cap), ctypes.byref(out_dtype), ctypes.byref(out_bytes)))
        raw = out[:out_bytes.value]
        return _to_f32(raw, out_dtype.value).reshape(rows, out_dim), out_dtype.value

    def forward(self, x, dtype, training=True):
        return self._run(lib().refl_forward, x, dtype, self.in_dim, self.out_dim, int(training))

    def backward(self, dy, dtype):
        return self._run(lib().refl_backward, dy, dtype, self.out_dim, self.in_dim)

    def gradient(self, index_from_end, shape, dtype):
        cap = int(np.prod(shape)) * 4
        out = np.empty(cap, np.uint8)
        nbytes = ctypes.c_size_t()
        _check(lib().refl_gradient(self.h, ctypes.c_uint32(index_from_end), _p(out), ctypes.c_size_t(cap),
                                   ctypes.byref(nbytes)))
        return _to_f32(out[:nbytes.value], dtype).reshape(shape)

    def time(self, x, x_dtype, dy, dy_dtype, backward, warm, iters):
        x = np.ascontiguousarray(x)
        rows = x.size * x.itemsize // (_ELEM[x_dtype] * self.in_dim)
        ms = ctypes.c_float()
        _check(lib().refl_time(self.h, _p(x), x_dtype, _p(np.ascontiguousarray(dy)) if dy is not None else None,
                               dy_dtype, ctypes.c_uint32(rows), ctypes.c_uint32(self.in_dim),
                               ctypes.c_uint32(self.out_dim), int(backward), int(warm), int(iters), ctypes.byref(ms)))
        return ms.value

    def close(self):
        if self.h:
            lib().refl_destroy(self.h)
            self.h = None


def _to_f32(raw, dtype):
    if dtype == F32:
        return raw.view(np.float32).copy()
    bits = raw.view(np.uint16)
    if dtype == BF16:
        return (bits.astype(np.uint32) << 16).view(np.float32)
    return bits.view(np.float16).astype(np.float32)


def to_raw(x_f32, dtype):
    """fp32 values (already representable in `dtype`) as the raw array the reference uploads."""
    x = np.ascontiguousarray(x_f32, np.float32)
    if dtype == F32:
        return x
    if dtype == BF16:
        return (x.view(np.uint32) >> 16).astype(np.uint16)
    return x.astype(np.float16).view(np.uint16)


def frozen_linear(in_dim, out_dim, storage, compute, codes, scales, group=128, cache_fp32=True, scheme=0):
    """codes: packed uint8 (int4), int8, or raw float array; scales: fp16 bits (uint16) / fp32 / None."""
    codes = np.ascontiguousarray(codes)
    if storage == I4:
        codes_dtype = U8
    elif storage == I8:
        codes_dtype = I8
    else:
        codes_dtype = storage
    h = ctypes.c_void_p()
    sc = np.ascontiguousarray(scales) if scales is not None else None
    _check(lib().refl_frozen_create(ctypes.c_uint32(in_dim), ctypes.c_uint32(out_dim), storage, compute,
                                    ctypes.c_uint32(group), int(cache_fp32), scheme, _p(codes), codes_dtype,
                                    ctypes.c_uint32(codes.size), _p(sc),
                                    ctypes.c_size_t(sc.nbytes if sc is not None else 0), ctypes.byref(h)))
    return Layer(h, in_dim, out_dim)


def lora_wrap(base, rank, alpha, storage, compute, a_raw, b_raw):
    h = ctypes.c_void_p()
    _check(lib().refl_lora_wrap(base.h, ctypes.c_uint32(rank), ctypes.c_float(alpha), ctypes.c_uint32(base.in_dim),
                                ctypes.c_uint32(base.out_dim), storage, compute, _p(np.ascontiguousarray(a_raw)),
                                _p(np.ascontiguousarray(b_raw)), ctypes.byref(h)))
    base.h = None
    return Layer(h, base.in_dim, base.out_dim)


def frozen_expert(gate, up, down, input_dim, hidden_dim, storage, compute):
    h = ctypes.c_void_p()
    _check(lib().refl_expert_create(gate.h if gate is not None else None, up.h, down.h, ctypes.c_uint32(input_dim),
                                    ctypes.c_uint32(hidden_dim), int(gate is not None), storage, compute,
                                    ctypes.byref(h)))
    for layer in (gate, up, down):
        if layer is not None:
            layer.h = None
    return Layer(h, input_dim, input_dim)


# ---- the reference's SafeTensors reader / writer and name mapper (oracle/ref_layers_shim.cpp) ----
_CAP = 1 << 22


def _strings(items):
    arr = (ctypes.c_char_p * max(1, len(items)))()
    for i, s in enumerate(items):
        arr[i] = s.encode()
    return arr


def st_tensor_infos(path):
    """{name: (dtype, shape, begin, end)} from CAIF_SafeTensorsFormat::TensorInfos (no device involved)."""
    buf = ctypes.create_string_buffer(_CAP)
    _check(lib().refl_st_tensor_infos(path.encode(), buf, ctypes.c_size_t(_CAP)))
    out = {}
    for line in buf.value.decode().split("\n"):
        if line:
            name, dtype, shape, begin, end = line.split("\t")
            out[name] = (dtype, [int(d) for d in shape.split(",") if d], int(begin), int(end))
    return out


def st_metadata(path):
    buf = ctypes.create_string_buffer(_CAP)
    _check(lib().refl_st_metadata(path.encode(), buf, ctypes.c_size_t(_CAP)))
    flat = buf.value.decode().split("\n")[:-1]
    return dict(zip(flat[0::2], flat[1::2]))


def st_save(path, tensors, metadata=None):
    """tensors: list of (name, CAIF_DataType_e value, shape, bytes); CAIF_SafeTensorsFormat::Save (needs a GPU)."""
    metadata = metadata or {}
    held = [bytes(t[3]) for t in tensors]
    data = (ctypes.c_void_p * max(1, len(tensors)))()
    for i, b in enumerate(held):
        data[i] = ctypes.cast(ctypes.c_char_p(b), ctypes.c_void_p)
    flat = [d for t in tensors for d in t[2]]
    ranks = (ctypes.c_uint32 * max(1, len(tensors)))(*[len(t[2]) for t in tensors])
    shapes = (ctypes.c_uint32 * max(1, len(flat)))(*flat)
    codes = (ctypes.c_int * max(1, len(tensors)))(*[int(t[1]) for t in tensors])
    keys = sorted(metadata)
    _check(lib().refl_st_save(path.encode(), ctypes.c_uint32(len(tensors)), _strings([t[0] for t in tensors]), codes,
                              ranks, shapes, data, ctypes.c_uint32(len(keys)), _strings(keys),
                              _strings([metadata[k] for k in keys])))


def st_load(path, name, capacity, from_directory=False):
    """(dtype code, bytes) of one tensor through CAIF_SafeTensorsFormat::Load / LoadTensorByName (needs a GPU)."""
    buf = ctypes.create_string_buffer(max(1, capacity))
    dtype, nbytes = ctypes.c_int(), ctypes.c_size_t()
    _check(lib().refl_st_load(path.encode(), int(from_directory), name.encode(), buf, ctypes.c_size_t(capacity),
                              ctypes.byref(dtype), ctypes.byref(nbytes)))
    return dtype.value, buf.raw[:nbytes.value]


class Mapper:
    def __init__(self):
        self.h = ctypes.c_void_p()
        _check(lib().refl_mapper_create(ctypes.byref(self.h)))

    def add(self, alias, hf, aif):
        _check(lib().refl_mapper_add(self.h, int(alias), hf.encode(), aif.encode()))

    def translate(self, hf_to_aif, name):
        buf = ctypes.create_string_buffer(4096)
        _check(lib().refl_mapper_translate(self.h, int(hf_to_aif), name.encode(), buf, ctypes.c_size_t(4096)))
        return buf.value.decode()

    def query(self, which, aif_names, hf_names):
        buf = ctypes.create_string_buffer(_CAP)
        _check(lib().refl_mapper_query(self.h, which, "\n".join(aif_names).encode(), "\n".join(hf_names).encode(),
                                       buf, ctypes.c_size_t(_CAP)))
        return [n for n in buf.value.decode().split("\n") if n]

    def close(self):
        lib().refl_mapper_destroy(self.h)


def moe_layer(experts, input_dim, hidden_dim, top_k, storage, compute, router_w_raw, router_b_raw=None,
              sigmoid_gate=False, norm_topk=True, scaling=1.0, balance_weight=0.0, z_weight=0.0):
    """The reference's CAIF_DeviceMoELayer over frozen experts (handles consumed): no shared experts, no noise,
    no token dropping; router weight [input_dim, num_experts] (and bias) set from raw bytes in `storage`."""
    h = ctypes.c_void_p()
    arr = (ctypes.c_void_p * len(experts))(*[e.h for e in experts])
    w = np.ascontiguousarray(router_w_raw)
    b = np.ascontiguousarray(router_b_raw) if router_b_raw is not None else None
    _check(lib().refl_moe_layer_create(arr, ctypes.c_uint32(len(experts)), ctypes.c_uint32(input_dim),
                                       ctypes.c_uint32(hidden_dim), ctypes.c_uint32(top_k), storage, compute, _p(w),
                                       _p(b), int(sigmoid_gate), int(norm_topk), ctypes.c_float(scaling),
                                       ctypes.c_float(balance_weight), ctypes.c_float(z_weight), ctypes.byref(h)))
    for e in experts:
        e.h = None
    return Layer(h, input_dim, input_dim)


def moe_layer_losses(layer):
    b, z = ctypes.c_float(), ctypes.c_float()
    _check(lib().refl_moe_layer_losses(layer.h, ctypes.byref(b), ctypes.byref(z)))
    return b.value, z.value
