"""Helpers shared by the GPU parity tests (test infrastructure)."""
import numpy as np
import torch

import caif_oracle as orc
from caif_b200 import native as nv

TORCH_DTYPE = {orc.F32: torch.float32, orc.F16: torch.float16, orc.BF16: torch.bfloat16}


def dev():
    return torch.device("cuda:0")


def to_dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev())
    if dtype is not None:
        t = t.to(dtype)
    return t.contiguous()


def f16_bits_to_dev(bits):
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).to(dev()).view(torch.float16)


def max_rel_err(got, want):
    """max |got - want| / max |want| -- the reference tests' rel-to-max measure
    (tests/test_device_frozen_linear.cpp:1080-1310)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    denom = max(float(np.max(np.abs(want))), 1e-30)
    return float(np.max(np.abs(got - want))) / denom


def make_weight(rng, out_dim, in_dim, storage, scheme=orc.PER_TENSOR, group=128, std=0.02, with_scales=True):
    """Seeded N(0, std) weight quantized by the ORACLE; returns (native Weight, oracle codes, oracle scales)."""
    w = (rng.standard_normal((out_dim, in_dim)) * std).astype(np.float32)
    if storage == orc.F32:
        codes, scales = w, None
        t_codes = to_dev(codes)
        t_scales = None
    elif storage == orc.F16:
        codes, scales = orc.f32_to_f16_bits(w), None
        t_codes = f16_bits_to_dev(codes)
        t_scales = None
    elif storage == orc.BF16:
        codes, scales = orc.f32_to_bf16_bits(w), None
        t_codes = torch.from_numpy(codes.view(np.int16)).to(dev()).view(torch.bfloat16)
        t_scales = None
    elif storage == orc.I8:
        if not with_scales:
            codes, scales = orc.cast_f32_to_int8(w * 3000.0), None
            t_scales = None
        elif scheme == orc.PER_TENSOR:
            codes, scales = orc.quantize_int8_per_tensor(w)
            t_scales = to_dev(scales)
        else:
            # the layer hands the [out,in] buffer to the per-channel kernels as rows=in, cols=out
            codes, scales = orc.quantize_int8_per_channel(w.reshape(in_dim, out_dim))
            codes = codes.reshape(out_dim, in_dim)
            t_scales = to_dev(scales)
        t_codes = to_dev(codes)
    elif storage == orc.I4:
        codes, scales = orc.quantize_int4(w, group)
        t_codes = to_dev(codes)
        t_scales = f16_bits_to_dev(scales)
    else:
        raise ValueError(storage)
    weight = nv.Weight(t_codes, storage, in_dim, out_dim, t_scales, scheme, group)
    return weight, codes, scales


def act(rng, m, k, dtype_code):
    """N(0,1) activations already rounded to the storage dtype; returns (fp32 numpy, device tensor)."""
    x = orc.round_through(rng.standard_normal((m, k)).astype(np.float32), dtype_code)
    return x, to_dev(x, TORCH_DTYPE[dtype_code])
