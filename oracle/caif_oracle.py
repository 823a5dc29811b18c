"""CPU oracle for the quantized frozen-linear path (numpy + the C restatement).

TEST INFRASTRUCTURE ONLY.  The shipped library never imports this module; it is
the checker for the tests and the smoke run, and the CPU baseline of the
benchmark.  Integer and bit-level work is done by ``caif_oracle.c``; the layer
dataflow (which tensor is rounded to which dtype where) is restated here with
numpy, citing the reference lines it follows.

dtype codes follow the reference's ``CAIF_DataType_e``
(include/caif/caif_data_type.h:32-48): 0 fp32, 2 fp16, 3 bf16, 4 int4, 5 int8.
"""
import ctypes
import os

import numpy as np

F32, F16, BF16, I4, I8 = 0, 2, 3, 4, 5
PER_TENSOR, PER_CHANNEL = 0, 1

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "_build", "libcaif_oracle.so")
        if not os.path.exists(path):
            import importlib.util

            spec = importlib.util.spec_from_file_location("_oracle_build", os.path.join(_HERE, "build.py"))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            mod.build_oracle()
        _LIB = ctypes.CDLL(path)
        _LIB.orc_f32_to_f16.restype = ctypes.c_uint16
        _LIB.orc_f32_to_f16.argtypes = [ctypes.c_float]
        _LIB.orc_f16_to_f32.restype = ctypes.c_float
        _LIB.orc_f16_to_f32.argtypes = [ctypes.c_uint16]
        _LIB.orc_build_dispatch_map.restype = ctypes.c_int32
        _LIB.orc_num_threads.restype = ctypes.c_int
    return _LIB


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def num_threads():
    return int(lib().orc_num_threads())


# --------------------------------------------------------------------------
# conversions
# --------------------------------------------------------------------------
def f32_to_f16_bits(x):
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_f16_array(_p(x), _p(y), ctypes.c_int64(x.size))
    return y


def f32_to_bf16_bits(x):
    x = _c(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().orc_f32_to_bf16_array(_p(x), _p(y), ctypes.c_int64(x.size))
    return y


def f16_bits_to_f32(b):
    b = _c(b, np.uint16)
    y = np.empty(b.shape, np.float32)
    lib().orc_f16_to_f32_array(_p(b), _p(y), ctypes.c_int64(b.size))
    return y


def bf16_bits_to_f32(b):
    b = _c(b, np.uint16)
    y = np.empty(b.shape, np.float32)
    lib().orc_bf16_to_f32_array(_p(b), _p(y), ctypes.c_int64(b.size))
    return y


def round_through(x, dtype):
    """fp32 values rounded (nearest even) through `dtype` and back."""
    y = np.array(x, dtype=np.float32, copy=True, order="C")
    if dtype in (F16, BF16):
        lib().orc_round_through(_p(y), ctypes.c_int64(y.size), ctypes.c_int(dtype))
    return y


# --------------------------------------------------------------------------
# quantize / dequantize
# --------------------------------------------------------------------------
def quantize_int8_per_tensor(x):
    x = _c(x, np.float32)
    q = np.zeros(x.shape, np.int8)
    s = np.zeros(1, np.float32)
    lib().orc_quantize_int8_per_tensor(_p(x), ctypes.c_int64(x.size), _p(q), _p(s))
    return q, s


def quantize_int8_per_channel(x):
    x = _c(x, np.float32)
    rows, cols = x.shape
    q = np.zeros(x.shape, np.int8)
    s = np.zeros(cols, np.float32)
    lib().orc_quantize_int8_per_channel(_p(x), ctypes.c_int(rows), ctypes.c_int(cols), _p(q), _p(s))
    return q, s


def quantize_int4(x, group=128):
    x = _c(x, np.float32)
    n = x.size
    packed = np.zeros((n + 1) // 2, np.uint8)
    scales = np.zeros((n + group - 1) // group, np.uint16)
    lib().orc_quantize_int4(_p(x), ctypes.c_int64(n), ctypes.c_int(group), _p(packed), _p(scales))
    return packed, scales


def dequantize_int8_per_tensor(q, s):
    q = _c(q, np.int8)
    s = _c(s, np.float32)
    out = np.empty(q.shape, np.float32)
    lib().orc_dequantize_int8_per_tensor(_p(q), ctypes.c_int64(q.size), _p(s), _p(out))
    return out


def dequantize_int8_per_channel(q, s):
    q = _c(q, np.int8)
    s = _c(s, np.float32)
    rows, cols = q.shape
    out = np.empty(q.shape, np.float32)
    lib().orc_dequantize_int8_per_channel(_p(q), ctypes.c_int(rows), ctypes.c_int(cols), _p(s), _p(out))
    return out


def dequantize_int4(packed, scales, n, group=128):
    packed = _c(packed, np.uint8)
    scales = _c(scales, np.uint16)
    out = np.empty(n, np.float32)
    lib().orc_dequantize_int4(_p(packed), _p(scales), ctypes.c_int64(n), ctypes.c_int(group), _p(out))
    return out


def cast_f32_to_int8(x):
    x = _c(x, np.float32)
    q = np.empty(x.shape, np.int8)
    lib().orc_cast_f32_to_int8(_p(x), ctypes.c_int64(x.size), _p(q))
    return q


# --------------------------------------------------------------------------
# frozen linear
# --------------------------------------------------------------------------
def weight_to_compute(codes, scales, storage, in_dim, out_dim, compute=F32, scheme=PER_TENSOR, group=128):
    """CAIF_DeviceFrozenLinear::ConvertToComputeDtype
    (src/caif_device_frozen_linear.cpp:288-378): the [out,in] fp32 matrix the
    GEMM sees, rounded through `compute`."""
    codes = np.ascontiguousarray(codes)
    w = np.empty((out_dim, in_dim), np.float32)
    sp = ctypes.c_void_p(None)
    if scales is not None:
        scales = np.ascontiguousarray(scales)
        sp = _p(scales)
    rc = lib().orc_weight_to_compute(_p(codes), sp, ctypes.c_int(storage), ctypes.c_int(scheme), ctypes.c_int(group),
                                     ctypes.c_int(in_dim), ctypes.c_int(out_dim), ctypes.c_int(compute), _p(w))
    if rc != 0:
        raise ValueError("orc_weight_to_compute failed: %d" % rc)
    return w


def gemm_nt(x, w, exact=True):
    """Y = X . W^T with fp32 operands.  exact=True accumulates in fp64 (C
    loop); exact=False is numpy's fp32 matmul, i.e. OpenBLAS sgemm -- the same
    routine the reference's host backend calls (src/caif_host_gemm.cpp:52)."""
    x = _c(x, np.float32)
    w = _c(w, np.float32)
    if not exact:
        return x @ w.T
    m, k = x.shape
    n = w.shape[0]
    y = np.empty((m, n), np.float32)
    lib().orc_gemm_nt(_p(x), _p(w), _p(y), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k))
    return y


def gemm_nn(a, b, exact=True):
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    if not exact:
        return a @ b
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    lib().orc_gemm_nn(_p(a), _p(b), _p(c), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k))
    return c


def gemm_tn(a, b, exact=True):
    """C[m,n] = A[k,m]^T . B[k,n]"""
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    if not exact:
        return a.T @ b
    k, m = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    lib().orc_gemm_tn(_p(a), _p(b), _p(c), ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(k))
    return c


def frozen_linear_forward(x, w_compute, compute=F32, exact=True):
    """CAIF_DeviceFrozenLinear::ForwardImpl
    (src/caif_device_frozen_linear.cpp:381-524): X is cast to the compute
    dtype, Y = X . W^T with fp32 accumulation, Y is fp32."""
    x2 = round_through(np.asarray(x, np.float32).reshape(-1, w_compute.shape[1]), compute)
    return gemm_nt(x2, w_compute, exact)


def frozen_linear_backward(dy, w_compute, compute=F32, exact=True):
    """CAIF_DeviceFrozenLinear::BackwardImpl
    (src/caif_device_frozen_linear.cpp:526-660): dX = dY . W, fp32 out."""
    g = round_through(np.asarray(dy, np.float32).reshape(-1, w_compute.shape[0]), compute)
    return gemm_nn(g, w_compute, exact)


# --------------------------------------------------------------------------
# LoRA adapter: src/caif_device_lora_adapter.cpp:119-281.  Every intermediate
# is materialised at the storage dtype `sd`; GEMM operands are at `sd` and
# accumulate in fp32.
# --------------------------------------------------------------------------
def lora_forward(x, base_out, a, b, alpha, sd=F32, exact=True):
    rank = a.shape[0]
    x2 = round_through(np.asarray(x, np.float32).reshape(-1, a.shape[1]), sd)
    a = round_through(a, sd)
    b = round_through(b, sd)
    hidden = round_through(gemm_nt(x2, a, exact), sd)                 # :162-163
    lora_out = round_through(gemm_nt(hidden, b, exact), sd)           # :172-173
    scale = np.float32(alpha) / np.float32(rank)
    lora_out = round_through(lora_out * scale, sd)                    # :176-177
    base = round_through(base_out, sd)                                # :189-198
    out = round_through(base + lora_out, sd)
    return out, hidden


def lora_backward(dy, x, hidden, dx_base, a, b, alpha, sd=F32, exact=True):
    rank = a.shape[0]
    g = round_through(np.asarray(dy, np.float32).reshape(-1, b.shape[0]), sd)
    x2 = round_through(np.asarray(x, np.float32).reshape(-1, a.shape[1]), sd)
    a = round_through(a, sd)
    b = round_through(b, sd)
    scale = np.float32(alpha) / np.float32(rank)
    gs = round_through(g * scale, sd)                                 # :235-236
    d_b = round_through(gemm_tn(gs, hidden, exact), sd)               # :240  [out, r]
    d_h = round_through(gemm_nn(gs, b, exact), sd)                    # :243-244 [n, r]
    d_a = round_through(gemm_tn(d_h, x2, exact), sd)                  # :248  [r, in]
    dx_lora = round_through(gemm_nn(d_h, a, exact), sd)               # :251-252
    dx = round_through(round_through(dx_base, sd) + dx_lora, sd)      # :267-276
    return dx, d_a, d_b


# --------------------------------------------------------------------------
# frozen SwiGLU expert: src/caif_device_moe_frozen_expert.cpp:91-332
# --------------------------------------------------------------------------
def silu(x):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    lib().orc_silu(_p(x), ctypes.c_int64(x.size), _p(y))
    return y


def silu_backward(grad, x):
    grad = _c(grad, np.float32)
    x = _c(x, np.float32)
    y = np.empty_like(x)
    lib().orc_silu_backward(_p(grad), _p(x), ctypes.c_int64(x.size), _p(y))
    return y


def frozen_expert_forward(x, wg, wu, wd, compute=F32, sd=F32, exact=True):
    """down( silu(gate(x)) * up(x) ); each frozen-linear output (fp32) is cast
    to the storage dtype before the elementwise step (:113-126).  wg=None is the
    non-gated form down( silu(up(x)) ) (:158-162); gate is then returned as None."""
    up = round_through(frozen_linear_forward(x, wu, compute, exact), sd)
    if wg is None:
        hid = round_through(silu(up), sd)
        out = round_through(frozen_linear_forward(hid, wd, compute, exact), sd)
        return out, None, up
    gate = round_through(frozen_linear_forward(x, wg, compute, exact), sd)
    act = round_through(silu(gate), sd)
    hid = round_through(act * up, sd)
    out = round_through(frozen_linear_forward(hid, wd, compute, exact), sd)
    return out, gate, up


def frozen_expert_backward(dy, gate, up, wg, wu, wd, compute=F32, sd=F32, exact=True):
    g_hidden = round_through(frozen_linear_backward(dy, wd, compute, exact), sd)
    if wg is None:
        # src/caif_device_moe_frozen_expert.cpp:318-331
        g_up = round_through(silu_backward(g_hidden, up), sd)
        return round_through(frozen_linear_backward(g_up, wu, compute, exact), sd)
    act = round_through(silu(gate), sd)
    g_up = round_through(g_hidden * act, sd)
    g_act = round_through(g_hidden * up, sd)
    g_gate = round_through(silu_backward(g_act, gate), sd)
    dx_up = round_through(frozen_linear_backward(g_up, wu, compute, exact), sd)
    dx_gate = round_through(frozen_linear_backward(g_gate, wg, compute, exact), sd)
    return round_through(dx_up + dx_gate, sd)


# --------------------------------------------------------------------------
# routing / dispatch
# --------------------------------------------------------------------------
def topk(probs, k):
    probs = _c(probs, np.float32)
    batch, dim = probs.shape
    idx = np.empty((batch, k), np.int32)
    val = np.empty((batch, k), np.float32)
    lib().orc_topk(_p(probs), ctypes.c_int(batch), ctypes.c_int(dim), ctypes.c_int(k), _p(idx), _p(val))
    return idx, val


def normalize_rows(x):
    x = _c(x, np.float32)
    batch, dim = x.shape
    out = np.empty_like(x)
    lib().orc_normalize_rows(_p(x), ctypes.c_int(batch), ctypes.c_int(dim), _p(out))
    return out


def router_softmax(logits, bias=None, dtype=F32):
    """Probabilities of CAIF_DeviceMoERouter::Route for SoftmaxTopK gating
    (src/caif_device_moe_router.cpp:233-303): optional AddBias (sum rounded through
    `dtype`), then the attention softmax kernel's operation order.  fp32 in, fp32 out
    (round the result through `dtype` for 16-bit storage)."""
    x = _c(logits, np.float32)
    rows, cols = x.shape
    out = np.empty_like(x)
    b = None if bias is None else _c(bias, np.float32)
    lib().orc_router_softmax(_p(x), None if b is None else _p(b), ctypes.c_int(rows), ctypes.c_int(cols),
                             ctypes.c_int(dtype), _p(out))
    return out


def router_backward(grad_w, probs, indices, balance_bias=None, z_lse_scaled=None, sigmoid_gate=False,
                    normalize=True, scaling=1.0, exact_jacobian=False, dtype=F32):
    """grad_logits and grad_topk of CAIF_DeviceMoERouter::BackwardRoutingAuxAware
    (src/caif_device_moe_router.cpp:529-733); inputs are fp32 arrays holding values already
    representable in `dtype`, intermediates are rounded through `dtype` as the reference stores them."""
    g = _c(grad_w, np.float32)
    p = _c(probs, np.float32)
    idx = _c(indices, np.int32)
    tokens, experts = p.shape
    top_k = idx.shape[1]
    bb = None if balance_bias is None else _c(balance_bias, np.float32)
    zl = None if z_lse_scaled is None else _c(z_lse_scaled, np.float32)
    grad_topk = np.empty((tokens, top_k), np.float32)
    grad_logits = np.empty((tokens, experts), np.float32)
    lib().orc_router_backward(_p(g), _p(p), _p(idx), None if bb is None else _p(bb), None if zl is None else _p(zl),
                              ctypes.c_int(tokens), ctypes.c_int(experts), ctypes.c_int(top_k),
                              ctypes.c_int(1 if sigmoid_gate else 0), ctypes.c_int(1 if normalize else 0),
                              ctypes.c_float(scaling), ctypes.c_int(1 if exact_jacobian else 0), ctypes.c_int(dtype),
                              _p(grad_topk), _p(grad_logits))
    return grad_logits, grad_topk


def moe_aux_losses(logits, probs, counts, top_k, balance_weight, z_weight, dtype=F32):
    """(losses[2], balance_bias, lse, z_lse_scaled) of CAIF_DeviceMoELayer's auxiliary losses
    (src/caif_device_moe_layer.cpp:792-835, 853-925)."""
    ref = probs if probs is not None else logits
    tokens, experts = ref.shape
    x = None if logits is None else _c(logits, np.float32)
    p = None if probs is None else _c(probs, np.float32)
    cnt = _c(counts, np.int32)
    losses = np.zeros(2, np.float32)
    bias = np.zeros(experts, np.float32)
    lse = np.zeros(tokens, np.float32)
    zls = np.zeros(tokens, np.float32)
    lib().orc_moe_aux_losses(None if x is None else _p(x), None if p is None else _p(p), _p(cnt),
                             ctypes.c_int(tokens), ctypes.c_int(experts), ctypes.c_int(top_k),
                             ctypes.c_float(balance_weight), ctypes.c_float(z_weight), ctypes.c_int(dtype),
                             _p(bias), _p(lse), _p(zls), _p(losses))
    return losses, bias, lse, zls


RMSNORM_FORM = 0   # how the reference build fuses dy * gamma - x_hat * sum_term (see orc_rmsnorm_backward)


def rmsnorm_forward(x, gamma, eps=1e-5, dtype=F32):
    """(y, rms) of the reference's RMSNorm forward kernel (src/caif_cuda_kernels_normalization.cu:46-119)."""
    x = _c(x, np.float32)
    g = _c(gamma, np.float32)
    rows, dim = x.shape
    y = np.empty_like(x)
    rms = np.empty(rows, np.float32)
    lib().orc_rmsnorm_forward(_p(x), _p(g), ctypes.c_int(rows), ctypes.c_int(dim), ctypes.c_float(eps),
                              ctypes.c_int(dtype), _p(y), _p(rms))
    return y, rms


def rmsnorm_backward(dy, x, gamma, rms, dtype=F32, form=None):
    """(dx, grad_gamma) of the reference's RMSNorm backward kernel (:129-203)."""
    dy = _c(dy, np.float32)
    x = _c(x, np.float32)
    g = _c(gamma, np.float32)
    r = _c(rms, np.float32)
    rows, dim = x.shape
    dx = np.empty_like(x)
    gg = np.empty(dim, np.float32)
    lib().orc_rmsnorm_backward(_p(dy), _p(x), _p(g), _p(r), ctypes.c_int(rows), ctypes.c_int(dim), ctypes.c_int(dtype),
                               ctypes.c_int(RMSNORM_FORM if form is None else form), _p(dx), _p(gg))
    return dx, gg


def build_dispatch_map(expert_indices, num_experts, capacity=0):
    idx = _c(expert_indices, np.int32)
    tokens, top_k = idx.shape
    dmap = np.empty((tokens, top_k), np.int32)
    offsets = np.empty(num_experts + 1, np.int32)
    total = lib().orc_build_dispatch_map(_p(idx), ctypes.c_int(tokens), ctypes.c_int(top_k),
                                         ctypes.c_int(num_experts), ctypes.c_int(capacity), _p(dmap), _p(offsets))
    return dmap, offsets, int(total)


def moe_dispatch(x, expert_indices, dispatch_map, expert_offsets, total_assigned):
    x = _c(x, np.float32)
    tokens, dim = x.shape
    top_k = expert_indices.shape[1]
    buf = np.zeros((total_assigned, dim), np.float32)
    lib().orc_moe_dispatch(_p(x), _p(_c(expert_indices, np.int32)), _p(_c(dispatch_map, np.int32)),
                           _p(_c(expert_offsets, np.int32)), ctypes.c_int(tokens), ctypes.c_int(dim),
                           ctypes.c_int(top_k), _p(buf))
    return buf


def moe_combine(buf, expert_indices, weights, dispatch_map, expert_offsets, num_tokens):
    buf = _c(buf, np.float32)
    dim = buf.shape[1]
    top_k = expert_indices.shape[1]
    out = np.empty((num_tokens, dim), np.float32)
    lib().orc_moe_combine(_p(buf), _p(_c(expert_indices, np.int32)), _p(_c(weights, np.float32)),
                          _p(_c(dispatch_map, np.int32)), _p(_c(expert_offsets, np.int32)),
                          ctypes.c_int(num_tokens), ctypes.c_int(dim), ctypes.c_int(top_k), _p(out))
    return out


def moe_combine_bwd_grad_expert(grad_output, expert_indices, weights, dispatch_map, expert_offsets, total):
    """fp32 values of the packed-buffer gradient (unassigned slots stay zero); round to storage outside."""
    g = _c(grad_output, np.float32)
    tokens, dim = g.shape
    top_k = expert_indices.shape[1]
    out = np.zeros((total, dim), np.float32)
    lib().orc_moe_combine_bwd_grad_expert(_p(g), _p(_c(expert_indices, np.int32)), _p(_c(weights, np.float32)),
                                          _p(_c(dispatch_map, np.int32)), _p(_c(expert_offsets, np.int32)),
                                          ctypes.c_int(tokens), ctypes.c_int(dim), ctypes.c_int(top_k), _p(out))
    return out


def moe_combine_bwd_grad_weights(grad_output, buf, expert_indices, dispatch_map, expert_offsets):
    g = _c(grad_output, np.float32)
    tokens, dim = g.shape
    top_k = expert_indices.shape[1]
    out = np.empty((tokens, top_k), np.float32)
    lib().orc_moe_combine_bwd_grad_weights(_p(g), _p(_c(buf, np.float32)), _p(_c(expert_indices, np.int32)),
                                           _p(_c(dispatch_map, np.int32)), _p(_c(expert_offsets, np.int32)),
                                           ctypes.c_int(tokens), ctypes.c_int(dim), ctypes.c_int(top_k), _p(out))
    return out


def moe_dispatch_bwd(grad_buf, expert_indices, dispatch_map, expert_offsets, num_tokens):
    gb = _c(grad_buf, np.float32)
    dim = gb.shape[1]
    top_k = expert_indices.shape[1]
    out = np.empty((num_tokens, dim), np.float32)
    lib().orc_moe_dispatch_bwd(_p(gb), _p(_c(expert_indices, np.int32)), _p(_c(dispatch_map, np.int32)),
                               _p(_c(expert_offsets, np.int32)), ctypes.c_int(num_tokens), ctypes.c_int(dim),
                               ctypes.c_int(top_k), _p(out))
    return out
