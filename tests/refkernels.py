"""ctypes binding of oracle/_ref/libcaif_ref_kernels.so: the reference's own
quantize and MoE kernels, compiled unmodified (oracle/build.py).  Test
infrastructure: used to pin the oracle and the product kernels against what the
reference itself computes on the GPU."""
import ctypes
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PATH = os.path.join(ROOT, "oracle", "_ref", "libcaif_ref_kernels.so")

_lib = None


def available():
    return os.path.exists(PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(PATH)
    return _lib


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _s():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def quantize_int8_per_tensor(x):
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(1, dtype=torch.float32, device=x.device)
    lib().ref_quantize_int8_per_tensor(_p(x), _p(q), _p(s), ctypes.c_int64(x.numel()), _s())
    return q, s


def dequantize_int8_per_tensor(q, s):
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    lib().ref_dequantize_int8_per_tensor(_p(q), _p(out), _p(s), ctypes.c_int64(q.numel()), _s())
    return out


def quantize_int8_per_channel(x):
    rows, cols = x.shape
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    s = torch.empty(cols, dtype=torch.float32, device=x.device)
    lib().ref_quantize_int8_per_channel(_p(x), _p(q), _p(s), ctypes.c_int(rows), ctypes.c_int(cols), _s())
    return q, s


def dequantize_int8_per_channel(q, s):
    rows, cols = q.shape
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    lib().ref_dequantize_int8_per_channel(_p(q), _p(out), _p(s), ctypes.c_int(rows), ctypes.c_int(cols), _s())
    return out


def quantize_int4(x, group=128):
    n = x.numel()
    packed = torch.zeros((n + 1) // 2, dtype=torch.uint8, device=x.device)
    scales = torch.zeros((n + group - 1) // group, dtype=torch.float16, device=x.device)
    lib().ref_quantize_int4(_p(x), _p(packed), _p(scales), ctypes.c_int64(n), ctypes.c_int(group), _s())
    return packed, scales


def dequantize_int4(packed, scales, n, group=128):
    out = torch.empty(n, dtype=torch.float32, device=packed.device)
    lib().ref_dequantize_int4(_p(packed), _p(scales), _p(out), ctypes.c_int64(n), ctypes.c_int(group), _s())
    return out


def topk(probs, k):
    batch, dim = probs.shape
    idx = torch.empty((batch, k), dtype=torch.int32, device=probs.device)
    val = torch.empty((batch, k), dtype=torch.float32, device=probs.device)
    lib().ref_topk_f32(_p(probs), _p(idx), _p(val), ctypes.c_int(batch), ctypes.c_int(dim), ctypes.c_int(k), _s())
    return idx, val


def normalize_rows(x):
    batch, dim = x.shape
    out = torch.empty_like(x)
    lib().ref_normalize_rows_f32(_p(x), _p(out), ctypes.c_int(batch), ctypes.c_int(dim), _s())
    return out


def moe_dispatch(x, idx, dmap, off, total):
    tokens, dim = x.shape
    buf = torch.zeros((total, dim), dtype=torch.float32, device=x.device)
    lib().ref_moe_dispatch_f32(_p(x), _p(buf), ctypes.c_int(tokens), ctypes.c_int(dim), ctypes.c_int(idx.shape[1]),
                               _p(idx), _p(dmap), _p(off), _s())
    return buf


def moe_combine(buf, idx, weights, dmap, off, tokens):
    dim = buf.shape[1]
    out = torch.empty((tokens, dim), dtype=torch.float32, device=buf.device)
    lib().ref_moe_combine_f32(_p(buf), _p(out), ctypes.c_int(tokens), ctypes.c_int(dim), ctypes.c_int(idx.shape[1]),
                              _p(idx), _p(weights), _p(dmap), _p(off), _s())
    return out


def moe_combine_bwd_grad_expert(grad_out, idx, weights, dmap, off, total):
    tokens, dim = grad_out.shape
    gbuf = torch.zeros((total, dim), dtype=torch.float32, device=grad_out.device)
    lib().ref_moe_combine_bwd_grad_expert_f32(_p(grad_out), _p(gbuf), ctypes.c_int(tokens), ctypes.c_int(dim),
                                              ctypes.c_int(idx.shape[1]), _p(idx), _p(weights), _p(dmap), _p(off), _s())
    return gbuf


def moe_combine_bwd_grad_weights(grad_out, buf, idx, dmap, off):
    tokens, dim = grad_out.shape
    gw = torch.empty((tokens, idx.shape[1]), dtype=torch.float32, device=grad_out.device)
    lib().ref_moe_combine_bwd_grad_weights_f32(_p(grad_out), _p(buf), _p(gw), ctypes.c_int(tokens), ctypes.c_int(dim),
                                               ctypes.c_int(idx.shape[1]), _p(idx), _p(dmap), _p(off), _s())
    return gw


def moe_dispatch_bwd(gbuf, idx, dmap, off, tokens):
    dim = gbuf.shape[1]
    gin = torch.empty((tokens, dim), dtype=torch.float32, device=gbuf.device)
    lib().ref_moe_dispatch_bwd_f32(_p(gbuf), _p(gin), ctypes.c_int(tokens), ctypes.c_int(dim),
                                   ctypes.c_int(idx.shape[1]), _p(idx), _p(dmap), _p(off), _s())
    return gin


def softmax(x):
    """launch_attention_softmax on fp32 or bf16 rows (the router's score function)."""
    rows, cols = x.shape
    out = torch.empty_like(x)
    fn = lib().ref_softmax_f32 if x.dtype == torch.float32 else lib().ref_softmax_bf16
    fn(_p(x), _p(out), ctypes.c_int(rows), ctypes.c_int(cols), _s())
    return out


def bias_add(x, bias):
    rows, cols = x.shape
    out = torch.empty_like(x)
    fn = lib().ref_bias_add_f32 if x.dtype == torch.float32 else lib().ref_bias_add_bf16
    fn(_p(x), _p(bias), _p(out), ctypes.c_int(rows), ctypes.c_int(cols), _s())
    return out


def scale_bf16(x, factor):
    out = torch.empty_like(x)
    lib().ref_scale_bf16(_p(x), _p(out), ctypes.c_float(factor), ctypes.c_int64(x.numel()), _s())
    return out


def fused_adam(param, grad, m, v, lr, beta1, beta2, epsilon, weight_decay, bc1, bc2):
    """The reference's launch_fused_adam (src/caif_cuda_kernels_optimizers.cu:217-245) in place on param, m, v."""
    fn = lib().ref_fused_adam_f32 if param.dtype == torch.float32 else lib().ref_fused_adam_bf16
    fn(_p(param), _p(grad), _p(m), _p(v), ctypes.c_float(lr), ctypes.c_float(beta1), ctypes.c_float(beta2),
       ctypes.c_float(epsilon), ctypes.c_float(weight_decay), ctypes.c_float(bc1), ctypes.c_float(bc2),
       ctypes.c_int64(param.numel()), _s())


def _typed(name, t):
    return getattr(lib(), name + ("_f32" if t.dtype == torch.float32 else "_bf16"))


def sigmoid(x):
    out = torch.empty_like(x)
    _typed("ref_sigmoid", x)(_p(x), _p(out), ctypes.c_int64(x.numel()), _s())
    return out


def group_mask_(sel, n_group, topk_group):
    """launch_moe_group_mask, in place on the [tokens, experts] selection scores."""
    tokens, experts = sel.shape
    _typed("ref_group_mask", sel)(_p(sel), ctypes.c_int(tokens), ctypes.c_int(experts), ctypes.c_int(n_group),
                                  ctypes.c_int(topk_group), _s())
    return sel


def topk_any(x, k):
    batch, dim = x.shape
    idx = torch.empty((batch, k), dtype=torch.int32, device=x.device)
    val = torch.empty((batch, k), dtype=x.dtype, device=x.device)
    _typed("ref_topk", x)(_p(x), _p(idx), _p(val), ctypes.c_int(batch), ctypes.c_int(dim), ctypes.c_int(k), _s())
    return idx, val


def gather_topk(scores, idx):
    tokens, experts = scores.shape
    k = idx.shape[1]
    out = torch.empty((tokens, k), dtype=scores.dtype, device=scores.device)
    _typed("ref_gather_topk", scores)(_p(scores), _p(idx), _p(out), ctypes.c_int(tokens), ctypes.c_int(experts),
                                      ctypes.c_int(k), _s())
    return out


def _pn(t):
    return ctypes.c_void_p(None) if t is None else _p(t)


def router_backward(grad_w, probs, idx, balance_bias=None, z_lse_scaled=None, sigmoid_gate=False, normalize=True,
                    scaling=1.0):
    """The launches of CAIF_DeviceMoERouter::BackwardRoutingAuxAware up to grad_logits, in its order and with
    its operand order (oracle/ref_shim.cu): returns (grad_logits, grad_topk)."""
    tokens, experts = probs.shape
    k = idx.shape[1]
    grad_topk = torch.empty_like(grad_w)
    grad_probs = torch.empty_like(probs)
    grad_logits = torch.empty_like(probs)
    _typed("ref_router_backward", probs)(_p(grad_w), _p(probs), _p(idx), _pn(balance_bias), _pn(z_lse_scaled),
                                         _p(grad_topk), _p(grad_probs), _p(grad_logits), ctypes.c_int(tokens),
                                         ctypes.c_int(experts), ctypes.c_int(k), ctypes.c_int(1 if sigmoid_gate else 0),
                                         ctypes.c_int(1 if normalize else 0), ctypes.c_float(scaling), _s())
    return grad_logits, grad_topk


def logsumexp(x):
    """launch_logsumexp: fp32 result per row."""
    rows, cols = x.shape
    out = torch.empty(rows, dtype=torch.float32, device=x.device)
    _typed("ref_logsumexp", x)(_p(x), _p(out), ctypes.c_int(rows), ctypes.c_int(cols), _s())
    return out


def sum_axis0(x):
    rows, cols = x.shape
    out = torch.empty(cols, dtype=torch.float32, device=x.device)
    _typed("ref_sum_axis0", x)(_p(x), _p(out), ctypes.c_int(rows), ctypes.c_int(cols), _s())
    return out


def bias_update_(bias, counts, rate):
    """launch_moe_bias_update, in place."""
    _typed("ref_bias_update", bias)(_p(bias), _p(counts), ctypes.c_int(bias.numel()), ctypes.c_float(rate), _s())
    return bias


def rmsnorm_fwd(x, gamma, eps):
    rows, dim = x.shape
    y = torch.empty_like(x)
    rms = torch.empty(rows, dtype=torch.float32, device=x.device)
    _typed("ref_rmsnorm_fwd", x)(_p(x), _p(gamma), _p(y), _p(rms), ctypes.c_float(eps), ctypes.c_int(rows),
                                 ctypes.c_int(dim), _s())
    return y, rms


def rmsnorm_bwd(dy, x, gamma, rms, eps):
    rows, dim = x.shape
    dx = torch.empty_like(x)
    gg = torch.zeros(dim, dtype=torch.float32, device=x.device)
    _typed("ref_rmsnorm_bwd", x)(_p(dy), _p(x), _p(gamma), _p(rms), _p(dx), _p(gg), ctypes.c_float(eps),
                                 ctypes.c_int(rows), ctypes.c_int(dim), _s())
    return dx, gg
