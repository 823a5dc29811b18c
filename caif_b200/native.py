"""ctypes binding of libcaifq.so (the C ABI in include/caifq.h) for torch tensors.

PyTorch is used for device memory and streams only: every function here hands
raw device pointers to the shared library.  There is no fallback: if the
library is missing or the call fails, a CaifqError is raised.
"""
import ctypes
import os

import torch

F32, F16, BF16, I4, I8 = 0, 2, 3, 4, 5
PER_TENSOR, PER_CHANNEL = 0, 1

_TORCH_TO_CODE = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.int8: I8}
_CODE_TO_TORCH = {F32: torch.float32, F16: torch.float16, BF16: torch.bfloat16, I8: torch.int8}

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libcaifq.so")


class CaifqError(RuntimeError):
    pass


class CWeight(ctypes.Structure):
    _fields_ = [
        ("codes", ctypes.c_void_p),
        ("scales", ctypes.c_void_p),
        ("storage", ctypes.c_int32),
        ("scheme", ctypes.c_int32),
        ("group_size", ctypes.c_int32),
        ("in_dim", ctypes.c_int32),
        ("out_dim", ctypes.c_int32),
    ]


class CLora(ctypes.Structure):
    _fields_ = [
        ("a", ctypes.c_void_p),
        ("b", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("rank", ctypes.c_int32),
        ("alpha", ctypes.c_float),
    ]


_lib = None

_vp = ctypes.c_void_p
_i32 = ctypes.c_int32
_i64 = ctypes.c_int64

_SIGNATURES = {
    "caifq_last_error": (ctypes.c_char_p, []),
    "caifq_last_path": (ctypes.c_char_p, []),
    "caifq_version": (ctypes.c_char_p, []),
    "caifq_device_ok": (ctypes.c_int, []),
    "caifq_device_status": (ctypes.c_int, []),
    "caifq_umma_pair_capacity": (ctypes.c_int32, []),
    "caifq_selftest_stall_next_decode": (None, []),
    "caifq_selftest_stall_next_umma": (None, []),
    "caifq_set_cta_limit": (None, [_i32]),
    "caifq_quantize_int8_per_tensor": (ctypes.c_int, [_vp, _vp, _vp, _i64, _vp]),
    "caifq_quantize_int8_per_channel": (ctypes.c_int, [_vp, _vp, _vp, _i32, _i32, _vp]),
    "caifq_quantize_int4_per_group": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "caifq_dequantize_int8_per_tensor": (ctypes.c_int, [_vp, _vp, _vp, _i64, _vp]),
    "caifq_dequantize_int8_per_channel": (ctypes.c_int, [_vp, _vp, _vp, _i32, _i32, _vp]),
    "caifq_dequantize_int4": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i32, _vp]),
    "caifq_cast": (ctypes.c_int, [_vp, _i32, _vp, _i32, _i64, _vp]),
    "caifq_weight_materialize": (ctypes.c_int, [ctypes.POINTER(CWeight), _vp, _i32, _vp]),
    "caifq_linear_fwd": (ctypes.c_int, [ctypes.POINTER(CWeight), _vp, _i32, _i64, _vp, _i32, _i32, _vp]),
    "caifq_linear_fwd_residual": (ctypes.c_int, [ctypes.POINTER(CWeight), _vp, _i32, _i64, _vp, _i32, _i32, _vp]),
    "caifq_linear_fwd_multi": (ctypes.c_int, [ctypes.POINTER(CWeight), _i32, _vp, _i32, _i64, _vp, _i32, _i32, _vp]),
    "caifq_linear_concat_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(CWeight), _i32]),
    "caifq_linear_fwd_concat": (ctypes.c_int, [ctypes.POINTER(CWeight), _i32, _vp, _i32, _i64, _vp, _i32, _i32, _vp,
                                               ctypes.c_size_t, _vp]),
    "caifq_linear_dx_concat": (ctypes.c_int, [ctypes.POINTER(CWeight), _i32, _vp, _i32, _i64, _vp, _i32, _i32, _vp,
                                              ctypes.c_size_t, _vp]),
    "caifq_linear_fwd_gather": (ctypes.c_int, [ctypes.POINTER(CWeight), _vp, _i32, _i64, ctypes.POINTER(_vp), _i32,
                                               _i64, _i64, _i32, _i32, _vp]),
    "caifq_linear_dx": (ctypes.c_int, [ctypes.POINTER(CWeight), _vp, _i32, _i64, _vp, _i32, _i32, _vp]),
    "caifq_lora_fwd_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _i64]),
    "caifq_lora_linear_fwd": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _vp, _i64, _vp, _vp,
                                             _vp, _i32, _vp]),
    "caifq_moe_route_grouped": (ctypes.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32, _vp]),
    "caifq_moe_router_bwd": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i32,
                                            ctypes.c_float, _i32, _vp]),
    "caifq_rmsnorm_fwd": (ctypes.c_int, [_vp, _vp, _vp, _vp, ctypes.c_float, _i32, _i32, _i32, _vp]),
    "caifq_rmsnorm_bwd": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_moe_bias_update": (ctypes.c_int, [_vp, _vp, _i32, _i32, _i32, ctypes.c_float, _vp]),
    "caifq_moe_aux_losses": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, ctypes.c_float,
                                            ctypes.c_float, _vp]),
    "caifq_lora_adamw_step": (ctypes.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32,
                                             ctypes.c_float, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                                             ctypes.c_float, ctypes.c_float, ctypes.c_float, _vp]),
    "caifq_lora_bwd_workspace_bytes": (ctypes.c_size_t, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _i64]),
    "caifq_lora_fwd_workspace_bytes_expanded": (ctypes.c_size_t, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _i64,
                                                                  _i32]),
    "caifq_lora_bwd_workspace_bytes_expanded": (ctypes.c_size_t, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _i64,
                                                                  _i32]),
    "caifq_lora_linear_fwd_expanded": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _vp, _i64, _vp,
                                                      _vp, _vp, _i32, _vp]),
    "caifq_lora_linear_bwd_expanded": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _vp, _vp, _vp,
                                                      _i64, _vp, _vp, _vp, _vp, _i32, _vp]),
    "caifq_lora_linear_bwd": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _vp, _vp, _vp, _i64,
                                             _vp, _vp, _vp, _vp, _i32, _vp]),
    "caifq_lora_bwd_noalloc_max_bytes": (ctypes.c_size_t, []),
    "caifq_lora_linear_bwd_noalloc": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CLora), _vp, _vp, _vp,
                                                     _i64, _vp, _vp, _vp, _i32, _vp]),
    "caifq_moe_topk": (ctypes.c_int, [_vp, _i32, _vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_moe_normalize_rows": (ctypes.c_int, [_vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_moe_router_softmax": (ctypes.c_int, [_vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_scale": (ctypes.c_int, [_vp, _vp, _i32, ctypes.c_float, _i64, _vp]),
    "caifq_moe_build_dispatch": (ctypes.c_int, [_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp]),
    "caifq_moe_dispatch": (ctypes.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_moe_combine": (ctypes.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_moe_combine_bwd_grad_expert": (ctypes.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_moe_combine_bwd_grad_weights": (ctypes.c_int, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_moe_dispatch_bwd": (ctypes.c_int, [_vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _vp]),
    "caifq_linear_fwd_sharded": (ctypes.c_int, [ctypes.POINTER(CWeight), _vp, _i32, _i64, _vp, _vp, _i32, _i32, _vp, _vp]),
    "caifq_linear_dx_sharded": (ctypes.c_int, [ctypes.POINTER(CWeight), _vp, _i32, _i64, _vp, _vp, _i32, _i32, _i32,
                                               _vp, _vp]),
    "caifq_rows_all_to_all": (ctypes.c_int, [_vp, ctypes.POINTER(_i64), _vp, ctypes.POINTER(_i64), _i64, _vp, _vp]),
    "caifq_grouped_expert_expanded_bytes": (ctypes.c_size_t, [ctypes.POINTER(CWeight), ctypes.POINTER(CWeight),
                                                              ctypes.POINTER(CWeight), _i32, _i32, _i32]),
    "caifq_grouped_expert_expand": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CWeight),
                                                   ctypes.POINTER(CWeight), _i32, _vp, _i32, _i32, _vp]),
    "caifq_grouped_expert_fwd_expanded": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CWeight),
                                                         ctypes.POINTER(CWeight), _i32, ctypes.POINTER(_i32), _vp, _vp,
                                                         _vp, _vp, _vp, _vp, _i32, _i32, _vp]),
    "caifq_grouped_expert_bwd_expanded": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CWeight),
                                                         ctypes.POINTER(CWeight), _i32, ctypes.POINTER(_i32), _vp, _vp,
                                                         _vp, _vp, _vp, _vp, _i32, _i32, _vp]),
    "caifq_grouped_expert_fwd": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CWeight),
                                                ctypes.POINTER(CWeight), _i32, ctypes.POINTER(_i32), _vp, _vp, _vp,
                                                _vp, _vp, _i32, _i32, _vp]),
    "caifq_grouped_expert_bwd": (ctypes.c_int, [ctypes.POINTER(CWeight), ctypes.POINTER(CWeight),
                                                ctypes.POINTER(CWeight), _i32, ctypes.POINTER(_i32), _vp, _vp, _vp,
                                                _vp, _vp, _i32, _i32, _vp]),
}


def exported_names():
    """Names this binding expects libcaifq.so to export."""
    return sorted(_SIGNATURES)


def lib():
    """The loaded shared library; raises CaifqError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CaifqError("%s is missing: run `python -m caif_b200.build` (there is no fallback path)" % LIB_PATH)
        loaded = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(loaded, name)
            fn.restype = res
            fn.argtypes = args
        _lib = loaded
    return _lib


def _check(rc, what):
    if rc != 0:
        raise CaifqError("%s failed (%d): %s" % (what, rc, lib().caifq_last_error().decode()))


def last_path():
    return lib().caifq_last_path().decode()


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    if t is None:
        return ctypes.c_void_p(None)
    return ctypes.c_void_p(t.data_ptr())


def _need_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise CaifqError("caifq works on CUDA tensors only (no CPU fallback)")
        if t is not None and not t.is_contiguous():
            raise CaifqError("caifq needs contiguous tensors")


def dtype_code(t):
    return _TORCH_TO_CODE[t] if isinstance(t, torch.dtype) else _TORCH_TO_CODE[t.dtype]


class Weight:
    """A frozen weight: codes + scales as the reference's quantize ops produce them."""

    def __init__(self, codes, storage, in_dim, out_dim, scales=None, scheme=PER_TENSOR, group_size=128):
        _need_cuda(codes, scales)
        self.codes = codes
        self.scales = scales
        self.storage = storage
        self.scheme = scheme
        self.group_size = group_size
        self.in_dim = in_dim
        self.out_dim = out_dim
        self.c = CWeight(codes.data_ptr(), scales.data_ptr() if scales is not None else None, storage, scheme,
                         group_size, in_dim, out_dim)

    def ref(self):
        return ctypes.byref(self.c)

    def rows(self, begin, end):
        """Column-parallel shard: output features [begin, end) -- a contiguous slice of codes and scales."""
        n = end - begin
        if self.storage == I4:
            if self.in_dim % self.group_size != 0 or (self.in_dim % 2) != 0:
                raise CaifqError("int4 row shards need in_dim to be a multiple of the group size")
            gpr = self.in_dim // self.group_size
            codes = self.codes.view(-1)[begin * self.in_dim // 2: end * self.in_dim // 2]
            scales = self.scales.view(-1)[begin * gpr: end * gpr]
            return Weight(codes, I4, self.in_dim, n, scales, self.scheme, self.group_size)
        codes = self.codes.view(-1)[begin * self.in_dim: end * self.in_dim]
        scales = self.scales
        if self.storage == I8 and self.scheme == PER_CHANNEL and scales is not None:
            raise CaifqError("per-channel int8 scales are indexed by flat % out_dim and do not shard by rows")
        return Weight(codes, self.storage, self.in_dim, n, scales, self.scheme, self.group_size)


# ---- quantize / dequantize ---------------------------------------------------

def quantize_int8_per_tensor(x):
    _need_cuda(x)
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scale = torch.empty(1, dtype=torch.float32, device=x.device)
    _check(lib().caifq_quantize_int8_per_tensor(_ptr(x), _ptr(q), _ptr(scale), x.numel(), _stream()),
           "quantize_int8_per_tensor")
    return q, scale


def quantize_int8_per_channel(x):
    _need_cuda(x)
    rows, cols = x.shape
    q = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    scales = torch.empty(cols, dtype=torch.float32, device=x.device)
    _check(lib().caifq_quantize_int8_per_channel(_ptr(x), _ptr(q), _ptr(scales), rows, cols, _stream()),
           "quantize_int8_per_channel")
    return q, scales


def quantize_int4(x, group_size=128):
    _need_cuda(x)
    n = x.numel()
    packed = torch.zeros((n + 1) // 2, dtype=torch.uint8, device=x.device)
    scales = torch.zeros((n + group_size - 1) // group_size, dtype=torch.float16, device=x.device)
    _check(lib().caifq_quantize_int4_per_group(_ptr(x), _ptr(packed), _ptr(scales), n, group_size, _stream()),
           "quantize_int4_per_group")
    return packed, scales


def dequantize_int8_per_tensor(q, scale):
    _need_cuda(q, scale)
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    _check(lib().caifq_dequantize_int8_per_tensor(_ptr(q), _ptr(out), _ptr(scale), q.numel(), _stream()),
           "dequantize_int8_per_tensor")
    return out


def dequantize_int8_per_channel(q, scales):
    _need_cuda(q, scales)
    rows, cols = q.shape
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    _check(lib().caifq_dequantize_int8_per_channel(_ptr(q), _ptr(out), _ptr(scales), rows, cols, _stream()),
           "dequantize_int8_per_channel")
    return out


def dequantize_int4(packed, scales, n, group_size=128):
    _need_cuda(packed, scales)
    out = torch.empty(n, dtype=torch.float32, device=packed.device)
    _check(lib().caifq_dequantize_int4(_ptr(packed), _ptr(scales), _ptr(out), n, group_size, _stream()),
           "dequantize_int4")
    return out


def cast(x, dtype):
    _need_cuda(x)
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _check(lib().caifq_cast(_ptr(x), dtype_code(x), _ptr(out), dtype_code(dtype), x.numel(), _stream()), "cast")
    return out


def weight_materialize(w, dtype=torch.float32):
    out = torch.empty((w.out_dim, w.in_dim), dtype=dtype, device=w.codes.device)
    _check(lib().caifq_weight_materialize(w.ref(), _ptr(out), dtype_code(dtype), _stream()), "weight_materialize")
    return out


# ---- frozen linear -----------------------------------------------------------

def linear_fwd(w, x, out_dtype=torch.float32, compute=F32, out=None):
    _need_cuda(x)
    m = x.numel() // w.in_dim
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (w.out_dim,), dtype=out_dtype, device=x.device)
    _check(lib().caifq_linear_fwd(w.ref(), _ptr(x), dtype_code(x), m, _ptr(out), dtype_code(out), compute, _stream()),
           "linear_fwd")
    return out


def linear_fwd_residual(w, x, residual, compute=F32):
    """residual [m, out] += W-path(x) in place, with the roundings of cast-then-Add; returns residual."""
    _need_cuda(x, residual)
    m = x.numel() // w.in_dim
    _check(lib().caifq_linear_fwd_residual(w.ref(), _ptr(x), dtype_code(x), m, _ptr(residual), dtype_code(residual),
                                           compute, _stream()), "caifq_linear_fwd_residual")
    return residual


def linear_fwd_multi(ws, x, out_dtype=torch.float32, compute=F32, out=None):
    """Few-token forward of several frozen linears that share x (q/k/v, gate/up) in one launch:
    y[m, sum out_i], weight i's outputs at columns sum_{j<i} out_j."""
    _need_cuda(x)
    m = x.numel() // ws[0].in_dim
    total = sum(w.out_dim for w in ws)
    y = out if out is not None else torch.empty((m, total), dtype=out_dtype, device=x.device)
    arr = _weight_array(ws)
    _check(lib().caifq_linear_fwd_multi(arr, len(ws), _ptr(x), dtype_code(x), m, _ptr(y), dtype_code(y), compute,
                                        _stream()), "caifq_linear_fwd_multi")
    return y


def linear_concat(ws, act, backward=False, out_dtype=torch.bfloat16, workspace=None):
    """Many-token product of several frozen linears that share their input as one launch over the concatenated
    weights: forward y[m, sum out_i] = x . [W_0; W_1; ...]^T, or backward dx[m, in] = dy[m, sum out_i] . [W_0; ...]."""
    _need_cuda(act, workspace)
    arr = _weight_array(ws)
    total = sum(w.out_dim for w in ws)
    need = lib().caifq_linear_concat_workspace_bytes(arr, len(ws))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=act.device)
    m = act.numel() // (total if backward else ws[0].in_dim)
    out = torch.empty((m, ws[0].in_dim if backward else total), dtype=out_dtype, device=act.device)
    fn = lib().caifq_linear_dx_concat if backward else lib().caifq_linear_fwd_concat
    _check(fn(arr, len(ws), _ptr(act), dtype_code(act), m, _ptr(out), dtype_code(out), BF16, _ptr(workspace),
              workspace.numel(), _stream()), "caifq_linear_concat")
    return out


def linear_fwd_gather(w, x, peer_ptrs, y_ld, y_col0, y_dtype=F32, compute=F32):
    """Few-token forward whose result goes straight into every buffer of `peer_ptrs` (raw device
    pointers: this GPU's own buffer and the peers' buffers mapped into this process)."""
    _need_cuda(x)
    m = x.shape[0]
    arr = (_vp * len(peer_ptrs))(*[_vp(int(q)) for q in peer_ptrs])
    _check(lib().caifq_linear_fwd_gather(w.ref(), _ptr(x), dtype_code(x), m, arr, len(peer_ptrs), int(y_ld),
                                         int(y_col0), y_dtype, compute, _stream()), "linear_fwd_gather")


def linear_dx(w, dy, out_dtype=torch.float32, compute=F32, out=None):
    _need_cuda(dy)
    m = dy.numel() // w.out_dim
    if out is None:
        out = torch.empty(tuple(dy.shape[:-1]) + (w.in_dim,), dtype=out_dtype, device=dy.device)
    _check(lib().caifq_linear_dx(w.ref(), _ptr(dy), dtype_code(dy), m, _ptr(out), dtype_code(out), compute, _stream()),
           "linear_dx")
    return out


# ---- LoRA --------------------------------------------------------------------

class Lora:
    def __init__(self, a, b, alpha):
        _need_cuda(a, b)
        self.a = a
        self.b = b
        self.alpha = float(alpha)
        self.rank = a.shape[0]
        self.c = CLora(a.data_ptr(), b.data_ptr(), dtype_code(a), self.rank, self.alpha)

    def ref(self):
        return ctypes.byref(self.c)


def lora_fwd_workspace_bytes(w, lora, m, compute=F32, expanded=False):
    if expanded:
        return int(lib().caifq_lora_fwd_workspace_bytes_expanded(w.ref(), lora.ref(), m, compute))
    return int(lib().caifq_lora_fwd_workspace_bytes(w.ref(), lora.ref(), m))


def lora_bwd_workspace_bytes(w, lora, m, compute=F32, expanded=False):
    if expanded:
        return int(lib().caifq_lora_bwd_workspace_bytes_expanded(w.ref(), lora.ref(), m, compute))
    return int(lib().caifq_lora_bwd_workspace_bytes(w.ref(), lora.ref(), m))


def lora_linear_fwd(w, lora, x, compute=F32, out=None, hidden=None, workspace=None, expanded=False):
    """y = W-path(x) + (alpha/r) . (x . A^T) . B^T.  `out`, `hidden` and `workspace` (a uint8 tensor of at
    least lora_fwd_workspace_bytes) may be passed in to keep the call free of allocations.  expanded=True
    uses the entry point that may expand the weight once per call into the (larger) workspace."""
    _need_cuda(x)
    m = x.numel() // w.in_dim
    y = out if out is not None else torch.empty(tuple(x.shape[:-1]) + (w.out_dim,), dtype=x.dtype, device=x.device)
    if hidden is None:
        hidden = torch.empty((m, lora.rank), dtype=x.dtype, device=x.device)
    ws_bytes = lora_fwd_workspace_bytes(w, lora, m, compute, expanded)
    if workspace is None:
        workspace = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
    elif workspace.numel() < ws_bytes:
        raise CaifqError("lora_linear_fwd: workspace of %d bytes, %d needed" % (workspace.numel(), ws_bytes))
    fn = lib().caifq_lora_linear_fwd_expanded if expanded else lib().caifq_lora_linear_fwd
    _check(fn(w.ref(), lora.ref(), _ptr(x), m, _ptr(y), _ptr(hidden), _ptr(workspace), compute, _stream()),
           "lora_linear_fwd")
    return y, hidden


def lora_linear_bwd(w, lora, dy, x, hidden, compute=F32, dx=None, d_a=None, d_b=None, workspace=None,
                    expanded=False):
    _need_cuda(dy, x, hidden)
    m = dy.numel() // w.out_dim
    if dx is None:
        dx = torch.empty(tuple(dy.shape[:-1]) + (w.in_dim,), dtype=dy.dtype, device=dy.device)
    if d_a is None:
        d_a = torch.empty_like(lora.a)
    if d_b is None:
        d_b = torch.empty_like(lora.b)
    ws_bytes = lora_bwd_workspace_bytes(w, lora, m, compute, expanded)
    if workspace is None:
        workspace = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dy.device)
    elif workspace.numel() < ws_bytes:
        raise CaifqError("lora_linear_bwd: workspace of %d bytes, %d needed" % (workspace.numel(), ws_bytes))
    fn = lib().caifq_lora_linear_bwd_expanded if expanded else lib().caifq_lora_linear_bwd
    _check(fn(w.ref(), lora.ref(), _ptr(dy), _ptr(x), _ptr(hidden), m, _ptr(dx), _ptr(d_a), _ptr(d_b),
              _ptr(workspace), compute, _stream()), "lora_linear_bwd")
    return dx, d_a, d_b


def lora_adamw_step(lora, d_a, d_b, m_a, v_a, m_b, v_b, lr, beta1, beta2, epsilon, weight_decay, step):
    """AdamW on the adapter's A and B in place (one launch); moments are fp32 tensors shaped like A and B."""
    _need_cuda(lora.a, lora.b, d_a, d_b, m_a, v_a, m_b, v_b)
    import numpy as _np
    bc1 = float(_np.float32(1.0) - _np.float32(beta1) ** _np.float32(step))
    bc2 = float(_np.float32(1.0) - _np.float32(beta2) ** _np.float32(step))
    rank, in_dim = lora.a.shape
    out_dim = lora.b.shape[0]
    _check(lib().caifq_lora_adamw_step(_ptr(lora.a), _ptr(lora.b), _ptr(d_a), _ptr(d_b), _ptr(m_a), _ptr(v_a),
                                       _ptr(m_b), _ptr(v_b), rank, in_dim, out_dim, dtype_code(lora.a), lr, beta1,
                                       beta2, epsilon, weight_decay, bc1, bc2, _stream()), "lora_adamw_step")
    return bc1, bc2


def lora_linear_bwd_noalloc(w, lora, dy, x, hidden, compute=F32):
    """caifq_lora_linear_bwd_noalloc: the scratch comes from the buffer built into the
    library, so this wrapper allocates only the three result tensors."""
    _need_cuda(dy, x, hidden)
    m = dy.numel() // w.out_dim
    dx = torch.empty(tuple(dy.shape[:-1]) + (w.in_dim,), dtype=dy.dtype, device=dy.device)
    d_a = torch.empty_like(lora.a)
    d_b = torch.empty_like(lora.b)
    _check(lib().caifq_lora_linear_bwd_noalloc(w.ref(), lora.ref(), _ptr(dy), _ptr(x), _ptr(hidden), m, _ptr(dx),
                                               _ptr(d_a), _ptr(d_b), compute, _stream()),
           "lora_linear_bwd_noalloc")
    return dx, d_a, d_b


# ---- MoE ---------------------------------------------------------------------

def moe_topk(probs, k):
    _need_cuda(probs)
    batch, dim = probs.shape
    idx = torch.empty((batch, k), dtype=torch.int32, device=probs.device)
    val = torch.empty((batch, k), dtype=probs.dtype, device=probs.device)
    _check(lib().caifq_moe_topk(_ptr(probs), dtype_code(probs), _ptr(idx), _ptr(val), batch, dim, k, _stream()),
           "moe_topk")
    return idx, val


def moe_normalize_rows(x):
    _need_cuda(x)
    batch, dim = x.shape
    out = torch.empty_like(x)
    _check(lib().caifq_moe_normalize_rows(_ptr(x), _ptr(out), dtype_code(x), batch, dim, _stream()),
           "moe_normalize_rows")
    return out


def moe_route_grouped(x, k, logits=True, bias=None, n_group=1, topk_group=1):
    """Sigmoid (logits=True) or given scores, selection-only bias, group mask, top-k, gathered weights:
    returns (scores, indices, weights)."""
    _need_cuda(x, bias)
    batch, dim = x.shape
    scores = torch.empty_like(x)
    idx = torch.empty((batch, k), dtype=torch.int32, device=x.device)
    wts = torch.empty((batch, k), dtype=x.dtype, device=x.device)
    _check(lib().caifq_moe_route_grouped(_ptr(x), 1 if logits else 0, _ptr(bias), _ptr(scores), _ptr(idx), _ptr(wts),
                                         dtype_code(x), batch, dim, k, n_group, topk_group, _stream()),
           "moe_route_grouped")
    return scores, idx, wts


def moe_router_bwd(grad_weights, probs, indices, balance_bias=None, z_lse_scaled=None, sigmoid_gate=False,
                   normalize=True, scaling=1.0, exact_jacobian=False):
    """Gradient of the routing weights back to the router's logits: returns (grad_logits [tokens, experts],
    grad_topk [tokens, top_k])."""
    _need_cuda(grad_weights, probs, indices, balance_bias, z_lse_scaled)
    tokens, experts = probs.shape
    top_k = indices.shape[1]
    grad_logits = torch.empty_like(probs)
    grad_topk = torch.empty_like(grad_weights)
    _check(lib().caifq_moe_router_bwd(_ptr(grad_weights), _ptr(probs), _ptr(indices), _ptr(balance_bias),
                                      _ptr(z_lse_scaled), _ptr(grad_topk), _ptr(grad_logits), dtype_code(probs),
                                      tokens, experts, top_k, 1 if sigmoid_gate else 0, 1 if normalize else 0,
                                      float(scaling), 1 if exact_jacobian else 0, _stream()), "moe_router_bwd")
    return grad_logits, grad_topk


def moe_aux_losses(logits, probs, expert_offsets, top_k, balance_weight, z_weight):
    """Load-balance and z loss with the operands of their gradients: returns (sums, balance_bias, lse,
    z_lse_scaled); sums[0], sums[1] are the two loss values, sums[2:] the column sums of probs."""
    _need_cuda(logits, probs, expert_offsets)
    ref = probs if probs is not None else logits
    tokens, experts = ref.shape
    sums = torch.empty(2 + experts, dtype=torch.float32, device=ref.device)
    bias = torch.empty(experts, dtype=ref.dtype, device=ref.device) if probs is not None else None
    lse = torch.empty(tokens, dtype=ref.dtype, device=ref.device) if logits is not None else None
    zls = torch.empty(tokens, dtype=ref.dtype, device=ref.device) if logits is not None else None
    _check(lib().caifq_moe_aux_losses(_ptr(logits), _ptr(probs), _ptr(expert_offsets), _ptr(bias), _ptr(lse),
                                      _ptr(zls), _ptr(sums), dtype_code(ref), tokens, experts, top_k,
                                      float(balance_weight), float(z_weight), _stream()), "moe_aux_losses")
    return sums, bias, lse, zls


def moe_bias_update(bias, counts, rate, from_offsets=False):
    """Aux-loss-free balancing: bias moves by `rate` towards the mean load, in place."""
    _need_cuda(bias, counts)
    _check(lib().caifq_moe_bias_update(_ptr(bias), _ptr(counts), 1 if from_offsets else 0, dtype_code(bias),
                                       bias.numel(), float(rate), _stream()), "moe_bias_update")
    return bias


def rmsnorm_fwd(x, gamma, epsilon=1e-5):
    """Returns (y, rms_cache)."""
    _need_cuda(x, gamma)
    dim = x.shape[-1]
    rows = x.numel() // dim
    y = torch.empty_like(x)
    rms = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(lib().caifq_rmsnorm_fwd(_ptr(x), _ptr(gamma), _ptr(y), _ptr(rms), float(epsilon), dtype_code(x), rows, dim,
                                   _stream()), "rmsnorm_fwd")
    return y, rms


def rmsnorm_bwd(dy, x, gamma, rms_cache, grad_gamma=None):
    """Returns (dx, grad_gamma); grad_gamma is accumulated onto the tensor given (zeros when None)."""
    _need_cuda(dy, x, gamma, rms_cache, grad_gamma)
    dim = x.shape[-1]
    rows = x.numel() // dim
    dx = torch.empty_like(x)
    if grad_gamma is None:
        grad_gamma = torch.zeros(dim, dtype=torch.float32, device=x.device)
    _check(lib().caifq_rmsnorm_bwd(_ptr(dy), _ptr(x), _ptr(gamma), _ptr(rms_cache), _ptr(dx), _ptr(grad_gamma),
                                   dtype_code(x), rows, dim, _stream()), "rmsnorm_bwd")
    return dx, grad_gamma


def moe_softmax(logits, bias=None):
    """Router probabilities: softmax over the experts of each row, optional bias added first."""
    _need_cuda(logits, bias)
    rows, cols = logits.shape
    probs = torch.empty_like(logits)
    _check(lib().caifq_moe_router_softmax(_ptr(logits), _ptr(bias), _ptr(probs), dtype_code(logits), rows, cols,
                                          _stream()), "moe_router_softmax")
    return probs


def scale(x, factor, out=None):
    _need_cuda(x)
    if out is None:
        out = torch.empty_like(x)
    _check(lib().caifq_scale(_ptr(x), _ptr(out), dtype_code(x), float(factor), x.numel(), _stream()), "scale")
    return out


def moe_build_dispatch(expert_indices, num_experts, capacity=0):
    _need_cuda(expert_indices)
    tokens, top_k = expert_indices.shape
    dmap = torch.empty((tokens, top_k), dtype=torch.int32, device=expert_indices.device)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=expert_indices.device)
    _check(lib().caifq_moe_build_dispatch(_ptr(expert_indices), tokens, top_k, num_experts, capacity, _ptr(dmap),
                                          _ptr(offsets), _stream()), "moe_build_dispatch")
    return dmap, offsets


def moe_dispatch(x, expert_indices, dispatch_map, expert_offsets, total_assigned):
    _need_cuda(x, expert_indices, dispatch_map, expert_offsets)
    tokens, dim = x.shape
    top_k = expert_indices.shape[1]
    # every row below expert_offsets[E] is written exactly once; like the reference's layer
    # (src/caif_device_moe_layer.cpp:457-462, Uninitialized workspaces) the buffer is not cleared first
    buf = torch.empty((total_assigned, dim), dtype=x.dtype, device=x.device)
    _check(lib().caifq_moe_dispatch(_ptr(x), dtype_code(x), _ptr(expert_indices), _ptr(dispatch_map),
                                    _ptr(expert_offsets), _ptr(buf), tokens, dim, top_k, _stream()), "moe_dispatch")
    return buf


def moe_combine(buf, expert_indices, weights, dispatch_map, expert_offsets, num_tokens):
    _need_cuda(buf, expert_indices, weights, dispatch_map, expert_offsets)
    dim = buf.shape[1]
    top_k = expert_indices.shape[1]
    out = torch.empty((num_tokens, dim), dtype=buf.dtype, device=buf.device)
    _check(lib().caifq_moe_combine(_ptr(buf), dtype_code(buf), _ptr(expert_indices), _ptr(weights),
                                   _ptr(dispatch_map), _ptr(expert_offsets), _ptr(out), num_tokens, dim, top_k,
                                   _stream()), "moe_combine")
    return out


def moe_combine_bwd_grad_expert(grad_output, expert_indices, weights, dispatch_map, expert_offsets, total_assigned):
    _need_cuda(grad_output, expert_indices, weights, dispatch_map, expert_offsets)
    tokens, dim = grad_output.shape
    top_k = expert_indices.shape[1]
    gbuf = torch.empty((total_assigned, dim), dtype=grad_output.dtype, device=grad_output.device)   # as above (:723-728)
    _check(lib().caifq_moe_combine_bwd_grad_expert(_ptr(grad_output), dtype_code(grad_output), _ptr(expert_indices),
                                                   _ptr(weights), _ptr(dispatch_map), _ptr(expert_offsets),
                                                   _ptr(gbuf), tokens, dim, top_k, _stream()),
           "moe_combine_bwd_grad_expert")
    return gbuf


def moe_combine_bwd_grad_weights(grad_output, buf, expert_indices, dispatch_map, expert_offsets):
    _need_cuda(grad_output, buf, expert_indices, dispatch_map, expert_offsets)
    tokens, dim = grad_output.shape
    top_k = expert_indices.shape[1]
    gw = torch.empty((tokens, top_k), dtype=grad_output.dtype, device=grad_output.device)
    _check(lib().caifq_moe_combine_bwd_grad_weights(_ptr(grad_output), _ptr(buf), dtype_code(grad_output),
                                                    _ptr(expert_indices), _ptr(dispatch_map), _ptr(expert_offsets),
                                                    _ptr(gw), tokens, dim, top_k, _stream()),
           "moe_combine_bwd_grad_weights")
    return gw


def moe_dispatch_bwd(grad_buf, expert_indices, dispatch_map, expert_offsets, num_tokens):
    _need_cuda(grad_buf, expert_indices, dispatch_map, expert_offsets)
    dim = grad_buf.shape[1]
    top_k = expert_indices.shape[1]
    gin = torch.empty((num_tokens, dim), dtype=grad_buf.dtype, device=grad_buf.device)
    _check(lib().caifq_moe_dispatch_bwd(_ptr(grad_buf), dtype_code(grad_buf), _ptr(expert_indices),
                                        _ptr(dispatch_map), _ptr(expert_offsets), _ptr(gin), num_tokens, dim, top_k,
                                        _stream()), "moe_dispatch_bwd")
    return gin


def _weight_array(ws):
    arr = (CWeight * len(ws))()
    for i, w in enumerate(ws):
        arr[i] = w.c
    return arr


def grouped_expert_expanded_bytes(gate, up, down, dtype=BF16, compute=F32):
    """Bytes of the scratch that holds the bf16 copies of these experts' weights (0: not expanded)."""
    return int(lib().caifq_grouped_expert_expanded_bytes(_weight_array(gate) if gate is not None else None,
                                                         _weight_array(up), _weight_array(down), len(up), dtype,
                                                         compute))


def grouped_expert_expand(gate, up, down, expanded, dtype=BF16, compute=F32):
    """Fill `expanded` (uint8 tensor of grouped_expert_expanded_bytes) with the bf16 copies, once per step."""
    _need_cuda(expanded)
    _check(lib().caifq_grouped_expert_expand(_weight_array(gate) if gate is not None else None, _weight_array(up),
                                             _weight_array(down), len(up), _ptr(expanded), dtype, compute, _stream()),
           "grouped_expert_expand")
    return expanded


def grouped_expert_fwd(gate, up, down, offsets_host, x, compute=F32, expanded=None):
    """gate/up/down: lists of Weight (gate=None: experts without a gate projection; the gate output
    returned is then None); offsets_host: list of E+1 ints; x: packed [total, in].  expanded: the buffer
    grouped_expert_expand filled for these tables (the launches then read bf16 weight tiles from it)."""
    _need_cuda(x)
    n_exp = len(up)
    total = int(offsets_host[-1])
    hid = up[0].out_dim
    out = torch.empty((total, up[0].in_dim), dtype=x.dtype, device=x.device)
    gate_out = torch.empty((total, hid), dtype=x.dtype, device=x.device) if gate is not None else None
    up_out = torch.empty((total, hid), dtype=x.dtype, device=x.device)
    hidden = torch.empty((total, hid), dtype=x.dtype, device=x.device)
    offs = (ctypes.c_int32 * (n_exp + 1))(*[int(v) for v in offsets_host])
    if expanded is not None:
        _check(lib().caifq_grouped_expert_fwd_expanded(_weight_array(gate) if gate is not None else None,
                                                       _weight_array(up), _weight_array(down), n_exp, offs, _ptr(x),
                                                       _ptr(out), _ptr(gate_out), _ptr(up_out), _ptr(hidden),
                                                       _ptr(expanded), dtype_code(x), compute, _stream()),
               "grouped_expert_fwd_expanded")
        return out, gate_out, up_out
    _check(lib().caifq_grouped_expert_fwd(_weight_array(gate) if gate is not None else None, _weight_array(up),
                                          _weight_array(down), n_exp, offs,
                                          _ptr(x), _ptr(out), _ptr(gate_out), _ptr(up_out), _ptr(hidden),
                                          dtype_code(x), compute, _stream()), "grouped_expert_fwd")
    return out, gate_out, up_out


def grouped_expert_bwd(gate, up, down, offsets_host, dy, gate_out, up_out, compute=F32, expanded=None):
    _need_cuda(dy, gate_out, up_out)
    n_exp = len(up)
    total = int(offsets_host[-1])
    hid = up[0].out_dim
    dx = torch.empty((total, up[0].in_dim), dtype=dy.dtype, device=dy.device)
    ws = torch.empty((3, max(total, 1), hid), dtype=dy.dtype, device=dy.device)
    offs = (ctypes.c_int32 * (n_exp + 1))(*[int(v) for v in offsets_host])
    if expanded is not None:
        _check(lib().caifq_grouped_expert_bwd_expanded(_weight_array(gate) if gate is not None else None,
                                                       _weight_array(up), _weight_array(down), n_exp, offs, _ptr(dy),
                                                       _ptr(gate_out), _ptr(up_out), _ptr(dx), _ptr(ws),
                                                       _ptr(expanded), dtype_code(dy), compute, _stream()),
               "grouped_expert_bwd_expanded")
        return dx
    _check(lib().caifq_grouped_expert_bwd(_weight_array(gate) if gate is not None else None, _weight_array(up),
                                          _weight_array(down), n_exp, offs,
                                          _ptr(dy), _ptr(gate_out), _ptr(up_out), _ptr(dx), _ptr(ws),
                                          dtype_code(dy), compute, _stream()), "grouped_expert_bwd")
    return dx
