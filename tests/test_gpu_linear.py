"""GPU parity of the frozen-linear forward and dX against the CPU oracle.

Tolerances (max |err| / max |want|, the reference tests' measure):
  fp32 compute 1e-4, bf16/fp16 compute 2e-2 -- the bounds the task states.
Where the kernel consumes exactly the operands the reference would (generic
path), the bound asserted is the tighter 1e-4 in every cell.
"""
import os

import numpy as np
import pytest
import torch

import caif_oracle as orc
from caif_b200 import native as nv
from gpu_util import TORCH_DTYPE, act, make_weight, max_rel_err, to_dev

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-4
TOL_16 = 2e-2

STORAGES = [orc.F32, orc.F16, orc.BF16, orc.I8, orc.I4]
COMPUTES = [orc.F32, orc.F16, orc.BF16]


def _oracle_w(weight, codes, scales, compute):
    return orc.weight_to_compute(codes, scales, weight.storage, weight.in_dim, weight.out_dim, compute,
                                 weight.scheme, weight.group_size)


@pytest.mark.parametrize("storage", STORAGES)
@pytest.mark.parametrize("compute", COMPUTES)
def test_every_cell_forward_and_dx(storage, compute, monkeypatch):
    """The reference's 3x5 (compute, storage) grid, shapes that hit every tail:
    in/out not multiples of the tile, int4 groups straddling rows."""
    monkeypatch.setenv("CAIFQ_FORCE_PATH", "generic")
    rng = np.random.default_rng(100 + storage * 10 + compute)
    in_dim, out_dim, m = 72, 52, 37
    weight, codes, scales = make_weight(rng, out_dim, in_dim, storage)
    x_np, x = act(rng, m, in_dim, compute if compute != orc.F32 else orc.F32)
    dy_np, dy = act(rng, m, out_dim, compute if compute != orc.F32 else orc.F32)
    wc = _oracle_w(weight, codes, scales, compute)
    y = nv.linear_fwd(weight, x, torch.float32, compute)
    dx = nv.linear_dx(weight, dy, torch.float32, compute)
    assert nv.last_path() == "generic"
    assert y.dtype == torch.float32 and tuple(y.shape) == (m, out_dim)
    assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc, compute)) <= TOL_F32
    assert max_rel_err(dx.cpu().numpy(), orc.frozen_linear_backward(dy_np, wc, compute)) <= TOL_F32


def test_config1_int8_fp32(monkeypatch):
    """in=1024, out=1024, M=64, fp32 compute, int8 per-tensor weights N(0,0.02):
    codes and scale bit-exact, Y and dX within 1e-4 of the host-sgemm path."""
    rng = np.random.default_rng(1234)
    w = (rng.standard_normal((1024, 1024)) * 0.02).astype(np.float32)
    q, s = nv.quantize_int8_per_tensor(to_dev(w))
    oq, os_ = orc.quantize_int8_per_tensor(w)
    assert np.array_equal(q.cpu().numpy(), oq) and np.array_equal(s.cpu().numpy().view(np.uint32), os_.view(np.uint32))
    weight = nv.Weight(q, nv.I8, 1024, 1024, s)
    x_np, x = act(rng, 64, 1024, orc.F32)
    dy_np, dy = act(rng, 64, 1024, orc.F32)
    wc = orc.weight_to_compute(oq, os_, orc.I8, 1024, 1024)
    y = nv.linear_fwd(weight, x)
    dx = nv.linear_dx(weight, dy)
    for exact in (True, False):  # fp64-accumulated loop and OpenBLAS sgemm (the reference's host GEMM)
        assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc, exact=exact)) <= TOL_F32
        assert max_rel_err(dx.cpu().numpy(), orc.frozen_linear_backward(dy_np, wc, exact=exact)) <= TOL_F32


@pytest.mark.parametrize("scheme,with_scales", [(orc.PER_CHANNEL, True), (orc.PER_TENSOR, False)])
def test_int8_per_channel_quirk_and_raw_cast(scheme, with_scales, monkeypatch):
    rng = np.random.default_rng(7)
    in_dim, out_dim, m = 96, 64, 20
    weight, codes, scales = make_weight(rng, out_dim, in_dim, orc.I8, scheme=scheme, with_scales=with_scales)
    x_np, x = act(rng, m, in_dim, orc.F32)
    wc = _oracle_w(weight, codes, scales, orc.F32)
    y = nv.linear_fwd(weight, x)
    assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc)) <= TOL_F32
    mat = nv.weight_materialize(weight)
    assert np.array_equal(mat.cpu().numpy(), wc)


def test_three_d_input_and_output_dtypes():
    rng = np.random.default_rng(8)
    weight, codes, scales = make_weight(rng, 48, 64, orc.I4)
    x_np = orc.round_through(rng.standard_normal((2, 5, 64)).astype(np.float32), orc.BF16)
    x = to_dev(x_np, torch.bfloat16)
    wc = _oracle_w(weight, codes, scales, orc.F32)
    want = orc.frozen_linear_forward(x_np, wc).reshape(2, 5, 48)
    y = nv.linear_fwd(weight, x, torch.float32, orc.F32)
    assert tuple(y.shape) == (2, 5, 48)
    assert max_rel_err(y.cpu().numpy(), want) <= TOL_F32
    yb = nv.linear_fwd(weight, x, torch.bfloat16, orc.F32)
    assert np.array_equal(yb.float().cpu().numpy(), orc.round_through(y.cpu().numpy(), orc.BF16))


def test_errors():
    rng = np.random.default_rng(9)
    weight, _, _ = make_weight(rng, 16, 16, orc.I8)
    x = torch.zeros((4, 16), device="cuda")
    bad = nv.Weight(weight.codes, 9, 16, 16)
    with pytest.raises(nv.CaifqError):
        nv.linear_fwd(bad, x)
    no_scales = nv.Weight(weight.codes, nv.I4, 16, 16, None)
    with pytest.raises(nv.CaifqError):
        nv.linear_fwd(no_scales, x)
    # m == 0 is a no-op
    y = nv.linear_fwd(weight, torch.zeros((0, 16), device="cuda"))
    assert y.shape[0] == 0


# --------------------------------------------------------------------- decode
@pytest.mark.parametrize("m", [1, 4, 16])
def test_decode_int4_config2(m):
    """in=4096, out=14336, int4 g128, bf16 activations: forward, weight-streaming kernel."""
    g = torch.Generator(device="cuda").manual_seed(1235)
    out_dim, in_dim = 14336, 4096
    wf = torch.randn(out_dim * in_dim, generator=g, device="cuda") * 0.02
    p, s = nv.quantize_int4(wf, 128)
    weight = nv.Weight(p, nv.I4, in_dim, out_dim, s, group_size=128)
    x = torch.randn(m, in_dim, generator=g, device="cuda").to(torch.bfloat16)
    y = nv.linear_fwd(weight, x, torch.float32, orc.F32)
    assert nv.last_path() == "decode"
    wc = orc.dequantize_int4(p.cpu().numpy(), s.cpu().view(torch.int16).numpy().view(np.uint16), out_dim * in_dim,
                             128).reshape(out_dim, in_dim)
    want = orc.gemm_nt(x.float().cpu().numpy(), wc)
    assert max_rel_err(y.cpu().numpy(), want) <= TOL_F32
    # bf16 compute: the reference rounds scale*code to bf16 first; bound 2e-2
    yb = nv.linear_fwd(weight, x, torch.float32, orc.BF16)
    want_b = orc.gemm_nt(x.float().cpu().numpy(), orc.round_through(wc, orc.BF16))
    assert max_rel_err(yb.cpu().numpy(), want_b) <= TOL_16
    os.environ["CAIFQ_FORCE_PATH"] = "generic"
    try:
        yg = nv.linear_fwd(weight, x, torch.float32, orc.F32)
        assert nv.last_path() == "generic"
    finally:
        del os.environ["CAIFQ_FORCE_PATH"]
    assert max_rel_err(y.cpu().numpy(), yg.cpu().numpy()) <= TOL_F32


@pytest.mark.parametrize("storage,in_dim,out_dim,m,group", [
    (orc.I4, 1024, 264, 3, 128),     # one chunk per warp, partial... out multiple of 8
    (orc.I4, 2048, 1000, 8, 256),    # group of two chunks
    (orc.I4, 8192, 128, 5, 128),     # four chunks per warp
    (orc.I4, 4096, 100, 16, 128),    # out not a multiple of 8 (ragged last unit), two token tiles
    (orc.I4, 384, 64, 9, 128),       # fewer chunks than warps
    (orc.I8, 4096, 512, 2, 0),
    (orc.I8, 1024, 136, 12, 0),
    (orc.I8, 5120, 64, 7, 0),       # five chunks per warp
    (orc.I8, 320, 72, 1, 0),
    (orc.I4, 1024, 40000, 16, 128),  # more items per CTA than partial sums can be parked: several rounds
    (orc.I4, 1024, 40000, 3, 128),
    (orc.I8, 512, 33000, 9, 0),
])
def test_decode_shapes(storage, in_dim, out_dim, m, group):
    rng = np.random.default_rng(in_dim + out_dim + m)
    weight, codes, scales = make_weight(rng, out_dim, in_dim, storage, group=group or 128)
    x_np, x = act(rng, m, in_dim, orc.BF16)
    y = nv.linear_fwd(weight, x, torch.float32, orc.F32)
    assert nv.last_path() == "decode"
    wc = _oracle_w(weight, codes, scales, orc.F32)
    assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc)) <= TOL_F32


def test_decode_int8_without_scales_and_bf16_out():
    rng = np.random.default_rng(77)
    weight, codes, scales = make_weight(rng, 256, 2048, orc.I8, with_scales=False)
    x_np, x = act(rng, 4, 2048, orc.BF16)
    y = nv.linear_fwd(weight, x, torch.bfloat16, orc.F32)
    assert nv.last_path() == "decode"
    want = orc.frozen_linear_forward(x_np, _oracle_w(weight, codes, scales, orc.F32))
    assert max_rel_err(y.float().cpu().numpy(), want) <= 1e-2  # bf16 output rounding


def test_decode_forward_gather_into_several_buffers():
    """The fused gather: two shards of a wider layer write their slices, at their column offsets,
    into two result buffers each (on one GPU both 'ranks' are local buffers); every buffer ends up
    holding the full-width result, equal to the plain forward of each shard bit for bit."""
    rng = np.random.default_rng(2024)
    in_dim, shard, m = 1024, 520, 5
    shards = [make_weight(rng, shard, in_dim, orc.I4)[0] for _ in range(2)]
    _, x = act(rng, m, in_dim, orc.BF16)
    bufs = [torch.full((m, 2 * shard), float("nan"), device="cuda") for _ in range(2)]
    ptrs = [b.data_ptr() for b in bufs]
    for r, w in enumerate(shards):
        nv.linear_fwd_gather(w, x, ptrs, 2 * shard, r * shard, orc.F32, orc.F32)
        assert nv.last_path() == "decode"
    torch.cuda.synchronize()
    want = torch.cat([nv.linear_fwd(w, x, torch.float32, orc.F32) for w in shards], dim=1)
    for b in bufs:
        assert torch.equal(b, want)
    # shapes the few-token kernel does not take are refused, not silently run elsewhere
    _, x_many = act(rng, 64, in_dim, orc.BF16)
    big = torch.empty((64, 2 * shard), device="cuda")
    with pytest.raises(nv.CaifqError):
        nv.linear_fwd_gather(shards[0], x_many, [big.data_ptr()], 2 * shard, 0, orc.F32, orc.F32)
    with pytest.raises(nv.CaifqError):   # the slice must fit the row pitch
        nv.linear_fwd_gather(shards[0], x, ptrs, shard, shard, orc.F32, orc.F32)


# ------------------------------------------------------------ tensor-core path
def _umma_case(storage, compute, m, in_dim, out_dim, seed, group=128):
    rng = np.random.default_rng(seed)
    weight, codes, scales = make_weight(rng, out_dim, in_dim, storage, group=group)
    x_np, x = act(rng, m, in_dim, orc.BF16)
    dy_np, dy = act(rng, m, out_dim, orc.BF16)
    wc = _oracle_w(weight, codes, scales, compute)
    return weight, wc, x_np, x, dy_np, dy


@pytest.mark.parametrize("storage,compute,tol", [
    (orc.I8, orc.F32, TOL_F32),     # exact products: holds the fp32 bound
    (orc.I8, orc.BF16, TOL_16),
    (orc.I4, orc.BF16, TOL_16),
    (orc.I4, orc.F32, TOL_F32),     # scale*code as two bf16 terms: holds the fp32 bound
    (orc.BF16, orc.F32, TOL_F32),
])
@pytest.mark.parametrize("m,in_dim,out_dim", [(300, 512, 384), (256, 128, 128), (77, 1408, 2048), (1000, 2048, 1408),
                                             (17, 256, 384)])
def test_umma_forward_and_dx(storage, compute, tol, m, in_dim, out_dim):
    weight, wc, x_np, x, dy_np, dy = _umma_case(storage, compute, m, in_dim, out_dim, 500 + storage + m)
    y = nv.linear_fwd(weight, x, torch.float32, compute)
    assert nv.last_path() == "umma"
    dx = nv.linear_dx(weight, dy, torch.float32, compute)
    assert nv.last_path() == "umma"
    assert nv.lib().caifq_device_status() == 0
    assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc, compute)) <= tol
    assert max_rel_err(dx.cpu().numpy(), orc.frozen_linear_backward(dy_np, wc, compute)) <= tol
    if storage == orc.I4 and compute == orc.BF16:
        # the operand is code * bf16(scale), the reference's is bf16(code * scale): they differ by the bf16
        # rounding of the fp16 scale, a small fraction of the bound
        assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc, compute)) <= 4e-3


def test_umma_int4_group_size_that_is_not_a_power_of_two():
    weight, wc, x_np, x, dy_np, dy = _umma_case(orc.I4, orc.BF16, 64, 384, 256, 4321, group=96)
    y = nv.linear_fwd(weight, x, torch.float32, orc.BF16)
    assert nv.last_path() == "umma"
    dx = nv.linear_dx(weight, dy, torch.float32, orc.BF16)
    assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc, orc.BF16)) <= 4e-3
    assert max_rel_err(dx.cpu().numpy(), orc.frozen_linear_backward(dy_np, wc, orc.BF16)) <= 4e-3


def test_umma_bf16_output_and_accumulate_epilogue():
    weight, wc, x_np, x, dy_np, dy = _umma_case(orc.I8, orc.F32, 200, 256, 256, 42)
    yb = nv.linear_fwd(weight, x, torch.bfloat16, orc.F32)
    assert nv.last_path() == "umma"
    want = orc.round_through(orc.frozen_linear_forward(x_np, wc), orc.BF16)
    assert max_rel_err(yb.float().cpu().numpy(), want) <= 1e-2


def test_umma_config3_shape_matches_generic_and_oracle_rows(monkeypatch):
    """4096 -> 4096 int8 per-tensor, M = 8192 bf16 tokens (the training config): the tensor-core
    path against the generic path on the whole output and against the oracle on 16 rows."""
    g = torch.Generator(device="cuda").manual_seed(1236)
    dim, m = 4096, 8192
    wf = torch.randn(dim * dim, generator=g, device="cuda") * 0.02
    q, s = nv.quantize_int8_per_tensor(wf)
    weight = nv.Weight(q.view(dim, dim), nv.I8, dim, dim, s)
    x = torch.randn(m, dim, generator=g, device="cuda").to(torch.bfloat16)
    dy = torch.randn(m, dim, generator=g, device="cuda").to(torch.bfloat16)
    y = nv.linear_fwd(weight, x, torch.float32, orc.F32)
    assert nv.last_path() == "umma"
    dx = nv.linear_dx(weight, dy, torch.float32, orc.F32)
    assert nv.lib().caifq_device_status() == 0
    monkeypatch.setenv("CAIFQ_FORCE_PATH", "generic")
    yg = nv.linear_fwd(weight, x, torch.float32, orc.F32)
    dxg = nv.linear_dx(weight, dy, torch.float32, orc.F32)
    assert nv.last_path() == "generic"
    assert float((y - yg).abs().max() / yg.abs().max()) <= TOL_F32
    assert float((dx - dxg).abs().max() / dxg.abs().max()) <= TOL_F32
    rows = torch.arange(0, m, m // 16, device="cuda")
    wc = orc.dequantize_int8_per_tensor(q.cpu().numpy().reshape(dim, dim), s.cpu().numpy())
    want = orc.gemm_nt(x[rows].float().cpu().numpy(), wc)
    assert max_rel_err(y[rows].cpu().numpy(), want) <= TOL_F32
    want_dx = orc.gemm_nn(dy[rows].float().cpu().numpy(), wc)
    assert max_rel_err(dx[rows].cpu().numpy(), want_dx) <= TOL_F32


def test_decode_misaligned_activations_fall_back():
    """bf16 activations that do not start on a 16-byte boundary (a row slice of a larger tensor)
    are a legal call: the few-token kernel declines them and another kernel family answers."""
    rng = np.random.default_rng(77)
    weight, codes, scales = make_weight(rng, 136, 1024, orc.I8)
    x_np, x = act(rng, 4, 1024, orc.BF16)
    big = torch.zeros(4 * 1024 + 8, dtype=torch.bfloat16, device="cuda")
    shifted = big[1:1 + 4 * 1024].view(4, 1024)     # starts 2 bytes past an aligned address
    shifted.copy_(x)
    assert shifted.data_ptr() % 16 == 2
    y = nv.linear_fwd(weight, shifted, torch.float32, orc.F32)
    assert nv.last_path() != "decode"
    wc = _oracle_w(weight, codes, scales, orc.F32)
    assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc)) <= TOL_F32


def test_decode_wait_that_runs_out_raises_the_flag_and_returns():
    """The library's self-test of its bounded waits: the next few-token launch announces bytes that
    never arrive, with a short wait limit.  The kernel must return (no hang, no fault), the status
    word must report the few-token kernel (bit 0), and the next call must be healthy again."""
    import time

    rng = np.random.default_rng(78)
    weight, codes, scales = make_weight(rng, 1024, 4096, orc.I4)
    x_np, x = act(rng, 4, 4096, orc.BF16)
    wc = _oracle_w(weight, codes, scales, orc.F32)
    want = orc.frozen_linear_forward(x_np, wc)
    y = nv.linear_fwd(weight, x, torch.float32, orc.F32)
    assert nv.last_path() == "decode"
    assert nv.lib().caifq_device_status() == 0
    nv.lib().caifq_selftest_stall_next_decode()
    t0 = time.time()
    nv.linear_fwd(weight, x, torch.float32, orc.F32)
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0
    assert nv.lib().caifq_device_status() & 1
    y = nv.linear_fwd(weight, x, torch.float32, orc.F32)
    assert nv.lib().caifq_device_status() == 0
    assert max_rel_err(y.cpu().numpy(), want) <= TOL_F32


def test_umma_wait_that_runs_out_raises_the_flag_and_returns():
    """The tensor-core kernel's give-up path: one activation tile announces bytes that never arrive.  The
    first wait that runs out makes every later wait of the CTA return at once, so the kernel ends within
    about one (short, self-test) limit instead of one limit per remaining wait; its tensor memory is
    released (the next launch can allocate it) and the status word reports bit 1."""
    import time

    weight, wc, x_np, x, dy_np, dy = _umma_case(orc.I8, orc.BF16, 512, 1024, 1024, 4242)
    y = nv.linear_fwd(weight, x, torch.float32, orc.BF16)
    assert nv.last_path() == "umma"
    assert nv.lib().caifq_device_status() == 0
    nv.lib().caifq_selftest_stall_next_umma()
    t0 = time.time()
    nv.linear_fwd(weight, x, torch.float32, orc.BF16)
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0
    assert nv.lib().caifq_device_status() & 2
    y2 = nv.linear_fwd(weight, x, torch.float32, orc.BF16)
    dx = nv.linear_dx(weight, dy, torch.float32, orc.BF16)
    assert nv.lib().caifq_device_status() == 0
    assert torch.equal(y, y2)
    assert max_rel_err(dx.cpu().numpy(), orc.frozen_linear_backward(dy_np, wc, orc.BF16)) <= TOL_16


@pytest.mark.parametrize("storage,compute,tol", [
    (orc.I8, orc.BF16, TOL_16),
    (orc.I8, orc.F32, TOL_F32),
    (orc.I4, orc.BF16, TOL_16),
    (orc.I4, orc.F32, TOL_F32),
    (orc.BF16, orc.F32, TOL_F32),
])
def test_umma_cta_pairs_equal_single_ctas(storage, compute, tol, monkeypatch):
    """256-wide tiles on CTA pairs (one `cta_group::2` MMA of 256 rows over two SMs, operands staged half
    and half, barriers of the leader CTA signalled across the cluster) accumulate every output element
    over k in the same order as a single CTA's two 128-row MMAs: the results are bit-equal, for the
    forward pass (K-major weights) and dX (MN-major), and sampled rows hold the oracle's bound."""
    m, in_dim, out_dim = 10007, 512, 1024
    weight, wc, x_np, x, dy_np, dy = _umma_case(storage, compute, m, in_dim, out_dim, 9100 + storage)
    monkeypatch.setenv("CAIFQ_UMMA_PAIR", "0")
    y1 = nv.linear_fwd(weight, x, torch.float32, compute)
    dx1 = nv.linear_dx(weight, dy, torch.bfloat16, compute)
    monkeypatch.setenv("CAIFQ_UMMA_PAIR", "1")
    y2 = nv.linear_fwd(weight, x, torch.float32, compute)
    assert nv.last_path() == "umma"
    dx2 = nv.linear_dx(weight, dy, torch.bfloat16, compute)
    assert nv.lib().caifq_device_status() == 0
    assert nv.lib().caifq_umma_pair_capacity() >= 1
    assert torch.equal(y1, y2)
    assert torch.equal(dx1, dx2)
    rows = np.r_[0:8, 5000:5008, m - 8:m]
    assert max_rel_err(y2[rows].cpu().numpy(), orc.frozen_linear_forward(x_np[rows], wc, compute)) <= tol
    want_dx = orc.round_through(orc.frozen_linear_backward(dy_np[rows], wc, compute), orc.BF16)
    assert max_rel_err(dx2[rows].float().cpu().numpy(), want_dx) <= max(tol, 1e-2)   # one bf16 rounding of the output


def test_umma_cta_pair_wait_that_runs_out_returns(monkeypatch):
    """The give-up path with CTA pairs: the leader's wait runs out, both CTAs of every pair leave their
    loops, meet at the cluster barrier, release their tensor memory, and the next launch is correct."""
    import time

    monkeypatch.setenv("CAIFQ_UMMA_PAIR", "1")
    weight, wc, x_np, x, dy_np, dy = _umma_case(orc.I8, orc.BF16, 10007, 512, 1024, 4243)
    y = nv.linear_fwd(weight, x, torch.float32, orc.BF16)
    assert nv.lib().caifq_device_status() == 0
    nv.lib().caifq_selftest_stall_next_umma()
    t0 = time.time()
    nv.linear_fwd(weight, x, torch.float32, orc.BF16)
    torch.cuda.synchronize()
    assert time.time() - t0 < 1.0
    assert nv.lib().caifq_device_status() & 2
    y2 = nv.linear_fwd(weight, x, torch.float32, orc.BF16)
    assert nv.lib().caifq_device_status() == 0
    assert torch.equal(y, y2)


@pytest.mark.parametrize("storage,outs,m", [
    (orc.I4, (4096, 1024, 1024), 1),        # q, k, v of the Llama-shaped block
    (orc.I4, (4096, 1024, 1024), 16),
    (orc.I4, (1416, 1032, 520), 4),         # boundaries that are multiples of 8 but not of 16: items straddle layers
    (orc.I8, (1416, 1032, 520, 264), 9),    # int8: every layer has its own per-tensor scale
    (orc.I4, (14336, 14336), 4),            # gate, up
])
def test_decode_several_layers_that_share_the_input_in_one_launch(storage, outs, m):
    """caifq_linear_fwd_multi: one persistent launch streams the code matrices of all layers; every output
    has the bits the layer's own caifq_linear_fwd call gives, and holds the oracle's bound."""
    in_dim = 4096 if outs[0] >= 4096 else 1024
    rng = np.random.default_rng(7700 + sum(outs) + m)
    ws, wcs = [], []
    for o in outs:
        w, codes, scales = make_weight(rng, o, in_dim, storage)
        ws.append(w)
        wcs.append(_oracle_w(w, codes, scales, orc.F32))
    x_np, x = act(rng, m, in_dim, orc.BF16)
    y = nv.linear_fwd_multi(ws, x, torch.float32, orc.F32)
    assert nv.last_path() == "decode"
    assert nv.lib().caifq_device_status() == 0
    col = 0
    for w, wc in zip(ws, wcs):
        single = nv.linear_fwd(w, x, torch.float32, orc.F32)
        assert nv.last_path() == "decode"
        assert torch.equal(y[:, col:col + w.out_dim], single)
        assert max_rel_err(single.cpu().numpy(), orc.frozen_linear_forward(x_np, wc, orc.F32)) <= TOL_F32
        col += w.out_dim
    # refused, not mis-computed: a layer (not the last) whose row count is not a multiple of 8, and many tokens
    odd = [make_weight(rng, 1028, in_dim, storage)[0], ws[0]]
    with pytest.raises(nv.CaifqError):
        nv.linear_fwd_multi(odd, x, torch.float32, orc.F32)
    with pytest.raises(nv.CaifqError):
        nv.linear_fwd_multi(ws, act(rng, 32, in_dim, orc.BF16)[1], torch.float32, orc.F32)


@pytest.mark.parametrize("storage,compute,sd,m", [
    (orc.I4, orc.BF16, orc.BF16, 300),    # tensor-core path, bf16 residual stream
    (orc.I8, orc.F32, orc.F32, 77),       # tensor-core path, fp32 stream
    (orc.I4, orc.BF16, orc.BF16, 4),      # few tokens: the accumulate epilogue lives on the other kernels
    (orc.F16, orc.F16, orc.F16, 20),      # generic kernel
])
def test_forward_with_the_residual_add_in_the_epilogue(storage, compute, sd, m):
    """caifq_linear_fwd_residual: the block's x = x + sub_out with sub_out the projection's output cast to
    the stream's dtype, computed in the product's epilogue: round(round(y) + residual)."""
    in_dim, out_dim = 512, 384
    rng = np.random.default_rng(8800 + storage + m)
    weight, codes, scales = make_weight(rng, out_dim, in_dim, storage)
    wc = _oracle_w(weight, codes, scales, compute)
    x_np, x = act(rng, m, in_dim, sd)
    res_np, res = act(rng, m, out_dim, sd)
    got = nv.linear_fwd_residual(weight, x, res.clone(), compute)
    y = orc.round_through(orc.frozen_linear_forward(x_np, wc, compute), sd)
    want = orc.round_through(y + res_np, sd)
    tol = TOL_F32 if compute == orc.F32 else TOL_16
    assert max_rel_err(got.float().cpu().numpy(), want) <= tol
    # the same bits as the separate product followed by an add in the stream's dtype
    sep = nv.linear_fwd(weight, x, TORCH_DTYPE[sd], compute)
    if nv.last_path() != "decode":     # (the few-token kernel sums in another order than the kernel that accumulates)
        assert torch.equal(got, (sep.float() + res.float()).to(TORCH_DTYPE[sd]))


@pytest.mark.parametrize("storage", [orc.I4, orc.I8, orc.BF16])
def test_layers_sharing_their_input_as_one_product_over_concatenated_weights(storage):
    """caifq_linear_fwd_concat / caifq_linear_dx_concat on the attention shapes of the Llama-like config scaled
    down (q of 1024, k and v of 256 features over 512 inputs, 4099 tokens): the columns of every layer hold what
    the oracle gives for that layer alone (weights as bf16 compute sees them), dX the sum over the layers, and
    both agree with the per-layer calls."""
    rng = np.random.default_rng(700 + storage)
    in_dim, outs, m = 512, (1024, 256, 256), 4099
    layers = [make_weight(rng, o, in_dim, storage, std=0.05) for o in outs]
    ws = [l[0] for l in layers]
    wc = [orc.weight_to_compute(l[1], l[2], storage, in_dim, o, orc.BF16, l[0].scheme, l[0].group_size)
          for l, o in zip(layers, outs)]
    x_np, x = act(rng, m, in_dim, orc.BF16)
    dy_np, dy = act(rng, m, sum(outs), orc.BF16)
    y = nv.linear_concat(ws, x, out_dtype=torch.float32)
    assert nv.last_path() == "umma"
    dx = nv.linear_concat(ws, dy, backward=True, out_dtype=torch.float32)
    assert nv.lib().caifq_device_status() == 0
    rows = np.r_[0:8, 2000:2008, m - 8:m]
    col = 0
    want_dx = np.zeros((rows.size, in_dim), np.float64)
    per_layer_dx = torch.zeros(m, in_dim, device="cuda")
    for w, c, o in zip(ws, wc, outs):
        want = orc.frozen_linear_forward(x_np[rows], c, orc.BF16)
        assert max_rel_err(y[rows, col:col + o].cpu().numpy(), want) <= TOL_16
        alone = nv.linear_fwd(w, x, torch.float32, orc.BF16)
        assert max_rel_err(y[:, col:col + o].cpu().numpy(), alone.cpu().numpy()) <= TOL_16
        want_dx += orc.frozen_linear_backward(dy_np[rows, col:col + o], c, orc.BF16)
        per_layer_dx += nv.linear_dx(w, dy[:, col:col + o].contiguous(), torch.float32, orc.BF16)
        col += o
    assert max_rel_err(dx[rows].cpu().numpy(), want_dx) <= TOL_16
    assert max_rel_err(dx.cpu().numpy(), per_layer_dx.cpu().numpy()) <= TOL_16
    # refusals: fp32 compute has no bf16 operand; a short workspace
    arr = nv._weight_array(ws)
    y2 = torch.empty(m, sum(outs), device="cuda")
    scratch = torch.empty(1024, dtype=torch.uint8, device="cuda")
    rc = nv.lib().caifq_linear_fwd_concat(arr, 3, nv._ptr(x), nv.BF16, m, nv._ptr(y2), nv.F32, nv.BF16, nv._ptr(scratch),
                                          1024, nv._stream())
    assert rc == 1 and b"workspace" in nv.lib().caifq_last_error()
    big = torch.empty(nv.lib().caifq_linear_concat_workspace_bytes(arr, 3), dtype=torch.uint8, device="cuda")
    rc = nv.lib().caifq_linear_fwd_concat(arr, 3, nv._ptr(x), nv.BF16, m, nv._ptr(y2), nv.F32, nv.F32, nv._ptr(big),
                                          big.numel(), nv._stream())
    assert rc == 1 and b"BF16" in nv.lib().caifq_last_error()
