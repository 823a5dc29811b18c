"""GPU parity of the LoRA adapter path, routing/dispatch kernels and the grouped
frozen experts against the CPU oracle (and the reference kernels where built)."""
import numpy as np
import pytest
import torch

import caif_oracle as orc
import refkernels as ref
from caif_b200 import native as nv
from gpu_util import TORCH_DTYPE, act, dev, make_weight, max_rel_err, to_dev

pytestmark = pytest.mark.gpu

TOL = {orc.F32: 1e-4, orc.BF16: 2e-2, orc.F16: 2e-2}


def _lora_case(rng, storage, sd, in_dim, out_dim, m, rank, alpha):
    weight, codes, scales = make_weight(rng, out_dim, in_dim, storage)
    bound = np.sqrt(1.0 / in_dim)
    a = orc.round_through(rng.uniform(-bound, bound, (rank, in_dim)).astype(np.float32), sd)
    b = orc.round_through((rng.standard_normal((out_dim, rank)) * 1e-3).astype(np.float32), sd)
    x_np, x = act(rng, m, in_dim, sd)
    dy_np, dy = act(rng, m, out_dim, sd)
    lora = nv.Lora(to_dev(a, TORCH_DTYPE[sd]), to_dev(b, TORCH_DTYPE[sd]), alpha)
    return weight, codes, scales, a, b, x_np, x, dy_np, dy, lora


@pytest.mark.parametrize("storage,sd,compute", [
    (orc.I8, orc.F32, orc.F32),
    (orc.I8, orc.BF16, orc.F32),   # the training config's cell: bf16 storage, fp32 compute
    (orc.I4, orc.BF16, orc.BF16),
    (orc.F16, orc.F16, orc.F16),
])
def test_lora_forward_backward(storage, sd, compute):
    rng = np.random.default_rng(300 + storage + sd)
    in_dim, out_dim, m, rank, alpha = 256, 192, 77, 16, 32.0
    weight, codes, scales, a, b, x_np, x, dy_np, dy, lora = _lora_case(rng, storage, sd, in_dim, out_dim, m, rank,
                                                                         alpha)
    wc = orc.weight_to_compute(codes, scales, storage, in_dim, out_dim, compute, weight.scheme, weight.group_size)
    base = orc.frozen_linear_forward(x_np, wc, compute)
    want_y, want_h = orc.lora_forward(x_np, base, a, b, alpha, sd)
    y, hidden = nv.lora_linear_fwd(weight, lora, x, compute)
    tol = max(TOL[sd], TOL[compute])
    assert y.dtype == TORCH_DTYPE[sd]
    assert max_rel_err(y.float().cpu().numpy(), want_y) <= tol
    assert max_rel_err(hidden.float().cpu().numpy(), want_h) <= tol
    dx_base = orc.frozen_linear_backward(dy_np, wc, compute)
    want_dx, want_da, want_db = orc.lora_backward(dy_np, x_np, want_h, dx_base, a, b, alpha, sd)
    dx, d_a, d_b = nv.lora_linear_bwd(weight, lora, dy, x, hidden, compute)
    assert max_rel_err(dx.float().cpu().numpy(), want_dx) <= tol
    assert max_rel_err(d_a.float().cpu().numpy(), want_da) <= tol
    assert max_rel_err(d_b.float().cpu().numpy(), want_db) <= tol


def test_lora_zero_b_equals_base_and_gradients_overwrite():
    rng = np.random.default_rng(301)
    weight, codes, scales, a, b, x_np, x, dy_np, dy, lora = _lora_case(rng, orc.I8, orc.F32, 128, 96, 33, 8, 16.0)
    zero_b = nv.Lora(lora.a, torch.zeros_like(lora.b), 16.0)
    y, hidden = nv.lora_linear_fwd(weight, zero_b, x)
    base = nv.linear_fwd(weight, x)
    assert torch.equal(y, base)   # reference: tests/test_device_lora_adapter.cpp:371-442
    dx1, da1, db1 = nv.lora_linear_bwd(weight, lora, dy, x, hidden)
    dx2, da2, db2 = nv.lora_linear_bwd(weight, lora, dy, x, hidden)
    assert float(da1.abs().max()) > 0 and float(db1.abs().max()) > 0
    assert max_rel_err(da2.cpu().numpy(), da1.cpu().numpy()) <= 1e-5  # overwritten, not accumulated


# -------------------------------------------------------------------- routing
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_topk_and_normalize_bit_exact(dtype):
    g = torch.Generator().manual_seed(17)
    probs = torch.softmax(torch.randn(1000, 68, generator=g), dim=-1).to(torch.bfloat16).to(dtype)
    pd = probs.to(dev()).contiguous()
    idx, val = nv.moe_topk(pd, 6)
    oidx, oval = orc.topk(probs.float().numpy(), 6)
    assert np.array_equal(idx.cpu().numpy(), oidx)
    assert np.array_equal(val.float().cpu().numpy(), oval)
    norm = nv.moe_normalize_rows(val)
    code = {torch.float32: orc.F32, torch.bfloat16: orc.BF16, torch.float16: orc.F16}[dtype]
    assert np.array_equal(norm.float().cpu().numpy(), orc.round_through(orc.normalize_rows(oval), code))
    if dtype == torch.float32 and ref.available():
        ridx, rval = ref.topk(pd, 6)
        assert torch.equal(ridx, idx) and torch.equal(rval, val)
        assert torch.equal(ref.normalize_rows(val), norm)


@pytest.mark.parametrize("dtype,rows,cols,with_bias", [
    (torch.float32, 16384, 68, False),     # the MoE config's router
    (torch.float32, 777, 64, True),
    (torch.bfloat16, 1000, 68, True),
    (torch.bfloat16, 300, 256, False),
    (torch.float32, 50, 300, True),        # more than 128 columns: the strided per-thread scan
    (torch.float32, 9, 1, False),
])
def test_router_softmax_bit_exact_with_the_reference_kernel(dtype, rows, cols, with_bias):
    """Router probabilities: bit-identical to the reference's softmax kernel run on the same GPU
    (so the top-k indices that follow are identical too), and within a few ulp of the CPU oracle,
    whose expf is the host's."""
    g = torch.Generator().manual_seed(rows + cols)
    logits = (torch.randn(rows, cols, generator=g) * 2.0).to(dtype)
    bias = (torch.randn(cols, generator=g) * 0.5).to(dtype) if with_bias else None
    ld = logits.to(dev()).contiguous()
    bd = bias.to(dev()).contiguous() if with_bias else None
    probs = nv.moe_softmax(ld, bd)
    code = orc.F32 if dtype == torch.float32 else orc.BF16
    want = orc.round_through(orc.router_softmax(logits.float().numpy(), None if bias is None else bias.float().numpy(),
                                                code), code)
    got = probs.float().cpu().numpy()
    assert np.max(np.abs(got - want)) <= (2e-7 if dtype == torch.float32 else 1e-2) * max(1.0, float(np.max(want)))
    if ref.available():
        biased = ref.bias_add(ld, bd) if with_bias else ld
        assert torch.equal(ref.softmax(biased), probs)
        k = min(6, cols)
        ridx, _ = ref.topk(ref.softmax(biased).float().contiguous(), k)
        idx, _ = nv.moe_topk(probs.float().contiguous(), k)
        assert torch.equal(ridx, idx)
    # in place
    again = ld.clone()
    nv._check(nv.lib().caifq_moe_router_softmax(nv._ptr(again), nv._ptr(bd), nv._ptr(again), nv.dtype_code(again),
                                                rows, cols, nv._stream()), "softmax in place")
    assert torch.equal(again, probs)


def test_scale_matches_the_reference_kernel():
    g = torch.Generator().manual_seed(5)
    w = torch.rand(1000, 6, generator=g).to(torch.bfloat16).to(dev())
    got = nv.scale(w, 16.0)
    want = orc.round_through(w.float().cpu().numpy() * np.float32(16.0), orc.BF16)
    assert np.array_equal(got.float().cpu().numpy(), want)
    if ref.available():
        assert torch.equal(ref.scale_bf16(w, 16.0), got)
    odd = nv.scale(w, 2.5)
    assert np.array_equal(odd.float().cpu().numpy(), orc.round_through(w.float().cpu().numpy() * np.float32(2.5), orc.BF16))


def test_topk_edge_cases():
    p = torch.tensor([[0.25, 0.25, 0.25, 0.25], [-2e30, -2e30, -2e30, -2e30], [0.0, 1.0, float("nan"), 1.0]])
    idx, val = nv.moe_topk(p.to(dev()), 2)
    assert idx.cpu().tolist() == [[0, 1], [0, 0], [1, 3]]
    wide = torch.rand(5, 1000).to(dev())
    idx, val = nv.moe_topk(wide, 8)
    oidx, _ = orc.topk(wide.cpu().numpy(), 8)
    assert np.array_equal(idx.cpu().numpy(), oidx)
    n = nv.moe_normalize_rows(wide)
    assert np.array_equal(n.cpu().numpy(), orc.normalize_rows(wide.cpu().numpy()))


@pytest.mark.parametrize("tokens,top_k,experts,capacity", [
    (16384, 6, 68, 0),     # the MoE config's size
    (1000, 2, 8, 100),     # capacity drops
    (37, 3, 5, 0),
    (1, 1, 1, 0),
    (3000, 4, 256, 0),
])
def test_dispatch_map_bit_exact(tokens, top_k, experts, capacity):
    rng = np.random.default_rng(tokens + experts)
    idx = rng.integers(0, experts, (tokens, top_k)).astype(np.int32)
    if tokens > 10:
        idx[5, 0] = -1          # ignored entries, as the reference's range check does
        idx[7, top_k - 1] = experts
    dmap, off = nv.moe_build_dispatch(to_dev(idx), experts, capacity)
    odmap, ooff, total = orc.build_dispatch_map(idx, experts, capacity)
    assert np.array_equal(off.cpu().numpy(), ooff)
    assert np.array_equal(dmap.cpu().numpy(), odmap)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dispatch_and_combine(dtype):
    rng = np.random.default_rng(19)
    tokens, dim, top_k, experts = 500, 96, 6, 68
    code = orc.F32 if dtype == torch.float32 else orc.BF16
    x_np, x = act(rng, tokens, dim, code)
    probs = rng.random((tokens, experts)).astype(np.float32)
    idx, val = orc.topk(probs, top_k)
    w_np = orc.round_through(orc.normalize_rows(val), code)
    dmap, off, total = orc.build_dispatch_map(idx, experts, capacity=40)
    d_idx, d_map, d_off = to_dev(idx), to_dev(dmap), to_dev(off)
    buf = nv.moe_dispatch(x, d_idx, d_map, d_off, total)
    obuf = orc.moe_dispatch(x_np, idx, dmap, off, total)
    assert np.array_equal(buf.float().cpu().numpy(), obuf)
    out = nv.moe_combine(buf, d_idx, to_dev(w_np, dtype), d_map, d_off, tokens)
    want = orc.round_through(orc.moe_combine(obuf, idx, w_np, dmap, off, tokens), code)
    assert np.array_equal(out.float().cpu().numpy(), want)
    if dtype == torch.float32 and ref.available():
        assert torch.equal(ref.moe_dispatch(x, d_idx, d_map, d_off, total), buf)
        assert torch.equal(ref.moe_combine(buf, d_idx, to_dev(w_np), d_map, d_off, tokens), out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim", [96, 2048, 37])
def test_combine_and_dispatch_backward(dtype, dim):
    """The three backward kernels of the dispatch/combine pair, bit for bit against the oracle
    (and the reference's kernels in fp32), with a capacity that drops some picks."""
    rng = np.random.default_rng(23 + dim)
    tokens, top_k, experts = 300, 6, 68
    code = orc.F32 if dtype == torch.float32 else orc.BF16
    g_np, g = act(rng, tokens, dim, code)
    probs = rng.random((tokens, experts)).astype(np.float32)
    idx, val = orc.topk(probs, top_k)
    w_np = orc.round_through(orc.normalize_rows(val), code)
    dmap, off, total = orc.build_dispatch_map(idx, experts, capacity=30)
    buf_np = orc.round_through(rng.standard_normal((total, dim)).astype(np.float32), code)
    d_idx, d_map, d_off = to_dev(idx), to_dev(dmap), to_dev(off)
    w, buf = to_dev(w_np, dtype), to_dev(buf_np, dtype)

    gbuf = nv.moe_combine_bwd_grad_expert(g, d_idx, w, d_map, d_off, total)
    want = orc.round_through(orc.moe_combine_bwd_grad_expert(g_np, idx, w_np, dmap, off, total), code)
    assert np.array_equal(gbuf.float().cpu().numpy(), want)

    gw = nv.moe_combine_bwd_grad_weights(g, buf, d_idx, d_map, d_off)
    want_gw = orc.round_through(orc.moe_combine_bwd_grad_weights(g_np, buf_np, idx, dmap, off), code)
    assert np.array_equal(gw.float().cpu().numpy(), want_gw)

    gin = nv.moe_dispatch_bwd(gbuf, d_idx, d_map, d_off, tokens)
    want_gin = orc.round_through(orc.moe_dispatch_bwd(want, idx, dmap, off, tokens), code)
    assert np.array_equal(gin.float().cpu().numpy(), want_gin)

    if dtype == torch.float32 and ref.available():
        assert torch.equal(ref.moe_combine_bwd_grad_expert(g, d_idx, w, d_map, d_off, total), gbuf)
        assert torch.equal(ref.moe_combine_bwd_grad_weights(g, buf, d_idx, d_map, d_off), gw)
        assert torch.equal(ref.moe_dispatch_bwd(gbuf, d_idx, d_map, d_off, tokens), gin)


# ------------------------------------------------------------ grouped experts
@pytest.mark.parametrize("storage,sd,compute", [(orc.I4, orc.BF16, orc.BF16), (orc.I8, orc.F32, orc.F32),
                                                (orc.I4, orc.F32, orc.F32)])
def test_grouped_frozen_experts(storage, sd, compute):
    rng = np.random.default_rng(400 + storage + sd)
    experts, in_dim, hid = 5, 128, 256
    counts = [13, 0, 40, 1, 27]
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    total = int(offsets[-1])
    gate, up, down, o_gate, o_up, o_down = [], [], [], [], [], []
    for _ in range(experts):
        for lst, olst, (o, i) in ((gate, o_gate, (hid, in_dim)), (up, o_up, (hid, in_dim)),
                                  (down, o_down, (in_dim, hid))):
            w, codes, scales = make_weight(rng, o, i, storage, std=0.05)
            lst.append(w)
            olst.append(orc.weight_to_compute(codes, scales, storage, i, o, compute, w.scheme, w.group_size))
    x_np, x = act(rng, total, in_dim, sd)
    dy_np, dy = act(rng, total, in_dim, sd)
    out, gate_out, up_out = nv.grouped_expert_fwd(gate, up, down, offsets.tolist(), x, compute)
    dx = nv.grouped_expert_bwd(gate, up, down, offsets.tolist(), dy, gate_out, up_out, compute)
    tol = max(TOL[sd], TOL[compute])
    for e in range(experts):
        lo, hi = offsets[e], offsets[e + 1]
        if lo == hi:
            continue
        want, g, u = orc.frozen_expert_forward(x_np[lo:hi], o_gate[e], o_up[e], o_down[e], compute, sd)
        assert max_rel_err(out[lo:hi].float().cpu().numpy(), want) <= tol
        assert max_rel_err(gate_out[lo:hi].float().cpu().numpy(), g) <= tol
        want_dx = orc.frozen_expert_backward(dy_np[lo:hi], g, u, o_gate[e], o_up[e], o_down[e], compute, sd)
        assert max_rel_err(dx[lo:hi].float().cpu().numpy(), want_dx) <= tol


@pytest.mark.parametrize("storage,sd,compute,rows", [
    (orc.I8, orc.F32, orc.F32, [13, 0, 40]),            # per-expert calls of the generic kernel
    (orc.I4, orc.BF16, orc.BF16, [300, 0, 700, 1]),     # grouped tensor-core launches
])
def test_frozen_experts_without_a_gate_projection(storage, sd, compute, rows):
    """UseGated() == false: down( silu(up(x)) ), dX = up.Bwd( SiLUBackward(up_out, down.Bwd(dy)) )
    (src/caif_device_moe_frozen_expert.cpp:158-162, 318-331), selected by gate == NULL."""
    rng = np.random.default_rng(450 + storage)
    in_dim, hid = 256, 384
    offsets = np.concatenate([[0], np.cumsum(rows)]).astype(np.int32)
    total = int(offsets[-1])
    up, down, o_up, o_down = [], [], [], []
    for _ in rows:
        for lst, olst, (o, i) in ((up, o_up, (hid, in_dim)), (down, o_down, (in_dim, hid))):
            w, codes, scales = make_weight(rng, o, i, storage, std=0.05)
            lst.append(w)
            olst.append(orc.weight_to_compute(codes, scales, storage, i, o, compute, w.scheme, w.group_size))
    x_np, x = act(rng, total, in_dim, sd)
    dy_np, dy = act(rng, total, in_dim, sd)
    out, gate_out, up_out = nv.grouped_expert_fwd(None, up, down, offsets.tolist(), x, compute)
    assert gate_out is None
    dx = nv.grouped_expert_bwd(None, up, down, offsets.tolist(), dy, None, up_out, compute)
    assert nv.lib().caifq_device_status() == 0
    tol = max(TOL[sd], TOL[compute])
    for e in range(len(rows)):
        lo, hi = offsets[e], offsets[e + 1]
        if lo == hi:
            continue
        want, _, u = orc.frozen_expert_forward(x_np[lo:hi], None, o_up[e], o_down[e], compute, sd)
        assert max_rel_err(out[lo:hi].float().cpu().numpy(), want) <= tol
        assert max_rel_err(up_out[lo:hi].float().cpu().numpy(), u) <= tol
        want_dx = orc.frozen_expert_backward(dy_np[lo:hi], None, u, None, o_up[e], o_down[e], compute, sd)
        assert max_rel_err(dx[lo:hi].float().cpu().numpy(), want_dx) <= tol


@pytest.mark.parametrize("storage,compute,experts,in_dim,hid,mean_rows", [
    (orc.I4, orc.BF16, 6, 2048, 1408, 300),    # the MoE config's expert shape, ragged row counts
    (orc.I4, orc.F32, 3, 512, 640, 200),       # fp32 compute: two-term int4 operand
    (orc.I8, orc.F32, 4, 256, 512, 700),
    (orc.I4, orc.BF16, 131, 128, 128, 5),      # more experts than one launch's table holds
])
def test_grouped_frozen_experts_single_launch(storage, compute, experts, in_dim, hid, mean_rows):
    """Quantized experts of one shape on bf16 rows: each of the six products is one grouped
    tensor-core launch over the packed buffer; per-expert results match the oracle's loop."""
    rng = np.random.default_rng(4100 + experts)
    counts = rng.integers(0, 2 * mean_rows, experts)
    counts[1] = 0
    counts[-1] = 1
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    total = int(offsets[-1])
    sd = orc.BF16
    gate, up, down, o_gate, o_up, o_down = [], [], [], [], [], []
    for _ in range(experts):
        for lst, olst, (o, i) in ((gate, o_gate, (hid, in_dim)), (up, o_up, (hid, in_dim)),
                                  (down, o_down, (in_dim, hid))):
            w, codes, scales = make_weight(rng, o, i, storage, std=0.05)
            lst.append(w)
            olst.append(orc.weight_to_compute(codes, scales, storage, i, o, compute, w.scheme, w.group_size))
    x_np, x = act(rng, total, in_dim, sd)
    dy_np, dy = act(rng, total, in_dim, sd)
    out, gate_out, up_out = nv.grouped_expert_fwd(gate, up, down, offsets.tolist(), x, compute)
    assert nv.last_path() == "umma-grouped"
    dx = nv.grouped_expert_bwd(gate, up, down, offsets.tolist(), dy, gate_out, up_out, compute)
    assert nv.last_path() == "umma-grouped"
    assert nv.lib().caifq_device_status() == 0
    tol = 2e-2
    check = range(experts) if experts <= 8 else list(range(0, experts, 13)) + [experts - 1]
    for e in check:
        lo, hi = offsets[e], offsets[e + 1]
        if lo == hi:
            continue
        want, g, u = orc.frozen_expert_forward(x_np[lo:hi], o_gate[e], o_up[e], o_down[e], compute, sd)
        assert max_rel_err(out[lo:hi].float().cpu().numpy(), want) <= tol
        assert max_rel_err(gate_out[lo:hi].float().cpu().numpy(), g) <= tol
        assert max_rel_err(up_out[lo:hi].float().cpu().numpy(), u) <= tol
        want_dx = orc.frozen_expert_backward(dy_np[lo:hi], g, u, o_gate[e], o_up[e], o_down[e], compute, sd)
        assert max_rel_err(dx[lo:hi].float().cpu().numpy(), want_dx) <= tol


def test_grouped_experts_at_the_moe_config_size_equal_single_expert_calls():
    """64 int4 experts 2048 -> 1408 -> 2048, 16384 tokens routed top-6 (98,304 packed rows): the grouped
    launches must give every expert's rows exactly what a call with that expert alone gives (an
    expert's tiles never mix rows or codes of its neighbours), forward and dX; one expert is also
    checked against the oracle."""
    g = torch.Generator(device="cuda").manual_seed(77)
    hidden, ffn, n_exp, tokens, top_k = 2048, 1408, 64, 16384, 6
    gate, up, down = [], [], []
    for _ in range(n_exp):
        for lst, (o, i) in ((gate, (ffn, hidden)), (up, (ffn, hidden)), (down, (hidden, ffn))):
            wf = torch.randn(o * i, generator=g, device="cuda") * 0.02
            pk, sc = nv.quantize_int4(wf, 128)
            lst.append(nv.Weight(pk, nv.I4, i, o, sc, group_size=128))
    probs = torch.softmax(torch.randn(tokens, n_exp, generator=g, device="cuda"), dim=-1)
    idx, _ = nv.moe_topk(probs, top_k)
    dmap, off = nv.moe_build_dispatch(idx, n_exp)
    offs = off.cpu().tolist()
    total = offs[-1]
    assert total == tokens * top_k
    x = torch.randn(tokens, hidden, generator=g, device="cuda").to(torch.bfloat16)
    buf = nv.moe_dispatch(x, idx, dmap, off, total)
    dy = torch.randn(total, hidden, generator=g, device="cuda").to(torch.bfloat16)
    out, g_out, u_out = nv.grouped_expert_fwd(gate, up, down, offs, buf, orc.BF16)
    assert nv.last_path() == "umma-grouped"
    dx = nv.grouped_expert_bwd(gate, up, down, offs, dy, g_out, u_out, orc.BF16)
    assert nv.lib().caifq_device_status() == 0
    for e in (0, 17, 63):
        lo, hi = offs[e], offs[e + 1]
        o1, g1, u1 = nv.grouped_expert_fwd([gate[e]], [up[e]], [down[e]], [0, hi - lo], buf[lo:hi].contiguous(),
                                           orc.BF16)
        d1 = nv.grouped_expert_bwd([gate[e]], [up[e]], [down[e]], [0, hi - lo], dy[lo:hi].contiguous(), g1, u1,
                                   orc.BF16)
        assert torch.equal(o1, out[lo:hi]) and torch.equal(g1, g_out[lo:hi]) and torch.equal(u1, u_out[lo:hi])
        assert torch.equal(d1, dx[lo:hi])
    # three experts (first, middle, last) against the oracle on 64 of their rows each, forward and dX
    for e in (0, 17, 63):
        lo = offs[e] + 5
        ws = []
        for w in (gate[e], up[e], down[e]):
            codes = w.codes.cpu().numpy()
            scales = w.scales.cpu().view(torch.int16).numpy().view(np.uint16)
            ws.append(orc.weight_to_compute(codes, scales, orc.I4, w.in_dim, w.out_dim, orc.BF16, 0, 128))
        xe = buf[lo:lo + 64].float().cpu().numpy()
        want, og, ou = orc.frozen_expert_forward(xe, ws[0], ws[1], ws[2], orc.BF16, orc.BF16, exact=False)
        assert max_rel_err(out[lo:lo + 64].float().cpu().numpy(), want) <= 2e-2
        assert max_rel_err(g_out[lo:lo + 64].float().cpu().numpy(), og) <= 2e-2
        # the backward from the kernel's own saved gate/up values, as the layer does it
        want_dx = orc.frozen_expert_backward(dy[lo:lo + 64].float().cpu().numpy(),
                                             g_out[lo:lo + 64].float().cpu().numpy(),
                                             u_out[lo:lo + 64].float().cpu().numpy(), ws[0], ws[1], ws[2], orc.BF16,
                                             orc.BF16, exact=False)
        assert max_rel_err(dx[lo:lo + 64].float().cpu().numpy(), want_dx) <= 2e-2


@pytest.mark.parametrize("storage,compute", [(orc.I8, orc.F32), (orc.I4, orc.BF16), (orc.I4, orc.F32)])
@pytest.mark.parametrize("m,in_dim,out_dim,rank", [(300, 512, 384, 16), (1024, 1024, 1024, 8), (130, 256, 640, 64)])
def test_lora_fused_tensor_core_path(storage, compute, m, in_dim, out_dim, rank):
    """bf16 adapter on a quantized base with enough tokens: the LoRA products ride in the tensor-core
    kernel (forward and dX) and the token reductions use the skinny kernels."""
    rng = np.random.default_rng(700 + storage + m)
    alpha, sd = 32.0, orc.BF16
    weight, codes, scales, a, b, x_np, x, dy_np, dy, lora = _lora_case(rng, storage, sd, in_dim, out_dim, m, rank,
                                                                         alpha)
    wc = orc.weight_to_compute(codes, scales, storage, in_dim, out_dim, compute, weight.scheme, weight.group_size)
    y, hidden = nv.lora_linear_fwd(weight, lora, x, compute)
    assert nv.last_path() == "umma"
    want_y, want_h = orc.lora_forward(x_np, orc.frozen_linear_forward(x_np, wc, compute), a, b, alpha, sd)
    assert max_rel_err(hidden.float().cpu().numpy(), want_h) <= TOL[sd]
    assert max_rel_err(y.float().cpu().numpy(), want_y) <= TOL[sd]
    dx, d_a, d_b = nv.lora_linear_bwd(weight, lora, dy, x, hidden, compute)
    assert nv.last_path() == "umma"
    assert nv.lib().caifq_device_status() == 0
    want_dx, want_da, want_db = orc.lora_backward(dy_np, x_np, want_h, orc.frozen_linear_backward(dy_np, wc, compute),
                                                  a, b, alpha, sd)
    assert max_rel_err(dx.float().cpu().numpy(), want_dx) <= TOL[sd]
    assert max_rel_err(d_a.float().cpu().numpy(), want_da) <= TOL[sd]
    assert max_rel_err(d_b.float().cpu().numpy(), want_db) <= TOL[sd]
    # the LoRA term must really be there: with B scaled up 100x the outputs move accordingly
    big = nv.Lora(lora.a, (lora.b.float() * 100).to(torch.bfloat16), alpha)
    y_big, _ = nv.lora_linear_fwd(weight, big, x, compute)
    want_big, _ = orc.lora_forward(x_np, orc.frozen_linear_forward(x_np, wc, compute), a,
                                   orc.round_through(b * 100, sd), alpha, sd)
    assert max_rel_err(y_big.float().cpu().numpy(), want_big) <= TOL[sd]


def test_lora_at_the_training_config_size():
    """4096 -> 4096 int8 per-tensor base, LoRA r16 a32, M = 8192 bf16 tokens, fp32 compute (config 3): Y and dX
    on 64 sampled rows and the whole dA and dB against the oracle (host sgemm for the big products)."""
    g = torch.Generator(device="cuda").manual_seed(1236)
    dim, m, rank, alpha = 4096, 8192, 16, 32.0
    wf = torch.randn(dim * dim, generator=g, device="cuda") * 0.02
    q, s = nv.quantize_int8_per_tensor(wf)
    weight = nv.Weight(q.view(dim, dim), nv.I8, dim, dim, s)
    a = ((torch.rand(rank, dim, generator=g, device="cuda") * 2 - 1) / 64).to(torch.bfloat16)
    b = (torch.randn(dim, rank, generator=g, device="cuda") * 1e-3).to(torch.bfloat16)
    lora = nv.Lora(a, b, alpha)
    x = torch.randn(m, dim, generator=g, device="cuda").to(torch.bfloat16)
    dy = torch.randn(m, dim, generator=g, device="cuda").to(torch.bfloat16)
    y, hidden = nv.lora_linear_fwd(weight, lora, x, nv.F32)
    assert nv.last_path() == "umma"
    dx, d_a, d_b = nv.lora_linear_bwd(weight, lora, dy, x, hidden, nv.F32)
    assert nv.lib().caifq_device_status() == 0
    wc = orc.dequantize_int8_per_tensor(q.cpu().numpy().reshape(dim, dim), s.cpu().numpy())
    a_np, b_np = a.float().cpu().numpy(), b.float().cpu().numpy()
    x_np, dy_np = x.float().cpu().numpy(), dy.float().cpu().numpy()
    rows = np.arange(0, m, m // 64)
    base = orc.frozen_linear_forward(x_np[rows], wc, orc.F32, exact=False)
    want_y, want_h = orc.lora_forward(x_np[rows], base, a_np, b_np, alpha, orc.BF16, exact=False)
    assert max_rel_err(hidden[rows].float().cpu().numpy(), want_h) <= 2e-2
    assert max_rel_err(y[rows].float().cpu().numpy(), want_y) <= 2e-2
    # backward over ALL tokens (dA and dB reduce over them); hidden is the kernel's own, as the layer caches it
    dx_base = orc.frozen_linear_backward(dy_np, wc, orc.F32, exact=False)
    want_dx, want_da, want_db = orc.lora_backward(dy_np, x_np, hidden.float().cpu().numpy(), dx_base, a_np, b_np, alpha,
                                                  orc.BF16, exact=False)
    assert max_rel_err(dx[rows].float().cpu().numpy(), want_dx[rows]) <= 2e-2
    assert max_rel_err(d_a.float().cpu().numpy(), want_da) <= 2e-2
    assert max_rel_err(d_b.float().cpu().numpy(), want_db) <= 2e-2


def test_lora_unfused_path_accumulates_into_the_tensor_core_epilogue():
    """A rank the fused path does not take (12): the base product then ADDS into the LoRA term that is already
    in y / dx (the reference's cast-then-Add, src/caif_device_lora_adapter.cpp:170-203), through the
    tensor-core kernel's accumulate epilogue."""
    rng = np.random.default_rng(812)
    in_dim, out_dim, m, rank, alpha, sd = 1024, 768, 512, 12, 24.0, orc.BF16
    weight, codes, scales, a, b, x_np, x, dy_np, dy, lora = _lora_case(rng, orc.I8, sd, in_dim, out_dim, m, rank, alpha)
    big_b = orc.round_through(b * 300, sd)     # a LoRA term of the base's magnitude: a lost Add would show
    lora = nv.Lora(lora.a, to_dev(big_b, torch.bfloat16), alpha)
    wc = orc.weight_to_compute(codes, scales, orc.I8, in_dim, out_dim, orc.BF16, weight.scheme, weight.group_size)
    y, hidden = nv.lora_linear_fwd(weight, lora, x, orc.BF16)
    assert nv.last_path() == "umma"
    want_y, want_h = orc.lora_forward(x_np, orc.frozen_linear_forward(x_np, wc, orc.BF16), a, big_b, alpha, sd)
    assert max_rel_err(y.float().cpu().numpy(), want_y) <= 2e-2
    lora_only = want_y - orc.round_through(orc.frozen_linear_forward(x_np, wc, orc.BF16), sd)
    assert np.max(np.abs(lora_only)) > 0.1 * np.max(np.abs(want_y))       # the Add matters in this case
    dx, d_a, d_b = nv.lora_linear_bwd(weight, lora, dy, x, hidden, orc.BF16)
    assert nv.last_path() == "umma"
    want_dx, want_da, want_db = orc.lora_backward(dy_np, x_np, want_h, orc.frozen_linear_backward(dy_np, wc, orc.BF16),
                                                  a, big_b, alpha, sd)
    assert max_rel_err(dx.float().cpu().numpy(), want_dx) <= 2e-2
    assert max_rel_err(d_a.float().cpu().numpy(), want_da) <= 2e-2
    assert max_rel_err(d_b.float().cpu().numpy(), want_db) <= 2e-2


@pytest.mark.parametrize("storage,compute", [(orc.I4, orc.BF16), (orc.I8, orc.F32)])
def test_grouped_experts_on_cta_pairs_equal_single_ctas(storage, compute, monkeypatch):
    """The grouped launches (fused gate/up/SwiGLU with 128 features of each projection per tile, down,
    and the three dX launches incl. the accumulating one) on CTA pairs give the single-CTA results
    bit for bit."""
    experts, in_dim, hid = 6, 512, 384
    rng = np.random.default_rng(6200 + storage)
    counts = rng.integers(2000, 3500, experts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    total = int(offsets[-1])
    gate, up, down = [], [], []
    for _ in range(experts):
        for lst, (o, i) in ((gate, (hid, in_dim)), (up, (hid, in_dim)), (down, (in_dim, hid))):
            lst.append(make_weight(rng, o, i, storage, std=0.05)[0])
    _, x = act(rng, total, in_dim, orc.BF16)
    _, dy = act(rng, total, in_dim, orc.BF16)
    results = []
    for pair in ("0", "1"):
        monkeypatch.setenv("CAIFQ_UMMA_PAIR", pair)
        out, g, u = nv.grouped_expert_fwd(gate, up, down, offsets.tolist(), x, compute)
        assert nv.last_path() == "umma-grouped"
        dx = nv.grouped_expert_bwd(gate, up, down, offsets.tolist(), dy, g, u, compute)
        assert nv.lib().caifq_device_status() == 0
        results.append((out, g, u, dx))
    for a, b in zip(*results):
        assert torch.equal(a, b)


@pytest.mark.parametrize("storage,compute", [(orc.I8, orc.F32), (orc.I8, orc.BF16), (orc.I4, orc.BF16),
                                             (orc.I4, orc.F32)])
@pytest.mark.parametrize("m", [4608, 5003])
def test_lora_entry_points_that_expand_the_weight_once_per_call(storage, compute, m):
    """caifq_lora_linear_fwd_expanded / _bwd_expanded at a many-token size: the weight goes through a bf16
    copy in the workspace and the CTA-pair tile form.  int8: bit-equal to the plain entry points (exact
    codes, scale in the epilogue).  int4 under bf16 compute: the reference's own operand bf16(scale * code),
    so sampled rows hold the tight bound against the oracle.  int4 under fp32 compute is not expanded
    (same workspace size, same bits)."""
    in_dim, out_dim, rank = 512, 768, 16
    rng = np.random.default_rng(9300 + storage + compute)
    weight, codes, scales = make_weight(rng, out_dim, in_dim, storage, std=0.05)
    a_np = orc.round_through(rng.uniform(-1 / 16, 1 / 16, (rank, in_dim)).astype(np.float32), orc.BF16)
    b_np = orc.round_through((rng.standard_normal((out_dim, rank)) * 0.05).astype(np.float32), orc.BF16)
    lora = nv.Lora(to_dev(a_np, torch.bfloat16), to_dev(b_np, torch.bfloat16), 32.0)
    x_np, x = act(rng, m, in_dim, orc.BF16)
    dy_np, dy = act(rng, m, out_dim, orc.BF16)
    plain_f = nv.lora_fwd_workspace_bytes(weight, lora, m, compute)
    big_f = nv.lora_fwd_workspace_bytes(weight, lora, m, compute, expanded=True)
    expands = not (storage == orc.I4 and compute == orc.F32)
    assert big_f == plain_f + (in_dim * out_dim * 2 if expands else 0)
    y0, h0 = nv.lora_linear_fwd(weight, lora, x, compute)
    dx0, da0, db0 = nv.lora_linear_bwd(weight, lora, dy, x, h0, compute)
    y1, h1 = nv.lora_linear_fwd(weight, lora, x, compute, expanded=True)
    dx1, da1, db1 = nv.lora_linear_bwd(weight, lora, dy, x, h1, compute, expanded=True)
    assert nv.lib().caifq_device_status() == 0
    assert torch.equal(h0, h1)
    # (dA and dB are token reductions with fp32 atomics: the same kernels in both calls, equal up to the order)
    assert max_rel_err(da1.float().cpu().numpy(), da0.float().cpu().numpy()) <= 1e-2
    assert max_rel_err(db1.float().cpu().numpy(), db0.float().cpu().numpy()) <= 1e-2
    if storage == orc.I8 or not expands:
        assert torch.equal(y0, y1) and torch.equal(dx0, dx1)
    rows = np.r_[0:16, m - 16:m]
    wc = orc.weight_to_compute(codes, scales, storage, in_dim, out_dim, compute, weight.scheme, weight.group_size)
    base = orc.frozen_linear_forward(x_np[rows], wc, compute)
    want_y, hid = orc.lora_forward(x_np[rows], base, a_np, b_np, 32.0, orc.BF16)
    tol = 1e-2    # results are stored in bf16: one rounding of the output
    assert max_rel_err(y1[rows].float().cpu().numpy(), want_y) <= tol
    assert max_rel_err(y0[rows].float().cpu().numpy(), want_y) <= tol
    # dx of the sampled rows (dA / dB need all rows and are equal to the plain entry point's, checked above)
    base_dx = orc.frozen_linear_backward(dy_np[rows], wc, compute)
    want_dx, _, _ = orc.lora_backward(dy_np[rows], x_np[rows], hid, base_dx, a_np, b_np, 32.0, orc.BF16)
    assert max_rel_err(dx1[rows].float().cpu().numpy(), want_dx) <= 2e-2


@pytest.mark.parametrize("storage,compute,gated", [(orc.I8, orc.F32, True), (orc.I8, orc.BF16, False),
                                                   (orc.I4, orc.BF16, True), (orc.I4, orc.BF16, False)])
def test_grouped_experts_on_bf16_copies_expanded_once_per_step(storage, compute, gated):
    """caifq_grouped_expert_expand + _fwd_expanded / _bwd_expanded: the grouped launches read stacked bf16
    copies of the experts' weights (one tensor map per projection, CTA pairs where the width allows).
    int8: bit-equal to the plain calls.  int4: the reference's own operand values; rows of three experts
    hold the bound against the oracle."""
    experts, in_dim, hid = 6, 512, 384
    rng = np.random.default_rng(9700 + storage + compute + gated)
    counts = rng.integers(2000, 3500, experts)
    counts[2] = 0
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    total = int(offsets[-1])
    gate, up, down, o_gate, o_up, o_down = [], [], [], [], [], []
    for _ in range(experts):
        for lst, olst, (o, i) in ((gate, o_gate, (hid, in_dim)), (up, o_up, (hid, in_dim)),
                                  (down, o_down, (in_dim, hid))):
            w, codes, scales = make_weight(rng, o, i, storage, std=0.05)
            lst.append(w)
            olst.append(orc.weight_to_compute(codes, scales, storage, i, o, compute, w.scheme, w.group_size))
    if not gated:
        gate, o_gate = None, [None] * experts
    x_np, x = act(rng, total, in_dim, orc.BF16)
    dy_np, dy = act(rng, total, in_dim, orc.BF16)
    nbytes = nv.grouped_expert_expanded_bytes(gate, up, down, nv.BF16, compute)
    assert nbytes == (3 if gated else 2) * experts * in_dim * hid * 2
    buf = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    nv.grouped_expert_expand(gate, up, down, buf, nv.BF16, compute)
    out0, g0, u0 = nv.grouped_expert_fwd(gate, up, down, offsets.tolist(), x, compute)
    dx0 = nv.grouped_expert_bwd(gate, up, down, offsets.tolist(), dy, g0, u0, compute)
    out1, g1, u1 = nv.grouped_expert_fwd(gate, up, down, offsets.tolist(), x, compute, expanded=buf)
    assert nv.last_path() == "umma-grouped"
    dx1 = nv.grouped_expert_bwd(gate, up, down, offsets.tolist(), dy, g1, u1, compute, expanded=buf)
    assert nv.last_path() == "umma-grouped"
    assert nv.lib().caifq_device_status() == 0
    if storage == orc.I8:
        assert torch.equal(out0, out1) and torch.equal(u0, u1) and torch.equal(dx0, dx1)
        assert (not gated) or torch.equal(g0, g1)
    for e in (0, 3, experts - 1):
        lo, hi = int(offsets[e]), int(offsets[e]) + 24
        want, g, u = orc.frozen_expert_forward(x_np[lo:hi], o_gate[e], o_up[e], o_down[e], compute, orc.BF16)
        assert max_rel_err(out1[lo:hi].float().cpu().numpy(), want) <= 2e-2
        assert max_rel_err(u1[lo:hi].float().cpu().numpy(), u) <= 2e-2
        want_dx = orc.frozen_expert_backward(dy_np[lo:hi], g, u, o_gate[e], o_up[e], o_down[e], compute, orc.BF16)
        assert max_rel_err(dx1[lo:hi].float().cpu().numpy(), want_dx) <= 2e-2
    # a non-bf16 row dtype is not expanded: size 0, and the expanded calls are the plain ones
    assert nv.grouped_expert_expanded_bytes(gate, up, down, nv.F32, compute) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("weight_decay", [0.0, 0.01])
def test_lora_adamw_step_bit_exact_with_the_reference_kernel(dtype, weight_decay):
    """caifq_lora_adamw_step (A and B in one launch) against the reference's fused_adam_kernel run once per
    factor: parameters and both moments bit for bit, over three steps."""
    if not ref.available():
        pytest.skip("reference kernels not built")
    rank, in_dim, out_dim = 16, 384, 520
    g = torch.Generator(device="cuda").manual_seed(31)
    a = (torch.rand(rank, in_dim, generator=g, device="cuda") - 0.5).to(dtype)
    b = (torch.randn(out_dim, rank, generator=g, device="cuda") * 0.01).to(dtype)
    lora = nv.Lora(a.clone(), b.clone(), 32.0)
    mine = [torch.zeros(rank, in_dim, device="cuda"), torch.zeros(rank, in_dim, device="cuda"),
            torch.zeros(out_dim, rank, device="cuda"), torch.zeros(out_dim, rank, device="cuda")]
    theirs = [t.clone() for t in mine]
    ra, rb = a.clone(), b.clone()
    lr, beta1, beta2, eps = 1e-3, 0.9, 0.999, 1e-8
    for step in (1, 2, 3):
        d_a = (torch.randn(rank, in_dim, generator=g, device="cuda") * 0.1).to(dtype)
        d_b = (torch.randn(out_dim, rank, generator=g, device="cuda") * 0.1).to(dtype)
        bc1, bc2 = nv.lora_adamw_step(lora, d_a, d_b, mine[0], mine[1], mine[2], mine[3], lr, beta1, beta2, eps,
                                      weight_decay, step)
        ref.fused_adam(ra, d_a, theirs[0], theirs[1], lr, beta1, beta2, eps, weight_decay, bc1, bc2)
        ref.fused_adam(rb, d_b, theirs[2], theirs[3], lr, beta1, beta2, eps, weight_decay, bc1, bc2)
        assert torch.equal(lora.a, ra) and torch.equal(lora.b, rb)
        for x, y in zip(mine, theirs):
            assert torch.equal(x, y)
    assert not torch.equal(lora.a, a)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("use_bias,n_group,topk_group,logits", [
    (True, 8, 3, True),      # DeepSeek-V3-style: sigmoid scores, selection-only bias, group-limited
    (True, 1, 1, True),      # sigmoid + bias, no groups
    (False, 8, 4, True),     # sigmoid, groups, no bias
    (False, 4, 2, False),    # softmax probabilities given, groups (DeepSeek-V2 group-limited greedy)
])
def test_grouped_sigmoid_routing_bit_exact_with_the_reference_kernels(dtype, use_bias, n_group, topk_group, logits):
    """caifq_moe_route_grouped against the reference's own kernel sequence (Sigmoid, AddBias, MoEGroupMask, TopK,
    GatherTopKValues as CAIF_DeviceMoERouter::Route chains them): scores, indices and weights bit for bit;
    ties (repeated scores) included."""
    if not ref.available():
        pytest.skip("reference kernels not built")
    tokens, experts, k = 777, 64, 6
    g = torch.Generator(device="cuda").manual_seed(77 + n_group)
    x = (torch.randn(tokens, experts, generator=g, device="cuda") * 2.0).to(dtype)
    x[5, 10:20] = x[5, 3]          # ties inside and across groups
    x[6] = 0.25
    if not logits:
        x = nv.moe_softmax(x)
    bias = (torch.randn(experts, generator=g, device="cuda") * 0.1).to(dtype) if use_bias else None
    scores, idx, wts = nv.moe_route_grouped(x, k, logits=logits, bias=bias, n_group=n_group, topk_group=topk_group)
    r_scores = ref.sigmoid(x) if logits else x
    sel = ref.bias_add(r_scores, bias) if use_bias else r_scores.clone()
    if n_group > 1:
        ref.group_mask_(sel, n_group, topk_group)
    r_idx, r_val = ref.topk_any(sel, k)
    r_wts = ref.gather_topk(r_scores, r_idx) if use_bias else r_val
    assert torch.equal(scores, r_scores)
    assert torch.equal(idx, r_idx)
    assert torch.equal(wts, r_wts)
    # every chosen expert lies in one of the topk_group groups the token kept
    if n_group > 1:
        groups = (idx // (experts // n_group)).cpu().numpy()
        assert max(len(set(row)) for row in groups) <= topk_group


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sigmoid_gate,normalize,scaling,with_aux,experts,top_k", [
    (False, True, 1.0, False, 64, 6),      # the MoE config's router
    (False, True, 2.5, True, 64, 6),       # load-balance and z-loss operands, scaled weights
    (True, True, 1.0, False, 64, 6),       # sigmoid gating, normalized
    (True, False, 16.0, False, 256, 8),    # sigmoid gating, scaled only; rows wider than the softmax block
    (False, True, 1.0, True, 160, 6),      # columns beyond 128: two per thread of the reference's block
    (False, True, 1.0, True, 8, 2),
    (False, True, 0.5, True, 3, 1),        # a single chosen expert: the normalize Jacobian is zero
    (True, False, 1.0, False, 5, 5),       # every expert chosen
])
def test_router_backward_bit_exact_with_the_reference_chain(dtype, sigmoid_gate, normalize, scaling, with_aux,
                                                            experts, top_k):
    """caifq_moe_router_bwd against the reference's own launches (NormalizeRowsBackwardTopKGather, Scale,
    Zeros + ScatterAdd, AddBias, SoftmaxBackward with the router's operand order, MoEZLossGradAdd;
    SigmoidBackward for sigmoid gating): grad_logits and grad_topk bit for bit; the oracle agrees bit for
    bit too; the softmax Jacobian proper (exact_jacobian) matches autograd."""
    tokens = 1111
    code = orc.F32 if dtype == torch.float32 else orc.BF16
    g = torch.Generator(device="cuda").manual_seed(900 + experts)
    logits = (torch.randn(tokens, experts, generator=g, device="cuda") * 2.0).to(dtype)
    probs = nv.moe_route_grouped(logits, top_k)[0] if sigmoid_gate else nv.moe_softmax(logits)
    idx, _ = nv.moe_topk(probs, top_k)
    grad_w = torch.randn(tokens, top_k, generator=g, device="cuda").to(dtype)
    bias = zls = None
    if with_aux:
        bias = (torch.rand(experts, generator=g, device="cuda") * 1e-3).to(dtype)
        zls = (torch.randn(tokens, generator=g, device="cuda") * 1e-2).to(dtype)
    got, got_topk = nv.moe_router_bwd(grad_w, probs, idx, bias, zls, sigmoid_gate, normalize, scaling)
    f = lambda t: None if t is None else t.float().cpu().numpy()
    want, want_topk = orc.router_backward(f(grad_w), f(probs), idx.cpu().numpy(), f(bias), f(zls), sigmoid_gate,
                                          normalize, scaling, dtype=code)
    assert np.array_equal(got_topk.float().cpu().numpy(), want_topk)
    assert np.array_equal(got.float().cpu().numpy(), want)
    if ref.available():
        r_logits, r_topk = ref.router_backward(grad_w, probs, idx, bias, zls, sigmoid_gate, normalize, scaling)
        assert torch.equal(r_topk, got_topk)
        assert torch.equal(r_logits, got)
    if dtype == torch.float32:
        x = logits.double().requires_grad_(True)
        scores = torch.sigmoid(x) if sigmoid_gate else torch.softmax(x, dim=-1)
        chosen = torch.gather(scores, 1, idx.long())
        w = chosen / chosen.sum(dim=-1, keepdim=True) if normalize else chosen
        (w * scaling).backward(grad_w.double())
        exact, _ = nv.moe_router_bwd(grad_w, probs, idx, None, None, sigmoid_gate, normalize, scaling,
                                     exact_jacobian=True)
        assert float((exact.double() - x.grad).abs().max()) <= 1e-4 * max(1.0, float(x.grad.abs().max()))


def test_router_backward_rejects_aux_operands_for_sigmoid_gating():
    probs = torch.rand(4, 8, device="cuda")
    idx, _ = nv.moe_topk(probs, 2)
    with pytest.raises(nv.CaifqError):
        nv.moe_router_bwd(torch.ones(4, 2, device="cuda"), probs, idx, torch.zeros(8, device="cuda"), None, True)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,top_k", [(16384, 64, 6), (777, 160, 4), (50, 8, 2)])
def test_aux_losses_against_the_reference_kernels_and_the_oracle(dtype, tokens, experts, top_k):
    """caifq_moe_aux_losses: logsumexp per row bit-identical to the reference's kernel (rounded to the storage
    type as its cached tensor), the scaled copy and the per-expert load-balance term bit-identical to the
    oracle's restatement of the host arithmetic, the two loss values within rounding of the reference's
    sequential sums."""
    code = orc.F32 if dtype == torch.float32 else orc.BF16
    g = torch.Generator(device="cuda").manual_seed(tokens)
    logits = (torch.randn(tokens, experts, generator=g, device="cuda") * 2.0).to(dtype)
    probs = nv.moe_softmax(logits)
    idx, _ = nv.moe_topk(probs, top_k)
    _, offsets = nv.moe_build_dispatch(idx, experts)
    bw, zw = 0.01, 0.001
    sums, bias, lse, zls = nv.moe_aux_losses(logits, probs, offsets, top_k, bw, zw)
    counts = np.diff(offsets.cpu().numpy())
    o_losses, o_bias, o_lse, o_zls = orc.moe_aux_losses(logits.float().cpu().numpy(), probs.float().cpu().numpy(),
                                                        counts, top_k, bw, zw, code)
    assert np.array_equal(bias.float().cpu().numpy(), o_bias)
    lse_np = lse.float().cpu().numpy()
    # the host's expf / logf may differ from the device's in the last bit: the oracle bounds, the reference pins
    assert np.max(np.abs(lse_np - o_lse)) <= (1e-6 if dtype == torch.float32 else 4e-2) * max(1.0, np.max(np.abs(o_lse)))
    if ref.available():
        r_lse = ref.logsumexp(logits).to(dtype)
        assert torch.equal(r_lse, lse)
        scale = np.float32(2.0) * np.float32(zw) / np.float32(tokens)
        assert np.array_equal(zls.float().cpu().numpy(), orc.round_through(r_lse.float().cpu().numpy() * scale, code))
        r_cols = ref.sum_axis0(probs)
        assert torch.allclose(sums[2:], r_cols, rtol=1e-5, atol=1e-6)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    got = sums[:2].cpu().numpy()
    assert abs(got[0] - o_losses[0]) <= tol * abs(o_losses[0])
    assert abs(got[1] - o_losses[1]) <= tol * abs(o_losses[1])
    # the pieces alone: no logits -> no z loss; no probs -> no balance loss
    only_b = nv.moe_aux_losses(None, probs, offsets, top_k, bw, zw)[0].cpu().numpy()
    only_z = nv.moe_aux_losses(logits, None, None, top_k, bw, zw)[0].cpu().numpy()
    assert only_b[1] == 0.0 and abs(only_b[0] - got[0]) <= 1e-6 * abs(got[0])
    assert only_z[0] == 0.0 and abs(only_z[1] - got[1]) <= 1e-6 * abs(got[1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts", [64, 257])
def test_aux_loss_free_bias_update_equals_the_reference_kernel(dtype, experts):
    g = torch.Generator(device="cuda").manual_seed(experts)
    counts = torch.randint(0, 3000, (experts,), generator=g, device="cuda", dtype=torch.int32)
    counts[3] = counts[4]
    if experts == 64:
        counts[:] = 1536           # every load equals the mean: nothing moves
        counts[0], counts[1] = 1530, 1542
    bias = (torch.randn(experts, generator=g, device="cuda") * 0.01).to(dtype)
    offsets = torch.cat([torch.zeros(1, dtype=torch.int32, device="cuda"), counts.cumsum(0).to(torch.int32)])
    got = nv.moe_bias_update(bias.clone(), counts, 1e-3)
    got_off = nv.moe_bias_update(bias.clone(), offsets, 1e-3, from_offsets=True)
    mean = np.float32(counts.cpu().numpy().astype(np.float32).sum() / np.float32(experts))
    err = mean - counts.cpu().numpy().astype(np.float32)
    code = orc.F32 if dtype == torch.float32 else orc.BF16
    want = orc.round_through(bias.float().cpu().numpy() + np.float32(1e-3) * np.sign(err).astype(np.float32), code)
    assert np.array_equal(got.float().cpu().numpy(), want)
    assert torch.equal(got, got_off)
    if ref.available():
        assert torch.equal(ref.bias_update_(bias.clone(), counts, 1e-3), got)


def test_router_backward_edge_cases():
    """No tokens: nothing is written.  One token.  Indices outside [0, experts) contribute nothing (the
    reference's scatter skips them too, src/caif_cuda_kernels_moe.cu:565-569)."""
    probs = torch.rand(0, 8, device="cuda")
    idx = torch.zeros(0, 2, dtype=torch.int32, device="cuda")
    out, _ = nv.moe_router_bwd(torch.zeros(0, 2, device="cuda"), probs, idx)
    assert out.shape == (0, 8)
    g = torch.Generator(device="cuda").manual_seed(3)
    probs = torch.softmax(torch.randn(1, 8, generator=g, device="cuda"), -1)
    idx = torch.tensor([[2, 99]], dtype=torch.int32, device="cuda")
    grad_w = torch.tensor([[0.5, -0.25]], device="cuda")
    got, got_topk = nv.moe_router_bwd(grad_w, probs, idx)
    want, want_topk = orc.router_backward(grad_w.cpu().numpy(), probs.cpu().numpy(), idx.cpu().numpy())
    assert np.array_equal(got.cpu().numpy(), want) and np.array_equal(got_topk.cpu().numpy(), want_topk)
    with pytest.raises(nv.CaifqError, match="top_k"):
        nv.moe_router_bwd(torch.zeros(2, 40, device="cuda"), torch.rand(2, 64, device="cuda"),
                          torch.zeros(2, 40, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("storage", [orc.I4, orc.I8])
def test_dense_gated_ffn_is_the_grouped_call_with_one_expert(storage):
    """CAIF_DeviceFFN with frozen gate / up / down projections (src/caif_device_ffn.cpp:324-349: gate, up, gated
    activation, down) is the grouped expert call with a single expert that owns every row: gate + up + SwiGLU in
    one launch, down in a second, and the mirror for dX."""
    rng = np.random.default_rng(88 + storage)
    in_dim, hid, rows = 512, 1408, 4099
    ws, oracle_ws = [], []
    for o, i in ((hid, in_dim), (hid, in_dim), (in_dim, hid)):
        w, codes, scales = make_weight(rng, o, i, storage, std=0.05)
        ws.append(w)
        oracle_ws.append(orc.weight_to_compute(codes, scales, storage, i, o, orc.BF16, w.scheme, w.group_size))
    x_np, x = act(rng, rows, in_dim, orc.BF16)
    dy_np, dy = act(rng, rows, in_dim, orc.BF16)
    out, g_out, u_out = nv.grouped_expert_fwd([ws[0]], [ws[1]], [ws[2]], [0, rows], x, orc.BF16)
    assert nv.last_path() == "umma-grouped"
    dx = nv.grouped_expert_bwd([ws[0]], [ws[1]], [ws[2]], [0, rows], dy, g_out, u_out, orc.BF16)
    sample = np.r_[0:8, 2048:2056, rows - 3:rows]
    want, g, u = orc.frozen_expert_forward(x_np[sample], oracle_ws[0], oracle_ws[1], oracle_ws[2], orc.BF16, orc.BF16)
    assert max_rel_err(out[sample].float().cpu().numpy(), want) <= 2e-2
    want_dx = orc.frozen_expert_backward(dy_np[sample], g, u, oracle_ws[0], oracle_ws[1], oracle_ws[2], orc.BF16,
                                         orc.BF16)
    assert max_rel_err(dx[sample].float().cpu().numpy(), want_dx) <= 2e-2
