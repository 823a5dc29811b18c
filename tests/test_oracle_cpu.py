"""CPU checks of the oracle: hand-derived known answers, the properties the
reference's own tests assert (tests/test_quantize_ops.cpp:161-330,
tests/test_device_moe.cpp), and the committed golden vectors captured from the
reference's kernels."""
import glob
import os

import numpy as np
import pytest

import caif_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


# ----------------------------------------------------------------- conversions
def test_fp16_matches_numpy_on_all_bit_patterns():
    bits = np.arange(65536, dtype=np.uint16)
    ours = orc.f16_bits_to_f32(bits)
    theirs = bits.view(np.float16).astype(np.float32)
    nan = np.isnan(theirs)
    assert np.array_equal(np.isnan(ours), nan)
    assert np.array_equal(ours[~nan].view(np.uint32), theirs[~nan].view(np.uint32))


def test_f32_to_f16_rounding_matches_numpy():
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(200000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 200000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e9, -1e9, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5,
                  np.inf, -np.inf], np.float32),
    ]).astype(np.float32)
    ours = orc.f32_to_f16_bits(x)
    with np.errstate(over="ignore"):
        theirs = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(ours, theirs)


def test_bf16_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 1e-40], np.float32)
    # 1 + 2^-8 is exactly half an ulp above 1.0 -> ties to even (1.0); 1 + 3*2^-8 ties up to 1 + 2^-6
    got = orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(x))
    assert got[0] == 1.0 and got[1] == 1.0 and got[2] == np.float32(1.015625)
    assert got[3] == -2.5
    import torch

    t = torch.from_numpy(np.random.default_rng(2).standard_normal(100000).astype(np.float32))
    ref = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.f32_to_bf16_bits(t.numpy()), ref)


# ------------------------------------------------------------------ int8 / int4
def test_int8_per_tensor_known_answer():
    x = np.array([0.0, 1.27, -1.27, 0.635, 0.005, -0.015, 0.6399], np.float32)
    q, s = orc.quantize_int8_per_tensor(x)
    assert s[0] == np.float32(1.27) / np.float32(127.0)
    assert q.tolist() == [0, 127, -127, 64, 0, -2, 64]  # 63.5 ties to even 64; 0.5 ties to 0; -1.5 ties to -2


def test_int8_zero_input_has_unit_scale():
    q, s = orc.quantize_int8_per_tensor(np.zeros(64, np.float32))
    assert s[0] == 1.0 and not q.any()
    q, s = orc.quantize_int8_per_channel(np.zeros((4, 8), np.float32))
    assert np.all(s == 1.0) and not q.any()


def test_int8_round_trip_error_bound():
    # tests/test_quantize_ops.cpp:186 -- |x - dq| <= max|x|/127 (+1e-6)
    rng = np.random.default_rng(3)
    x = rng.standard_normal(4096).astype(np.float32)
    q, s = orc.quantize_int8_per_tensor(x)
    dq = orc.dequantize_int8_per_tensor(q, s)
    assert np.max(np.abs(x - dq)) <= np.max(np.abs(x)) / 127.0 + 1e-6
    x2 = rng.standard_normal((32, 48)).astype(np.float32)
    q2, s2 = orc.quantize_int8_per_channel(x2)
    dq2 = orc.dequantize_int8_per_channel(q2, s2)
    assert np.all(np.abs(x2 - dq2) <= np.max(np.abs(x2), axis=0) / 127.0 + 1e-6)
    assert np.array_equal(s2, np.max(np.abs(x2), axis=0) / np.float32(127.0))


def test_int4_known_answer_and_packing():
    x = np.zeros(8, np.float32)
    x[:] = [7.0, -7.0, 3.5, -3.5, 0.49, 2.5, 1.0, -1.0]
    packed, scales = orc.quantize_int4(x, group=8)
    assert orc.f16_bits_to_f32(scales)[0] == 1.0
    # 3.5 -> 4 (even), -3.5 -> -4, 0.49 -> 0, 2.5 -> 2 (even)
    codes = [7, -7, 4, -4, 0, 2, 1, -1]
    expect = [(codes[i] & 0xF) | ((codes[i + 1] & 0xF) << 4) for i in range(0, 8, 2)]
    assert packed.tolist() == expect
    assert orc.dequantize_int4(packed, scales, 8, group=8).tolist() == [float(c) for c in codes]


def test_int4_groups_are_flat_and_tail_is_padded():
    rng = np.random.default_rng(4)
    x = rng.standard_normal(16 * 8 + 3).astype(np.float32)  # 131 elements: groups of 128 and 3
    packed, scales = orc.quantize_int4(x, group=128)
    assert packed.size == 66 and scales.size == 2
    assert packed[-1] >> 4 == 0  # lone last element: high nibble zero
    s = orc.f16_bits_to_f32(scales)
    assert s[0] == np.float32(np.float16(np.max(np.abs(x[:128])) / np.float32(7.0)))
    assert s[1] == np.float32(np.float16(np.max(np.abs(x[128:])) / np.float32(7.0)))
    dq = orc.dequantize_int4(packed, scales, x.size, group=128)
    # tests/test_quantize_ops.cpp:296 -- error <= max|x|/7 (+1e-3)
    assert np.max(np.abs(x - dq)) <= np.max(np.abs(x)) / 7.0 + 1e-3


def test_int4_zero_group_has_zero_scale():
    packed, scales = orc.quantize_int4(np.zeros(256, np.float32), group=128)
    assert not packed.any() and not scales.any()


def test_int4_reciprocal_uses_unrounded_scale():
    # max = 0.7000001 -> scale just above 0.1 in fp32 but fp16(scale) differs; codes come from the fp32 scale
    x = np.full(128, 0.05, np.float32)
    x[0] = np.float32(0.7000001)
    packed, scales = orc.quantize_int4(x, group=128)
    scale32 = x[0] / np.float32(7.0)
    inv = np.float32(1.0) / scale32
    want = int(np.rint(np.float32(0.05) * inv))
    assert (packed[0] >> 4) == want
    assert orc.f16_bits_to_f32(scales)[0] == np.float32(np.float16(scale32))


# ------------------------------------------------------------- weight / linear
def test_weight_to_compute_cells():
    rng = np.random.default_rng(5)
    in_dim, out_dim = 24, 16
    w = (rng.standard_normal((out_dim, in_dim)) * 0.02).astype(np.float32)
    # int8 per tensor
    q, s = orc.quantize_int8_per_tensor(w)
    w8 = orc.weight_to_compute(q, s, orc.I8, in_dim, out_dim)
    assert np.array_equal(w8, q.astype(np.float32) * s[0])
    # int8 without scales = raw cast
    assert np.array_equal(orc.weight_to_compute(q, None, orc.I8, in_dim, out_dim), q.astype(np.float32))
    # per-channel quirk: scale index = flat % out_dim over the [out,in] buffer
    qc = rng.integers(-127, 128, (out_dim, in_dim)).astype(np.int8)
    sc = rng.random(out_dim).astype(np.float32)
    wc = orc.weight_to_compute(qc, sc, orc.I8, in_dim, out_dim, scheme=orc.PER_CHANNEL)
    flat = np.arange(in_dim * out_dim)
    assert np.array_equal(wc.reshape(-1), qc.reshape(-1).astype(np.float32) * sc[flat % out_dim])
    # int4 group straddling rows (in_dim=24, group 128 over 384 elements)
    p4, s4 = orc.quantize_int4(w, group=128)
    w4 = orc.weight_to_compute(p4, s4, orc.I4, in_dim, out_dim, group=128)
    assert np.array_equal(w4.reshape(-1), orc.dequantize_int4(p4, s4, w.size, 128))
    # bf16 compute: values rounded through bf16
    w4b = orc.weight_to_compute(p4, s4, orc.I4, in_dim, out_dim, compute=orc.BF16)
    assert np.array_equal(w4b, orc.round_through(w4, orc.BF16))


def test_linear_forward_backward_against_numpy():
    rng = np.random.default_rng(6)
    w = rng.standard_normal((48, 32)).astype(np.float32)
    x = rng.standard_normal((5, 32)).astype(np.float32)
    dy = rng.standard_normal((5, 48)).astype(np.float32)
    y = orc.frozen_linear_forward(x, w)
    dx = orc.frozen_linear_backward(dy, w)
    assert np.allclose(y, x.astype(np.float64) @ w.T.astype(np.float64), rtol=1e-6, atol=1e-6)
    assert np.allclose(dx, dy.astype(np.float64) @ w.astype(np.float64), rtol=1e-6, atol=1e-6)
    assert np.allclose(orc.gemm_tn(dy, x), dy.T.astype(np.float64) @ x.astype(np.float64), rtol=1e-6, atol=1e-6)
    # sgemm flavour agrees within fp32 accumulation error
    assert np.allclose(orc.gemm_nt(x, w, exact=False), y, rtol=1e-5, atol=1e-5)


def test_lora_zero_b_equals_base():
    # tests/test_device_lora_adapter.cpp:371-442 -- B = 0 => output == base output
    rng = np.random.default_rng(7)
    x = rng.standard_normal((6, 32)).astype(np.float32)
    a = rng.uniform(-0.1, 0.1, (4, 32)).astype(np.float32)
    b = np.zeros((16, 4), np.float32)
    base = rng.standard_normal((6, 16)).astype(np.float32)
    out, hidden = orc.lora_forward(x, base, a, b, alpha=8.0)
    assert np.array_equal(out, base)
    assert hidden.shape == (6, 4)


def test_lora_gradients_match_autograd():
    import torch

    rng = np.random.default_rng(8)
    x = rng.standard_normal((7, 20)).astype(np.float32)
    w = rng.standard_normal((12, 20)).astype(np.float32)
    a = rng.uniform(-0.2, 0.2, (3, 20)).astype(np.float32)
    b = rng.standard_normal((12, 3)).astype(np.float32)
    dy = rng.standard_normal((7, 12)).astype(np.float32)
    alpha = 6.0
    base = orc.frozen_linear_forward(x, w)
    out, hidden = orc.lora_forward(x, base, a, b, alpha)
    dx, d_a, d_b = orc.lora_backward(dy, x, hidden, orc.frozen_linear_backward(dy, w), a, b, alpha)
    tx = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    ta = torch.tensor(a, dtype=torch.float64, requires_grad=True)
    tb = torch.tensor(b, dtype=torch.float64, requires_grad=True)
    tw = torch.tensor(w, dtype=torch.float64)
    ty = tx @ tw.T + (alpha / 3) * ((tx @ ta.T) @ tb.T)
    ty.backward(torch.tensor(dy, dtype=torch.float64))
    assert np.allclose(out, ty.detach().numpy(), atol=1e-5)
    assert np.allclose(dx, tx.grad.numpy(), atol=1e-5)
    assert np.allclose(d_a, ta.grad.numpy(), atol=1e-5)
    assert np.allclose(d_b, tb.grad.numpy(), atol=1e-5)


def test_frozen_expert_matches_autograd():
    import torch

    rng = np.random.default_rng(9)
    x = rng.standard_normal((5, 16)).astype(np.float32)
    wg = (rng.standard_normal((24, 16)) * 0.3).astype(np.float32)
    wu = (rng.standard_normal((24, 16)) * 0.3).astype(np.float32)
    wd = (rng.standard_normal((16, 24)) * 0.3).astype(np.float32)
    dy = rng.standard_normal((5, 16)).astype(np.float32)
    out, gate, up = orc.frozen_expert_forward(x, wg, wu, wd)
    dx = orc.frozen_expert_backward(dy, gate, up, wg, wu, wd)
    tx = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    tg, tu, td = (torch.tensor(v, dtype=torch.float64) for v in (wg, wu, wd))
    ty = (torch.nn.functional.silu(tx @ tg.T) * (tx @ tu.T)) @ td.T
    ty.backward(torch.tensor(dy, dtype=torch.float64))
    assert np.allclose(out, ty.detach().numpy(), atol=1e-5)
    assert np.allclose(dx, tx.grad.numpy(), atol=1e-5)


# -------------------------------------------------------------------- routing
def test_topk_ties_go_to_lowest_index_and_match_argmax():
    p = np.array([[0.1, 0.4, 0.4, 0.1], [0.25, 0.25, 0.25, 0.25], [0.0, 0.0, 1.0, 0.0]], np.float32)
    idx, val = orc.topk(p, 2)
    assert idx.tolist() == [[1, 2], [0, 1], [2, 0]]
    assert val[0].tolist() == [np.float32(0.4), np.float32(0.4)]
    rng = np.random.default_rng(10)
    probs = rng.random((64, 68)).astype(np.float32)
    idx, _ = orc.topk(probs, 6)
    assert np.array_equal(idx[:, 0], np.argmax(probs, axis=1))  # tests/test_device_moe.cpp TopKIndicesMatchArgmax
    order = np.argsort(-probs, axis=1, kind="stable")[:, :6]
    assert np.array_equal(idx, order)


def test_topk_sentinel_rows():
    p = np.full((1, 4), -2e30, np.float32)
    idx, val = orc.topk(p, 2)
    assert idx.tolist() == [[0, 0]] and np.all(val == np.float32(-1e30))


def test_normalize_rows_sums_to_one():
    rng = np.random.default_rng(11)
    x = rng.random((32, 6)).astype(np.float32)
    out = orc.normalize_rows(x)
    assert np.allclose(out.sum(axis=1), 1.0, atol=1e-6)  # WeightsNormalized
    z = orc.normalize_rows(np.zeros((2, 6), np.float32))
    assert not z.any()
    # wide rows exercise the strided partial sums and the tree
    wide = rng.random((3, 1000)).astype(np.float32)
    assert np.allclose(orc.normalize_rows(wide).sum(axis=1), 1.0, atol=1e-5)


def test_dispatch_map_known_answer_and_capacity():
    idx = np.array([[0, 2], [2, 0], [2, 1], [5, 2]], np.int32)  # 5 is out of range for E=3
    dmap, off, total = orc.build_dispatch_map(idx, num_experts=3)
    assert off.tolist() == [0, 2, 3, 7] and total == 7
    assert dmap.tolist() == [[0, 0], [1, 1], [2, 0], [-1, 3]]
    dmap, off, total = orc.build_dispatch_map(idx, num_experts=3, capacity=2)
    assert off.tolist() == [0, 2, 3, 5] and total == 5
    assert dmap.tolist() == [[0, 0], [1, 1], [-1, 0], [-1, -1]]


def test_dispatch_then_combine_with_unit_weights_is_a_sum_of_copies():
    rng = np.random.default_rng(12)
    tokens, dim, k, experts = 40, 8, 3, 7
    x = rng.standard_normal((tokens, dim)).astype(np.float32)
    idx = np.stack([rng.permutation(experts)[:k] for _ in range(tokens)]).astype(np.int32)
    dmap, off, total = orc.build_dispatch_map(idx, experts)
    assert total == tokens * k
    buf = orc.moe_dispatch(x, idx, dmap, off, total)
    # each expert segment holds its tokens in arrival order
    for e in range(experts):
        toks = [t for t in range(tokens) for kk in range(k) if idx[t, kk] == e]
        assert np.array_equal(buf[off[e]:off[e + 1]], x[toks])
    w = np.full((tokens, k), 1.0 / k, np.float32)
    out = orc.moe_combine(buf, idx, w, dmap, off, tokens)
    assert np.allclose(out, x, atol=1e-6)


# ------------------------------------------------------------ golden fixtures
# (the layer_*.npz files hold whole-layer vectors in another format: tests/test_layer_golden.py replays those)
@pytest.mark.parametrize("path", sorted(f for f in glob.glob(os.path.join(GOLDEN, "*.npz"))
                                        if not os.path.basename(f).startswith("layer_")) or [None])
def test_oracle_reproduces_reference_golden_vectors(path):
    """Fixtures under tests/golden/ hold inputs and the outputs of the reference's
    own kernels (captured on a B200 by tests/golden/make_golden.py)."""
    if path is None:
        pytest.skip("no golden fixtures committed yet")
    g = np.load(path)
    kind = str(g["kind"])
    if kind == "int8_per_tensor":
        q, s = orc.quantize_int8_per_tensor(g["x"])
        assert np.array_equal(q, g["q"]) and np.array_equal(s.view(np.uint32), g["scale"].view(np.uint32))
        assert np.array_equal(orc.dequantize_int8_per_tensor(q, s).view(np.uint32), g["dq"].view(np.uint32))
    elif kind == "int8_per_channel":
        q, s = orc.quantize_int8_per_channel(g["x"])
        assert np.array_equal(q, g["q"]) and np.array_equal(s.view(np.uint32), g["scales"].view(np.uint32))
        assert np.array_equal(orc.dequantize_int8_per_channel(q, s).view(np.uint32), g["dq"].view(np.uint32))
    elif kind == "int4":
        group = int(g["group"])
        p, s = orc.quantize_int4(g["x"], group)
        assert np.array_equal(p, g["packed"]) and np.array_equal(s, g["scales"])
        assert np.array_equal(orc.dequantize_int4(p, s, g["x"].size, group).view(np.uint32), g["dq"].view(np.uint32))
    elif kind == "routing":
        idx, val = orc.topk(g["probs"], int(g["k"]))
        assert np.array_equal(idx, g["indices"]) and np.array_equal(val.view(np.uint32), g["values"].view(np.uint32))
        assert np.array_equal(orc.normalize_rows(val).view(np.uint32), g["normalized"].view(np.uint32))
    elif kind == "dispatch":
        idx = g["indices"]
        dmap, off, total = orc.build_dispatch_map(idx, int(g["num_experts"]))
        buf = orc.moe_dispatch(g["x"], idx, dmap, off, total)
        assert np.array_equal(buf.view(np.uint32), g["buffer"].view(np.uint32))
        out = orc.moe_combine(buf, idx, g["weights"], dmap, off, g["x"].shape[0])
        assert np.array_equal(out.view(np.uint32), g["combined"].view(np.uint32))
    elif kind == "dispatch_backward":
        idx = g["indices"]
        dmap, off, total = orc.build_dispatch_map(idx, int(g["num_experts"]))
        gbuf = orc.moe_combine_bwd_grad_expert(g["grad_output"], idx, g["weights"], dmap, off, total)
        assert np.array_equal(gbuf.view(np.uint32), g["grad_buffer"].view(np.uint32))
        gw = orc.moe_combine_bwd_grad_weights(g["grad_output"], g["buffer"], idx, dmap, off)
        assert np.array_equal(gw.view(np.uint32), g["grad_weights"].view(np.uint32))
        gin = orc.moe_dispatch_bwd(gbuf, idx, dmap, off, g["grad_output"].shape[0])
        assert np.array_equal(gin.view(np.uint32), g["grad_input"].view(np.uint32))
    else:
        raise AssertionError("unknown fixture kind %s" % kind)


def test_dispatch_backward_is_the_adjoint_of_dispatch_and_combine():
    """<combine(B), G> = <B, combine_bwd_expert(G)> and <dispatch(X), GB> = <X, dispatch_bwd(GB)> in
    exact integer arithmetic (small integers keep every fp32 sum exact); the routing-weight gradient
    of an all-ones buffer is the row sum of G."""
    rng = np.random.default_rng(5)
    tokens, dim, top_k, experts = 40, 24, 3, 7
    idx = np.stack([rng.permutation(experts)[:top_k] for _ in range(tokens)]).astype(np.int32)
    dmap, off, total = orc.build_dispatch_map(idx, experts, capacity=12)
    w = rng.integers(-3, 4, (tokens, top_k)).astype(np.float32)
    b = rng.integers(-4, 5, (total, dim)).astype(np.float32)
    g = rng.integers(-4, 5, (tokens, dim)).astype(np.float32)
    x = rng.integers(-4, 5, (tokens, dim)).astype(np.float32)
    gb = orc.moe_combine_bwd_grad_expert(g, idx, w, dmap, off, total)
    assert float((orc.moe_combine(b, idx, w, dmap, off, tokens) * g).sum()) == float((b * gb).sum())
    assert float((orc.moe_dispatch(x, idx, dmap, off, total) * b).sum()) == \
        float((x * orc.moe_dispatch_bwd(b, idx, dmap, off, tokens)).sum())
    gw = orc.moe_combine_bwd_grad_weights(g, np.ones((total, dim), np.float32), idx, dmap, off)
    want = np.where(dmap >= 0, g.sum(axis=1, keepdims=True), 0.0)
    assert np.array_equal(gw, want.astype(np.float32))


def test_router_softmax_restatement():
    """The oracle's router softmax keeps the kernel's operation order; against a float64 softmax it is
    exact to a few fp32 ulp, rows sum to one, and a bias is added before the score function."""
    rng = np.random.default_rng(41)
    for rows, cols in ((33, 68), (5, 300), (4, 1), (7, 128)):
        x = (rng.standard_normal((rows, cols)) * 3).astype(np.float32)
        b = rng.standard_normal(cols).astype(np.float32)
        for bias in (None, b):
            p = orc.router_softmax(x, bias)
            z = x.astype(np.float64) + (0 if bias is None else bias.astype(np.float32).astype(np.float64))
            e = np.exp(z - z.max(axis=1, keepdims=True))
            want = e / e.sum(axis=1, keepdims=True)
            assert np.max(np.abs(p - want)) <= 3e-7
            assert np.allclose(p.sum(axis=1), 1.0, atol=1e-6)
    # the biased logit is rounded through the storage dtype before the softmax, as AddBias stores it
    x = np.array([[1.0, 1.0]], np.float32)
    b = np.array([2 ** -10, 0.0], np.float32)
    p = orc.router_softmax(x, b, orc.BF16)
    assert p[0, 0] == p[0, 1]          # 1 + 2^-10 rounds to 1 in bf16
    p = orc.router_softmax(x, b, orc.F32)
    assert p[0, 0] > p[0, 1]
    # a row of equal logits gives the uniform distribution; -inf-like entries vanish
    assert np.array_equal(orc.router_softmax(np.zeros((1, 4), np.float32)), np.full((1, 4), 0.25, np.float32))
    p = orc.router_softmax(np.array([[0.0, -1e30, 0.0]], np.float32))
    assert p[0, 1] == 0.0 and p[0, 0] == 0.5


@pytest.mark.parametrize("sigmoid_gate,normalize,scaling", [(False, True, 1.0), (False, True, 2.5), (True, True, 1.0),
                                                            (True, False, 16.0)])
def test_router_backward_restatement_against_autograd(sigmoid_gate, normalize, scaling):
    """The oracle's router backward with the softmax Jacobian proper equals autograd through
    scores -> gather at the chosen experts -> normalize -> scale; with the reference's operand
    order (probs in the grad_output slot) it equals grad_probs * (probs - dot) instead."""
    import torch
    rng = np.random.default_rng(31)
    tokens, experts, top_k = 37, 64, 6
    logits = torch.tensor(rng.standard_normal((tokens, experts)), dtype=torch.float64, requires_grad=True)
    scores = torch.sigmoid(logits) if sigmoid_gate else torch.softmax(logits, dim=-1)
    idx = torch.topk(scores, top_k, dim=-1).indices
    chosen = torch.gather(scores, 1, idx)
    weights = chosen / chosen.sum(dim=-1, keepdim=True) if normalize else chosen
    weights = weights * scaling
    grad_w = torch.tensor(rng.standard_normal((tokens, top_k)), dtype=torch.float64)
    weights.backward(grad_w)
    got, _ = orc.router_backward(grad_w.numpy().astype(np.float32), scores.detach().numpy().astype(np.float32),
                                 idx.numpy().astype(np.int32), sigmoid_gate=sigmoid_gate, normalize=normalize,
                                 scaling=scaling, exact_jacobian=True)
    want = logits.grad.numpy()
    assert np.max(np.abs(got - want)) <= 1e-5 * max(1.0, np.max(np.abs(want)))
    if not sigmoid_gate:
        ref_form, grad_topk = orc.router_backward(grad_w.numpy().astype(np.float32),
                                                  scores.detach().numpy().astype(np.float32),
                                                  idx.numpy().astype(np.int32), normalize=normalize, scaling=scaling)
        p = scores.detach().numpy()
        gp = np.zeros_like(p)
        np.put_along_axis(gp, idx.numpy(), grad_topk.astype(np.float64), axis=1)
        dot = (p * gp).sum(axis=1, keepdims=True)
        assert np.max(np.abs(ref_form - gp * (p - dot))) <= 1e-5


def test_aux_losses_restatement_against_formulas():
    rng = np.random.default_rng(5)
    tokens, experts, top_k = 200, 64, 6
    logits = rng.standard_normal((tokens, experts)).astype(np.float32) * 2
    ex = np.exp(logits.astype(np.float64) - logits.max(axis=1, keepdims=True))
    probs = (ex / ex.sum(axis=1, keepdims=True)).astype(np.float32)
    counts = np.bincount(np.argsort(-probs, axis=1)[:, :top_k].ravel(), minlength=experts).astype(np.int32)
    bw, zw = 0.01, 0.001
    losses, bias, lse, zls = orc.moe_aux_losses(logits, probs, counts, top_k, bw, zw)
    lse64 = np.log(np.exp(logits.astype(np.float64)).sum(axis=1))
    assert np.allclose(lse, lse64, rtol=1e-6, atol=1e-6)
    assert np.isclose(losses[1], zw * (lse64 ** 2).sum() / tokens, rtol=1e-5)
    want_balance = bw * experts * ((counts / (tokens * top_k)) * (probs.astype(np.float64).sum(axis=0) / tokens)).sum()
    assert np.isclose(losses[0], want_balance, rtol=1e-5)
    assert np.allclose(bias, bw * experts * counts / (tokens * tokens * top_k), rtol=1e-6)
    assert np.allclose(zls, lse64 * 2 * zw / tokens, rtol=1e-5)


def test_rmsnorm_restatement_against_autograd():
    import torch
    rng = np.random.default_rng(17)
    rows, dim = 9, 700
    x = rng.standard_normal((rows, dim)).astype(np.float32)
    gamma = (1.0 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    dy = rng.standard_normal((rows, dim)).astype(np.float32)
    y, rms = orc.rmsnorm_forward(x, gamma, 1e-5)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    gt = torch.tensor(gamma, dtype=torch.float64, requires_grad=True)
    yt = xt / torch.sqrt((xt * xt).mean(-1, keepdim=True) + 1e-5) * gt
    yt.backward(torch.tensor(dy, dtype=torch.float64))
    assert np.max(np.abs(y - yt.detach().numpy())) <= 1e-5
    for form in (0, 1, 2):
        dx, gg = orc.rmsnorm_backward(dy, x, gamma, rms, form=form)
        assert np.max(np.abs(dx - xt.grad.numpy())) <= 1e-5
        assert np.max(np.abs(gg - gt.grad.numpy())) <= 1e-4
