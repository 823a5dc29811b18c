"""GPU parity: quantize / dequantize / cast kernels are bit-exact against the
CPU oracle and against the reference's own kernels (oracle/_ref)."""
import numpy as np
import pytest
import torch

import caif_oracle as orc
import refkernels as ref
from caif_b200 import native as nv
from gpu_util import dev, to_dev

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.detach().cpu().contiguous().view(torch.int32).numpy() if t.dtype == torch.float32 else t.cpu().numpy()


def _f16bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


INT8_CASES = {
    "c1_1024x1024": lambda g: (torch.randn(1024, 1024, generator=g) * 0.02),
    "odd_length": lambda g: torch.randn(100003, generator=g),
    "unaligned_view": lambda g: torch.randn(4099, generator=g)[3:],
    "zeros": lambda g: torch.zeros(777),
    "ties": lambda g: torch.arange(-127, 128).float() * 0.5,
    "one": lambda g: torch.tensor([0.3]),
    "with_inf_nan": lambda g: torch.tensor([1.0, float("nan"), -2.0, 0.5]),
}


@pytest.mark.parametrize("name", sorted(INT8_CASES))
def test_int8_per_tensor_bit_exact(name):
    g = torch.Generator().manual_seed(11)
    x = INT8_CASES[name](g).float()
    xd = x.to(dev())
    if name == "unaligned_view":
        xd = torch.randn(4099, generator=g).to(dev())[3:]
        x = xd.cpu()
    else:
        xd = xd.contiguous()
    q, s = nv.quantize_int8_per_tensor(xd)
    dq = nv.dequantize_int8_per_tensor(q, s)
    oq, os_ = orc.quantize_int8_per_tensor(x.numpy())
    assert np.array_equal(q.cpu().numpy(), oq)
    assert np.array_equal(_bits(s), os_.view(np.int32))
    assert np.array_equal(_bits(dq), orc.dequantize_int8_per_tensor(oq, os_).view(np.int32))
    if ref.available():
        rq, rs = ref.quantize_int8_per_tensor(xd.contiguous())
        assert torch.equal(rq, q) and torch.equal(rs.view(torch.int32), s.view(torch.int32))
        assert torch.equal(ref.dequantize_int8_per_tensor(rq, rs).view(torch.int32), dq.view(torch.int32))


def test_int8_empty_is_a_no_op():
    x = torch.empty(0, device=dev())
    q, s = nv.quantize_int8_per_tensor(x)
    assert q.numel() == 0


@pytest.mark.parametrize("shape", [(1024, 1024), (48, 80), (1, 7), (513, 3)])
def test_int8_per_channel_bit_exact(shape):
    g = torch.Generator().manual_seed(12)
    x = (torch.randn(*shape, generator=g) * 0.02).float()
    if shape[1] > 3:
        x[:, 3] = 0.0
    xd = x.to(dev()).contiguous()
    q, s = nv.quantize_int8_per_channel(xd)
    dq = nv.dequantize_int8_per_channel(q, s)
    oq, os_ = orc.quantize_int8_per_channel(x.numpy())
    assert np.array_equal(q.cpu().numpy(), oq)
    assert np.array_equal(_bits(s), os_.view(np.int32))
    assert np.array_equal(_bits(dq), orc.dequantize_int8_per_channel(oq, os_).view(np.int32))
    if ref.available():
        rq, rs = ref.quantize_int8_per_channel(xd)
        assert torch.equal(rq, q) and torch.equal(rs.view(torch.int32), s.view(torch.int32))


INT4_CASES = [
    ((14336 // 8, 4096), 128),   # an eighth of the decode config's weight
    ((16, 8), 128),              # the reference tests' shape: one group straddles all rows
    ((37, 24), 128),
    ((131,), 128),               # ragged tail, lone last nibble
    ((32, 96), 64),
    ((2048, 1408), 128),         # expert projection
    ((5, 30), 6),                # small even group
    ((1,), 128),
]


@pytest.mark.parametrize("shape,group", INT4_CASES)
def test_int4_bit_exact(shape, group):
    g = torch.Generator().manual_seed(13)
    x = (torch.randn(*shape, generator=g) * 0.02).float().reshape(-1)
    if x.numel() >= 512:
        x[128:256] = 0.0
    xd = x.to(dev()).contiguous()
    p, s = nv.quantize_int4(xd, group)
    dq = nv.dequantize_int4(p, s, x.numel(), group)
    op, os_ = orc.quantize_int4(x.numpy(), group)
    assert np.array_equal(p.cpu().numpy(), op)
    assert np.array_equal(_f16bits(s), os_)
    assert np.array_equal(_bits(dq), orc.dequantize_int4(op, os_, x.numel(), group).view(np.int32))
    if ref.available():
        rp, rs = ref.quantize_int4(xd, group)
        assert torch.equal(rp, p) and torch.equal(rs.view(torch.int16), s.view(torch.int16))
        assert torch.equal(ref.dequantize_int4(rp, rs, x.numel(), group).view(torch.int32), dq.view(torch.int32))


def test_int4_full_size_round_trip_properties():
    """Decode config weight (14336 x 4096): error bound of the reference's test
    (tests/test_quantize_ops.cpp:296) and idempotence of quantize(dequantize(.))."""
    g = torch.Generator(device="cuda").manual_seed(14)
    x = torch.randn(14336 * 4096, generator=g, device=dev()) * 0.02
    p, s = nv.quantize_int4(x, 128)
    dq = nv.dequantize_int4(p, s, x.numel(), 128)
    gmax = x.view(-1, 128).abs().amax(dim=1, keepdim=True)
    assert bool(((x.view(-1, 128) - dq.view(-1, 128)).abs() <= gmax / 7.0 * 0.5 + gmax * 1e-3 + 1e-7).all())
    p2, s2 = nv.quantize_int4(dq, 128)
    dq2 = nv.dequantize_int4(p2, s2, x.numel(), 128)
    assert float((dq2 - dq).abs().max()) <= float(gmax.max()) * 2e-3


@pytest.mark.parametrize("src,dst", [(torch.float32, torch.bfloat16), (torch.float32, torch.float16),
                                     (torch.bfloat16, torch.float32), (torch.float16, torch.float32),
                                     (torch.float16, torch.bfloat16), (torch.float32, torch.int8),
                                     (torch.int8, torch.float32)])
def test_cast_matches_oracle(src, dst):
    g = torch.Generator().manual_seed(15)
    x = torch.randn(10007, generator=g) * 50.0
    xs = x.to(src) if src != torch.int8 else x.clamp(-127, 127).round().to(torch.int8)
    got = nv.cast(xs.to(dev()).contiguous(), dst).cpu()
    base = xs.float().numpy()
    if dst == torch.int8:
        assert np.array_equal(got.numpy(), orc.cast_f32_to_int8(base))
    elif dst == torch.float32:
        assert np.array_equal(got.numpy(), base)
    else:
        code = orc.BF16 if dst == torch.bfloat16 else orc.F16
        assert np.array_equal(got.float().numpy(), orc.round_through(base, code))


def test_oracle_matches_reference_kernels_on_routing():
    if not ref.available():
        pytest.skip("reference kernels not built")
    g = torch.Generator().manual_seed(16)
    probs = torch.softmax(torch.randn(512, 68, generator=g), dim=-1).to(torch.bfloat16).float()
    pd = probs.to(dev()).contiguous()
    ridx, rval = ref.topk(pd, 6)
    rnorm = ref.normalize_rows(rval)
    oidx, oval = orc.topk(probs.numpy(), 6)
    assert np.array_equal(ridx.cpu().numpy(), oidx)
    assert np.array_equal(_bits(rval), oval.view(np.int32))
    assert np.array_equal(_bits(rnorm), orc.normalize_rows(oval).view(np.int32))
    wide = torch.rand(7, 1000, generator=g).to(dev())
    assert np.array_equal(_bits(ref.normalize_rows(wide)), orc.normalize_rows(wide.cpu().numpy()).view(np.int32))
