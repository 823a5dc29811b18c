"""RMSNorm in front of the frozen projections (caif_b200/csrc/norm.cu) against the reference's own kernels
(src/caif_cuda_kernels_normalization.cu, compiled unmodified into oracle/_ref) and the oracle: y, the cached rms
and dx bit for bit, grad_gamma to rounding (the reference adds it with atomics in no fixed order)."""
import numpy as np
import pytest
import torch

import caif_oracle as orc
import refkernels as ref
from caif_b200 import native as nv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,dim", [(333, 4096), (1, 4096), (1100, 14336), (50, 700), (7, 33), (3, 8192)])
def test_rmsnorm_bit_exact_with_the_reference_kernels(dtype, rows, dim):
    if dtype == torch.float32 and dim * 8 > 96 * 1024:
        pytest.skip("two fp32 rows of this width exceed the backward's row buffers")
    code = orc.F32 if dtype == torch.float32 else orc.BF16
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + dim)
    x = (torch.randn(rows, dim, generator=g, device="cuda") * 1.5).to(dtype)
    dy = torch.randn(rows, dim, generator=g, device="cuda").to(dtype)
    gamma = 1.0 + 0.1 * torch.randn(dim, generator=g, device="cuda")
    eps = 1e-5
    y, rms = nv.rmsnorm_fwd(x, gamma, eps)
    f = lambda t: t.float().cpu().numpy()
    o_y, o_rms = orc.rmsnorm_forward(f(x), f(gamma), eps, code)
    assert np.array_equal(f(rms), o_rms)
    assert np.array_equal(f(y), o_y)
    if dim > 8192:      # the backward keeps a thread's share of grad_gamma in registers: rows up to 8192 wide
        if ref.available():
            r_y, r_rms = ref.rmsnorm_fwd(x, gamma, eps)
            assert torch.equal(r_rms, rms) and torch.equal(r_y, y)
        with pytest.raises(nv.CaifqError, match="too long"):
            nv.rmsnorm_bwd(dy, x, gamma, rms)
        return
    dx, gg = nv.rmsnorm_bwd(dy, x, gamma, rms)
    o_dx, o_gg = orc.rmsnorm_backward(f(dy), f(x), f(gamma), o_rms, code)
    assert np.array_equal(f(dx), o_dx)
    assert np.max(np.abs(f(gg) - o_gg)) <= 1e-4 * max(1.0, float(np.max(np.abs(o_gg))))
    if ref.available():
        r_y, r_rms = ref.rmsnorm_fwd(x, gamma, eps)
        assert torch.equal(r_rms, rms) and torch.equal(r_y, y)
        r_dx, r_gg = ref.rmsnorm_bwd(dy, x, gamma, rms, eps)
        assert torch.equal(r_dx, dx)
        assert torch.allclose(r_gg, gg, rtol=1e-4, atol=1e-4 * float(gg.abs().max()))
    # in place, and accumulation onto an existing grad_gamma
    x2 = x.clone()
    nv._check(nv.lib().caifq_rmsnorm_fwd(nv._ptr(x2), nv._ptr(gamma), nv._ptr(x2), None, eps, nv.dtype_code(x2), rows,
                                         dim, nv._stream()), "in place")
    assert torch.equal(x2, y)
    _, gg2 = nv.rmsnorm_bwd(dy, x, gamma, rms, grad_gamma=gg.clone())
    assert torch.allclose(gg2, 2 * gg, rtol=1e-5, atol=1e-5 * float(gg.abs().max()))


def test_rmsnorm_edge_cases():
    gamma = torch.ones(16, device="cuda")
    y, rms = nv.rmsnorm_fwd(torch.zeros(0, 16, device="cuda"), gamma)
    assert y.shape == (0, 16) and rms.numel() == 0
    z, rms = nv.rmsnorm_fwd(torch.zeros(2, 16, device="cuda"), gamma, 1e-6)
    assert torch.equal(z, torch.zeros(2, 16, device="cuda")) and torch.all(rms == np.float32(1e-6) ** 0.5)
    with pytest.raises(nv.CaifqError, match="row buffer"):
        nv.rmsnorm_fwd(torch.zeros(1, 30000, device="cuda"), torch.ones(30000, device="cuda"))
