"""caifq_lora_linear_bwd_noalloc against caifq_lora_linear_bwd.

The no-allocation entry point serves callers that own no device allocator (a
plugin inside another runtime) or must not call cudaMalloc in their step (it
synchronises the device): its scratch is a fixed buffer inside the library.
Both entry points run the same kernels, so their results agree to the
tolerance of the other LoRA tests; the token reductions add with fp32 atomics,
whose order is free, hence no bit-equality claim.  The check runs twice in a
row because the buffer is shared between calls and keeps what the last call
left in it.

Collected last (file name) so that a run that stops at the first failure has
already gone through every other test.
"""
import numpy as np
import pytest
import torch

import caif_oracle as orc
from caif_b200 import native as nv
from gpu_util import TORCH_DTYPE, act, make_weight, max_rel_err, to_dev

pytestmark = pytest.mark.gpu

TOL = {orc.F32: 1e-4, orc.BF16: 2e-2}


def _case(seed, storage, sd, in_dim, out_dim, m, rank):
    rng = np.random.default_rng(seed)
    weight, _, _ = make_weight(rng, out_dim, in_dim, storage)
    bound = np.sqrt(1.0 / in_dim)
    a = orc.round_through(rng.uniform(-bound, bound, (rank, in_dim)).astype(np.float32), sd)
    b = orc.round_through((rng.standard_normal((out_dim, rank)) * 1e-2).astype(np.float32), sd)
    lora = nv.Lora(to_dev(a, TORCH_DTYPE[sd]), to_dev(b, TORCH_DTYPE[sd]), 32.0)
    _, x = act(rng, m, in_dim, sd)
    _, dy = act(rng, m, out_dim, sd)
    return weight, lora, x, dy


@pytest.mark.parametrize("storage,sd,compute", [(orc.I8, orc.F32, orc.F32), (orc.I4, orc.BF16, orc.BF16)])
def test_noalloc_matches_workspace_entry_point_twice(storage, sd, compute):
    weight, lora, x, dy = _case(900 + storage, storage, sd, 256, 192, 333, 16)
    _, hidden = nv.lora_linear_fwd(weight, lora, x, compute)
    want = nv.lora_linear_bwd(weight, lora, dy, x, hidden, compute)
    for call in range(2):
        if call == 1:
            # a different problem in between leaves other contents in the shared buffer
            w2, l2, x2, dy2 = _case(77, orc.I8, orc.F32, 128, 320, 50, 8)
            _, h2 = nv.lora_linear_fwd(w2, l2, x2)
            nv.lora_linear_bwd_noalloc(w2, l2, dy2, x2, h2)
        got = nv.lora_linear_bwd_noalloc(weight, lora, dy, x, hidden, compute)
        torch.cuda.synchronize()
        for g, w_, name in zip(got, want, ("dx", "d_a", "d_b")):
            err = max_rel_err(g.float().cpu().numpy(), w_.float().cpu().numpy())
            assert err <= TOL[sd], (call, name, err)


def test_noalloc_tensor_core_branch_allocates_no_device_memory():
    """A bf16 adapter of rank 16 on an int8 base with enough tokens takes the fused tensor-core branch, whose
    scratch holds the padded and transposed factors next to dH: the layout that matters inside the built-in
    buffer.  Checked against the oracle as well as the workspace entry point, and the free device memory
    must not move across a call made with caller-owned result tensors."""
    rng = np.random.default_rng(4321)
    in_dim, out_dim, m, rank, alpha = 512, 768, 320, 16, 32.0
    weight, codes, scales = make_weight(rng, out_dim, in_dim, orc.I8)
    a = orc.round_through(rng.uniform(-0.05, 0.05, (rank, in_dim)).astype(np.float32), orc.BF16)
    b = orc.round_through((rng.standard_normal((out_dim, rank)) * 1e-2).astype(np.float32), orc.BF16)
    lora = nv.Lora(to_dev(a, torch.bfloat16), to_dev(b, torch.bfloat16), alpha)
    x_np, x = act(rng, m, in_dim, orc.BF16)
    dy_np, dy = act(rng, m, out_dim, orc.BF16)
    _, hidden = nv.lora_linear_fwd(weight, lora, x, nv.F32)
    want = nv.lora_linear_bwd(weight, lora, dy, x, hidden, nv.F32)
    assert nv.last_path() == "umma"
    dx = torch.empty(m, in_dim, dtype=torch.bfloat16, device="cuda")
    d_a = torch.empty_like(lora.a)
    d_b = torch.empty_like(lora.b)

    def call():
        nv._check(nv.lib().caifq_lora_linear_bwd_noalloc(weight.ref(), lora.ref(), nv._ptr(dy), nv._ptr(x),
                                                         nv._ptr(hidden), m, nv._ptr(dx), nv._ptr(d_a), nv._ptr(d_b),
                                                         nv.F32, nv._stream()), "lora_linear_bwd_noalloc")
        torch.cuda.synchronize()

    call()                                    # the first call on a device may look up the buffer's address
    assert nv.last_path() == "umma"
    free_before, _ = torch.cuda.mem_get_info()
    call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    for g, w_, name in zip((dx, d_a, d_b), want, ("dx", "d_a", "d_b")):
        assert max_rel_err(g.float().cpu().numpy(), w_.float().cpu().numpy()) <= TOL[orc.BF16], name
    wc = orc.weight_to_compute(codes, scales, orc.I8, in_dim, out_dim, orc.F32, weight.scheme, weight.group_size)
    o_dx, o_da, o_db = orc.lora_backward(dy_np, x_np, hidden.float().cpu().numpy(),
                                         orc.frozen_linear_backward(dy_np, wc, orc.F32), a, b, alpha, orc.BF16)
    assert max_rel_err(dx.float().cpu().numpy(), o_dx) <= TOL[orc.BF16]
    assert max_rel_err(d_a.float().cpu().numpy(), o_da) <= TOL[orc.BF16]
    assert max_rel_err(d_b.float().cpu().numpy(), o_db) <= TOL[orc.BF16]


def test_noalloc_rejects_oversized_calls_without_launching():
    limit = int(nv.lib().caifq_lora_bwd_noalloc_max_bytes())
    assert limit == 8 << 20
    weight, lora, x, dy = _case(5, orc.I8, orc.F32, 64, 64, 8, 4)
    # describe a problem far beyond the built-in buffer (m * rank * 4 bytes alone exceeds it); the
    # entry point must refuse before touching any pointer
    big_m = limit  # tokens
    rc = nv.lib().caifq_lora_linear_bwd_noalloc(weight.ref(), lora.ref(), None, None, None, big_m, None, None, None,
                                               nv.F32, None)
    assert rc == 3
    msg = nv.lib().caifq_last_error().decode()
    assert "scratch" in msg and str(limit) in msg
