"""Device times of the kernels either side of the frozen-linear path, next to the reference's own kernels for
the same step (oracle/_ref/libcaif_ref_kernels.so, its unmodified sources): RMSNorm forward / backward, the
router backward (one launch against the reference's chain of launches), the auxiliary losses.  Not a test: run

    python tests/aux_kernel_timing.py

on a GPU box.  CUDA events over 30 calls after 3 warm-up calls; operands rotate over three buffer sets where
one set would fit the L2."""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "oracle"))

import refkernels as ref  # noqa: E402
from caif_b200 import native as nv  # noqa: E402


def timed(fn, n=30):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(n):
        fn(i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n * 1e3


def main():
    g = torch.Generator(device="cuda").manual_seed(5)
    rows, dim = 16384, 4096
    xs = [torch.randn(rows, dim, generator=g, device="cuda").to(torch.bfloat16) for _ in range(3)]
    dys = [torch.randn(rows, dim, generator=g, device="cuda").to(torch.bfloat16) for _ in range(3)]
    gamma = 1.0 + 0.1 * torch.randn(dim, generator=g, device="cuda")
    _, rms = nv.rmsnorm_fwd(xs[0], gamma)
    have_ref = ref.available()
    out = []
    fwd_bytes, bwd_bytes = rows * dim * 2 * 2, rows * dim * 2 * 3
    out.append(("RMSNorm forward 16384 x 4096 bf16", timed(lambda i: nv.rmsnorm_fwd(xs[i % 3], gamma)), fwd_bytes,
                timed(lambda i: ref.rmsnorm_fwd(xs[i % 3], gamma, 1e-5)) if have_ref else None))
    out.append(("RMSNorm backward", timed(lambda i: nv.rmsnorm_bwd(dys[i % 3], xs[i % 3], gamma, rms)), bwd_bytes,
                timed(lambda i: ref.rmsnorm_bwd(dys[i % 3], xs[i % 3], gamma, rms, 1e-5)) if have_ref else None))
    tokens, experts, k = 16384, 64, 6
    logits = (torch.randn(tokens, experts, generator=g, device="cuda") * 2).to(torch.bfloat16)
    probs = nv.moe_softmax(logits)
    idx, _ = nv.moe_topk(probs, k)
    _, off = nv.moe_build_dispatch(idx, experts)
    gw = torch.randn(tokens, k, generator=g, device="cuda").to(torch.bfloat16)
    _, bias, _, zls = nv.moe_aux_losses(logits, probs, off, k, 0.01, 0.001)
    rb_bytes = tokens * experts * 2 * 2 + tokens * k * (2 + 4 + 2)
    out.append(("router backward 16384 tokens x 64 experts, top-6, both aux terms",
                timed(lambda i: nv.moe_router_bwd(gw, probs, idx, bias, zls, False, True, 2.5)), rb_bytes,
                timed(lambda i: ref.router_backward(gw, probs, idx, bias, zls, False, True, 2.5)) if have_ref else None))
    out.append(("auxiliary losses (same shapes)", timed(lambda i: nv.moe_aux_losses(logits, probs, off, k, 0.01, 0.001)),
                tokens * experts * 2 * 2, None))
    print("| kernel | this library | algorithmic GB/s | reference kernels |")
    print("|---|---|---|---|")
    for name, us, nbytes, ref_us in out:
        print("| %s | %.1f us | %.0f | %s |" % (name, us, nbytes / us / 1e3, "%.1f us" % ref_us if ref_us else "-"))


if __name__ == "__main__":
    main()
