"""Capture golden vectors from the reference's own kernels.

Run on a machine with a GPU and oracle/_ref/libcaif_ref_kernels.so built
(`python oracle/build.py` where the reference checkout is present):

    python tests/golden/make_golden.py <output-dir>

Each .npz holds seeded inputs and what the reference's unmodified kernels
(src/caif_cuda_kernels_quant.cu, src/caif_cuda_kernels_moe.cu) produced for
them.  tests/test_oracle_cpu.py replays them through the CPU oracle without a
GPU.  Sizes are small on purpose (a few hundred KB in total).
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "oracle"))

import refkernels as ref  # noqa: E402
import caif_oracle as orc  # noqa: E402


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(20260101)

    def randn(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).float()

    # int8 per tensor: weights N(0, 0.02) as in the 1024x1024 config, scaled down to 96x128,
    # with exact ties and a zero tensor
    for name, x in (("w", randn(96, 128, std=0.02)), ("zero", torch.zeros(40)),
                    ("ties", torch.arange(-127, 128).float() * 0.5)):
        xd = x.to(dev).contiguous()
        q, s = ref.quantize_int8_per_tensor(xd)
        dq = ref.dequantize_int8_per_tensor(q, s)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, "int8_per_tensor_%s.npz" % name), kind="int8_per_tensor",
                            x=x.numpy(), q=q.cpu().numpy(), scale=s.cpu().numpy(), dq=dq.cpu().numpy())

    x = randn(48, 80, std=0.02)
    x[:, 3] = 0.0
    xd = x.to(dev).contiguous()
    q, s = ref.quantize_int8_per_channel(xd)
    dq = ref.dequantize_int8_per_channel(q, s)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "int8_per_channel.npz"), kind="int8_per_channel", x=x.numpy(),
                        q=q.cpu().numpy(), scales=s.cpu().numpy(), dq=dq.cpu().numpy())

    # int4: group 128 rows aligned (64x256), groups straddling rows (16x8 as in the reference's
    # tests, plus 37x24), ragged tail (131 elements), group 64, a zero group
    cases = {"aligned": (randn(64, 256, std=0.02), 128), "straddle16x8": (randn(16, 8, std=0.02), 128),
             "straddle37x24": (randn(37, 24, std=0.02), 128), "ragged131": (randn(131), 128),
             "group64": (randn(32, 96, std=0.02), 64)}
    z = randn(512, std=0.02)
    z[128:256] = 0.0
    cases["zero_group"] = (z, 128)
    for name, (x, group) in cases.items():
        xd = x.to(dev).contiguous()
        p, s = ref.quantize_int4(xd.view(-1), group)
        dq = ref.dequantize_int4(p, s, x.numel(), group)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, "int4_%s.npz" % name), kind="int4", group=group,
                            x=x.numpy().reshape(-1), packed=p.cpu().numpy(),
                            scales=s.cpu().view(torch.int16).numpy().view(np.uint16), dq=dq.cpu().numpy())

    # routing: softmax-like probabilities rounded through bf16 (creates ties), 68 experts, top-6
    logits = randn(256, 68)
    probs = torch.softmax(logits, dim=-1).to(torch.bfloat16).float()
    pd = probs.to(dev).contiguous()
    idx, val = ref.topk(pd, 6)
    norm = ref.normalize_rows(val)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "routing_68x6.npz"), kind="routing", k=6, probs=probs.numpy(),
                        indices=idx.cpu().numpy(), values=val.cpu().numpy(), normalized=norm.cpu().numpy())

    # dispatch + combine over the reference's kernels with the dispatch map of the host algorithm
    # (CAIF_Ops::MoEBuildDispatchMap is host code; the oracle restates it)
    xs = randn(256, 32)
    dmap, off, total = orc.build_dispatch_map(idx.cpu().numpy(), 68)
    idx_d = idx.contiguous()
    buf = ref.moe_dispatch(xs.to(dev), idx_d, torch.from_numpy(dmap).to(dev), torch.from_numpy(off).to(dev), total)
    comb = ref.moe_combine(buf, idx_d, norm.contiguous(), torch.from_numpy(dmap).to(dev), torch.from_numpy(off).to(dev),
                           256)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "dispatch_68x6.npz"), kind="dispatch", num_experts=68, x=xs.numpy(),
                        indices=idx.cpu().numpy(), weights=norm.cpu().numpy(), buffer=buf.cpu().numpy(),
                        combined=comb.cpu().numpy())
    # backward of the pair: packed-buffer gradient, routing-weight gradient, token gradient
    go = randn(256, 32)
    dmap_d, off_d = torch.from_numpy(dmap).to(dev), torch.from_numpy(off).to(dev)
    gbuf = ref.moe_combine_bwd_grad_expert(go.to(dev), idx_d, norm.contiguous(), dmap_d, off_d, total)
    gw = ref.moe_combine_bwd_grad_weights(go.to(dev), buf, idx_d, dmap_d, off_d)
    gin = ref.moe_dispatch_bwd(gbuf, idx_d, dmap_d, off_d, 256)
    torch.cuda.synchronize()
    np.savez_compressed(os.path.join(out_dir, "dispatch_backward_68x6.npz"), kind="dispatch_backward",
                        num_experts=68, indices=idx.cpu().numpy(), weights=norm.cpu().numpy(),
                        buffer=buf.cpu().numpy(), grad_output=go.numpy(), grad_buffer=gbuf.cpu().numpy(),
                        grad_weights=gw.cpu().numpy(), grad_input=gin.cpu().numpy())
    print("wrote", sorted(os.listdir(out_dir)))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py OUTPUT_DIR   (run on a box with a GPU)")
    main(sys.argv[1])
