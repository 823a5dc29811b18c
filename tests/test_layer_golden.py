"""Golden vectors captured from the EXECUTING reference layers (tests/golden/make_layer_golden.py:
CAIF_DeviceFrozenLinear, CAIF_DeviceLoRAAdapter, CAIF_DeviceMoEFrozenExpert compiled from the
reference's unmodified sources, MatmulMode Accuracy_e) replayed

  * through the CPU oracle (every box): pins the oracle's layer dataflow -- which tensor is rounded
    to which dtype where -- against what the reference itself computes;
  * through the C ABI on the GPU: the product against the reference on the same inputs.

Tolerances (max |err| / max |want|): 1e-4 for fp32 compute, 2e-2 for bf16 compute; where storage is
bf16 a result can differ by one bf16 rounding (2^-8 relative) between two correct implementations, so
bf16-stored results are held to 1e-2 even under fp32 compute.
"""
import glob
import os

import numpy as np
import pytest

import caif_oracle as orc

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "layer_*.npz")))


def _tol(compute, stored):
    if compute != orc.F32:
        return 2e-2
    return 1e-2 if stored != orc.F32 else 1e-4


def _rel(got, want):
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(np.asarray(got, np.float64) - want))) / max(float(np.max(np.abs(want))), 1e-30)


def _weight(codes, scales, storage, in_dim, out_dim, compute):
    return orc.weight_to_compute(codes, scales, storage, in_dim, out_dim, compute, orc.PER_TENSOR, 128)


def test_layer_goldens_are_present():
    kinds = sorted(str(np.load(f)["kind"]) for f in GOLDEN)
    assert kinds.count("frozen_linear") >= 3 and kinds.count("lora") >= 3 and kinds.count("expert") >= 3, kinds


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_replays_the_reference_layers(path):
    g = np.load(path)
    kind = str(g["kind"])
    storage, compute = int(g["storage"]), int(g["compute"])
    if kind == "frozen_linear":
        in_dim, out_dim = int(g["in_dim"]), int(g["out_dim"])
        wc = _weight(g["codes"], g["scales"], storage, in_dim, out_dim, compute)
        assert _rel(orc.frozen_linear_forward(g["x"], wc, compute), g["y"]) <= _tol(compute, orc.F32)
        assert _rel(orc.frozen_linear_backward(g["dy"], wc, compute), g["dx"]) <= _tol(compute, orc.F32)
        assert int(g["y_dtype"]) == orc.F32 and int(g["dx_dtype"]) == orc.F32    # the layer returns fp32
    elif kind == "lora":
        in_dim, out_dim, sd = int(g["in_dim"]), int(g["out_dim"]), int(g["sd"])
        wc = _weight(g["codes"], g["scales"], storage, in_dim, out_dim, compute)
        base = orc.frozen_linear_forward(g["x"], wc, compute)
        y, hidden = orc.lora_forward(g["x"], base, g["a"], g["b"], float(g["alpha"]), sd)
        tol = _tol(compute, sd)
        assert _rel(y, g["y"]) <= tol
        dx, d_a, d_b = orc.lora_backward(g["dy"], g["x"], hidden, orc.frozen_linear_backward(g["dy"], wc, compute),
                                         g["a"], g["b"], float(g["alpha"]), sd)
        assert _rel(dx, g["dx"]) <= tol
        assert _rel(d_a, g["d_a"]) <= tol
        assert _rel(d_b, g["d_b"]) <= tol
    else:
        in_dim, hid, sd, gated = int(g["in_dim"]), int(g["hid"]), int(g["sd"]), bool(int(g["gated"]))
        wu = _weight(g["up_codes"], g["up_scales"], storage, in_dim, hid, compute)
        wd = _weight(g["down_codes"], g["down_scales"], storage, hid, in_dim, compute)
        wg = _weight(g["gate_codes"], g["gate_scales"], storage, in_dim, hid, compute) if gated else None
        y, gate, up = orc.frozen_expert_forward(g["x"], wg, wu, wd, compute, sd)
        tol = _tol(compute, sd)
        assert _rel(y, g["y"]) <= tol
        assert _rel(orc.frozen_expert_backward(g["dy"], gate, up, wg, wu, wd, compute, sd), g["dx"]) <= tol


@pytest.mark.gpu
@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_c_abi_matches_the_reference_layers(path):
    import torch

    from caif_b200 import native as nv
    from gpu_util import TORCH_DTYPE, f16_bits_to_dev, to_dev

    g = np.load(path)
    kind = str(g["kind"])
    storage, compute = int(g["storage"]), int(g["compute"])

    def weight(codes, scales, in_dim, out_dim):
        if storage == orc.I4:
            return nv.Weight(to_dev(codes), nv.I4, in_dim, out_dim, f16_bits_to_dev(scales), group_size=128)
        return nv.Weight(to_dev(codes), nv.I8, in_dim, out_dim, to_dev(scales))

    if kind == "frozen_linear":
        in_dim, out_dim, act = int(g["in_dim"]), int(g["out_dim"]), int(g["act_dtype"])
        w = weight(g["codes"], g["scales"], in_dim, out_dim)
        y = nv.linear_fwd(w, to_dev(g["x"], TORCH_DTYPE[act]), torch.float32, compute)
        dx = nv.linear_dx(w, to_dev(g["dy"], TORCH_DTYPE[act]), torch.float32, compute)
        assert _rel(y.cpu().numpy(), g["y"]) <= _tol(compute, orc.F32)
        assert _rel(dx.cpu().numpy(), g["dx"]) <= _tol(compute, orc.F32)
    elif kind == "lora":
        in_dim, out_dim, sd = int(g["in_dim"]), int(g["out_dim"]), int(g["sd"])
        w = weight(g["codes"], g["scales"], in_dim, out_dim)
        lora = nv.Lora(to_dev(g["a"], TORCH_DTYPE[sd]), to_dev(g["b"], TORCH_DTYPE[sd]), float(g["alpha"]))
        x, dy = to_dev(g["x"], TORCH_DTYPE[sd]), to_dev(g["dy"], TORCH_DTYPE[sd])
        y, hidden = nv.lora_linear_fwd(w, lora, x, compute)
        dx, d_a, d_b = nv.lora_linear_bwd(w, lora, dy, x, hidden, compute)
        tol = _tol(compute, sd)
        assert _rel(y.float().cpu().numpy(), g["y"]) <= tol
        assert _rel(dx.float().cpu().numpy(), g["dx"]) <= tol
        assert _rel(d_a.float().cpu().numpy(), g["d_a"]) <= tol
        assert _rel(d_b.float().cpu().numpy(), g["d_b"]) <= tol
    else:
        in_dim, hid, sd, gated = int(g["in_dim"]), int(g["hid"]), int(g["sd"]), bool(int(g["gated"]))
        up = [weight(g["up_codes"], g["up_scales"], in_dim, hid)]
        down = [weight(g["down_codes"], g["down_scales"], hid, in_dim)]
        gate = [weight(g["gate_codes"], g["gate_scales"], in_dim, hid)] if gated else None
        x, dy = to_dev(g["x"], TORCH_DTYPE[sd]), to_dev(g["dy"], TORCH_DTYPE[sd])
        rows = x.shape[0]
        out, g_out, u_out = nv.grouped_expert_fwd(gate, up, down, [0, rows], x, compute)
        dx = nv.grouped_expert_bwd(gate, up, down, [0, rows], dy, g_out, u_out, compute)
        tol = _tol(compute, sd)
        assert _rel(out.float().cpu().numpy(), g["y"]) <= tol
        assert _rel(dx.float().cpu().numpy(), g["dx"]) <= tol
