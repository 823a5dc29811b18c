"""The C++ layer classes that mirror the reference's interface (caif_b200/host/):
what a CPU box can check (library loads, exports, argument errors) and, on a GPU,
the reference's own layer tests restated: shapes and output dtype
(tests/test_device_frozen_linear.cpp), zero trainable parameters, description
and name strings, LoRA with B = 0 equals the base, parameter order
(tests/test_device_lora_adapter.cpp:371-530), int4 path against
dequantize-then-fp32 within 2e-2 (tests/test_device_frozen_linear.cpp:1234-1310)."""
import ctypes

import numpy as np
import pytest
import torch

import caif_oracle as orc
from caif_b200 import host_layers as hl
from caif_b200 import native as nv


def test_host_library_exports():
    lib = hl.lib()
    missing = [n for n in hl.EXPORTS if not hasattr(lib, n)]
    assert not missing, missing


def test_factory_rejects_illegal_pairs_without_a_gpu():
    with pytest.raises(hl.HostLayerError, match="unsupported"):
        hl.Layer(16, 16, storage=1)      # Float64 storage is not a cell
    with pytest.raises(hl.HostLayerError, match="unsupported"):
        hl.Layer(16, 16, storage=nv.I8, compute=nv.I8)
    with pytest.raises(hl.HostLayerError):
        hl.Layer(0, 16, storage=nv.F32)


def test_description_and_counts_without_a_gpu():
    layer = hl.Layer(24, 40, storage=nv.I4, compute=nv.BF16)
    assert layer.description() == "FrozenLinear(24,40,int4)"
    assert layer.counts() == (0, 0, 1)
    assert layer.parameter_names("blk.") == []
    layer.close()


@pytest.mark.gpu
def test_frozen_linear_layer_every_storage():
    from gpu_util import act, make_weight, max_rel_err

    rng = np.random.default_rng(3)
    for storage in (orc.F32, orc.F16, orc.BF16, orc.I8, orc.I4):
        in_dim, out_dim, m = 64, 48, 10
        weight, codes, scales = make_weight(rng, out_dim, in_dim, storage)
        layer = hl.Layer(in_dim, out_dim, storage)
        with pytest.raises(hl.HostLayerError, match="weight not loaded"):
            layer.forward(torch.zeros(m, in_dim, device="cuda"))
        layer.load_weight(weight.codes, storage if storage != orc.I4 else nv.I4)
        if scales is not None:
            layer.load_scales_from_host(np.ascontiguousarray(scales).tobytes())
        x_np, x = act(rng, m, in_dim, orc.F32)
        dy_np, dy = act(rng, m, out_dim, orc.F32)
        with pytest.raises(hl.HostLayerError, match="Forward"):
            layer.backward(dy)                       # no training-mode forward yet
        y = layer.forward(x.view(2, 5, in_dim).contiguous())   # 3-D input flattens to rows
        assert y.dtype == torch.float32 and tuple(y.shape) == (m, out_dim)
        dx = layer.backward(dy)
        wc = orc.weight_to_compute(codes, scales, storage, in_dim, out_dim, orc.F32, weight.scheme, weight.group_size)
        assert max_rel_err(y.cpu().numpy(), orc.frozen_linear_forward(x_np, wc)) <= 1e-4
        assert max_rel_err(dx.cpu().numpy(), orc.frozen_linear_backward(dy_np, wc)) <= 1e-4
        assert np.array_equal(layer.frozen_tensor_fp32().cpu().numpy(), wc)
        with pytest.raises(hl.HostLayerError, match="last dim"):
            layer.forward(torch.zeros(m, in_dim + 1, device="cuda"))
        layer.close()


@pytest.mark.gpu
def test_int4_layer_against_dequantize_then_fp32_within_2e2():
    from gpu_util import act, make_weight, max_rel_err

    rng = np.random.default_rng(4)
    in_dim, out_dim, m = 256, 128, 64
    weight, codes, scales = make_weight(rng, out_dim, in_dim, orc.I4)
    layer = hl.Layer(in_dim, out_dim, orc.I4, compute=nv.BF16)
    layer.load_weight(weight.codes, nv.I4)
    layer.load_scales_from_host(np.ascontiguousarray(scales).tobytes())
    x_np, x = act(rng, m, in_dim, orc.BF16)
    y = layer.forward(x)
    want = orc.gemm_nt(x_np, orc.dequantize_int4(codes, scales, in_dim * out_dim, 128).reshape(out_dim, in_dim))
    assert max_rel_err(y.cpu().numpy(), want) <= 2e-2
    layer.close()


@pytest.mark.gpu
def test_lora_adapter_layer():
    from gpu_util import act, make_weight, max_rel_err

    rng = np.random.default_rng(5)
    in_dim, out_dim, m, rank, alpha = 128, 96, 40, 8, 16.0
    weight, codes, scales = make_weight(rng, out_dim, in_dim, orc.I8)
    layer = hl.Layer(in_dim, out_dim, orc.I8)
    layer.load_weight(weight.codes, nv.I8)
    layer.load_scales_from_host(np.ascontiguousarray(scales).tobytes())
    x_np, x = act(rng, m, in_dim, orc.F32)
    base = layer.forward(x).clone()
    layer.wrap_lora(rank, alpha, storage=nv.F32, seed=7)
    assert layer.description() == "LoRA(rank=8,alpha=16,128,96)+FrozenLinear(128,96,int8)"
    assert layer.parameter_names("q.") == ["q.lora_a.weight", "q.lora_b.weight"]
    assert layer.counts() == (2, rank * in_dim + out_dim * rank, 1)
    # A: Kaiming-uniform from mt19937(seed) within +-sqrt(1/in); B zero => output equals the base
    a = layer.parameter(0, torch.empty(rank, in_dim, device="cuda"))
    b = layer.parameter(1, torch.empty(out_dim, rank, device="cuda"))
    assert float(a.abs().max()) <= np.sqrt(1.0 / in_dim) and float(a.abs().max()) > 0 and float(b.abs().max()) == 0
    assert torch.equal(layer.forward(x), base)
    # non-zero B: forward/backward against the oracle
    b_new = torch.from_numpy((rng.standard_normal((out_dim, rank)) * 1e-2).astype(np.float32)).cuda()
    layer.set_parameter(1, b_new)
    wc = orc.weight_to_compute(codes, scales, orc.I8, in_dim, out_dim)
    want_y, hidden = orc.lora_forward(x_np, orc.frozen_linear_forward(x_np, wc), a.cpu().numpy(), b_new.cpu().numpy(),
                                      alpha)
    y = layer.forward(x)
    assert max_rel_err(y.cpu().numpy(), want_y) <= 1e-4
    dy_np, dy = act(rng, m, out_dim, orc.F32)
    dx = layer.backward(dy)
    want_dx, want_da, want_db = orc.lora_backward(dy_np, x_np, hidden, orc.frozen_linear_backward(dy_np, wc),
                                                  a.cpu().numpy(), b_new.cpu().numpy(), alpha)
    assert max_rel_err(dx.cpu().numpy(), want_dx) <= 1e-4
    assert max_rel_err(layer.parameter(0, a, gradient=True).cpu().numpy(), want_da) <= 1e-4
    assert max_rel_err(layer.parameter(1, b, gradient=True).cpu().numpy(), want_db) <= 1e-4
    layer.close()


@pytest.mark.gpu
@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("storage,sd,compute", [(orc.I4, orc.BF16, orc.BF16), (orc.I8, orc.F32, orc.F32)])
def test_moe_frozen_expert_layer(gated, storage, sd, compute):
    """CAIF_DeviceMoEFrozenExpert over three frozen linears, gated and not
    (src/caif_device_moe_frozen_expert.cpp:91-332): forward, backward after a training forward,
    no trainable parameters, backward before forward refused."""
    from gpu_util import TORCH_DTYPE, act, make_weight, max_rel_err

    rng = np.random.default_rng(60 + storage + int(gated))
    in_dim, hid, m = 256, 384, 70
    subs, oracle_w = [], []
    for (o, i) in ((hid, in_dim), (hid, in_dim), (in_dim, hid)):
        weight, codes, scales = make_weight(rng, o, i, storage, std=0.05)
        layer = hl.Layer(i, o, storage, compute)
        layer.load_weight(weight.codes, storage)
        layer.load_scales_from_host(np.ascontiguousarray(scales).tobytes())
        subs.append(layer)
        oracle_w.append(orc.weight_to_compute(codes, scales, storage, i, o, compute, weight.scheme, weight.group_size))
    gate, up, down = subs
    wg, wu, wd = oracle_w
    if not gated:
        gate.close()
        gate, wg = None, None
    expert = hl.FrozenExpert(gate, up, down, in_dim, hid, sd, compute)
    assert expert.counts()[:2] == (0, 0)
    assert expert.description() == "MoEFrozenExpert(%d,%d)" % (in_dim, hid)
    x_np, x = act(rng, m, in_dim, sd)
    dy_np, dy = act(rng, m, in_dim, sd)
    with pytest.raises(hl.HostLayerError, match="Forward"):
        expert.backward(dy)
    y = expert.forward(x, training=True)
    assert y.dtype == TORCH_DTYPE[sd] and tuple(y.shape) == (m, in_dim)
    want, g, u = orc.frozen_expert_forward(x_np, wg, wu, wd, compute, sd)
    tol = 2e-2 if sd == orc.BF16 else 1e-4
    assert max_rel_err(y.float().cpu().numpy(), want) <= tol
    dx = expert.backward(dy)
    want_dx = orc.frozen_expert_backward(dy_np, g, u, wg, wu, wd, compute, sd)
    assert max_rel_err(dx.float().cpu().numpy(), want_dx) <= tol
    with pytest.raises(hl.HostLayerError, match="input_dim"):
        expert.forward(torch.zeros(m, in_dim + 1, dtype=TORCH_DTYPE[sd], device="cuda"))
    expert.close()


@pytest.mark.gpu
@pytest.mark.parametrize("sd", [nv.F32, nv.BF16])
def test_adapter_checkpoint_round_trip(tmp_path, sd):
    """The trainable tensors of an adapter go to a SafeTensors file under their parameter names and come back into
    a fresh adapter over the same frozen base: same outputs bit for bit; the file is what the safetensors package
    reads; a file with another rank is refused."""
    from safetensors.torch import load_file
    from gpu_util import act, make_weight

    rng = np.random.default_rng(21)
    in_dim, out_dim, m, rank = 128, 96, 33, 8
    tdt = nv._CODE_TO_TORCH[sd]
    weight, codes, scales = make_weight(rng, out_dim, in_dim, orc.I4)

    def fresh(r, seed):
        layer = hl.Layer(in_dim, out_dim, orc.I4, compute=sd)
        layer.load_weight(weight.codes, nv.I4)
        layer.load_scales_from_host(np.ascontiguousarray(scales).tobytes())
        return layer.wrap_lora(r, 16.0, storage=sd, compute=sd, seed=seed)

    trained = fresh(rank, 3)
    b = (torch.randn(out_dim, rank, device="cuda") * 0.02).to(tdt)
    trained.set_parameter(1, b)
    _, x = act(rng, m, in_dim, sd)
    want = trained.forward(x).clone()
    path = str(tmp_path / "adapter.safetensors")
    trained.save_parameters(path, "blk.q.")
    on_disk = load_file(path)
    assert sorted(on_disk) == ["blk.q.lora_a.weight", "blk.q.lora_b.weight"]
    assert on_disk["blk.q.lora_b.weight"].dtype == tdt and torch.equal(on_disk["blk.q.lora_b.weight"].cuda(), b)
    restored = fresh(rank, 99)                    # another seed: A differs until the file is loaded
    assert not torch.equal(restored.forward(x), want)
    f = hl.SafeTensors(path)
    restored.load_parameters(f, "blk.q.")
    assert torch.equal(restored.forward(x), want)
    other = fresh(4, 3)
    with pytest.raises(hl.HostLayerError, match="does not match"):
        other.load_parameters(f, "blk.q.")
    with pytest.raises(hl.HostLayerError, match="not found"):
        restored.load_parameters(f, "elsewhere.")
    f.close()
    for layer in (trained, restored, other):
        layer.close()
