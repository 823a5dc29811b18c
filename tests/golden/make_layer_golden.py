"""Golden vectors of the LAYER dataflow, captured from the executing reference.

Run on a box with a GPU, after `python oracle/build_ref_layers.py` has built the reference's own
layer classes (unmodified sources) into oracle/_ref/libcaif_ref_layers.so:

    python tests/golden/make_layer_golden.py OUTPUT_DIR

Every case draws seeded inputs, quantizes the weights with the CPU oracle (whose codes and scales are
pinned bit for bit against the reference's kernels elsewhere), runs the reference's
CAIF_DeviceFrozenLinear / CAIF_DeviceLoRAAdapter / CAIF_DeviceMoEFrozenExpert on them
(CAIF_Settings::MatmulMode Accuracy_e, so fp32 compute means full fp32 products) and stores inputs and
outputs.  tests/test_layer_golden.py replays the files through the oracle on the CPU and through the
C ABI on the GPU.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

import caif_oracle as orc  # noqa: E402
import reflayers as rl  # noqa: E402


def quantized(rng, out_dim, in_dim, storage, std=0.05):
    w = (rng.standard_normal((out_dim, in_dim)) * std).astype(np.float32)
    if storage == orc.I8:
        codes, scales = orc.quantize_int8_per_tensor(w)
    else:
        codes, scales = orc.quantize_int4(w, 128)
    return codes, scales


def activations(rng, rows, dim, dtype):
    return orc.round_through(rng.standard_normal((rows, dim)).astype(np.float32), dtype)


def frozen_case(path, seed, storage, act_dtype, compute, in_dim, out_dim, rows):
    rng = np.random.default_rng(seed)
    codes, scales = quantized(rng, out_dim, in_dim, storage)
    x = activations(rng, rows, in_dim, act_dtype)
    dy = activations(rng, rows, out_dim, act_dtype)
    layer = rl.frozen_linear(in_dim, out_dim, storage, compute, codes, scales)
    y, y_dtype = layer.forward(rl.to_raw(x, act_dtype), act_dtype, training=True)
    dx, dx_dtype = layer.backward(rl.to_raw(dy, act_dtype), act_dtype)
    layer.close()
    np.savez_compressed(path, kind="frozen_linear", storage=storage, act_dtype=act_dtype, compute=compute,
                        in_dim=in_dim, out_dim=out_dim, codes=codes, scales=scales, x=x, dy=dy, y=y, dx=dx,
                        y_dtype=y_dtype, dx_dtype=dx_dtype)


def lora_case(path, seed, storage, sd, compute, in_dim, out_dim, rows, rank, alpha):
    rng = np.random.default_rng(seed)
    codes, scales = quantized(rng, out_dim, in_dim, storage)
    a = orc.round_through(rng.uniform(-1 / 16, 1 / 16, (rank, in_dim)).astype(np.float32), sd)
    b = orc.round_through((rng.standard_normal((out_dim, rank)) * 0.05).astype(np.float32), sd)
    x = activations(rng, rows, in_dim, sd)
    dy = activations(rng, rows, out_dim, sd)
    base = rl.frozen_linear(in_dim, out_dim, storage, compute, codes, scales)
    layer = rl.lora_wrap(base, rank, alpha, sd, compute, rl.to_raw(a, sd), rl.to_raw(b, sd))
    y, _ = layer.forward(rl.to_raw(x, sd), sd, training=True)
    dx, _ = layer.backward(rl.to_raw(dy, sd), sd)
    d_b = layer.gradient(1, (out_dim, rank), sd)
    d_a = layer.gradient(2, (rank, in_dim), sd)
    layer.close()
    np.savez_compressed(path, kind="lora", storage=storage, sd=sd, compute=compute, in_dim=in_dim, out_dim=out_dim,
                        rank=rank, alpha=alpha, codes=codes, scales=scales, a=a, b=b, x=x, dy=dy, y=y, dx=dx, d_a=d_a,
                        d_b=d_b)


def expert_case(path, seed, storage, sd, compute, in_dim, hid, rows, gated):
    rng = np.random.default_rng(seed)
    subs = {}
    layers = {}
    for name, (o, i) in (("gate", (hid, in_dim)), ("up", (hid, in_dim)), ("down", (in_dim, hid))):
        if name == "gate" and not gated:
            continue
        codes, scales = quantized(rng, o, i, storage)
        subs[name] = (codes, scales)
        layers[name] = rl.frozen_linear(i, o, storage, compute, codes, scales)
    x = activations(rng, rows, in_dim, sd)
    dy = activations(rng, rows, in_dim, sd)
    expert = rl.frozen_expert(layers.get("gate"), layers["up"], layers["down"], in_dim, hid, sd, compute)
    y, _ = expert.forward(rl.to_raw(x, sd), sd, training=True)
    dx, _ = expert.backward(rl.to_raw(dy, sd), sd)
    expert.close()
    out = {"kind": "expert", "storage": storage, "sd": sd, "compute": compute, "in_dim": in_dim, "hid": hid,
           "gated": int(gated), "x": x, "dy": dy, "y": y, "dx": dx}
    for name, (codes, scales) in subs.items():
        out[name + "_codes"] = codes
        out[name + "_scales"] = scales
    np.savez_compressed(path, **out)


def main(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    rl.set_accuracy(True)
    j = lambda name: os.path.join(out_dir, name)
    frozen_case(j("layer_frozen_int8_f32.npz"), 11, orc.I8, orc.F32, orc.F32, 256, 192, 37)
    frozen_case(j("layer_frozen_int4_bf16.npz"), 12, orc.I4, orc.BF16, orc.BF16, 256, 192, 37)
    frozen_case(j("layer_frozen_int4_f32.npz"), 13, orc.I4, orc.F32, orc.F32, 384, 128, 20)
    lora_case(j("layer_lora_int8_bf16_f32.npz"), 21, orc.I8, orc.BF16, orc.F32, 256, 192, 64, 16, 32.0)
    lora_case(j("layer_lora_int4_bf16_bf16.npz"), 22, orc.I4, orc.BF16, orc.BF16, 256, 128, 48, 8, 16.0)
    lora_case(j("layer_lora_int8_f32_f32.npz"), 23, orc.I8, orc.F32, orc.F32, 128, 160, 33, 4, 8.0)
    expert_case(j("layer_expert_gated_int4_bf16.npz"), 31, orc.I4, orc.BF16, orc.BF16, 256, 384, 40, True)
    expert_case(j("layer_expert_plain_int8_f32.npz"), 32, orc.I8, orc.F32, orc.F32, 128, 256, 25, False)
    expert_case(j("layer_expert_gated_int8_f32.npz"), 33, orc.I8, orc.F32, orc.F32, 128, 256, 25, True)
    print("wrote", sorted(f for f in os.listdir(out_dir) if f.startswith("layer_")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_layer_golden.py OUTPUT_DIR   (run on a box with a GPU)")
    main(sys.argv[1])
