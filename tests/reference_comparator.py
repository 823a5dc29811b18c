"""GPU comparator: the reference's own device path timed on the same GPU.

Not a pytest file; run on a box with a GPU after `python oracle/build_ref_layers.py`:

    python tests/reference_comparator.py > comparator.json

It times, with CUDA events around loops of calls on the reference's stream,
  c2  CAIF_DeviceFrozenLinear int4 g128, 4096 -> 14336, bf16 activations, M = 1, 4, 16 forward, with the
      reference's default cache_fp32=true after the first call (a cuBLAS product on the cached dequantized
      weight) and with cache_fp32=false (dequantize kernel + cast + cuBLAS every call);
  c3  CAIF_DeviceLoRAAdapter over an int8 frozen linear 4096 -> 4096, rank 16, M = 8192 bf16 tokens,
      forward + backward, cache on and off;
  c5  one CAIF_DeviceMoEFrozenExpert (int4, 2048 -> 1408 -> 2048, bf16) on 1536 rows, forward + backward:
      what the reference's MoE layer runs 64 times per step, one expert after the other.
and prints one JSON object with the milliseconds and the derived GB/s and TFLOP/s.  Weights are seeded
N(0, 0.02) quantized by the CPU oracle; MatmulMode stays Performance_e (the reference's default).
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

import caif_oracle as orc  # noqa: E402
import reflayers as rl  # noqa: E402


def int4_weight(rng, out_dim, in_dim):
    w = (rng.standard_normal((out_dim, in_dim)) * 0.02).astype(np.float32)
    return orc.quantize_int4(w, 128)


def bf16(rng, rows, dim):
    return rl.to_raw(orc.round_through(rng.standard_normal((rows, dim)).astype(np.float32), orc.BF16), rl.BF16)


def main():
    rl.set_accuracy(False)
    rng = np.random.default_rng(7)
    out = {}

    in_dim, out_dim = 4096, 14336
    codes, scales = int4_weight(rng, out_dim, in_dim)
    c2 = {}
    for cache in (True, False):
        layer = rl.frozen_linear(in_dim, out_dim, rl.I4, rl.BF16, codes, scales, cache_fp32=cache)
        for m in (1, 4, 16):
            ms = layer.time(bf16(rng, m, in_dim), rl.BF16, None, rl.BF16, False, 3, 20)
            algo_bytes = out_dim * in_dim // 2 + out_dim * 32 * 2 + m * in_dim * 2 + m * out_dim * 4
            c2["cache_%s_m%d" % ("on" if cache else "off", m)] = {"ms": ms, "algorithmic_gbs": algo_bytes / ms / 1e6}
        layer.close()
    out["c2"] = c2

    dim, m, rank = 4096, 8192, 16
    w = (rng.standard_normal((dim, dim)) * 0.02).astype(np.float32)
    q, s = orc.quantize_int8_per_tensor(w)
    a = rl.to_raw(orc.round_through(rng.uniform(-1 / 64, 1 / 64, (rank, dim)).astype(np.float32), orc.BF16), rl.BF16)
    b = rl.to_raw(orc.round_through((rng.standard_normal((dim, rank)) * 1e-3).astype(np.float32), orc.BF16), rl.BF16)
    flops = 2 * (2 * m * dim * dim) + 6 * (2 * m * dim * rank)
    c3 = {}
    for cache in (True, False):
        base = rl.frozen_linear(dim, dim, rl.I8, rl.F32, q, s, cache_fp32=cache)
        layer = rl.lora_wrap(base, rank, 32.0, rl.BF16, rl.F32, a, b)
        ms = layer.time(bf16(rng, m, dim), rl.BF16, bf16(rng, m, dim), rl.BF16, True, 3, 10)
        c3["cache_%s" % ("on" if cache else "off")] = {"ms": ms, "tflops": flops / ms / 1e9}
        layer.close()
    out["c3"] = c3

    hidden, ffn, rows = 2048, 1408, 1536
    subs = []
    for (o, i) in ((ffn, hidden), (ffn, hidden), (hidden, ffn)):
        cds, scs = int4_weight(rng, o, i)
        subs.append(rl.frozen_linear(i, o, rl.I4, rl.BF16, cds, scs, cache_fp32=True))
    expert = rl.frozen_expert(subs[0], subs[1], subs[2], hidden, ffn, rl.BF16, rl.BF16)
    ms = expert.time(bf16(rng, rows, hidden), rl.BF16, bf16(rng, rows, hidden), rl.BF16, True, 3, 20)
    eflops = 2 * 3 * 2.0 * rows * hidden * ffn
    out["c5"] = {"one_expert_1536_rows_ms": ms, "tflops": eflops / ms / 1e9,
                 "step_of_64_experts_ms": 64 * ms,
                 "note": "cache_fp32=true: the fp32 copies of 64 x 3 expert weights (2.2 GB) stay resident"}
    expert.close()
    print(json.dumps(out))


if __name__ == "__main__":
    main()
