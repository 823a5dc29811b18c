#!/usr/bin/env python
"""Benchmark of the quantized frozen-linear hot path on B200.

`python bench.py --gpus N --steps K --warmup W` prints ONE JSON line from rank 0.  The headline
of the line is the decode workload (c2); the same line carries, under `workloads`, every
workload of the path, each with its own value, roofline, end-to-end figure and CPU baseline:

  c2     decode-shaped int4 frozen linear in=4096, out=14336, group 128, bf16 activations,
         M in {1,4,16}, forward only.  A step is 32 passes ("layers") over 8 independent weight
         copies at each M: 768 launches.  The copies total 242 MB, more than the 126 MB L2, and
         consecutive launches use different copies, so every launch streams its codes from HBM.
         Metric: algorithmic bytes per second (codes + scales + x + y).
  c3     training-shaped int8 frozen linear 4096->4096 with a rank-16 LoRA adapter, M=8192 bf16:
         forward + dX/dA/dB.  Metric TFLOP/s.  One GPU only.
  c5     the frozen int4 experts of the MoE config: 64 experts 2048->1408->2048 (SwiGLU), 16384
         tokens routed top-6: dispatch, grouped forward, combine, and the whole backward
         (combine-backward, grouped dX, dispatch-backward).  Metric TFLOP/s over the expert GEMMs.
         N > 1: experts sharded by expert, tokens sharded by rank, NCCL all-to-all both ways.
  c4lin  the frozen-linear part of the Llama-3-8B-shaped fine-tune step: 32 layers x 7 projections
         (q, k, v, o, gate, up, down), int4 g128 base + LoRA r16, 16384 tokens, forward +
         dX/dA/dB.  Metric tokens/s of that linear path.  N > 1: every projection column-parallel
         by output features (strong scaling): NCCL all-gather of Y, reduce-scatter of dX,
         all-reduce of dA, on a second stream beside the next projection's kernels.

Weights are seeded N(0, 0.02) quantized by the library's own (reference bit-exact) quantizers;
activations seeded N(0,1); LoRA A uniform(+-1/64), B N(0,1e-3).  Nothing is read from disk.

`--impl reference` times the reference's CPU path for the same workloads (dequantize once, as the
reference's cache_fp32=true does, then OpenBLAS sgemm per product) on all host cores, each step a
bounded sample of the workload, and prints the same line shape with "impl": "reference".
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

C2_IN, C2_OUT, C2_GROUP = 4096, 14336, 128
C2_MS = (1, 4, 16)
C2_COPIES = 8
C2_LAYERS = 32

# (name, out, in) of the seven projections of one Llama-3-8B-shaped layer
C4_PROJ = (("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
           ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336))
C4_LAYERS, C4_TOKENS, C4_RANK, C4_ALPHA = 32, 16384, 16, 32.0

C5_HIDDEN, C5_FFN, C5_EXPERTS, C5_TOKENS, C5_TOPK = 2048, 1408, 64, 16384, 6

WORKLOADS = ("c2", "c3", "c5", "c4lin")

METRIC = {
    "c2": ("decode int4 frozen-linear forward, algorithmic HBM bytes per second", "GB/s"),
    "c3": ("int8 frozen linear + LoRA r16, forward + dX/dA/dB, TFLOP/s", "TFLOP/s"),
    "c5": ("frozen int4 experts, grouped forward + dX, TFLOP/s", "TFLOP/s"),
    "c4lin": ("int4 frozen linears + LoRA r16 of a Llama-3-8B-shaped step, linear-path tokens per second", "tokens/s"),
}
SCALING = {"c2": "weak", "c3": "weak", "c5": "strong", "c4lin": "strong"}


def config_for(workload, world):
    """The workload description; the two arms of the benchmark print the same dict."""
    if workload == "c2":
        par = "1 GPU" if world == 1 else (
            "column-parallel x%d: a layer of out=%d, one [14336, 4096] shard per GPU; every launch stores its slice "
            "of Y into all ranks' result buffers over NVLink (peer memory), one 4-byte all-reduce per step as the "
            "completion signal" % (world, world * C2_OUT))
        return {"workload": "c2: in=4096 out=14336 int4 g128, M in {1,4,16}, forward; step = 32 layers x 8 weight "
                            "copies x 3 M = 768 launches",
                "l2": "8 weight copies = 242 MB > 126 MB L2; consecutive launches use different copies, a copy "
                      "returns 8 launches later",
                "parallelism": par}
    if workload == "c3":
        return {"workload": "c3: 4096->4096 int8 per-tensor + LoRA r16 a32, M=8192 bf16, fwd + dX/dA/dB",
                "l2": "two activation sets (268 MB) alternated between steps, larger than L2",
                "parallelism": "1 GPU"}
    if workload == "c5":
        par = "1 GPU" if world == 1 else (
            "experts sharded x%d (%d per GPU), tokens sharded x%d; counts exchanged, then NCCL all-to-all of the "
            "packed rows to the experts' owners and back, forward and backward" % (world, C5_EXPERTS // world, world))
        return {"workload": "c5: 64 frozen int4 experts 2048->1408->2048 (SwiGLU), 16384 tokens top-6: dispatch, "
                            "grouped fwd, combine, combine-bwd, grouped dX, dispatch-bwd",
                "l2": "packed buffers of 98304 rows (403 MB each) stream through L2 every step",
                "parallelism": par}
    par = "1 GPU" if world == 1 else (
        "every projection column-parallel x%d by output features (strong scaling): NCCL all-gather of Y, "
        "reduce-scatter of dX, all-reduce of dA on a second stream beside the next projection" % world)
    return {"workload": "c4lin: 32 layers x (q,k,v,o,gate,up,down) int4 g128 + LoRA r16 a32, 16384 tokens bf16, "
                        "fwd + dX/dA/dB of every projection",
            "l2": "3.6 GB of codes and 134-470 MB activations per projection: nothing stays in L2",
            "parallelism": par}


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def _recorded_traffic():
    """DRAM bytes per launch of the dominant kernels, as recorded from ncu captures (read + write)."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except Exception:
        return {}


def c2_bytes(m, out_dim=C2_OUT):
    """Algorithmic bytes of one decode forward: packed codes + fp16 scales + bf16 x + fp32 y."""
    return out_dim * C2_IN // 2 + (out_dim * C2_IN // C2_GROUP) * 2 + m * C2_IN * 2 + m * out_dim * 4


def c3_flops(m, dim=4096, rank=16):
    return 2 * (2 * m * dim * dim) + 6 * (2 * m * dim * rank)


def c5_flops(rows, hidden=C5_HIDDEN, ffn=C5_FFN):
    # three products forward and three for dX, 2 flops per multiply-add
    return 2 * 3 * 2.0 * rows * hidden * ffn


def c4_flops(tokens, layers=C4_LAYERS, rank=C4_RANK):
    per_layer = 0.0
    for _, o, i in C4_PROJ:
        per_layer += 2 * (2.0 * tokens * o * i) + 6.0 * tokens * rank * (o + i)
    return layers * per_layer


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        try:
            with open(self.path) as f:
                for line in f:
                    parts = [p.strip() for p in line.split(",")]
                    if len(parts) < 9:
                        continue
                    try:
                        sm.append(float(parts[1]))
                        mx = float(parts[2])
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                         parts[5:9]):
                        if val.lower().startswith("active"):
                            reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            sm.sort()
            # median of the upper half: samples taken while the GPU was busy
            busy = sm[len(sm) // 2:]
            out["sm_mhz"] = busy[len(busy) // 2]
            out["sm_max_mhz"] = mx
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ----------------------------------------------------------------------- CPU arm
def _cpu_threads():
    """Give the host BLAS and the oracle's OpenMP loops every core.  A launcher may export
    OMP_NUM_THREADS=1 for its ranks; the CPU arm is one process and takes the whole host."""
    n = os.cpu_count() or 1
    for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[var] = str(n)
    used = n
    try:
        import threadpoolctl

        threadpoolctl.threadpool_limits(limits=n)
        counts = [int(d.get("num_threads", 0)) for d in threadpoolctl.threadpool_info()
                  if d.get("user_api") == "blas"]
        if counts:
            used = max(counts)
    except Exception:
        pass
    return used


def _cpu_loop(step, steps, warmup, budget_s):
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        step()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    return time.perf_counter() - t0, done


class _RefHostOps:
    """The reference's own Host_e matmul (CAIF_Ops::MatMulTransposeB on host tensors ->
    src/caif_host_gemm.cpp -> cblas_sgemm), from the reference's unmodified sources compiled into
    oracle/_ref/libcaif_ref_layers.so.  Raises when that library cannot be loaded."""

    def __init__(self):
        import ctypes

        import numpy as np

        self.ct, self.np = ctypes, np
        self.lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libcaif_ref_layers.so"))
        self.lib.refl_last_error.restype = ctypes.c_char_p

    def tensor(self, rows, cols, init=None):
        ct = self.ct
        h, d = ct.c_void_p(), ct.POINTER(ct.c_float)()
        if self.lib.refl_host_tensor(ct.c_uint32(rows), ct.c_uint32(cols), ct.byref(h), ct.byref(d)) != 0:
            raise RuntimeError(self.lib.refl_last_error().decode())
        view = self.np.ctypeslib.as_array(d, shape=(rows, cols))
        if init is not None:
            view[:] = init
        return h, view

    def matmul_nt(self, a, b, out):
        if self.lib.refl_host_matmul(2, a, b, out) != 0:
            raise RuntimeError(self.lib.refl_last_error().decode())


def cpu_reference_c2(steps, warmup, budget_s=20.0):
    """The reference's Host_e path for this layer with its default cache_fp32=true: the int4 weights are
    dequantized to fp32 once (restated kernel, OpenMP, outside the timed loop, as the reference's cache does
    after the first call), then every forward is CAIF_Ops::MatMulTransposeB on host tensors (OpenBLAS sgemm):
    the reference's own code where its library is available (kind "reference"), numpy's sgemm otherwise
    (kind "port").  One sample step = one of the 32 layer passes: a forward at each M in {1,4,16} on each
    of the 8 copies."""
    cores = _cpu_threads()
    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import caif_oracle as orc

    try:
        ref = _RefHostOps()
    except Exception:
        ref = None
    rng = np.random.default_rng(1235)
    wds = []
    for _ in range(C2_COPIES):
        w = (rng.standard_normal((C2_OUT, C2_IN)) * 0.02).astype(np.float32)
        packed, scales = orc.quantize_int4(w, C2_GROUP)
        del w
        wd = orc.dequantize_int4(packed, scales, C2_OUT * C2_IN, C2_GROUP).reshape(C2_OUT, C2_IN)
        wds.append(ref.tensor(C2_OUT, C2_IN, wd)[0] if ref is not None else wd)
    xs = [orc.round_through(rng.standard_normal((m, C2_IN)).astype(np.float32), orc.BF16) for m in C2_MS]
    if ref is not None:
        xt = [ref.tensor(x.shape[0], C2_IN, x)[0] for x in xs]
        yt = [ref.tensor(x.shape[0], C2_OUT)[0] for x in xs]

        def step():
            for x, y in zip(xt, yt):
                for wd in wds:
                    ref.matmul_nt(x, wd, y)
    else:
        def step():
            for x in xs:
                for wd in wds:
                    orc.gemm_nt(x, wd, exact=False)

    dt, done = _cpu_loop(step, steps, warmup, budget_s)
    bytes_per_step = C2_COPIES * sum(c2_bytes(m) for m in C2_MS)
    how = ("the reference's CAIF_Ops::MatMulTransposeB on host tensors (its own sources, OpenBLAS sgemm)"
           if ref is not None else "numpy sgemm (OpenBLAS)")
    return {"value": bytes_per_step * done / dt / 1e9, "ms_per_step": dt / done * 1e3, "steps": done, "cores": cores,
            "kind": "reference" if ref is not None else "port",
            "sample": "%d sample steps, each ONE of the 32 layer passes of the step: %s at M=1,4,16 on 8 cached fp32 "
                      "14336x4096 weights (dequantized once)" % (done, how)}


def cpu_reference_c3(steps, warmup, budget_s=25.0):
    """Reference Host_e path for the training config on a bounded sample: M=512 of the 8192 tokens (1/16 of a
    step): the fp32 weight is dequantized once (the reference's default cache_fp32=true), each step is sgemm
    forward and dX + the six LoRA matmuls."""
    cores = _cpu_threads()
    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import caif_oracle as orc

    rng = np.random.default_rng(1236)
    dim, rank, m = 4096, 16, 512
    w = (rng.standard_normal((dim, dim)) * 0.02).astype(np.float32)
    q, s = orc.quantize_int8_per_tensor(w)
    a = rng.uniform(-1 / 64, 1 / 64, (rank, dim)).astype(np.float32)
    b = (rng.standard_normal((dim, rank)) * 1e-3).astype(np.float32)
    x = orc.round_through(rng.standard_normal((m, dim)).astype(np.float32), orc.BF16)
    dy = orc.round_through(rng.standard_normal((m, dim)).astype(np.float32), orc.BF16)
    wd = orc.dequantize_int8_per_tensor(q, s)  # cache_fp32=true: dequantized once, outside the loop

    def step():
        base = orc.gemm_nt(x, wd, exact=False)
        _, hidden = orc.lora_forward(x, base, a, b, 32.0, orc.BF16, exact=False)
        dx_base = orc.gemm_nn(dy, wd, exact=False)
        orc.lora_backward(dy, x, hidden, dx_base, a, b, 32.0, orc.BF16, exact=False)

    dt, done = _cpu_loop(step, steps, warmup, budget_s)
    flops = c3_flops(m)
    return {"value": flops * done / dt / 1e12, "ms_per_step": dt / done * 1e3, "steps": done, "cores": cores,
            "sample": "%d sample steps at M=%d tokens (1/16 of the 8192-token step): sgemm fwd/dX on the cached fp32 "
                      "weight + LoRA" % (done, m)}


def cpu_reference_c5(steps, warmup, budget_s=25.0):
    """Reference Host_e path for the frozen experts on a bounded sample: 4 of the 64 experts with 256 rows each
    (1024 of the 98,304 packed rows): cached fp32 weights (dequantized once), the expert loop of the layer with
    sgemm for the six products and the elementwise steps in numpy."""
    cores = _cpu_threads()
    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import caif_oracle as orc

    rng = np.random.default_rng(1238)
    hidden, ffn, n_exp, rows = C5_HIDDEN, C5_FFN, 4, 256
    ws = []
    for _ in range(n_exp):
        trio = []
        for (o, i) in ((ffn, hidden), (ffn, hidden), (hidden, ffn)):
            w = (rng.standard_normal((o, i)) * 0.02).astype(np.float32)
            pk, sc = orc.quantize_int4(w, 128)
            trio.append(orc.dequantize_int4(pk, sc, o * i, 128).reshape(o, i))
        ws.append(trio)
    x = orc.round_through(rng.standard_normal((n_exp * rows, hidden)).astype(np.float32), orc.BF16)
    dy = orc.round_through(rng.standard_normal((n_exp * rows, hidden)).astype(np.float32), orc.BF16)

    def step():
        for e in range(n_exp):
            xe = x[e * rows:(e + 1) * rows]
            _, g, u = orc.frozen_expert_forward(xe, ws[e][0], ws[e][1], ws[e][2], orc.F32, orc.BF16, exact=False)
            orc.frozen_expert_backward(dy[e * rows:(e + 1) * rows], g, u, ws[e][0], ws[e][1], ws[e][2], orc.F32,
                                       orc.BF16, exact=False)

    dt, done = _cpu_loop(step, steps, warmup, budget_s)
    flops = c5_flops(n_exp * rows)
    return {"value": flops * done / dt / 1e12, "ms_per_step": dt / done * 1e3, "steps": done, "cores": cores,
            "sample": "%d sample steps over %d experts x %d rows (1/96 of the packed rows): per-expert loop, sgemm on "
                      "cached fp32 weights, forward + dX" % (done, n_exp, rows)}


def cpu_reference_c4lin(steps, warmup, budget_s=25.0):
    """Reference Host_e path for the Llama-shaped linear path on a bounded sample: ONE of the 32 layers at 128 of
    the 16384 tokens: cached fp32 weights (dequantized once), sgemm forward and dX of the seven projections plus
    the LoRA matmuls of each."""
    cores = _cpu_threads()
    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import caif_oracle as orc

    rng = np.random.default_rng(1239)
    m = 128
    layer = []
    for _, o, i in C4_PROJ:
        w = (rng.standard_normal((o, i)) * 0.02).astype(np.float32)
        pk, sc = orc.quantize_int4(w, 128)
        del w
        wd = orc.dequantize_int4(pk, sc, o * i, 128).reshape(o, i)
        a = rng.uniform(-1 / 64, 1 / 64, (C4_RANK, i)).astype(np.float32)
        b = (rng.standard_normal((o, C4_RANK)) * 1e-3).astype(np.float32)
        x = orc.round_through(rng.standard_normal((m, i)).astype(np.float32), orc.BF16)
        dy = orc.round_through(rng.standard_normal((m, o)).astype(np.float32), orc.BF16)
        layer.append((wd, a, b, x, dy))

    def step():
        for wd, a, b, x, dy in layer:
            base = orc.gemm_nt(x, wd, exact=False)
            _, hidden = orc.lora_forward(x, base, a, b, C4_ALPHA, orc.BF16, exact=False)
            dx_base = orc.gemm_nn(dy, wd, exact=False)
            orc.lora_backward(dy, x, hidden, dx_base, a, b, C4_ALPHA, orc.BF16, exact=False)

    dt, done = _cpu_loop(step, steps, warmup, budget_s)
    # one sample step = 1 of 32 layers at m tokens: tokens per second of the full 32-layer linear path
    value = m * done / (dt * C4_LAYERS)
    return {"value": value, "ms_per_step": dt / done * 1e3, "steps": done, "cores": cores,
            "tflops": c4_flops(m, layers=1) * done / dt / 1e12,
            "sample": "%d sample steps, each ONE of the 32 layers at %d of the 16384 tokens: sgemm fwd/dX on cached "
                      "fp32 weights + LoRA for the seven projections; tokens/s scaled to 32 layers" % (done, m)}


CPU_ARM = {"c2": cpu_reference_c2, "c3": cpu_reference_c3, "c5": cpu_reference_c5, "c4lin": cpu_reference_c4lin}


def _cpu_baseline(workload, unit, budget_s=15.0):
    cb = CPU_ARM[workload](steps=50, warmup=1, budget_s=budget_s)
    return {"value": cb["value"], "unit": unit, "cores": cb["cores"], "kind": cb.get("kind", "port"),
            "sample": cb["sample"]}


# ----------------------------------------------------------------------- GPU arm
class Ctx:
    """What every workload needs: the binding, torch, the process group and the peaks."""

    def __init__(self, args, nv, torch, dist, dev, world, rank, peaks):
        self.args, self.nv, self.torch, self.dist = args, nv, torch, dist
        self.dev, self.world, self.rank, self.peaks = dev, world, rank, peaks
        self.traffic = _recorded_traffic()


def _timed(ctx, fn, steps):
    """Barrier + synchronize on both sides, CUDA events on the current stream, max over ranks."""
    torch, dist = ctx.torch, ctx.dist
    if ctx.world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    if ctx.world > 1:
        t = torch.tensor([ms], device=ctx.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def _gpu_uuid(torch, dev):
    try:
        return "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        return str(dev.index or 0)


def _keep_busy(torch, step, ms_per_step, target_ms=1200.0):
    """The timed region can be shorter than the sampler's 200 ms period: run the same step,
    untimed, straight after it so that the clock samples are taken under the same load.
    The step count depends only on the max-over-ranks time, so every rank runs the same number."""
    extra = int(min(max(target_ms / max(ms_per_step, 1e-3), 1), 50000))
    for _ in range(extra):
        step()
    torch.cuda.synchronize()


def _measure(ctx, step, steps, sample_clocks=True):
    """Times `steps` steps; on rank 0 the clocks are sampled during the timed region and a tail of the
    same load.  Returns (ms_total, clocks)."""
    sampler = ClockSampler(_gpu_uuid(ctx.torch, ctx.dev))
    if ctx.rank == 0 and sample_clocks:
        sampler.start()
        time.sleep(0.3)
    ms = _timed(ctx, step, steps)
    if sample_clocks:
        _keep_busy(ctx.torch, step, ms / steps)
    clocks = sampler.stop() if (ctx.rank == 0 and sample_clocks) else None
    return ms, clocks


def bench_c2(ctx):
    nv, torch, dist, dev, world, rank, args = ctx.nv, ctx.torch, ctx.dist, ctx.dev, ctx.world, ctx.rank, ctx.args
    # N > 1: a layer N times as wide, column-parallel: every rank holds a [14336, 4096] shard (its rows of
    # the 1-GPU quantization of the wide weight), so per-GPU work is the config's and the job grows with N.
    shard = C2_OUT
    gen = torch.Generator(device=dev).manual_seed(1235)
    weights = []
    wide0 = None     # rank 0, N > 1: copy 0 of the whole wide layer, for the parity check against one GPU
    wide_parts = []
    for c in range(C2_COPIES):
        for r in range(world):
            # every rank makes the same draws and keeps its own rows; int4 groups never straddle rows
            # here (4096 % 128 == 0), so quantizing a row block alone gives the wide weight's codes
            wf = torch.randn(C2_OUT * C2_IN, generator=gen, device=dev) * 0.02
            if r == rank or (world > 1 and c == 0 and rank == 0):
                packed, scales = nv.quantize_int4(wf, C2_GROUP)
                if r == rank:
                    weights.append(nv.Weight(packed, nv.I4, C2_IN, C2_OUT, scales, group_size=C2_GROUP))
                if world > 1 and c == 0 and rank == 0:
                    wide_parts.append((packed, scales))
            del wf
    if wide_parts:
        wide0 = nv.Weight(torch.cat([p for p, _ in wide_parts]), nv.I4, C2_IN, world * C2_OUT,
                          torch.cat([s for _, s in wide_parts]), group_size=C2_GROUP)
    torch.cuda.empty_cache()
    xs = {m: torch.randn(m, C2_IN, generator=gen, device=dev).to(torch.bfloat16) for m in C2_MS}
    rows_all = sum(C2_MS)
    # one output block per weight copy: the rows of M = 1, 4, 16 back to back
    yblk = [torch.empty(rows_all, shard, dtype=torch.float32, device=dev) for _ in range(C2_COPIES)]
    ys = []
    for c in range(C2_COPIES):
        views, r0 = {}, 0
        for m in C2_MS:
            views[m] = yblk[c][r0:r0 + m]
            r0 += m
        ys.append(views)
    # N > 1: every rank owns a [copies, 21, N * 14336] result block mapped into all ranks; the kernel
    # stores its slice into every rank's block (the all-gather is the kernel's own stores over NVLink)
    peer = None
    gathered = None
    if world > 1:
        from caif_b200.sharded import PeerBuffer
        ok = torch.ones(1, device=dev)
        try:
            peer = PeerBuffer(C2_COPIES * rows_all * world * shard * 4, dev)
        except Exception as e:   # no peer mapping on this box: gather with NCCL instead
            sys.stderr.write("rank %d: peer buffers unavailable (%s); gathering Y with NCCL\n" % (rank, e))
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0.0:
            peer = None
            gathered = [torch.empty(world * rows_all, shard, dtype=torch.float32, device=dev)
                        for _ in range(C2_COPIES)]
    comm = torch.cuda.Stream() if gathered is not None else None
    signal = torch.zeros(1, device=dev) if world > 1 else None
    row0 = {}
    r0 = 0
    for m in C2_MS:
        row0[m] = r0
        r0 += m

    def one_pass():
        # M-major: consecutive launches use different weight copies, a copy comes back 8 launches
        # (242 MB) later, so no launch finds its codes in L2
        for m in C2_MS:
            for c, w in enumerate(weights):
                if peer is not None:
                    off = (c * rows_all + row0[m]) * world * shard * 4
                    nv.linear_fwd_gather(w, xs[m], [q + off for q in peer.ptrs], world * shard, rank * shard,
                                         nv.F32, nv.F32)
                else:
                    nv.linear_fwd(w, xs[m], compute=nv.F32, out=ys[c][m])

    def step_eager():
        for _ in range(C2_LAYERS):
            one_pass()
        if gathered is not None:
            main = torch.cuda.current_stream()
            comm.wait_stream(main)
            with torch.cuda.stream(comm):
                for c in range(C2_COPIES):
                    dist.all_gather_into_tensor(gathered[c], yblk[c])
            main.wait_stream(comm)
        elif peer is not None:
            # completion signal: this collective ends on a rank only after every rank's kernels of the step,
            # and with them their stores into this rank's buffer, are complete; it also keeps a fast rank's
            # next step from overwriting a buffer a slower rank's consumers would still be reading
            dist.all_reduce(signal)

    launches_per_step = C2_LAYERS * C2_COPIES * len(C2_MS)
    one_pass()
    torch.cuda.synchronize()
    assert nv.last_path() == "decode", nv.last_path()

    # N > 1: the gathered result must equal what ONE GPU computes for the whole wide layer
    parity = None
    if world > 1:
        if peer is not None:
            dist.all_reduce(signal)
            torch.cuda.synchronize()
            got = peer.read(torch.float32, (C2_COPIES, rows_all, world * shard))[0]
        else:
            step_gather = [torch.empty(world * rows_all, shard, dtype=torch.float32, device=dev)]
            dist.all_gather_into_tensor(step_gather[0], yblk[0])
            got = step_gather[0].view(world, rows_all, shard).permute(1, 0, 2).reshape(rows_all, world * shard)
        err = torch.zeros(1, device=dev)
        if rank == 0:
            worst = 0.0
            for m in C2_MS:
                want = nv.linear_fwd(wide0, xs[m], compute=nv.F32)
                have = got[row0[m]:row0[m] + m]
                worst = max(worst, float((have - want).abs().max() / want.abs().max()))
            err.fill_(worst)
        dist.broadcast(err, 0)
        parity = {"checked": "gathered Y of weight copy 0 at M=1,4,16 against one GPU running the whole wide layer",
                  "max_rel_err": float(err.item()), "parity_ok": bool(float(err.item()) == 0.0)}
        del wide0
    for _ in range(max(args.warmup, 3) - 1):
        step_eager()
    torch.cuda.synchronize()

    step = step_eager
    graphed = False
    if not args.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_eager()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_eager()
            step = graph.replay
            graphed = True
            for _ in range(3):
                step()
            torch.cuda.synchronize()
        except Exception as e:  # capture of the collective can be refused; time eagerly then
            if rank == 0:
                sys.stderr.write("graph capture unavailable (%s); timing eager launches\n" % e)
            step = step_eager
            torch.cuda.synchronize()

    ms, clocks = _measure(ctx, step, args.steps)
    bytes_per_step = world * C2_LAYERS * C2_COPIES * sum(c2_bytes(m) for m in C2_MS)   # whole job (all shards)
    ms_per_step = ms / args.steps
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # dominant kernel: per-launch algorithmic bytes / average launch duration over the timed region
    per_launch_bytes = sum(c2_bytes(m, shard) for m in C2_MS) / len(C2_MS)
    per_launch_s = ms_per_step * 1e-3 / launches_per_step
    achieved = per_launch_bytes / per_launch_s / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": ctx.peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / ctx.peaks["hbm_gbs"],
                "traffic": ctx.traffic.get("linear_decode_kernel_c2") if world == 1 else None,
                "peak_source": ctx.peaks["source"], "kernel": "linear_decode_kernel<4,*,2>",
                "note": "algorithmic bytes per launch (mean of M=1,4,16) over the average launch duration in the "
                        "timed region (CUDA events around the step / 768 launches; includes inter-launch gaps)"}

    # end to end: host buffers in, host buffers out, through the C ABI, copies inside the timed region
    # One pinned block of inputs and one of results per pass (the 24 launches of one layer: M = 1, 4, 16 on the 8
    # weight copies, every launch with its own input rows): one copy in before the pass and one copy out after
    # it, on two side streams beside the kernels, so that the launches of a pass follow one another without a
    # copy between them.  Two sets of device blocks alternate between passes: the copy-in of a pass runs while
    # the pass before it computes, its copy-out while the next one does; a set is reused two passes later,
    # ordered by one event per pass and direction.
    hx = torch.cat([xs[m].cpu() for m in C2_MS for _ in range(C2_COPIES)]).pin_memory()
    hy = torch.empty(C2_COPIES * rows_all, shard, dtype=torch.float32).pin_memory()
    dx = [torch.empty(C2_COPIES * rows_all, C2_IN, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    dy_out = [torch.empty(C2_COPIES * rows_all, shard, dtype=torch.float32, device=dev) for _ in range(2)]
    slot = {}
    r0 = 0
    for m in C2_MS:
        for c in range(C2_COPIES):
            slot[(m, c)] = (r0, r0 + m)
            r0 += m
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_h2d = [torch.cuda.Event() for _ in range(2)]            # the inputs of the pass on set b have arrived
    ev_pass_kernels = [torch.cuda.Event() for _ in range(2)]   # the kernels of the last pass on set b are done
    ev_pass_d2h = [torch.cuda.Event() for _ in range(2)]       # ... and so is its copy to the host

    def e2e_pass(p):
        main = torch.cuda.current_stream()
        b = p & 1
        if p >= 2:
            s_in.wait_event(ev_pass_kernels[b])    # inputs of set b are free again
            main.wait_event(ev_pass_d2h[b])        # results of set b have left for the host
        with torch.cuda.stream(s_in):
            dx[b].copy_(hx, non_blocking=True)
            ev_h2d[b].record(s_in)
        main.wait_event(ev_h2d[b])
        for m in C2_MS:
            for c, w in enumerate(weights):
                lo, hi = slot[(m, c)]
                nv.linear_fwd(w, dx[b][lo:hi], compute=nv.F32, out=dy_out[b][lo:hi])
        ev_pass_kernels[b].record(main)
        s_out.wait_event(ev_pass_kernels[b])
        with torch.cuda.stream(s_out):
            hy.copy_(dy_out[b], non_blocking=True)
            ev_pass_d2h[b].record(s_out)

    def e2e_body():
        main = torch.cuda.current_stream()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for p in range(C2_LAYERS):
            e2e_pass(p)
        main.wait_stream(s_in)
        main.wait_stream(s_out)

    e2e_graph = None
    if graphed:
        # the same calls, copies included, recorded once and replayed: what a serving loop does
        try:
            warm = torch.cuda.Stream()
            warm.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(warm):
                e2e_body()
            torch.cuda.current_stream().wait_stream(warm)
            torch.cuda.synchronize()
            e2e_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(e2e_graph):
                e2e_body()
        except Exception as e:
            if rank == 0:
                sys.stderr.write("graph capture of the end-to-end step unavailable (%s)\n" % e)
            e2e_graph = None
            torch.cuda.synchronize()

    def step_e2e():
        if e2e_graph is not None:
            e2e_graph.replay()
        else:
            e2e_body()
        torch.cuda.synchronize()

    for _ in range(2):
        step_e2e()
    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = _timed(ctx, step_e2e, e2e_steps)
    e2e = {"value": bytes_per_step / (ms_e2e / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": C2_LAYERS * C2_COPIES * sum(m * C2_IN * 2 for m in C2_MS),
           "d2h_bytes_per_step": C2_LAYERS * C2_COPIES * sum(m * shard * 4 for m in C2_MS)}
    if world > 1:
        e2e["note"] = "times the local slice only (no gather)"

    result = {
        "metric": METRIC["c2"][0], "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": SCALING["c2"],
        "vs_baseline": None, "dtype": "bf16 x int4 -> fp32", "data": "synthetic", "config": config_for("c2", world),
        "run": {"launch": "CUDA graph replay" if graphed else "eager",
                "gather": None if world == 1 else ("peer stores" if peer is not None else "NCCL all-gather")},
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
    }
    if parity is not None:
        result["parity"] = parity
    if peer is not None:
        peer.close()
    if world == 1:
        # beside the single-call figure, never instead of it: layers that share their input in one launch
        result["multi_weight"] = _c2_multi_weight(ctx, weights, xs)
        try:
            result["multi_stream"] = _c2_multi_stream(ctx, weights, xs)
        except Exception as e:   # informative only: never takes the headline down
            result["multi_stream"] = {"error": "%s: %s" % (type(e).__name__, e)}
    return result


def _c2_multi_stream(ctx, weights, xs, streams=3):
    """The step's own launches (same calls, same weights and outputs of their own), issued round robin on three
    streams inside one CUDA graph: what a host gets that keeps the independent projections of a block (q / k / v,
    gate / up) or of several requests in flight together.  The tail of one launch then overlaps the ramp of the
    next.  Reported beside the headline, which stays the one-launch-after-the-other figure."""
    nv, torch, dev = ctx.nv, ctx.torch, ctx.dev
    outs = {(m, c): torch.empty(m, C2_OUT, dtype=torch.float32, device=dev) for m in C2_MS for c in range(C2_COPIES)}
    lanes = [torch.cuda.Stream() for _ in range(streams)]
    passes = 16

    def body():
        main = torch.cuda.current_stream()
        for s in lanes:
            s.wait_stream(main)
        k = 0
        for _ in range(passes):
            for m in C2_MS:
                for c, w in enumerate(weights):
                    with torch.cuda.stream(lanes[k % streams]):
                        nv.linear_fwd(w, xs[m], compute=nv.F32, out=outs[(m, c)])
                    k += 1
        for s in lanes:
            main.wait_stream(s)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        body()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        body()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    launches = reps * passes * len(C2_MS) * len(weights)
    us = a.elapsed_time(b) * 1e3 / launches
    algo = sum(c2_bytes(m) for m in C2_MS) / len(C2_MS)
    gbs = algo / us / 1e3
    return {"workload": "the c2 launches issued round robin on %d streams in one CUDA graph" % streams,
            "value": gbs, "unit": "GB/s", "us_per_launch_of_throughput": us, "launches_timed": launches,
            "frac_of_hbm_peak": gbs / ctx.peaks["hbm_gbs"]}


def _c2_multi_weight(ctx, weights, xs):
    """Two [14336, 4096] int4 layers that share x (gate and up of the Llama-shaped FFN) per launch of
    caifq_linear_fwd_multi, four pairs of weight copies (235 MB > L2) in turn, M in {1, 4, 16}."""
    nv, torch, dev = ctx.nv, ctx.torch, ctx.dev
    pairs = [weights[2 * i:2 * i + 2] for i in range(C2_COPIES // 2)]
    outs = {m: [torch.empty(m, 2 * C2_OUT, dtype=torch.float32, device=dev) for _ in pairs] for m in C2_MS}

    def one_pass():
        for m in C2_MS:
            for i, pair in enumerate(pairs):
                nv.linear_fwd_multi(pair, xs[m], torch.float32, nv.F32, out=outs[m][i])

    passes = 16
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        one_pass()
        one_pass()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(passes):
                one_pass()
    torch.cuda.synchronize()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    launches = reps * passes * len(C2_MS) * len(pairs)
    us = a.elapsed_time(b) * 1e3 / launches
    algo = sum(c2_bytes(m, 2 * C2_OUT) for m in C2_MS) / len(C2_MS)
    gbs = algo / us / 1e3
    return {"workload": "gate+up: two [14336, 4096] int4 g128 layers sharing x per launch, M in {1,4,16}",
            "value": gbs, "unit": "GB/s", "us_per_launch": us, "launches_timed": launches,
            "frac_of_hbm_peak": gbs / ctx.peaks["hbm_gbs"]}


def bench_c3(ctx):
    nv, torch, dev, args = ctx.nv, ctx.torch, ctx.dev, ctx.args
    dim, rank_r, m, alpha = 4096, 16, 8192, 32.0
    gen = torch.Generator(device=dev).manual_seed(1236)
    wf = torch.randn(dim * dim, generator=gen, device=dev) * 0.02
    q, s = nv.quantize_int8_per_tensor(wf)
    weight = nv.Weight(q.view(dim, dim), nv.I8, dim, dim, s)
    del wf
    a = ((torch.rand(rank_r, dim, generator=gen, device=dev) * 2 - 1) / 64).to(torch.bfloat16)
    b = (torch.randn(dim, rank_r, generator=gen, device=dev) * 1e-3).to(torch.bfloat16)
    lora = nv.Lora(a, b, alpha)
    n_sets = 2  # 2 x (X + dY) = 268 MB of activations > L2, alternated between steps
    xs = [torch.randn(m, dim, generator=gen, device=dev).to(torch.bfloat16) for _ in range(n_sets)]
    dys = [torch.randn(m, dim, generator=gen, device=dev).to(torch.bfloat16) for _ in range(n_sets)]
    state = {"i": 0}

    def step():
        i = state["i"] % n_sets
        state["i"] += 1
        # (the entry points that may expand the weight once per call into their workspace)
        _, hidden = nv.lora_linear_fwd(weight, lora, xs[i], compute=nv.F32, expanded=True)
        dx, _, _ = nv.lora_linear_bwd(weight, lora, dys[i], xs[i], hidden, compute=nv.F32, expanded=True)
        return dx

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    path = nv.last_path()
    steps = max(3, args.steps)
    ms, clocks = _measure(ctx, step, steps)
    ms_per_step = ms / steps
    flops = c3_flops(m)
    value = flops / (ms_per_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": value, "peak": ctx.peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": value / ctx.peaks["bf16_tflops"], "frac_of_sustained": value / ctx.peaks["bf16_tflops_sustained"],
                "traffic": ctx.traffic.get("linear_umma_kernel_c3_fwd"), "peak_source": ctx.peaks["source"],
                "kernel": "frozen linear path '%s'" % path,
                "note": "whole step (fwd + dX + LoRA) over its duration; peak is the burst cuBLAS bf16 figure"}

    hx = xs[0].cpu().pin_memory()
    hdy = dys[0].cpu().pin_memory()
    hdx = torch.empty(m, dim, dtype=torch.bfloat16).pin_memory()
    dxb, dyb = torch.empty_like(xs[0]), torch.empty_like(dys[0])

    def step_e2e():
        dxb.copy_(hx, non_blocking=True)
        dyb.copy_(hdy, non_blocking=True)
        xs[0], dys[0] = dxb, dyb
        state["i"] = 0
        out = step()
        hdx.copy_(out, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(2):
        step_e2e()
    e2e_steps = max(3, min(steps, 10))
    ms_e2e = _timed(ctx, step_e2e, e2e_steps)
    e2e = {"value": flops / (ms_e2e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": 2 * m * dim * 2, "d2h_bytes_per_step": m * dim * 2}
    return {
        "metric": METRIC["c3"][0], "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": SCALING["c3"],
        "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)", "data": "synthetic", "config": config_for("c3", 1),
        "roofline": roofline, "e2e": e2e, "gpu_launches": 10 * steps, "clocks": clocks,   # forward 3, backward 7 kernels
    }


class _NativeMoeOps:
    """The operations ExpertParallelFrozenMoE needs, over the C ABI, for one rank's experts."""

    def __init__(self, nv, torch, gate, up, down, num_experts, compute):
        self.nv, self.torch = nv, torch
        self.gate, self.up, self.down = gate, up, down
        self.num_experts = num_experts
        self.compute = compute
        self.saved = None
        # scratch for the bf16 copies of this rank's experts, filled once per step (in the forward pass, inside
        # the timed step) and read by the grouped launches of forward and backward
        nbytes = nv.grouped_expert_expanded_bytes(gate, up, down, nv.BF16, compute)
        self.expanded = torch.empty(nbytes, dtype=torch.uint8, device=up[0].codes.device) if nbytes > 0 else None

    def build_dispatch(self, idx):
        return self.nv.moe_build_dispatch(idx, self.num_experts, 0)

    def dispatch(self, x, idx, dmap, offsets, total):
        return self.nv.moe_dispatch(x, idx, dmap, offsets, total)

    def experts(self, packed, local_offsets):
        offs = [int(v) for v in local_offsets]
        if self.expanded is not None:
            self.nv.grouped_expert_expand(self.gate, self.up, self.down, self.expanded, self.nv.BF16, self.compute)
        out, g_out, u_out = self.nv.grouped_expert_fwd(self.gate, self.up, self.down, offs, packed,
                                                       compute=self.compute, expanded=self.expanded)
        self.saved = (offs, g_out, u_out)
        return out

    def experts_bwd(self, packed_dy, local_offsets):
        offs, g_out, u_out = self.saved
        return self.nv.grouped_expert_bwd(self.gate, self.up, self.down, offs, packed_dy, g_out, u_out,
                                          compute=self.compute, expanded=self.expanded)

    def combine(self, buf, idx, wts, dmap, offsets, tokens):
        return self.nv.moe_combine(buf, idx, wts, dmap, offsets, tokens)

    def combine_bwd(self, dy, idx, wts, dmap, offsets, total):
        return self.nv.moe_combine_bwd_grad_expert(dy, idx, wts, dmap, offsets, total)

    def dispatch_bwd(self, gbuf, idx, dmap, offsets, tokens):
        return self.nv.moe_dispatch_bwd(gbuf, idx, dmap, offsets, tokens)


def bench_c5(ctx):
    """Frozen int4 experts of the MoE config.  One GPU: the layer's frozen-expert dataflow forward and
    backward.  N GPUs: the same with experts and tokens sharded and the rows exchanged by all-to-all."""
    nv, torch, dist, dev, world, rank, args = ctx.nv, ctx.torch, ctx.dist, ctx.dev, ctx.world, ctx.rank, ctx.args
    hidden, ffn, n_exp, tokens, top_k = C5_HIDDEN, C5_FFN, C5_EXPERTS, C5_TOKENS, C5_TOPK
    local = n_exp // world
    gen = torch.Generator(device=dev).manual_seed(1238)
    gate, up, down = [], [], []
    for e in range(n_exp):
        for lst, (o, i) in ((gate, (ffn, hidden)), (up, (ffn, hidden)), (down, (hidden, ffn))):
            wf = torch.randn(o * i, generator=gen, device=dev) * 0.02   # same draws on every rank
            if e // local == rank:
                pk, sc = nv.quantize_int4(wf, 128)
                lst.append(nv.Weight(pk, nv.I4, i, o, sc, group_size=128))
            del wf
    logits = torch.randn(tokens, n_exp, generator=gen, device=dev)
    x_all = torch.randn(tokens, hidden, generator=gen, device=dev).to(torch.bfloat16)
    dy_all = torch.randn(tokens, hidden, generator=gen, device=dev).to(torch.bfloat16)
    probs = nv.moe_softmax(logits)
    idx_all, wts_all = nv.moe_topk(probs, top_k)
    wts_all = nv.moe_normalize_rows(wts_all).to(torch.bfloat16)
    # this rank's tokens
    t_local = tokens // world
    sl = slice(rank * t_local, (rank + 1) * t_local)
    x, dy = x_all[sl].contiguous(), dy_all[sl].contiguous()
    idx, wts = idx_all[sl].contiguous(), wts_all[sl].contiguous()
    del x_all, dy_all, logits, probs
    ops = _NativeMoeOps(nv, torch, gate, up, down, n_exp, nv.BF16)
    total_rows = tokens * top_k
    launches = 0

    if world == 1:
        dmap, offs = ops.build_dispatch(idx)
        offs_host = [int(v) for v in offs.cpu().tolist()]

        def step():
            buf = ops.dispatch(x, idx, dmap, offs, total_rows)
            out = ops.experts(buf, offs_host)
            y = ops.combine(out, idx, wts, dmap, offs, tokens)
            gbuf = ops.combine_bwd(dy, idx, wts, dmap, offs, total_rows)
            gx = ops.experts_bwd(gbuf, offs_host)
            dx = ops.dispatch_bwd(gx, idx, dmap, offs, tokens)
            return y, dx
        parity = None
    else:
        from caif_b200.sharded import ExpertParallelFrozenMoE
        moe = ExpertParallelFrozenMoE(ops, n_exp)
        routing = moe.route(idx)     # the routing is held fixed across iterations

        def step():
            y = moe.forward(x, idx, wts, routing)
            dx = moe.backward(dy)
            return y, dx
        # the exchange is checked by a round trip: every packed row goes to its expert's owner and comes
        # back unchanged (the experts themselves are the one-GPU kernels on the rows that arrive)
        probe = moe.round_trip_check(x, idx, routing)
        err = torch.tensor([probe], device=dev)
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        parity = {"checked": "every packed row sent to its expert's owner and returned by the two all-to-alls "
                             "arrives back bit-identical (max abs difference over all ranks)",
                  "max_abs_err": float(err.item()), "parity_ok": bool(float(err.item()) == 0.0)}

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    path = nv.last_path()
    steps = max(3, args.steps)
    ms, clocks = _measure(ctx, step, steps)
    ms_per_step = ms / steps
    flops = c5_flops(total_rows)
    value = flops / (ms_per_step * 1e-3) / 1e12

    hx = x.cpu().pin_memory()
    hdy = dy.cpu().pin_memory()
    hy = torch.empty(t_local, hidden, dtype=torch.bfloat16).pin_memory()
    hdx = torch.empty(t_local, hidden, dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        x.copy_(hx, non_blocking=True)
        dy.copy_(hdy, non_blocking=True)
        y, dx = step()
        hy.copy_(y, non_blocking=True)
        hdx.copy_(dx, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(2):
        step_e2e()
    e2e_steps = max(3, min(steps, 10))
    ms_e2e = _timed(ctx, step_e2e, e2e_steps)
    e2e = {"value": flops / (ms_e2e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": world * 2 * t_local * hidden * 2, "d2h_bytes_per_step": world * 2 * t_local * hidden * 2}
    result = {
        "metric": METRIC["c5"][0], "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": SCALING["c5"],
        "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)", "data": "synthetic", "config": config_for("c5", world),
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": ctx.peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": value / world / ctx.peaks["bf16_tflops"],
                     "frac_of_sustained": value / world / ctx.peaks["bf16_tflops_sustained"],
                     "traffic": ctx.traffic.get("linear_umma_kernel_c5_grouped") if world == 1 else None,
                     "peak_source": ctx.peaks["source"], "kernel": "frozen experts path '%s'" % path,
                     "note": "expert GEMM flops over the whole step (dispatch, SwiGLU, combine and their backward "
                             "kernels%s included in the time)" % (", both all-to-alls" if world > 1 else "")},
        "e2e": e2e, "gpu_launches": (11 if ops.expanded is not None else 9) * steps, "clocks": clocks,
    }
    if parity is not None:
        result["parity"] = parity
    return result


def bench_c4lin(ctx):
    nv, torch, dist, dev, world, rank, args = ctx.nv, ctx.torch, ctx.dist, ctx.dev, ctx.world, ctx.rank, ctx.args
    tokens, layers, r_lora = C4_TOKENS, C4_LAYERS, C4_RANK
    gen = torch.Generator(device=dev).manual_seed(1239 + 7919 * rank)   # each rank draws its own shards
    shared = torch.Generator(device=dev).manual_seed(1240)             # replicated tensors: same on every rank
    model = []
    for _ in range(layers):
        layer = []
        for name, o, i in C4_PROJ:
            o_loc = o // world
            wf = torch.randn(o_loc * i, generator=gen, device=dev) * 0.02
            pk, sc = nv.quantize_int4(wf, 128)
            del wf
            a = ((torch.rand(r_lora, i, generator=shared, device=dev) * 2 - 1) / 64).to(torch.bfloat16)
            b = (torch.randn(o_loc, r_lora, generator=gen, device=dev) * 1e-3).to(torch.bfloat16)
            layer.append((nv.Weight(pk, nv.I4, i, o_loc, sc, group_size=128), nv.Lora(a, b, C4_ALPHA)))
        model.append(layer)
    torch.cuda.empty_cache()
    # activations: one input per distinct in-dim, one dY per distinct local out-dim
    x_by_in = {i: torch.randn(tokens, i, generator=shared, device=dev).to(torch.bfloat16) for i in (4096, 14336)}
    dy_by_out = {o // world: torch.randn(tokens, o // world, generator=shared, device=dev).to(torch.bfloat16)
                 for o in (4096, 1024, 14336)}
    y_by_out = {o // world: torch.empty(tokens, o // world, dtype=torch.bfloat16, device=dev) for o in (4096, 1024, 14336)}
    dx_by_in = {i: torch.empty(tokens, i, dtype=torch.bfloat16, device=dev) for i in (4096, 14336)}
    hid = [[torch.empty(tokens, r_lora, dtype=torch.bfloat16, device=dev) for _ in C4_PROJ] for _ in range(2)]
    d_a = {i: torch.empty(r_lora, i, dtype=torch.bfloat16, device=dev) for i in (4096, 14336)}
    d_b = {o // world: torch.empty(o // world, r_lora, dtype=torch.bfloat16, device=dev) for o in (4096, 1024, 14336)}
    ws_bytes = 0
    for w, l in model[0]:
        ws_bytes = max(ws_bytes, nv.lora_fwd_workspace_bytes(w, l, tokens, nv.BF16, expanded=True),
                       nv.lora_bwd_workspace_bytes(w, l, tokens, nv.BF16, expanded=True))
    workspace = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=dev)
    comm = torch.cuda.Stream() if world > 1 else None
    group = None
    if world > 1:
        # The collectives run beside the persistent tensor-core kernels: they get SMs of their own.  The
        # kernels' grids are capped (caifq_set_cta_limit) and this workload's communicator is held to
        # as many CTAs as the kernels leave free; other workloads keep the default communicator.
        nccl_ctas = args.c4_nccl_ctas if args.c4_nccl_ctas else (16 if world < 4 else 32)
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        nv.lib().caifq_set_cta_limit(sms - nccl_ctas)
        try:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = nccl_ctas
            group = dist.new_group(ranks=list(range(world)), pg_options=opts)
        except Exception as e:   # older bindings: fall back to the default communicator
            if rank == 0:
                sys.stderr.write("per-group NCCL CTA cap unavailable (%s)\n" % e)
            group = None
        # double-buffered collective operands: the collective of projection p reads what projection p wrote
        # while projection p+1 already writes the other buffer
        y_full = [{o: torch.empty(world * tokens, o // world, dtype=torch.bfloat16, device=dev)
                   for o in (4096, 1024, 14336)} for _ in range(2)]
        y_send = [{o // world: torch.empty(tokens, o // world, dtype=torch.bfloat16, device=dev)
                   for o in (4096, 1024, 14336)} for _ in range(2)]
        dx_send = [{i: torch.empty(tokens, i, dtype=torch.bfloat16, device=dev) for i in (4096, 14336)}
                   for _ in range(2)]
        dx_part = {i: torch.empty(tokens // world, i, dtype=torch.bfloat16, device=dev) for i in (4096, 14336)}
        da_send = [{i: torch.empty(r_lora, i, dtype=torch.bfloat16, device=dev) for i in (4096, 14336)}
                   for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]       # collective that read buffer set b has finished
        coll_bytes = {"all_gather_y": 0, "reduce_scatter_dx": 0, "all_reduce_da": 0}
        for _, o, i in C4_PROJ:
            coll_bytes["all_gather_y"] += layers * tokens * o * 2 * (world - 1) // world
            coll_bytes["reduce_scatter_dx"] += layers * tokens * i * 2 * (world - 1) // world
            coll_bytes["all_reduce_da"] += layers * r_lora * i * 2

    def step():
        main = torch.cuda.current_stream()
        n = 0
        # forward, layer by layer
        for layer in model:
            for p, ((w, l), (_, o, i)) in enumerate(zip(layer, C4_PROJ)):
                if world == 1:
                    nv.lora_linear_fwd(w, l, x_by_in[i], compute=nv.BF16, out=y_by_out[o], hidden=hid[0][p],
                                       workspace=workspace, expanded=True)
                    continue
                b = n & 1
                if n >= 2:
                    main.wait_event(ev_done[b])
                nv.lora_linear_fwd(w, l, x_by_in[i], compute=nv.BF16, out=y_send[b][o // world], hidden=hid[0][p],
                                   workspace=workspace, expanded=True)
                comm.wait_stream(main)
                with torch.cuda.stream(comm):
                    dist.all_gather_into_tensor(y_full[b][o], y_send[b][o // world], group=group)
                    ev_done[b].record(comm)
                n += 1
        # backward, in reverse
        for layer in reversed(model):
            for p in range(len(C4_PROJ) - 1, -1, -1):
                (w, l), (_, o, i) = layer[p], C4_PROJ[p]
                if world == 1:
                    nv.lora_linear_bwd(w, l, dy_by_out[o], x_by_in[i], hid[0][p], compute=nv.BF16, dx=dx_by_in[i],
                                       d_a=d_a[i], d_b=d_b[o], workspace=workspace, expanded=True)
                    continue
                b = n & 1
                main.wait_event(ev_done[b])
                nv.lora_linear_bwd(w, l, dy_by_out[o // world], x_by_in[i], hid[0][p], compute=nv.BF16,
                                   dx=dx_send[b][i], d_a=da_send[b][i], d_b=d_b[o // world], workspace=workspace, expanded=True)
                comm.wait_stream(main)
                with torch.cuda.stream(comm):
                    dist.reduce_scatter_tensor(dx_part[i], dx_send[b][i], group=group)
                    dist.all_reduce(da_send[b][i], group=group)
                    ev_done[b].record(comm)
                n += 1
        if world > 1:
            main.wait_stream(comm)

    # hidden is produced by the forward of the LAST layer visited for each projection slot; the backward of
    # every layer reuses it (same shapes, synthetic values): the traffic and the work are those of the real step
    step()
    torch.cuda.synchronize()
    path = nv.last_path()

    parity = None
    if world > 1:
        # one projection against one GPU: rank 0 gathers the shards of layer 0's q projection and runs the whole
        # layer alone; Y must be bit-identical, dX equal up to the bf16 rounding of the partial sums
        w, l = model[0][0]
        xq = x_by_in[4096][:256].contiguous()
        y_loc, h_loc = nv.lora_linear_fwd(w, l, xq, compute=nv.BF16)
        y_all = torch.empty(world * 256, 4096 // world, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(y_all, y_loc)
        codes = [torch.empty_like(w.codes) for _ in range(world)]
        scales = [torch.empty_like(w.scales) for _ in range(world)]
        bs = [torch.empty_like(l.b) for _ in range(world)]
        dist.all_gather(codes, w.codes)
        dist.all_gather(scales, w.scales)
        dist.all_gather(bs, l.b)
        err = torch.zeros(2, device=dev)
        dy_full = torch.randn(256, 4096, generator=shared, device=dev).to(torch.bfloat16)
        dy_loc = dy_full[:, rank * (4096 // world):(rank + 1) * (4096 // world)].contiguous()
        dx_loc, _, _ = nv.lora_linear_bwd(w, l, dy_loc, xq, h_loc, compute=nv.BF16)
        dx_sum = dx_loc.float()
        dist.all_reduce(dx_sum)
        if rank == 0:
            wide = nv.Weight(torch.cat(codes), nv.I4, 4096, 4096, torch.cat(scales), group_size=128)
            lw = nv.Lora(l.a, torch.cat(bs).contiguous(), C4_ALPHA)
            y_one, h_one = nv.lora_linear_fwd(wide, lw, xq, compute=nv.BF16)
            got = y_all.view(world, 256, 4096 // world).permute(1, 0, 2).reshape(256, 4096)
            err[0] = (got.float() - y_one.float()).abs().max() / y_one.float().abs().max()
            dx_one, _, _ = nv.lora_linear_bwd(wide, lw, dy_full, xq, h_one, compute=nv.BF16)
            err[1] = (dx_sum - dx_one.float()).abs().max() / dx_one.float().abs().max()
        dist.broadcast(err, 0)
        parity = {"checked": "layer 0 q projection, 256 tokens: all-gathered Y and all-reduced dX against one GPU "
                             "running the unsharded projection",
                  "y_max_rel_err": float(err[0].item()), "dx_max_rel_err": float(err[1].item()),
                  "parity_ok": bool(float(err[0].item()) == 0.0 and float(err[1].item()) <= 2e-2)}

    for _ in range(max(min(args.warmup, 3), 1)):
        step()
    torch.cuda.synchronize()
    steps = max(2, args.steps // 5)

    ms, clocks = _measure(ctx, step, steps)
    ms_per_step = ms / steps
    value = tokens / (ms_per_step * 1e-3)
    tflops = c4_flops(tokens) / (ms_per_step * 1e-3) / 1e12

    # end to end: the step's host-visible inputs are the token activations and the gradient; its result dX
    hx = x_by_in[4096].cpu().pin_memory()
    hdy = dy_by_out[4096 // world].cpu().pin_memory()
    hdx = torch.empty(tokens, 4096, dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        x_by_in[4096].copy_(hx, non_blocking=True)
        dy_by_out[4096 // world].copy_(hdy, non_blocking=True)
        step()
        hdx.copy_(dx_by_in[4096] if world == 1 else dx_send[0][4096], non_blocking=True)
        torch.cuda.synchronize()

    step_e2e()
    e2e_steps = 2
    ms_e2e = _timed(ctx, step_e2e, e2e_steps)
    e2e = {"value": tokens / (ms_e2e / e2e_steps * 1e-3), "unit": "tokens/s",
           "h2d_bytes_per_step": tokens * 4096 * 2 + tokens * (4096 // world) * 2, "d2h_bytes_per_step": tokens * 4096 * 2}
    result = {
        "metric": METRIC["c4lin"][0], "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": max(min(args.warmup, 3), 1) + 1, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": SCALING["c4lin"], "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)", "data": "synthetic",
        "config": config_for("c4lin", world), "tflops": tflops,
        "roofline": {"bound": "tensor", "achieved": tflops / world, "peak": ctx.peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": tflops / world / ctx.peaks["bf16_tflops"],
                     "frac_of_sustained": tflops / world / ctx.peaks["bf16_tflops_sustained"],
                     "traffic": None, "peak_source": ctx.peaks["source"], "kernel": "frozen linear path '%s'" % path,
                     "note": "flops of the 224 projections (fwd + dX + LoRA) over the whole step; the step is seconds "
                             "long, so the sustained peak is the fair denominator"},
        "e2e": e2e, "gpu_launches": layers * len(C4_PROJ) * 10 * steps, "clocks": clocks,
    }
    if world > 1:
        total = sum(coll_bytes.values())
        result["collectives"] = {"bytes_per_rank_per_step": coll_bytes,
                                 "limiting": max(coll_bytes, key=coll_bytes.get),
                                 "note": "bytes each rank sends per step; at 770 GB/s per direction they alone take "
                                         "%.0f ms" % (total / 770e9 * 1e3)}
    if parity is not None:
        result["parity"] = parity
    nv.lib().caifq_set_cta_limit(0)
    return result


BENCH = {"c2": bench_c2, "c3": bench_c3, "c5": bench_c5, "c4lin": bench_c4lin}


def run_gpu(args):
    import torch
    import torch.distributed as dist

    from caif_b200 import native as nv

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torchrun with that many ranks" % args.gpus)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    if not nv.lib().caifq_device_ok():
        raise SystemExit("caifq needs an sm_100 device; there is no fallback")

    ctx = Ctx(args, nv, torch, dist, dev, world, rank, _peaks())
    wanted = [w for w in args.workloads.split(",") if w]
    for w in wanted:
        if w not in WORKLOADS:
            raise SystemExit("unknown workload %r" % w)
    if world > 1:
        wanted = [w for w in wanted if w != "c3"]     # the one-GPU training shape; c4lin is its sharded form
    results = {}
    for w in wanted:
        try:
            results[w] = BENCH[w](ctx)
        except Exception as e:   # a secondary workload must not take the headline down
            if w == wanted[0]:
                raise
            results[w] = {"error": "%s: %s" % (type(e).__name__, e)}
            if world > 1:
                raise
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_cpu:
        for w in wanted:
            if "error" not in results[w]:
                results[w]["cpu_baseline"] = _cpu_baseline(w, results[w]["unit"])
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        head = dict(results[wanted[0]])
        head["workloads"] = {w: results[w] for w in wanted}
        print(json.dumps(head))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = args.gpus
    wanted = [w for w in args.workloads.split(",") if w]
    if world > 1:
        wanted = [w for w in wanted if w != "c3"]
    lines = {}
    for i, w in enumerate(wanted):
        # the headline gets the caller's steps and warm-up; the others a bounded 15 s each
        if i == 0:
            cb = CPU_ARM[w](steps=args.steps, warmup=args.warmup, budget_s=120.0)
        else:
            cb = CPU_ARM[w](steps=max(args.steps, 3), warmup=1, budget_s=15.0)
        metric, unit = METRIC[w]
        lines[w] = {
            "impl": "reference", "metric": metric, "value": cb["value"], "unit": unit, "n_gpus": world,
            "steps": cb["steps"], "warmup": args.warmup if i == 0 else 1, "ms_per_step": cb["ms_per_step"],
            "higher_is_better": True, "scaling": SCALING[w], "vs_baseline": None, "dtype": "fp32 (host sgemm)",
            "data": "synthetic", "config": config_for(w, world),
            "cpu_baseline": {"value": cb["value"], "unit": unit, "cores": cb["cores"], "kind": cb.get("kind", "port"),
                             "sample": cb["sample"]},
            "e2e": {"value": cb["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
    head = dict(lines[wanted[0]])
    head["workloads"] = lines
    print(json.dumps(head))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workloads", default=",".join(WORKLOADS),
                    help="comma-separated subset of c2,c3,c5,c4lin; the first one is the headline of the line")
    ap.add_argument("--workload", default=None, help="shorthand for --workloads with one entry")
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA-graph replay")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--c4-nccl-ctas", type=int, default=None,
                    help="c4lin on several GPUs: CTAs left to NCCL (default 16 below 4 GPUs, else 32)")
    ap.add_argument("--c2-layers", type=int, default=None,
                    help="layer passes per c2 step instead of 32 (a short step for profiler captures; the line "
                         "then does not describe the configured workload)")
    args = ap.parse_args()
    if args.workload:
        args.workloads = args.workload
    if args.c2_layers is not None and args.c2_layers >= 1:
        global C2_LAYERS
        C2_LAYERS = args.c2_layers
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
