#!/usr/bin/env python
"""Benchmark of the quantized frozen-linear hot path on B200.

Default workload (`--workload c2`): the decode-shaped int4 frozen linear
in=4096, out=14336, group 128, bf16 activations, M in {1,4,16}, forward only.
One step = one forward at each M over each of 8 independent weight copies
(24 kernel launches); the copies total 242 MB, larger than the 126 MB L2, so
every launch streams its codes from HBM.  Metric: algorithmic bytes per second
(codes + scales + x + y).  Weights are seeded N(0, 0.02) quantized by the
library's own (reference bit-exact) int4 quantizer; activations seeded N(0,1).

`--workload c3`: the training-shaped int8 frozen linear 4096->4096 with a
rank-16 LoRA adapter, M=8192 bf16: forward + dX (+dA, dB); metric TFLOP/s.
`--workload c5`: the frozen int4 experts of the MoE config (dispatch, grouped
forward, combine, grouped dX); metric TFLOP/s.

Contract: `python bench.py --gpus N --steps K --warmup W` prints ONE JSON line
from rank 0.  With N > 1 (under torchrun) the layer is N times as wide and
column-sharded by output features: every rank holds a shard of the config's
shape (weak scaling; `value` is the whole job over all ranks).  The decode
workload gathers Y with the kernel's own stores into every rank's buffer over
NVLink; the training workload all-gathers Y and all-reduces dX with NCCL.  `--impl reference` times the reference's CPU
path (dequantize + OpenBLAS sgemm) on the host cores instead.
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


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def c2_bytes(m, out_dim=C2_OUT):
    """Algorithmic bytes of one decode forward: packed codes + fp16 scales + bf16 x + fp32 y."""
    return out_dim * C2_IN // 2 + (out_dim * C2_IN // C2_GROUP) * 2 + m * C2_IN * 2 + m * out_dim * 4


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
def cpu_reference_c2(steps, warmup, budget_s=20.0):
    """The reference's Host_e path for this layer with its default cache_fp32=true: the int4
    weight is dequantized to fp32 once (restated kernel, OpenMP, outside the timed loop, as the
    reference's cache does after the first call), then every forward is
    CAIF_Ops::MatMulTransposeB = OpenBLAS sgemm (numpy).  One step = one forward at each M in
    {1,4,16} on ONE weight copy."""
    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import caif_oracle as orc

    rng = np.random.default_rng(1235)
    w = (rng.standard_normal((C2_OUT, C2_IN)) * 0.02).astype(np.float32)
    packed, scales = orc.quantize_int4(w, C2_GROUP)
    del w
    xs = [orc.round_through(rng.standard_normal((m, C2_IN)).astype(np.float32), orc.BF16) for m in C2_MS]

    wd = orc.dequantize_int4(packed, scales, C2_OUT * C2_IN, C2_GROUP).reshape(C2_OUT, C2_IN)

    def step():
        for x in xs:
            orc.gemm_nt(x, wd, exact=False)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        step()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    bytes_per_step = sum(c2_bytes(m) for m in C2_MS)
    return {"value": bytes_per_step * done / dt / 1e9, "ms_per_step": dt / done * 1e3, "steps": done,
            "cores": orc.num_threads(),
            "sample": "%d steps of sgemm at M=1,4,16 on one cached fp32 14336x4096 weight (dequantized once)" % done}


def cpu_reference_c3(steps, warmup, budget_s=25.0):
    """Reference Host_e path for the training config on a bounded sample: M=512 of the 8192
    tokens (1/16 of a step): the fp32 weight is dequantized once (the reference's default
    cache_fp32=true), each step is sgemm forward and dX + the six LoRA matmuls."""
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
        out, hidden = orc.lora_forward(x, base, a, b, 32.0, orc.BF16, exact=False)
        dx_base = orc.gemm_nn(dy, wd, exact=False)
        orc.lora_backward(dy, x, hidden, dx_base, a, b, 32.0, orc.BF16, exact=False)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        step()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    flops = c3_flops(m)
    return {"value": flops * done / dt / 1e12, "ms_per_step": dt / done * 1e3, "steps": done,
            "cores": orc.num_threads(),
            "sample": "%d steps at M=%d tokens (1/16 of the 8192-token step): sgemm fwd/dX on the cached fp32 weight + LoRA"
                      % (done, m)}


def cpu_reference_c5(steps, warmup, budget_s=25.0):
    """Reference Host_e path for the frozen experts on a bounded sample: 4 of the 64 experts with 256
    rows each (1024 of the 98,304 packed rows): cached fp32 weights (dequantized once), the expert
    loop of the layer with sgemm for the six products and the elementwise steps in numpy."""
    import numpy as np

    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import caif_oracle as orc

    rng = np.random.default_rng(1238)
    hidden, ffn, n_exp, rows = 2048, 1408, 4, 256
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

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    for _ in range(steps):
        step()
        done += 1
        if time.perf_counter() - t0 > budget_s:
            break
    dt = time.perf_counter() - t0
    flops = c5_flops(n_exp * rows)
    return {"value": flops * done / dt / 1e12, "ms_per_step": dt / done * 1e3, "steps": done,
            "cores": orc.num_threads(),
            "sample": "%d steps over %d experts x %d rows (1/96 of the packed rows): per-expert loop, sgemm on cached "
                      "fp32 weights, forward + dX" % (done, n_exp, rows)}


def c3_flops(m, dim=4096, rank=16):
    return 2 * (2 * m * dim * dim) + 6 * (2 * m * dim * rank)


# ----------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import torch
    import torch.distributed as dist

    from caif_b200 import native as nv

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and args.workload == "c3":
        # the collectives run beside the persistent tensor-core kernels: give them SMs of their own
        # (measured: 132 CTAs + 16 channels best on 2 GPUs, 116 + 32 on 8, where the gather volume is larger)
        os.environ.setdefault("NCCL_MAX_NCHANNELS", "16" if world < 4 else "32")
        os.environ.setdefault("CAIFQ_UMMA_CTAS", "132" if world < 4 else "116")
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

    peaks = _peaks()
    if args.workload == "c2":
        result = bench_c2(args, nv, torch, dist, dev, world, rank, peaks)
    elif args.workload == "c3":
        result = bench_c3(args, nv, torch, dist, dev, world, rank, peaks)
    else:
        result = bench_c5(args, nv, torch, dist, dev, world, rank, peaks)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result))


def _timed(torch, dist, world, fn, steps, dev):
    """Barrier + synchronize on both sides, CUDA events on the current stream, max over ranks."""
    if world > 1:
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
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms


def _gpu_uuid(torch, dev):
    try:
        return "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        return str(dev.index or 0)


def _keep_busy(torch, step, ms_per_step, target_ms=1600.0):
    """The timed region can be shorter than the sampler's 200 ms period: run the same step,
    untimed, straight after it so that the clock samples are taken under the same load.
    The step count depends only on the max-over-ranks time, so every rank runs the same number."""
    extra = int(min(max(target_ms / max(ms_per_step, 1e-3), 1), 50000))
    for _ in range(extra):
        step()
    torch.cuda.synchronize()


def bench_c2(args, nv, torch, dist, dev, world, rank, peaks):
    # N > 1: a layer N times as wide, column-parallel: every rank holds a [14336, 4096] shard (its rows of
    # the 1-GPU quantization of the wide weight), so per-GPU work is the config's and the job grows with N.
    shard = C2_OUT
    gen = torch.Generator(device=dev).manual_seed(1235)
    weights = []
    for c in range(C2_COPIES):
        for r in range(world):
            # every rank makes the same draws and keeps its own rows; int4 groups never straddle rows
            # here (4096 % 128 == 0), so quantizing a row block alone gives the wide weight's codes
            wf = torch.randn(C2_OUT * C2_IN, generator=gen, device=dev) * 0.02
            if r == rank:
                packed, scales = nv.quantize_int4(wf, C2_GROUP)
                weights.append(nv.Weight(packed, nv.I4, C2_IN, C2_OUT, scales, group_size=C2_GROUP))
            del wf
    torch.cuda.empty_cache()
    xs = {m: torch.randn(m, C2_IN, generator=gen, device=dev).to(torch.bfloat16) for m in C2_MS}
    rows_all = sum(C2_MS)
    # one output block per weight copy: the rows of M = 1, 4, 16 back to back, gathered in one collective
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
    row0 = {}
    r0 = 0
    for m in C2_MS:
        row0[m] = r0
        r0 += m

    def step_eager():
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
        if gathered is not None:
            main = torch.cuda.current_stream()
            comm.wait_stream(main)
            with torch.cuda.stream(comm):
                for c in range(C2_COPIES):
                    dist.all_gather_into_tensor(gathered[c], yblk[c])
            main.wait_stream(comm)

    launches_per_step = C2_COPIES * len(C2_MS)
    # warm-up (also sets the kernel's shared-memory attribute outside any capture)
    for _ in range(max(args.warmup, 3)):
        step_eager()
    torch.cuda.synchronize()
    assert nv.last_path() == "decode", nv.last_path()

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

    sampler = ClockSampler(_gpu_uuid(torch, dev))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = _timed(torch, dist, world, step, args.steps, dev)
    _keep_busy(torch, step, ms / args.steps)
    clocks = sampler.stop() if rank == 0 else None

    bytes_per_step = world * C2_COPIES * sum(c2_bytes(m) for m in C2_MS)   # whole job (all shards)
    ms_per_step = ms / args.steps
    value = bytes_per_step / (ms_per_step * 1e-3) / 1e9

    # dominant kernel: per-launch algorithmic bytes / average launch duration over the timed region
    per_launch_bytes = sum(c2_bytes(m, shard) for m in C2_MS) / len(C2_MS)
    per_launch_s = ms_per_step * 1e-3 / launches_per_step
    achieved = per_launch_bytes / per_launch_s / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"], "traffic": NCU_TRAFFIC_C2 if world == 1 else None,
                "peak_source": peaks["source"], "kernel": "linear_decode_kernel<4,*,2>",
                "note": "average over the step's 24 launches (M=1,4,16); includes inter-launch gaps"}

    # end to end: host buffers in, host buffers out, through the C ABI, copies inside the timed region
    e2e = None
    if rank == 0 or world > 1:
        hx = {m: xs[m].cpu().pin_memory() for m in C2_MS}
        hy = {m: torch.empty(m, shard, dtype=torch.float32).pin_memory() for m in C2_MS}
        # one device copy of x per launch, so that the copy-in of a launch can run while the launch before
        # it still reads its own; copies ride two side streams (one per direction) beside the kernels
        dx = {m: [torch.empty_like(xs[m]) for _ in range(C2_COPIES)] for m in C2_MS}
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = {m: [torch.cuda.Event() for _ in range(C2_COPIES)] for m in C2_MS}
        ev_k = {m: [torch.cuda.Event() for _ in range(C2_COPIES)] for m in C2_MS}

        def e2e_body():
            main = torch.cuda.current_stream()
            s_in.wait_stream(main)
            s_out.wait_stream(main)
            for m in C2_MS:
                for c, w in enumerate(weights):
                    with torch.cuda.stream(s_in):
                        dx[m][c].copy_(hx[m], non_blocking=True)
                        ev_in[m][c].record(s_in)
                    main.wait_event(ev_in[m][c])
                    nv.linear_fwd(w, dx[m][c], compute=nv.F32, out=ys[c][m])
                    ev_k[m][c].record(main)
                    s_out.wait_event(ev_k[m][c])
                    with torch.cuda.stream(s_out):
                        hy[m].copy_(ys[c][m], non_blocking=True)
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

        for _ in range(3):
            step_e2e()
        e2e_steps = max(3, min(args.steps, 20))
        ms_e2e = _timed(torch, dist, world, step_e2e, e2e_steps, dev)
        e2e = {"value": bytes_per_step / (ms_e2e / e2e_steps * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": C2_COPIES * sum(m * C2_IN * 2 for m in C2_MS),
               "d2h_bytes_per_step": C2_COPIES * sum(m * shard * 4 for m in C2_MS)}

    result = {
        "metric": "decode int4 frozen-linear forward, algorithmic HBM bytes per second", "value": value,
        "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 x int4 -> fp32", "data": "synthetic",
        "config": {"workload": "c2: in=4096 out=14336 int4 g128, M in {1,4,16}, forward; step = 8 weight copies x 3 M",
                   "l2": "8 weight copies = 242 MB > 126 MB L2; consecutive launches use different copies, a copy returns 8 launches later",
                   "launch": "CUDA graph replay" if graphed else "eager",
                   "parallelism": "1 GPU" if world == 1 else
                   ("column-parallel x%d: a layer of out=%d, one [14336, 4096] shard per GPU; " % (world, world * C2_OUT)) +
                   ("every launch stores its slice of Y into all ranks' result buffers over NVLink (peer memory), "
                    "no separate collective" if peer is not None else "NCCL all-gather of Y at the end of the step") +
                   "; e2e times the local slice only"},
        "roofline": roofline, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
    }
    if peer is not None:
        peer.close()
    if rank == 0 and world == 1 and not args.no_cpu:
        cb = cpu_reference_c2(steps=50, warmup=1, budget_s=15.0)
        result["cpu_baseline"] = {"value": cb["value"], "unit": "GB/s", "cores": cb["cores"], "kind": "port",
                                  "sample": cb["sample"]}
    return result


# ncu dram__bytes_read.sum + dram__bytes_write.sum per launch of the decode kernel (see profiles/); None until captured
NCU_TRAFFIC_C2 = 30.37e6  # bytes per launch, mean of the M=1,4,16 captures in profiles/linear_decode_int4_c2.md
NCU_TRAFFIC_C3 = 116.6e6  # bytes per launch of the forward tensor-core kernel (profiles/linear_umma_int8_c3.md)


def bench_c3(args, nv, torch, dist, dev, world, rank, peaks):
    # N > 1: a projection 4096 -> 4096*N, column-parallel: every rank holds a [4096, 4096] int8 shard and
    # the matching rows of LoRA B; Y is all-gathered, dX and dA are partial sums and all-reduced.
    dim, rank_r, m, alpha = 4096, 16, 8192, 32.0
    gen = torch.Generator(device=dev).manual_seed(1236)
    weight = None
    for r in range(world):
        wf = torch.randn(dim * dim, generator=gen, device=dev) * 0.02
        if r == rank:
            q, s = nv.quantize_int8_per_tensor(wf)   # one scale per shard: what a per-rank layer object holds
            weight = nv.Weight(q.view(dim, dim), nv.I8, dim, dim, s)
        del wf
    a = ((torch.rand(rank_r, dim, generator=gen, device=dev) * 2 - 1) / 64).to(torch.bfloat16)
    b_full = (torch.randn(world * dim, rank_r, generator=gen, device=dev) * 1e-3).to(torch.bfloat16)
    b = b_full[rank * dim:(rank + 1) * dim].contiguous()
    lora = nv.Lora(a, b, alpha)
    n_sets = 2  # 2 x (X + dY) = 268 MB of activations > L2, alternated between steps
    xs = [torch.randn(m, dim, generator=gen, device=dev).to(torch.bfloat16) for _ in range(n_sets)]
    dys = [torch.randn(m, dim, generator=gen, device=dev).to(torch.bfloat16) for _ in range(n_sets)]
    state = {"i": 0}
    gathered = torch.empty(world * m, dim, dtype=torch.bfloat16, device=dev) if world > 1 else None
    comm = torch.cuda.Stream() if world > 1 else None
    overlap = os.environ.get("BENCH_C3_OVERLAP", "1") != "0"

    def step():
        i = state["i"] % n_sets
        state["i"] += 1
        main = torch.cuda.current_stream()
        y, hidden = nv.lora_linear_fwd(weight, lora, xs[i], compute=nv.F32)
        if world > 1 and overlap:
            # the gather of Y runs beside the backward pass
            comm.wait_stream(main)
            with torch.cuda.stream(comm):
                dist.all_gather_into_tensor(gathered, y)
        elif world > 1:
            dist.all_gather_into_tensor(gathered, y)
        dx, d_a, d_b = nv.lora_linear_bwd(weight, lora, dys[i], xs[i], hidden, compute=nv.F32)
        if world > 1 and overlap:
            comm.wait_stream(main)
            with torch.cuda.stream(comm):
                dist.all_reduce(dx)
                dist.all_reduce(d_a)
            main.wait_stream(comm)
            y.record_stream(comm)
        elif world > 1:
            dist.all_reduce(dx)
            dist.all_reduce(d_a)
        return dx

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    path = nv.last_path()
    sampler = ClockSampler(_gpu_uuid(torch, dev))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = _timed(torch, dist, world, step, args.steps, dev)
    _keep_busy(torch, step, ms / args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    flops = c3_flops(m) * world
    value = flops / (ms_per_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "achieved": value / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": value / world / peaks["bf16_tflops"], "traffic": NCU_TRAFFIC_C3,
                "peak_source": peaks["source"], "kernel": "frozen linear path '%s'" % path,
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
    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = _timed(torch, dist, world, step_e2e, e2e_steps, dev)
    e2e = {"value": flops / (ms_e2e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": 2 * m * dim * 2, "d2h_bytes_per_step": m * dim * 2}
    result = {
        "metric": "int8 frozen linear + LoRA r16, forward + dX/dA/dB, TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": "c3: 4096->4096 int8 per-tensor + LoRA r16 a32, M=8192 bf16, fwd + dX/dA/dB",
                   "l2": "two activation sets (268 MB) alternated between steps, larger than L2",
                   "parallelism": "1 GPU" if world == 1 else
                   "column-parallel x%d: a 4096 -> %d projection, one [4096, 4096] shard per GPU; all-gather of Y "
                   "beside the backward pass, all-reduce of dX and dA" % (world, world * dim)},
        "roofline": roofline, "e2e": e2e, "gpu_launches": 11 * args.steps, "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        cb = cpu_reference_c3(steps=20, warmup=1, budget_s=20.0)
        result["cpu_baseline"] = {"value": cb["value"], "unit": "TFLOP/s", "cores": cb["cores"], "kind": "port",
                                  "sample": cb["sample"]}
    return result


def c5_flops(rows, hidden=2048, ffn=1408):
    # three products forward and three for dX, 2 flops per multiply-add
    return 2 * 3 * 2.0 * rows * hidden * ffn


def bench_c5(args, nv, torch, dist, dev, world, rank, peaks):
    """Frozen int4 experts of the MoE config: 64 experts (sharded by expert over the ranks), hidden 2048,
    expert FFN 1408, 16384 tokens routed top-6.  Step = dispatch, grouped forward, combine, grouped dX."""
    hidden, ffn, n_exp, tokens, top_k = 2048, 1408, 64, 16384, 6
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
    probs = torch.softmax(logits, dim=-1)
    idx, wts = nv.moe_topk(probs, top_k)
    wts = nv.moe_normalize_rows(wts).to(torch.bfloat16)
    # this rank keeps the (token, k) picks that land on its experts: the rows an all-to-all would deliver
    mine = (idx // local) == rank
    idx_local = torch.where(mine, idx - rank * local, torch.full_like(idx, local))   # one overflow bin
    dmap, offs = nv.moe_build_dispatch(idx_local.to(torch.int32).contiguous(), local + 1, 0)
    offs_host = offs.cpu().tolist()
    rows = int(offs_host[local])
    offs_local = offs_host[:local + 1]
    x = torch.randn(tokens, hidden, generator=gen, device=dev).to(torch.bfloat16)
    dy = torch.randn(rows, hidden, generator=gen, device=dev).to(torch.bfloat16)
    idx_i32 = idx_local.to(torch.int32).contiguous()
    total_with_bin = int(offs_host[local + 1])

    def step():
        buf = nv.moe_dispatch(x, idx_i32, dmap, offs, total_with_bin)
        out, g_out, u_out = nv.grouped_expert_fwd(gate, up, down, offs_local, buf[:rows], compute=nv.BF16)
        buf[:rows].copy_(out)
        y = nv.moe_combine(buf, idx_i32, wts, dmap, offs, tokens)
        dx = nv.grouped_expert_bwd(gate, up, down, offs_local, dy, g_out, u_out, compute=nv.BF16)
        return y, dx

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    path = nv.last_path()
    sampler = ClockSampler(_gpu_uuid(torch, dev))
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ms = _timed(torch, dist, world, step, args.steps, dev)
    _keep_busy(torch, step, ms / args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    rows_t = torch.tensor([rows], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(rows_t)
    flops = c5_flops(int(rows_t.item()))
    value = flops / (ms_per_step * 1e-3) / 1e12

    hx = x.cpu().pin_memory()
    hdy = dy.cpu().pin_memory()
    hy = torch.empty(tokens, hidden, dtype=torch.bfloat16).pin_memory()

    def step_e2e():
        x.copy_(hx, non_blocking=True)
        dy.copy_(hdy, non_blocking=True)
        y, _ = step()
        hy.copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(2):
        step_e2e()
    e2e_steps = max(3, min(args.steps, 10))
    ms_e2e = _timed(torch, dist, world, step_e2e, e2e_steps, dev)
    e2e = {"value": flops / (ms_e2e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": (tokens + rows) * hidden * 2, "d2h_bytes_per_step": tokens * hidden * 2}
    result = {
        "metric": "frozen int4 experts, grouped forward + dX, TFLOP/s", "value": value, "unit": "TFLOP/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16 (fp32 accumulate)",
        "data": "synthetic",
        "config": {"workload": "c5: 64 frozen int4 experts 2048->1408->2048 (SwiGLU), 16384 tokens top-6, "
                               "dispatch + grouped fwd + combine + grouped dX",
                   "l2": "packed buffers of %d rows (>= 400 MB) stream through L2 every step" % int(rows_t.item()),
                   "parallelism": "1 GPU" if world == 1 else "experts sharded x%d (rows pre-routed per rank)" % world},
        "roofline": {"bound": "tensor", "achieved": value / world, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                     "frac": value / world / peaks["bf16_tflops"], "traffic": None, "peak_source": peaks["source"],
                     "kernel": "frozen experts path '%s'" % path,
                     "note": "whole step incl. dispatch, SwiGLU and combine kernels over its duration"},
        "e2e": e2e, "gpu_launches": 11 * args.steps, "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        cb = cpu_reference_c5(steps=20, warmup=1, budget_s=20.0)
        result["cpu_baseline"] = {"value": cb["value"], "unit": "TFLOP/s", "cores": cb["cores"], "kind": "port",
                                  "sample": cb["sample"]}
    return result


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    if args.workload == "c2":
        cb = cpu_reference_c2(steps=args.steps, warmup=min(args.warmup, 2), budget_s=120.0)
        unit, metric = "GB/s", "decode int4 frozen-linear forward, algorithmic HBM bytes per second"
        workload = "c2: in=4096 out=14336 int4 g128, M in {1,4,16}, forward; step = 8 weight copies x 3 M"
    elif args.workload == "c3":
        cb = cpu_reference_c3(steps=args.steps, warmup=min(args.warmup, 1), budget_s=120.0)
        unit, metric = "TFLOP/s", "int8 frozen linear + LoRA r16, forward + dX/dA/dB, TFLOP/s"
        workload = "c3: 4096->4096 int8 per-tensor + LoRA r16 a32, M=8192 bf16, fwd + dX/dA/dB"
    else:
        cb = cpu_reference_c5(steps=args.steps, warmup=min(args.warmup, 1), budget_s=120.0)
        unit, metric = "TFLOP/s", "frozen int4 experts, grouped forward + dX, TFLOP/s"
        workload = ("c5: 64 frozen int4 experts 2048->1408->2048 (SwiGLU), 16384 tokens top-6, "
                    "dispatch + grouped fwd + combine + grouped dX")
    line = {
        "impl": "reference", "metric": metric, "value": cb["value"], "unit": unit, "n_gpus": args.gpus,
        "steps": cb["steps"], "warmup": min(args.warmup, 2), "ms_per_step": cb["ms_per_step"],
        "higher_is_better": True, "scaling": "strong" if args.workload == "c5" else "weak", "vs_baseline": None,
        "dtype": "fp32 (host sgemm)",
        "data": "synthetic", "config": {"workload": workload},
        "cpu_baseline": {"value": cb["value"], "unit": unit, "cores": cb["cores"], "kind": "port",
                         "sample": cb["sample"]},
        "e2e": {"value": cb["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=["c2", "c3", "c5"])
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA-graph replay")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
