"""World-size-2 gloo tests (CPU) of the multi-GPU bookkeeping: the sharded result equals the
single-process result.  The compute is the numpy oracle here; on a GPU box the same classes
run over the CUDA library."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _init(rank, world, port):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _column_parallel_worker(rank, world, port, out_q):
    _init(rank, world, port)
    import caif_oracle as orc
    from caif_b200.sharded import ColumnParallelFrozenLinear, shard_range

    rng = np.random.default_rng(11)                         # same draws on every rank
    in_dim, out_dim, m = 256, 64, 9
    w = (rng.standard_normal((out_dim, in_dim)) * 0.02).astype(np.float32)
    packed, scales = orc.quantize_int4(w, 128)
    x = rng.standard_normal((m, in_dim)).astype(np.float32)
    dy = rng.standard_normal((m, out_dim)).astype(np.float32)
    full = orc.dequantize_int4(packed, scales, w.size, 128).reshape(out_dim, in_dim)
    b, e = shard_range(out_dim, world, rank)
    # the shard is a contiguous slice of codes and scales, bit-identical to the full tensor's
    gpr = in_dim // 128
    shard = orc.dequantize_int4(packed[b * in_dim // 2:e * in_dim // 2], scales[b * gpr:e * gpr],
                                (e - b) * in_dim, 128).reshape(e - b, in_dim)
    assert np.array_equal(shard, full[b:e])
    layer = ColumnParallelFrozenLinear(lambda t: torch.from_numpy(orc.gemm_nt(t.numpy(), shard)),
                                       lambda g: torch.from_numpy(orc.gemm_nn(g.numpy(), shard)), out_dim, in_dim)
    y = layer.forward(torch.from_numpy(x))
    dx = layer.backward(torch.from_numpy(dy))
    ok_y = np.array_equal(y.numpy(), orc.gemm_nt(x, full))          # same K loop per element: identical
    ok_dx = np.allclose(dx.numpy(), orc.gemm_nn(dy, full), rtol=1e-5, atol=1e-6)
    out_q.put((rank, bool(ok_y), bool(ok_dx)))
    dist.destroy_process_group()


def _expert_parallel_worker(rank, world, port, out_q):
    _init(rank, world, port)
    import caif_oracle as orc
    from caif_b200.sharded import ExpertParallelFrozenMoE

    num_experts, dim, hid, top_k, tokens_per_rank = 8, 16, 24, 3, 20
    rng = np.random.default_rng(21)
    experts = [tuple((rng.standard_normal(s) * 0.3).astype(np.float32) for s in ((hid, dim), (hid, dim), (dim, hid)))
               for _ in range(num_experts)]
    x_all = rng.standard_normal((world * tokens_per_rank, dim)).astype(np.float32)
    probs = rng.random((world * tokens_per_rank, num_experts)).astype(np.float32)
    idx_all, val_all = orc.topk(probs, top_k)
    w_all = orc.normalize_rows(val_all)

    def run_experts(packed, offsets, first_expert, saved=None):
        out = np.zeros_like(packed)
        for e in range(len(offsets) - 1):
            lo, hi = int(offsets[e]), int(offsets[e + 1])
            if hi > lo:
                g, u, d = experts[first_expert + e]
                o, gate, up = orc.frozen_expert_forward(packed[lo:hi], g, u, d)
                out[lo:hi] = o
                if saved is not None:
                    saved[e] = (gate, up)
        return out

    def run_experts_bwd(packed_dy, offsets, first_expert, saved):
        dx = np.zeros_like(packed_dy)
        for e in range(len(offsets) - 1):
            lo, hi = int(offsets[e]), int(offsets[e + 1])
            if hi > lo:
                g, u, d = experts[first_expert + e]
                gate, up = saved[e]
                dx[lo:hi] = orc.frozen_expert_backward(packed_dy[lo:hi], gate, up, g, u, d)
        return dx

    class Ops:
        def build_dispatch(self, indices):
            dmap, off, _ = orc.build_dispatch_map(indices.numpy(), num_experts)
            return torch.from_numpy(dmap), torch.from_numpy(off)

        def dispatch(self, x, indices, dmap, off, total):
            return torch.from_numpy(orc.moe_dispatch(x.numpy(), indices.numpy(), dmap.numpy(), off.numpy(), total))

        def experts(self, packed, local_offsets):
            first = rank * (num_experts // world)
            self.saved = {}
            return torch.from_numpy(run_experts(packed.numpy(), local_offsets.numpy(), first, self.saved))

        def experts_bwd(self, packed_dy, local_offsets):
            first = rank * (num_experts // world)
            return torch.from_numpy(run_experts_bwd(packed_dy.numpy(), local_offsets.numpy(), first, self.saved))

        def combine_bwd(self, dy, indices, weights, dmap, off, total):
            return torch.from_numpy(orc.moe_combine_bwd_grad_expert(dy.numpy(), indices.numpy(), weights.numpy(),
                                                                    dmap.numpy(), off.numpy(), total))

        def dispatch_bwd(self, gbuf, indices, dmap, off, tokens):
            return torch.from_numpy(orc.moe_dispatch_bwd(gbuf.numpy(), indices.numpy(), dmap.numpy(), off.numpy(),
                                                         tokens))

        def combine(self, buf, indices, weights, dmap, off, tokens):
            return torch.from_numpy(orc.moe_combine(buf.numpy(), indices.numpy(), weights.numpy(), dmap.numpy(),
                                                    off.numpy(), tokens))

    sl = slice(rank * tokens_per_rank, (rank + 1) * tokens_per_rank)
    moe = ExpertParallelFrozenMoE(Ops(), num_experts)
    got = moe.forward(torch.from_numpy(x_all[sl]), torch.from_numpy(idx_all[sl]), torch.from_numpy(w_all[sl]))
    # single-process reference on this rank's tokens with all experts local
    dmap, off, total = orc.build_dispatch_map(idx_all[sl], num_experts)
    packed = orc.moe_dispatch(x_all[sl], idx_all[sl], dmap, off, total)
    saved = {}
    want = orc.moe_combine(run_experts(packed, off, 0, saved), idx_all[sl], w_all[sl], dmap, off, tokens_per_rank)
    ok_fwd = bool(np.array_equal(got.numpy(), want))
    # backward: the gradient of this rank's tokens through combine, the experts' dX and dispatch
    dy = np.random.default_rng(31 + rank).standard_normal((tokens_per_rank, dim)).astype(np.float32)
    got_dx = moe.backward(torch.from_numpy(dy))
    gbuf = orc.moe_combine_bwd_grad_expert(dy, idx_all[sl], w_all[sl], dmap, off, total)
    want_dx = orc.moe_dispatch_bwd(run_experts_bwd(gbuf, off, 0, saved), idx_all[sl], dmap, off, tokens_per_rank)
    ok_bwd = bool(np.array_equal(got_dx.numpy(), want_dx))
    # a cached routing gives the same result, and the exchange alone returns every row unchanged
    routing = moe.route(torch.from_numpy(idx_all[sl]))
    again = moe.forward(torch.from_numpy(x_all[sl]), torch.from_numpy(idx_all[sl]), torch.from_numpy(w_all[sl]), routing)
    ok_fwd = ok_fwd and bool(np.array_equal(again.numpy(), want))
    ok_fwd = ok_fwd and moe.round_trip_check(torch.from_numpy(x_all[sl]), torch.from_numpy(idx_all[sl]), routing) == 0.0
    out_q.put((rank, ok_fwd, ok_bwd))
    dist.destroy_process_group()


def _spawn(worker, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(results)


def test_shard_range_and_owner():
    from caif_b200.sharded import expert_owner, shard_range

    assert [shard_range(14336, 8, r) for r in (0, 7)] == [(0, 1792), (12544, 14336)]
    assert expert_owner(0, 64, 8) == 0 and expert_owner(63, 64, 8) == 7 and expert_owner(8, 64, 8) == 1
    with pytest.raises(ValueError):
        shard_range(100, 8, 0)


def test_regroup_index():
    from caif_b200.sharded import ExpertParallelFrozenMoE

    incoming = torch.tensor([[2, 0, 1], [1, 3, 0]])       # [source, local expert]
    perm, off = ExpertParallelFrozenMoE.regroup_index(incoming)
    # arrival order: s0:e0,e0,e2 | s1:e0,e1,e1,e1 -> per expert: e0: 0,1,3  e1: 4,5,6  e2: 2
    assert perm.tolist() == [0, 1, 3, 4, 5, 6, 2]
    assert off.tolist() == [0, 3, 6, 7]


def test_column_parallel_world2_gloo():
    for rank, ok_y, ok_dx in _spawn(_column_parallel_worker):
        assert ok_y and ok_dx, rank


def test_expert_parallel_world2_gloo():
    """Forward and backward of the expert-parallel frozen experts equal the one-process dataflow bit for bit."""
    for rank, ok_fwd, ok_bwd in _spawn(_expert_parallel_worker):
        assert ok_fwd, rank
        assert ok_bwd, rank
