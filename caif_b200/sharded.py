"""Multi-GPU forms of the path: one process per GPU, torch.distributed for the plumbing.

The reference is single-device (no collective anywhere), so the contract is
"same numbers as one GPU":

* ColumnParallelFrozenLinear -- rank r holds output features [r*out/N, (r+1)*out/N) of the
  [out, in] codes and their scales (a contiguous slice of both: the codes stay bit-identical
  to the 1-GPU tensor).  Forward: local product on replicated X, all-gather of the Y slices
  along the feature axis.  Backward: dX is a partial sum over the local features, all-reduce.
* ExpertParallelFrozenMoE -- experts [r*E/N, (r+1)*E/N) live on rank r.  Each rank routes
  its own tokens, packs them by expert, sends every row to the expert's owner with an
  all-to-all (row counts are exchanged first), runs the grouped frozen experts on what it
  received, returns the rows with the mirror all-to-all and combines locally.

The compute itself is injected (`ops`): on a GPU box it is caif_b200.native (the CUDA
library); the CPU tests of the collectives' bookkeeping pass the numpy oracle instead.
No kernel of this package reads another GPU's memory: remote data always lands in local
memory through the collective first.  One kernel WRITES to it: the few-token forward can store
its slice of Y straight into every rank's result buffer (PeerBuffer below maps the buffers with
CUDA IPC), which replaces the all-gather for decode-sized calls.
"""
import ctypes
import ctypes.util

import torch
import torch.distributed as dist


class _IpcMemHandle(ctypes.Structure):
    """cudaIpcMemHandle_t: 64 opaque bytes, passed to the runtime BY VALUE."""
    _fields_ = [("reserved", ctypes.c_ubyte * 64)]


class PeerBuffer:
    """One device buffer per rank, each mapped into every process of the group (CUDA IPC with lazy
    peer access).  `ptrs[r]` is rank r's buffer as seen from this process; `local()` views this
    rank's own buffer as a tensor.  Collective constructor: every rank of the group calls it."""

    _IPC_LAZY_PEER_ACCESS = 1
    _cudart = None

    @classmethod
    def cudart(cls):
        if cls._cudart is None:
            last = None
            for name in ("libcudart.so.12", "libcudart.so", ctypes.util.find_library("cudart")):
                if not name:
                    continue
                try:
                    rt = ctypes.CDLL(name)
                    rt.cudaIpcGetMemHandle.argtypes = [ctypes.POINTER(_IpcMemHandle), ctypes.c_void_p]
                    rt.cudaIpcOpenMemHandle.argtypes = [ctypes.POINTER(ctypes.c_void_p), _IpcMemHandle, ctypes.c_uint]
                    rt.cudaIpcCloseMemHandle.argtypes = [ctypes.c_void_p]
                    rt.cudaMalloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_size_t]
                    rt.cudaMemset.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t]
                    rt.cudaFree.argtypes = [ctypes.c_void_p]
                    rt.cudaMemcpyAsync.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int,
                                                   ctypes.c_void_p]
                    cls._cudart = rt
                    break
                except OSError as e:
                    last = e
            if cls._cudart is None:
                raise RuntimeError("the CUDA runtime library is needed for peer buffers: %s" % last)
        return cls._cudart

    def __init__(self, nbytes, device, group=None):
        rt = self.cudart()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nbytes = int(nbytes)
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        base = ctypes.c_void_p()
        self._check(rt.cudaMalloc(ctypes.byref(base), self.nbytes), "cudaMalloc")
        self._check(rt.cudaMemset(base, 0, self.nbytes), "cudaMemset")
        handle = _IpcMemHandle()
        self._check(rt.cudaIpcGetMemHandle(ctypes.byref(handle), base), "cudaIpcGetMemHandle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.reserved), group=group)
        self.ptrs = []
        self._opened = []
        for r, raw in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(base.value)
                continue
            peer = ctypes.c_void_p()
            h = _IpcMemHandle()
            ctypes.memmove(h.reserved, raw, 64)
            self._check(rt.cudaIpcOpenMemHandle(ctypes.byref(peer), h, self._IPC_LAZY_PEER_ACCESS),
                        "cudaIpcOpenMemHandle")
            self.ptrs.append(peer.value)
            self._opened.append(peer)
        self._base = base
        dist.barrier(group=group)

    @staticmethod
    def _check(rc, what):
        if rc != 0:
            raise RuntimeError("%s failed with CUDA error %d" % (what, rc))

    def read(self, dtype, shape, offset=0):
        """A copy of this rank's buffer (from byte `offset`) as a tensor: a device-to-device copy on the
        current stream."""
        out = torch.empty(shape, dtype=dtype, device=self.device)
        nbytes = out.numel() * out.element_size()
        if offset + nbytes > self.nbytes:
            raise ValueError("the buffer holds %d bytes, %d asked at offset %d" % (self.nbytes, nbytes, offset))
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        src = ctypes.c_void_p(self._base.value + offset)
        self._check(self.cudart().cudaMemcpyAsync(out.data_ptr(), src, nbytes, 3, stream),   # 3: device to device
                    "cudaMemcpyAsync")
        return out

    def close(self):
        """Collective: unmaps the peers' buffers, then frees this rank's."""
        rt = self.cudart()
        torch.cuda.synchronize(self.device)
        for peer in self._opened:
            rt.cudaIpcCloseMemHandle(peer)
        self._opened = []
        dist.barrier(group=self.group)
        if self._base is not None:
            rt.cudaFree(self._base)
            self._base = None


def shard_range(total, world, rank, quantum=1):
    """Contiguous [begin, end) of `total` items for `rank`; every shard a multiple of `quantum`."""
    if total % (world * quantum) != 0:
        raise ValueError("%d does not split into %d shards of a multiple of %d" % (total, world, quantum))
    per = total // world
    return rank * per, (rank + 1) * per


def expert_owner(expert, num_experts, world):
    per = num_experts // world
    return expert // per


class ColumnParallelFrozenLinear:
    """y = x . W^T with W's rows sharded over the ranks of `group`."""

    def __init__(self, fwd, dx, out_dim, in_dim, group=None):
        """fwd(x) -> local Y slice [m, out/N]; dx(dy_slice) -> partial dX [m, in] (fp32)."""
        self.fwd = fwd
        self.dx = dx
        self.out_dim = out_dim
        self.in_dim = in_dim
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.begin, self.end = shard_range(out_dim, self.world, self.rank)
        self._gather_calls = 0

    def forward(self, x):
        y_local = self.fwd(x)                                    # [m, out/N]
        m = y_local.shape[0]
        shard = y_local.shape[1]
        # concatenated along dim 0 (the form every backend accepts): rows [r*m, (r+1)*m) come from rank r
        gathered = torch.empty((self.world * m, shard), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(gathered, y_local.contiguous(), group=self.group)
        # [N, m, out/N] -> [m, N, out/N] -> [m, out]: rank r's features land at columns [r*out/N, ...)
        return gathered.view(self.world, m, shard).permute(1, 0, 2).reshape(m, self.out_dim)

    def forward_gather(self, fwd_gather, x, peer_buffer, out_dtype=torch.float32):
        """Few-token forward with the gather fused into the kernel: fwd_gather(x, ptrs, y_ld, y_col0)
        stores this rank's [m, out/N] slice into every rank's [m, out] buffer.  Returns this rank's
        full Y once all ranks' kernels are complete (a stream-ordered barrier collective).

        Buffer reuse: the peer buffer is used as two halves, alternating per call.  A rank can only
        start call n+2 (which writes the half that call n used) after it has passed the barrier of
        call n+1, and that barrier completes on it only after every rank has enqueued its own barrier of
        call n+1, which is ordered behind that rank's read of call n on its stream.  So a fast rank
        never overwrites a result a slower rank is still reading, without a second barrier per call.
        The buffer must hold 2 * m * out elements of `out_dtype`."""
        m = x.shape[0]
        elem = torch.empty((), dtype=out_dtype).element_size()
        half_bytes = m * self.out_dim * elem
        if 2 * half_bytes > peer_buffer.nbytes:
            raise ValueError("the peer buffer holds %d bytes; two results of %d bytes are needed"
                             % (peer_buffer.nbytes, half_bytes))
        half = self._gather_calls & 1
        self._gather_calls += 1
        off = half * half_bytes
        fwd_gather(x, [q + off for q in peer_buffer.ptrs], self.out_dim, self.begin)
        dist.barrier(group=self.group)   # NCCL: a collective kernel behind this rank's stores on the stream
        return peer_buffer.read(out_dtype, (m, self.out_dim), offset=off)

    def backward(self, dy):
        part = self.dx(dy[:, self.begin:self.end].contiguous())  # partial sum over this rank's features
        dist.all_reduce(part, op=dist.ReduceOp.SUM, group=self.group)
        return part


class ExpertParallelFrozenMoE:
    """Routed frozen experts sharded by expert.  `ops` supplies, with the semantics of the
    C ABI entry points of the same names: build_dispatch(indices) -> (dispatch_map, offsets),
    dispatch(x, indices, dmap, offsets, total) -> packed rows, experts(packed, offsets_local)
    -> packed outputs for the experts this rank owns, combine(buf, indices, weights, dmap,
    offsets, tokens) -> [tokens, dim]; for backward() also combine_bwd(dy, indices, weights, dmap,
    offsets, total) -> packed gradients, experts_bwd(packed_dy, offsets_local) -> packed dX of the
    owned experts, dispatch_bwd(grad_buf, indices, dmap, offsets, tokens) -> [tokens, dim]."""

    def __init__(self, ops, num_experts, group=None):
        self.ops = ops
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.num_experts = num_experts
        self.e_begin, self.e_end = shard_range(num_experts, self.world, self.rank)
        self.local_experts = self.e_end - self.e_begin

    def plan(self, offsets):
        """From this rank's per-expert offsets [E+1]: rows sent to every rank, rows received from
        every rank, and the per-(source, local expert) counts of what arrives."""
        counts_dev = (offsets[1:] - offsets[:-1]).to(torch.int64)                # rows per expert, local tokens
        per = self.local_experts
        # the exchange runs where the offsets live (device memory under NCCL, host memory under gloo)
        all_counts = [torch.empty_like(counts_dev) for _ in range(self.world)]
        dist.all_gather(all_counts, counts_dev, group=self.group)                # small: E ints per rank
        counts = counts_dev.cpu()
        send_counts = counts.view(self.world, per).sum(dim=1)                    # rows to each owner
        incoming = torch.stack([c[self.e_begin:self.e_end].cpu() for c in all_counts])  # [source, local expert]
        recv_counts = incoming.sum(dim=1)
        return send_counts, recv_counts, incoming

    @staticmethod
    def regroup_index(incoming):
        """Rows arrive grouped by source rank, each source's rows ordered by expert.  Returns the
        permutation that makes them contiguous per expert (sources in rank order inside an
        expert), and the local offsets [E_local+1]."""
        sources, experts = incoming.shape
        src_start = torch.zeros(sources, dtype=torch.int64)
        src_start[1:] = torch.cumsum(incoming.sum(dim=1), 0)[:-1]
        within = torch.zeros_like(incoming)
        within[:, 1:] = torch.cumsum(incoming, dim=1)[:, :-1]
        order = []
        for e in range(experts):
            for s in range(sources):
                n = int(incoming[s, e])
                if n:
                    start = int(src_start[s] + within[s, e])
                    order.append(torch.arange(start, start + n, dtype=torch.int64))
        perm = torch.cat(order) if order else torch.zeros(0, dtype=torch.int64)
        local_offsets = torch.zeros(experts + 1, dtype=torch.int32)
        local_offsets[1:] = torch.cumsum(incoming.sum(dim=0), 0).to(torch.int32)
        return perm, local_offsets

    def route(self, expert_indices):
        """Everything about a routing decision that the exchange needs, computed once: dispatch map and
        offsets of this rank's tokens, rows per destination and per source, the permutation that groups
        arriving rows by expert.  Reusable as long as `expert_indices` does not change."""
        dmap, offsets = self.ops.build_dispatch(expert_indices)
        total = int(offsets[-1])
        send_counts, recv_counts, incoming = self.plan(offsets)
        perm, local_offsets = self.regroup_index(incoming)
        return {"indices": expert_indices, "dmap": dmap, "offsets": offsets, "total": total,
                "send": send_counts.tolist(), "recv": recv_counts.tolist(), "perm": perm.to(dmap.device),
                "local_offsets": local_offsets, "received_rows": int(recv_counts.sum())}

    def _to_owners(self, packed, routing):
        """Rows packed by (global) expert -> rows grouped by local expert on the experts' owners."""
        received = torch.empty((routing["received_rows"], packed.shape[1]), dtype=packed.dtype, device=packed.device)
        dist.all_to_all_single(received, packed, output_split_sizes=routing["recv"],
                               input_split_sizes=routing["send"], group=self.group)
        return received.index_select(0, routing["perm"])

    def _from_owners(self, grouped, routing):
        """The mirror exchange: rows grouped by local expert -> the senders' packed order."""
        arrival = torch.empty_like(grouped)
        arrival.index_copy_(0, routing["perm"], grouped)                              # back to arrival order
        returned = torch.empty((routing["total"], grouped.shape[1]), dtype=grouped.dtype, device=grouped.device)
        dist.all_to_all_single(returned, arrival, output_split_sizes=routing["send"],
                               input_split_sizes=routing["recv"], group=self.group)
        return returned

    def forward(self, x, expert_indices, expert_weights, routing=None):
        """The frozen experts' part of the layer forward (src/caif_device_moe_layer.cpp:534-557) with the
        experts on their owners.  Keeps what backward() needs."""
        tokens = x.shape[0]
        if routing is None:
            routing = self.route(expert_indices)
        packed = self.ops.dispatch(x, expert_indices, routing["dmap"], routing["offsets"], routing["total"])
        grouped = self._to_owners(packed, routing)
        out_grouped = self.ops.experts(grouped, routing["local_offsets"])
        returned = self._from_owners(out_grouped, routing)
        self._saved = (routing, expert_weights, tokens)
        return self.ops.combine(returned, expert_indices, expert_weights, routing["dmap"], routing["offsets"], tokens)

    def backward(self, dy):
        """The mirror of the layer backward over frozen experts (src/caif_device_moe_layer.cpp:754-778):
        the gradient of every (token, k) pick goes to the expert's owner, which runs the experts' dX on the
        rows it owns (`ops.experts_bwd`, using what its forward saved); the rows come back and are summed
        over k per token.  dX only: frozen experts have no weight gradient."""
        routing, expert_weights, tokens = self._saved
        idx = routing["indices"]
        gbuf = self.ops.combine_bwd(dy, idx, expert_weights, routing["dmap"], routing["offsets"], routing["total"])
        grouped = self._to_owners(gbuf, routing)
        gx_grouped = self.ops.experts_bwd(grouped, routing["local_offsets"])
        returned = self._from_owners(gx_grouped, routing)
        return self.ops.dispatch_bwd(returned, idx, routing["dmap"], routing["offsets"], tokens)

    def round_trip_check(self, x, expert_indices, routing=None):
        """Sends every packed row to its expert's owner and straight back: the largest absolute
        difference between what was sent and what returned (0.0 when the exchange is exact)."""
        if routing is None:
            routing = self.route(expert_indices)
        packed = self.ops.dispatch(x, expert_indices, routing["dmap"], routing["offsets"], routing["total"])
        back = self._from_owners(self._to_owners(packed, routing), routing)
        if packed.numel() == 0:
            return 0.0
        return float((back.float() - packed.float()).abs().max())
