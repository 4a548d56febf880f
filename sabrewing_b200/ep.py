"""Expert-parallel driver: experts sharded contiguously across the ranks of one node.

Each rank brings its own T token rows (data-parallel attention side), owns experts
[rank*E/N, (rank+1)*E/N) of every layer, and holds the router and the shared expert
replicated.  One step is: all-gather the token rows -> every rank routes all N*T
rows identically (same kernels, same bits) -> each rank runs only the (row, expert)
pairs of its resident experts -> reduce-scatter of the partial routed sums hands
every rank the routed sum of its own rows -> scale, shared expert, residual.  The
reference has no multi-process layer (its only multi-device code moves one row per
device with cudaMemcpyPeer, c/backend_cuda.cu:1444-1466); routing ids and the
dispatch arrays stay bit-identical on every rank, the cross-rank sum order differs
from pure rank order within the output tolerance.

Two exchange schemes (`scheme`): "replicate" as above, and "alltoall" for large
batches: every rank routes only its own rows, sends each row once to every rank that
holds one of its experts (with its ids and weights, ids of other ranks' experts
blanked to -1), the destination groups what it received by expert, runs its experts
and returns one pre-weighted partial sum per received row, and the owner adds the
partial sums of a row in rank order.

On CUDA the whole step is ONE call into the library (`sw_ep_forward`, which enqueues
the NCCL collectives itself); `forward()` below falls back to the Python exchange over
`torch.distributed` only for compute objects without that entry -- the CPU tests run
the same partition / permutation logic over gloo with a stand-in built on the checker.
"""
import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

SCHEMES = {"replicate": 0, "alltoall": 1}


def shard_range(n_experts, world, rank):
    """Contiguous expert range [lo, lo+cnt) of `rank`; the first n_experts % world ranks hold one more."""
    base, rem = divmod(n_experts, world)
    lo = rank * base + min(rank, rem)
    return lo, base + (1 if rank < rem else 0)


def plan_all_to_all(sel, ranges):
    """Which own rows go to which rank, each row once.  sel [T,K] int; ranges [(lo, cnt)] per rank.
    Returns (send_idx: list of int arrays in ascending row order, rank_of [T, world]: position of the row in
    that rank's send list or -1).  The device kernel k_ep_plan builds the same two arrays."""
    T = sel.shape[0]
    send_idx, rank_of = [], np.full((T, len(ranges)), -1, np.int64)
    for g, (lo, cnt) in enumerate(ranges):
        rows = np.nonzero(((sel >= lo) & (sel < lo + cnt)).any(axis=1))[0]
        send_idx.append(rows)
        rank_of[rows, g] = np.arange(len(rows))
    return send_idx, rank_of


class ExpertParallelMoe:
    def __init__(self, block, desc, group=None, scheme="replicate"):
        self.block, self.desc, self.group, self.scheme = block, desc, group, scheme
        assert scheme in SCHEMES
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._bufs = {}
        self._side = None
        self._graphs = {}
        self._ep = None          # SwEp handle of the in-library step (CUDA)

    # ---- the in-library step (CUDA): one host call per step, NCCL enqueued by the library ----
    def native_init(self, rows_per_rank, D, device):
        """Create the library's exchange state: rank 0 draws the NCCL id, every rank receives it over the default
        process group, then joins the library's own communicator."""
        lib = self.block.lib
        idbuf = torch.zeros(128, dtype=torch.uint8)
        if self.rank == 0:
            raw = (C.c_ubyte * 128)()
            self.block._chk(lib.sw_ep_unique_id(raw), "sw_ep_unique_id")
            idbuf = torch.tensor(list(raw), dtype=torch.uint8)
        idbuf = idbuf.to(device)
        dist.broadcast(idbuf, src=0, group=self.group)
        raw = (C.c_ubyte * 128)(*idbuf.cpu().tolist())
        h = C.c_void_p()
        self.block._chk(lib.sw_ep_create(C.byref(h), self.block.ctx, raw, self.world, self.rank, rows_per_rank, D, self.desc.topk),
                        "sw_ep_create")
        self._ep = h

    def native_forward(self, layer, x, out, timed=False, stream=None):
        d, l = self.desc.c(), layer.c()
        self.block._last = (x.shape[0] * self.world, self.desc.topk, self.desc.n_experts)
        self.block._chk(self.block.lib.sw_ep_forward(self._ep, C.byref(d), C.byref(l), x.data_ptr(), out.data_ptr(), x.shape[0],
                                                     SCHEMES[self.scheme], 1 if timed else 0, self.block._stream(stream)), "sw_ep_forward")
        return out

    def native_segments(self):
        ms = (C.c_float * 8)()
        n = self.block.lib.sw_ep_segments(self._ep, ms, SCHEMES[self.scheme])
        self.block._chk(0 if n > 0 else -1, "sw_ep_segments")
        names = (("all_gather", "route_experts", "reduce_scatter", "finish") if self.scheme == "replicate" else
                 ("route_plan_pack_counts", "rows_out", "experts", "partials_back_add", "finish"))
        return {k: float(ms[i]) for i, k in enumerate(names[:n])}

    def close(self):
        if self._ep is not None:
            self.block.lib.sw_ep_destroy(self._ep)
            self._ep = None

    def _buf(self, name, shape, like):
        b = self._bufs.get(name)
        if b is None or b.shape != tuple(shape) or b.device != like.device:
            b = torch.empty(shape, dtype=like.dtype, device=like.device)
            self._bufs[name] = b
        return b

    def prepare(self, layer, x, out):
        """Record this rank's kernels of one step for (layer, x, out) as three graphs -- shared expert; route +
        resident experts; finish -- which forward() then launches between the collectives instead of a dozen
        kernels one by one.  The collectives themselves stay ordinary NCCL calls.  CUDA block only."""
        if self.world == 1 or not x.is_cuda or not hasattr(self.block, "capture"):
            return
        self.forward(layer, x, out)                      # set-up work and buffers, eagerly
        torch.cuda.synchronize(x.device)
        T, D = x.shape
        b, d = self.block, self.desc
        X, partial, routed = self._bufs["X"], self._bufs["partial"], self._bufs["routed"]
        g_shared = b.capture(lambda s: b.shared(d, layer, x, stream=s))
        g_experts = b.capture(lambda s: (b.route(d, layer, X, stream=s), b.experts(d, layer, X, partial, stream=s)))
        # finish is recorded after a shared() of the same row count so that it takes the shared rows from there
        b.shared(d, layer, x)
        g_finish = b.capture(lambda s: b.finish(d, layer, x, routed, out, stream=s))
        torch.cuda.synchronize(x.device)
        self._graphs[(id(layer), x.data_ptr(), out.data_ptr())] = (g_shared, g_experts, g_finish, layer)

    def forward(self, layer, x, out):
        """out[T,D] += MoE(x[T,D]) for this rank's rows; `layer` is this rank's shard."""
        T, D = x.shape
        if self._ep is not None:
            return self.native_forward(layer, x, out)
        if self.scheme == "alltoall" and self.world > 1:
            return self._forward_alltoall(layer, x, out)
        gs = self._graphs.get((id(layer), x.data_ptr(), out.data_ptr()))
        if gs is not None:
            return self._forward_graphs(gs, x, out)
        # The shared expert needs only this rank's rows: on a second stream it runs beside the exchange and the
        # routed experts (CUDA block only; the CPU stand-in has no streams).
        side = None
        if self.world > 1 and x.is_cuda and hasattr(self.block, "shared"):
            if self._side is None:
                self._side = torch.cuda.Stream(device=x.device)
            side, cur = self._side, torch.cuda.current_stream(x.device)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                self.block.shared(self.desc, layer, x)
        if self.world == 1:
            X = x
        else:
            X = self._buf("X", (self.world * T, D), x)
            dist.all_gather_into_tensor(X, x, group=self.group)
        self.block.route(self.desc, layer, X)
        partial = self._buf("partial", X.shape, x)
        self.block.experts(self.desc, layer, X, partial)
        if self.world == 1:
            routed = partial
        else:
            routed = self._buf("routed", (T, D), x)
            dist.reduce_scatter_tensor(routed, partial, op=dist.ReduceOp.SUM, group=self.group)
        if side is not None:
            torch.cuda.current_stream(x.device).wait_stream(side)
        self.block.finish(self.desc, layer, x, routed, out)
        return out

    def _forward_alltoall(self, layer, x, out):
        """The all-to-all scheme over torch.distributed point-to-point calls (any backend): the host-side twin of
        sw_ep_forward(SW_EP_ALLTOALL).  The compute object needs route(), routing() -> {sel, w}, experts_routed() and
        finish()."""
        from .ep import shard_range as _sr
        T, D = x.shape
        W, me, K = self.world, self.rank, self.desc.topk if self.desc is not None else None
        self.block.route(self.desc, layer, x)
        r = self.block.routing()
        sel, w = np.asarray(r["sel"]), np.asarray(r["w"], np.float32)
        K = sel.shape[1]
        E = self.block.n_experts if self.desc is None else self.desc.n_experts
        ranges = [_sr(E, W, g) for g in range(W)]
        send_idx, rank_of = plan_all_to_all(sel, ranges)
        counts = torch.zeros(W, dtype=torch.int64, device=x.device)
        for g in range(W):
            counts[g] = len(send_idx[g])
        allc = [torch.zeros_like(counts) for _ in range(W)]
        dist.all_gather(allc, counts, group=self.group)
        allc = torch.stack(allc).cpu().numpy()                      # [src][dst]
        sx, ssel, sw_ = [], [], []
        for g, (lo, cnt) in enumerate(ranges):
            rows = send_idx[g]
            sx.append(x[torch.from_numpy(rows).to(x.device)].contiguous())
            sg = sel[rows].copy(); sg[(sg < lo) | (sg >= lo + cnt)] = -1
            ssel.append(torch.from_numpy(sg.astype(np.int32)).to(x.device)); sw_.append(torch.from_numpy(w[rows]).to(x.device))
        rx = [torch.empty((int(allc[g][me]), D), dtype=x.dtype, device=x.device) for g in range(W)]
        rsel = [torch.empty((int(allc[g][me]), K), dtype=torch.int32, device=x.device) for g in range(W)]
        rw = [torch.empty((int(allc[g][me]), K), dtype=torch.float32, device=x.device) for g in range(W)]
        ops = []
        for g in range(W):
            if g == me:
                rx[g], rsel[g], rw[g] = sx[g], ssel[g], sw_[g]
                continue
            for snd, rcv in ((sx, rx), (ssel, rsel), (sw_, rw)):
                if snd[g].numel():
                    ops.append(dist.P2POp(dist.isend, snd[g], g, group=self.group))
                if rcv[g].numel():
                    ops.append(dist.P2POp(dist.irecv, rcv[g], g, group=self.group))
        if ops:
            for q in dist.batch_isend_irecv(ops):
                q.wait()
        X = torch.cat(rx); S = torch.cat(rsel); Wt = torch.cat(rw)
        partial = torch.zeros_like(X)
        if X.shape[0]:
            self.block.experts_routed(self.desc, layer, X, S, Wt, partial)
        offs = np.concatenate([[0], np.cumsum([t.shape[0] for t in rx])])
        back = [partial[offs[g]:offs[g + 1]].contiguous() for g in range(W)]
        ret = [torch.empty((len(send_idx[g]), D), dtype=x.dtype, device=x.device) for g in range(W)]
        ops = []
        for g in range(W):
            if g == me:
                ret[g] = back[g]
                continue
            if back[g].numel():
                ops.append(dist.P2POp(dist.isend, back[g], g, group=self.group))
            if ret[g].numel():
                ops.append(dist.P2POp(dist.irecv, ret[g], g, group=self.group))
        if ops:
            for q in dist.batch_isend_irecv(ops):
                q.wait()
        routed = torch.zeros_like(x)
        for g in range(W):                                          # partial sums of a row are added in rank order
            rows = send_idx[g]
            if len(rows):
                routed[torch.from_numpy(rows).to(x.device)] += ret[g]
        self.block.finish(self.desc, layer, x, routed, out)
        return out

    def _forward_graphs(self, gs, x, out):
        g_shared, g_experts, g_finish, _ = gs
        T, D = x.shape
        X, partial, routed = self._bufs["X"], self._bufs["partial"], self._bufs["routed"]
        side, cur = self._side, torch.cuda.current_stream(x.device)
        side.wait_stream(cur)
        g_shared.replay(side)
        dist.all_gather_into_tensor(X, x, group=self.group)
        g_experts.replay()
        dist.reduce_scatter_tensor(routed, partial, op=dist.ReduceOp.SUM, group=self.group)
        cur.wait_stream(side)
        g_finish.replay()
        return out

    def timed_segments(self, layers, xs, outs, steps):
        """Mean ms of the five segments of a step on this rank, from CUDA events on the launching streams: the
        all-gather, the route + resident-experts graph, the reduce-scatter, the shared-expert graph (side stream) and
        the finish graph.  Needs prepare() to have recorded the graphs of every (layer, batch) pair used."""
        names = ("all_gather", "route_experts", "reduce_scatter", "shared", "finish")
        tot = dict.fromkeys(names, 0.0)
        dev = xs[0].device
        cur = torch.cuda.current_stream(dev)
        n = 0
        for i in range(steps):
            layer, x, out = layers[i % len(layers)], xs[i % len(xs)], outs[i % len(outs)]
            gs = self._graphs.get((id(layer), x.data_ptr(), out.data_ptr()))
            if gs is None:
                continue
            g_shared, g_experts, g_finish, _ = gs
            X, partial, routed = self._bufs["X"], self._bufs["partial"], self._bufs["routed"]
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(8)]
            side = self._side
            side.wait_stream(cur)
            ev[0].record(side); g_shared.replay(side); ev[1].record(side)
            ev[2].record(cur)
            dist.all_gather_into_tensor(X, x, group=self.group); ev[3].record(cur)
            g_experts.replay(); ev[4].record(cur)
            dist.reduce_scatter_tensor(routed, partial, op=dist.ReduceOp.SUM, group=self.group); ev[5].record(cur)
            cur.wait_stream(side); ev[6].record(cur)
            g_finish.replay(); ev[7].record(cur)
            torch.cuda.synchronize(dev)
            tot["shared"] += ev[0].elapsed_time(ev[1]); tot["all_gather"] += ev[2].elapsed_time(ev[3])
            tot["route_experts"] += ev[3].elapsed_time(ev[4]); tot["reduce_scatter"] += ev[4].elapsed_time(ev[5])
            tot["finish"] += ev[6].elapsed_time(ev[7])
            n += 1
        if n == 0:
            raise RuntimeError("no recorded graphs: call prepare() first")
        return {k: v / n for k, v in tot.items()}
