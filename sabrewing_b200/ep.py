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

The compute object only needs route / experts / finish, so the same driver runs
over the CUDA block (NCCL) and, in CPU tests, over a stand-in built on the checker
(gloo).
"""
import torch
import torch.distributed as dist


def shard_range(n_experts, world, rank):
    """Contiguous expert range [lo, lo+cnt) of `rank`; the first n_experts % world ranks hold one more."""
    base, rem = divmod(n_experts, world)
    lo = rank * base + min(rank, rem)
    return lo, base + (1 if rank < rem else 0)


class ExpertParallelMoe:
    def __init__(self, block, desc, group=None):
        self.block, self.desc, self.group = block, desc, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._bufs = {}
        self._side = None
        self._graphs = {}

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
