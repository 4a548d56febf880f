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

    def _buf(self, name, shape, like):
        b = self._bufs.get(name)
        if b is None or b.shape != tuple(shape) or b.device != like.device:
            b = torch.empty(shape, dtype=like.dtype, device=like.device)
            self._bufs[name] = b
        return b

    def forward(self, layer, x, out):
        """out[T,D] += MoE(x[T,D]) for this rank's rows; `layer` is this rank's shard."""
        T, D = x.shape
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
