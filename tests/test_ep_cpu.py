"""Expert-parallel driver over world_size-2 (and 4) gloo ranks on CPU.

The CUDA block is replaced by a stand-in with the same route/experts/finish
interface built on the CPU checker, so the partitioning, the all-gather /
reduce-scatter exchange and the final combine are exercised without a GPU.
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, synth_case, rel_l2


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


class CheckerBlock:
    """route / experts / finish of the CUDA block, computed by the CPU checker for one expert shard."""

    def __init__(self, case, lo, cnt):
        import oracle
        self.orc = oracle.load(); self.case, self.lo, self.cnt = case, lo, cnt

    def route(self, desc, layer, X):
        x = np.ascontiguousarray(X.numpy())
        self.sel, self.w = self.orc.route(self.case.host, x, exact=1)

    def routing(self):
        return {"sel": self.sel, "w": self.w}

    @property
    def n_experts(self):
        return self.case.cfg.E

    def experts_routed(self, desc, layer, X, sel, w, partial):
        """Routing given by the sender: -1 ids contribute nothing; only resident experts are computed here."""
        x = np.ascontiguousarray(X.numpy()); sel = sel.numpy().copy(); w = w.numpy().copy()
        keep = (sel >= self.lo) & (sel < self.lo + self.cnt)
        assert ((sel == -1) | keep).all()                       # the sender blanked every id that does not live here
        w = np.where(keep, w, 0.0).astype(np.float32); sel[~keep] = self.lo
        partial.copy_(torch.from_numpy(self.orc.experts_given_routing(self.case.host, x, sel, w, exact=1)))

    def experts(self, desc, layer, X, partial):
        x = np.ascontiguousarray(X.numpy())
        w = np.where((self.sel >= self.lo) & (self.sel < self.lo + self.cnt), self.w, 0.0).astype(np.float32)
        partial.copy_(torch.from_numpy(self.orc.experts_given_routing(self.case.host, x, self.sel, w, exact=1)))

    def finish(self, desc, layer, x, routed, out):
        cfg = self.case.cfg
        acc = routed.numpy() * np.float32(cfg.route_scale)
        if cfg.shared_mode:
            acc = acc + self.orc.shared_rows(self.case.host, np.ascontiguousarray(x.numpy()), exact=1)
        out += torch.from_numpy(acc.astype(np.float32))


def _worker(rank, world, port, base, kw, T, q, scheme="replicate"):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sabrewing_b200.ep import ExpertParallelMoe, shard_range
        case = synth_case(base, corr_bias_std=0.01, T=T * world, **kw)
        lo, cnt = shard_range(case.cfg.E, world, rank)
        ep = ExpertParallelMoe(CheckerBlock(case, lo, cnt), None, scheme=scheme)
        x = torch.from_numpy(case.x[rank * T:(rank + 1) * T].copy())
        out = torch.from_numpy(case.hin[rank * T:(rank + 1) * T].copy())
        ep.forward(None, x, out)
        q.put((rank, out.numpy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("scheme", ["replicate", "alltoall"])
@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("base,kw", [("c4", dict(D=128, E=12, K=4, I=64)), ("c2", dict(D=128, E=10, K=3, I=64, SI=64))])
def test_expert_parallel_matches_single_rank(orc, world, base, kw, scheme):
    T = 3 if scheme == "replicate" else 5
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, base, kw, T, q, scheme)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    case = synth_case(base, corr_bias_std=0.01, T=T * world, **kw)
    want = orc.moe_group(case.host, case.x, case.hin, exact=1)["out"]
    full = np.concatenate([got[r] for r in range(world)])
    # the cross-rank sum order differs from pure rank order: float-noise, far inside the output bar
    assert rel_l2(full - case.hin, want - case.hin) < 1e-5


def test_shard_ranges_cover_all_experts():
    from sabrewing_b200.ep import shard_range
    for E in (8, 10, 256, 384, 512):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(E, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == E
            assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))


def test_all_to_all_plan_sends_each_row_once_per_rank():
    from sabrewing_b200.ep import plan_all_to_all, shard_range
    rng = np.random.default_rng(3)
    E, K, T, W = 24, 4, 50, 4
    sel = np.stack([rng.permutation(E)[:K] for _ in range(T)]).astype(np.int32)
    ranges = [shard_range(E, W, g) for g in range(W)]
    send_idx, rank_of = plan_all_to_all(sel, ranges)
    for g, (lo, cnt) in enumerate(ranges):
        want = [t for t in range(T) if any(lo <= e < lo + cnt for e in sel[t])]
        assert send_idx[g].tolist() == want                               # ascending rows, each once
        assert [rank_of[t, g] for t in want] == list(range(len(want)))
        assert (rank_of[[t for t in range(T) if t not in want], g] == -1).all()
    # every (row, expert) pair is covered by exactly one destination
    assert sum(len(s) for s in send_idx) == sum(len({next(g for g, (lo, c) in enumerate(ranges) if lo <= e < lo + c) for e in sel[t]}) for t in range(T))
