"""The in-library expert-parallel step (sw_ep_forward: NCCL enqueued by the library) on real GPUs, both exchange
schemes, against the single-GPU CPU checker.  One process per GPU, spawned here; needs two or more devices."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, synth_case, rel_l2

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, T, q):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from sabrewing_b200.ep import ExpertParallelMoe, shard_range
        from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
        res = {}
        for base, kw in (("c2", dict(D=512, E=32, K=4, I=128, SI=128)), ("c4", dict(D=256, E=12, K=4, I=128))):
            case = synth_case(base, corr_bias_std=0.01, T=T * world, **kw)
            cfg = case.cfg
            lo, cnt = shard_range(cfg.E, world, rank)
            layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, dev, expert_lo=lo, expert_cnt=cnt)
            x = torch.from_numpy(case.x[rank * T:(rank + 1) * T].copy()).to(dev)
            for scheme in ("replicate", "alltoall"):
                blk = MoeBlock(dev, T * world, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
                ep = ExpertParallelMoe(blk, desc_from_config(cfg), scheme=scheme)
                ep.native_init(T, cfg.D, dev)
                out = torch.from_numpy(case.hin[rank * T:(rank + 1) * T].copy()).to(dev)
                ep.forward(layer, x, out)
                ep.native_forward(layer, x, out, timed=True)          # a second step on the same buffers (adds again)
                torch.cuda.synchronize(dev)
                assert blk.status() == 0
                seg = ep.native_segments()
                assert all(v >= 0 for v in seg.values())
                res[(base, scheme)] = out.cpu().numpy()
                ep.close(); blk.close()
        q.put((rank, res))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_native_expert_parallel_step_matches_single_gpu_checker(orc):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    T = 24
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=600) for _ in range(world))
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for base, kw in (("c2", dict(D=512, E=32, K=4, I=128, SI=128)), ("c4", dict(D=256, E=12, K=4, I=128))):
        case = synth_case(base, corr_bias_std=0.01, T=T * world, **kw)
        want = orc.moe_group(case.host, case.x, case.hin, exact=1)["out"]
        for scheme in ("replicate", "alltoall"):
            full = np.concatenate([got[r][(base, scheme)] for r in range(world)])
            # two steps were run: out = hin + 2 * MoE(x)
            assert rel_l2((full - case.hin) / 2.0, want - case.hin) < 1e-3, (base, scheme)
