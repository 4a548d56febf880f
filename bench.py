"""MoE-block benchmark: tokens/s of one Laguna-shaped MoE layer call at a decode batch.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload c1|c2|c3|c4|c5] [--batch T] [--layers L]

A step is one pass of the MoE block (route -> top-k -> group-by-expert -> int4
gate/up -> SiLU*up -> int4 down -> combine + shared expert) over one batch of T
synthetic token rows.  Steps cycle over L resident layers and 8 token batches so no
step finds its weights in L2.  N > 1 shards the experts over the ranks (one process
per GPU) with T rows per rank (weak scaling).  Prints one JSON line on rank 0.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "moe_block_tokens_per_s"
UNIT = "tokens/s"
LAYER_KEYS = ("router_w", "corr_bias", "logit_bias", "gu_q", "gu_s", "dn_q", "dn_s", "sh_gate", "sh_up", "sh_down")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2")
    ap.add_argument("--batch", type=int, default=0, help="token rows per rank and step (0 = the config's)")
    ap.add_argument("--layers", type=int, default=4, help="resident layers the steps cycle over")
    ap.add_argument("--cpu-reps", type=int, default=12)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch the kernels of every step one by one instead of replaying CUDA graphs")
    return ap.parse_args()


def workload_name(cfg, T, world):
    return "%s: D=%d E=%d top%d I=%d shared_I=%d, decode batch %d%s" % (
        cfg.name, cfg.D, cfg.E, cfg.K, cfg.I, cfg.SI, T, " per rank, experts sharded over %d ranks" % world if world > 1 else "")


# ---------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML while the bench runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.marks, self.stop_flag = [], {}, False
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, rs))
            except Exception:
                pass
            time.sleep(self.period)

    def mark(self, name):
        self.marks[name] = time.perf_counter()

    def summary(self, t0, t1):
        inside = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-3:]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        bits = 0
        for s in inside:
            bits |= s[2]
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(v for k, v in self.REASONS.items() if bits & k), "samples": len(inside)}


def host_layer_from(cfg, arrays):
    import numpy as np
    import oracle
    a = {}
    for k in LAYER_KEYS:
        v = arrays.get(k)
        if v is None:
            a[k] = None
        else:
            v = v.cpu().numpy() if hasattr(v, "cpu") else v
            a[k] = v.view(np.uint16) if v.dtype == np.int16 else v
    return oracle.HostLayer(cfg.D, cfg.I, cfg.SI, cfg.E, cfg.K, cfg.route_act, cfg.use_corr_bias, cfg.norm_topk,
                            cfg.route_scale, cfg.shared_mode, cfg.gs, **a)


def cpu_step_fn(cfg, host):
    """The reference's CPU implementation of one block call (its timed default: AVX-512 f32), or the port."""
    import oracle
    ref = oracle.load_ref()
    laguna_ok = cfg.route_act == 0 and cfg.shared_mode == 1 and cfg.gs == 0 and host.a.get("logit_bias") is None
    if ref is not None:
        ref.omp_autotune()                    # one thread per physical core, c/moe_util.h:78-87
        if laguna_ok:
            return "reference", ref.threads(), (lambda x, h: ref.laguna_moe_rows(host, x, h, exact=0, group_on=1))
        return "reference", ref.threads(), (lambda x, h: ref.moe_block_rows(host, x, h, exact=0))
    orc = oracle.load()
    return "port", orc.threads(), (lambda x, h: orc.moe_group(host, x, h, exact=0)["out"])


def time_cpu(fn, x, reps, budget_s=30.0):
    import numpy as np
    h = np.zeros_like(x)
    fn(x, h)                                  # warm-up
    best, done, t_start = None, 0, time.perf_counter()
    while done < reps and (time.perf_counter() - t_start) < budget_s:
        t0 = time.perf_counter(); fn(x, h); dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        done += 1
    return best, done


# ---------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import torch
    from sabrewing_b200 import synth
    cfg = synth.CONFIGS[args.workload]
    T = args.batch or cfg.T
    arrays = synth.make_layer_device(cfg, "cpu", 0)
    host = host_layer_from(cfg, arrays)
    kind, cores, fn = cpu_step_fn(cfg, host)
    xs = [synth.make_tokens(cfg, T, seed_offset=1000 + i) for i in range(4)]
    h = np.zeros_like(xs[0])
    for i in range(args.warmup):
        fn(xs[i % 4], h)
    t0 = time.perf_counter()
    for i in range(args.steps):
        fn(xs[i % 4], h)
    dt = time.perf_counter() - t0
    val = T * args.steps / dt
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32 activations x int4 weights (AVX-512 f32 accumulate)" if kind == "reference" else "f32",
            "data": "synthetic", "config": {"workload": workload_name(cfg, T, 1)},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind,
                             "sample": "every step = one full block call of the workload (T=%d rows, one layer)" % T},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from sabrewing_b200 import synth, capi
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    from sabrewing_b200.ep import ExpertParallelMoe, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    capi.lib()

    cfg = synth.CONFIGS[args.workload]
    T = args.batch or cfg.T
    desc = desc_from_config(cfg)
    lo, cnt = shard_range(cfg.E, world, rank)
    NB = 8

    sampler = ClockSampler(local)
    sampler.start()

    layers, host0 = [], None
    for li in range(args.layers):
        arrays = synth.make_layer_device(cfg, dev, li)
        if li == 0 and rank == 0 and world == 1 and not args.no_cpu_baseline:
            host0 = host_layer_from(cfg, arrays)
        layers.append(MoeLayer(cfg.D, cfg.I, cfg.SI, arrays, dev, expert_lo=lo if world > 1 else 0,
                               expert_cnt=cnt if world > 1 else 0))
        del arrays
    torch.cuda.empty_cache()
    xs_host = [torch.from_numpy(synth.make_tokens(cfg, T, seed_offset=1000 + 97 * rank + i)).pin_memory() for i in range(NB)]
    xs = [x.to(dev) for x in xs_host]
    outs = [torch.zeros_like(x) for x in xs]
    block = MoeBlock(dev, T * world, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    ep = ExpertParallelMoe(block, desc) if world > 1 else None

    # one captured CUDA graph per (layer, batch) pair the steps cycle over (single GPU)
    graphs = {}
    if ep is None and not args.no_graph:
        for li in range(len(layers)):
            for bi in range(NB):
                if (li - bi) % np.gcd(len(layers), NB) == 0:     # only the pairs (i % L, i % NB) that occur
                    graphs[(li, bi)] = block.graph(desc, layers[li], xs[bi], outs[bi])
        torch.cuda.synchronize()
    # expert parallel: this rank's kernels of a step as three graphs per pair (the collectives stay NCCL calls)
    if ep is not None and not args.no_graph:
        try:
            for li in range(len(layers)):
                for bi in range(NB):
                    if (li - bi) % np.gcd(len(layers), NB) == 0:
                        ep.prepare(layers[li], xs[bi], outs[bi])
        except Exception as e:                                  # every rank runs the same code: all fall back together
            print("stage capture failed (%s); launching the kernels one by one" % e, file=sys.stderr, flush=True)
            ep._graphs.clear()
        torch.cuda.synchronize()

    def step(i, use_graph=True):
        li, bi = i % len(layers), i % NB
        layer, x, out = layers[li], xs[bi], outs[bi]
        if ep is None:
            g = graphs.get((li, bi)) if use_graph else None
            if g is not None:
                g.replay()
            else:
                block.forward(desc, layer, x, out)
        else:
            ep.forward(layer, x, out)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        step(i)
    barrier()
    l0 = block.lib.sw_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_a = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    t_b = time.perf_counter()
    launches = block.lib.sw_launch_count() - l0
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.summary(t_a, t_b)
    value = T * world * args.steps / (ms * 1e-3)

    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 activations x int4 weights (f32 accumulate)", "data": "synthetic",
            "config": {"workload": workload_name(cfg, T, world), "global_batch": T * world, "layers_cycled": len(layers),
                       "l2": "inputs larger than L2: steps cycle over %d layers (%.2f GB of expert blobs each per GPU) and %d token batches"
                             % (len(layers), layers[0].expert_bytes() / 1e9, NB),
                       "parallelism": "ep%d" % world if world > 1 else "single",
                       "launch": "cuda graph replay per step" if graphs else ("three graph replays and two NCCL calls per step" if (ep is not None and not args.no_graph) else "one launch per kernel")},
            "clocks": clocks, "gpu_launches": int(launches)}

    # ---- roofline of the dominant kernel: per-stage CUDA events over the same steps (1 GPU) ----
    if world == 1:
        block.profile(True)
        for i in range(min(args.steps, 500)):
            step(i, use_graph=False)
        torch.cuda.synchronize()
        stage_ms, calls = block.profile_read()
        block.profile(False)
        Gs = []
        for i in range(min(NB * len(layers), 16)):
            block.route(desc, layers[i % len(layers)], xs[i % NB]); Gs.append(block.routing()["G"])
        G = float(np.mean(Gs))
        per = {k: v / max(calls, 1) for k, v in stage_ms.items()}
        dom = max(per, key=per.get)
        P, D, I, SI, E = T * cfg.K, cfg.D, cfg.I, cfg.SI, cfg.E
        alg = {"q4_gateup": G * (I * D + 8 * I) + T * D * 4 + P * I * 4,
               "q4_down": G * (I * D // 2 + 4 * D) + P * I * 4 + P * D * 4,
               "shared_gateup": 2 * SI * D * 2 + T * D * 4 + T * SI * 4,
               "shared_down": SI * D * 2 + T * SI * 4 + T * D * 4,
               "router_logits": E * D * 2 + T * D * 4 + T * E * 4,
               "combine": P * D * 4 + 2 * T * D * 4, "route_topk": 2 * T * E * 4, "dispatch": 3 * P * 4}
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        ach = alg[dom] / (per[dom] * 1e-3) / 1e9
        # DRAM bytes of one launch from an ncu capture of this workload, as a ratio to that launch's algorithmic
        # bytes (the capture and its command are summarised under profiles/); scaled to this run's launch.
        ncu_ratio = {("c2", 32, "q4_gateup"): 776.06 / 776.67, ("c2", 32, "q4_down"): 395.97 / 389.0,
                     ("c3", 4096, "q4_gateup"): 1929.8 / 1291.3, ("c3", 4096, "q4_down"): 1340.2 / 1364.0}
        ratio = ncu_ratio.get((args.workload, T, dom))
        flops = {"q4_gateup": 4.0 * P * I * D, "q4_down": 2.0 * P * I * D}
        block_bytes = G * (1.5 * I * D + 8 * I + 4 * D) + (3 * SI * D * 2 if SI else 0) + E * D * 2 + 2 * T * D * 4
        line["roofline"] = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                            "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                            "traffic": ratio * alg[dom] if ratio else None,
                            "traffic_source": "ncu dram read+write bytes of one launch of this workload / its algorithmic bytes, "
                                              "times this run's algorithmic bytes" if ratio else None,
                            "algorithmic_bytes_per_launch": alg[dom], "kernel_ms": per[dom],
                            "distinct_experts_per_step": G}
        # large groups: the expert GEMMs are bound by the tensor cores, not by HBM
        tpeak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        if dom in flops and flops[dom] / (tpeak * 1e12) > alg[dom] / (peak * 1e9):
            tach = flops[dom] / (per[dom] * 1e-3) / 1e12
            line["roofline"].update({"bound": "tensor", "achieved": tach, "peak": tpeak, "unit": "TFLOP/s", "frac": tach / tpeak,
                                     "algorithmic_flops_per_launch": flops[dom], "hbm_gbs_achieved": ach,
                                     "peak_source": ("measured, sustained bf16 (MEASURED_PEAKS.json)" if peaks else "fallback")})
        exp_ms = per["q4_gateup"] + per["q4_down"]
        line["int4_expert_gbs"] = G * (1.5 * I * D + 8 * I + 4 * D) / (exp_ms * 1e-3) / 1e9
        line["block_hbm_frac"] = block_bytes / (line["ms_per_step"] * 1e-3) / 1e9 / peak
        line["stage_ms"] = {k: round(v, 5) for k, v in per.items()}

    # ---- expert parallel: rows and int4 bytes per GPU of one step (imbalance = max / mean rows per GPU) ----
    if world > 1:
        try:
            ep.forward(layers[0], xs[0], outs[0])
            torch.cuda.synchronize()
            r = block.routing()
            mine = (r["gexp"] >= lo) & (r["gexp"] < lo + cnt)
            rows_here, experts_here = int(r["gcnt"][mine].sum()), int(mine.sum())
            tt = torch.tensor([rows_here, experts_here], device=dev, dtype=torch.float64)
            allr = [torch.zeros_like(tt) for _ in range(world)]
            dist.all_gather(allr, tt)
            rows = [float(a[0].item()) for a in allr]; exps = [float(a[1].item()) for a in allr]
            per_expert = 1.5 * cfg.I * cfg.D + 8 * cfg.I + 4 * cfg.D
            line["expert_parallel"] = {"rows_per_gpu": rows, "distinct_experts_per_gpu": exps,
                                       "imbalance": max(rows) / (sum(rows) / world) if sum(rows) else None,
                                       "int4_gbs_per_gpu": [e * per_expert / (line["ms_per_step"] * 1e-3) / 1e9 for e in exps]}
        except Exception as e:                      # a reporting extra: never lose the bench line over it
            line["expert_parallel"] = {"error": str(e)[:120]}

    # ---- end to end through host buffers: pinned x -> H2D, block, D2H of the result, every step ----
    if world == 1:
        hx = [x.numpy() for x in xs_host]
        ho_t = [torch.zeros_like(x).pin_memory() for x in xs_host]      # residual rows, page-locked like the inputs
        ho = [t.numpy() for t in ho_t]
        n_e2e = max(3, min(args.steps, 200))
        for i in range(3):
            block.forward_host(desc, layers[i % len(layers)], hx[i % NB], ho[i % NB])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(n_e2e):
            block.forward_host(desc, layers[i % len(layers)], hx[i % NB], ho[i % NB])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        nbytes = T * cfg.D * 4
        line["e2e"] = {"value": T * n_e2e / dt, "unit": UNIT, "h2d_bytes_per_step": 2 * nbytes, "d2h_bytes_per_step": nbytes,
                       "steps": n_e2e, "api": "sw_moe_forward_host (page-locked host rows: x up, residual rows up beside the kernels, residual + MoE(x) down; one sync per call)"}
    else:
        # expert-parallel: every rank copies its rows in from pinned memory and its result back out each step
        n_e2e = max(3, min(args.steps, 200))
        hout = [torch.zeros_like(h).pin_memory() for h in xs_host]
        barrier()
        t0 = time.perf_counter()
        for i in range(n_e2e):
            xs[i % NB].copy_(xs_host[i % NB], non_blocking=True)
            step(i)
            hout[i % NB].copy_(outs[i % NB], non_blocking=True)
            torch.cuda.current_stream().synchronize()
        barrier()
        dt = time.perf_counter() - t0
        t = torch.tensor([dt], device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); dt = float(t.item())
        nbytes = T * cfg.D * 4
        line["e2e"] = {"value": T * world * n_e2e / dt, "unit": UNIT, "h2d_bytes_per_step": nbytes * world,
                       "d2h_bytes_per_step": nbytes * world, "steps": n_e2e,
                       "api": "ExpertParallelMoe.forward with per-step pinned H2D of x and D2H of out on every rank"}

    # ---- CPU baseline on the host cores (rank 0, N=1): the reference's own CPU code on the same layer ----
    if host0 is not None:
        kind, cores, fn = cpu_step_fn(cfg, host0)
        xh = xs_host[0].numpy()
        best, done = time_cpu(fn, xh, args.cpu_reps)
        line["cpu_baseline"] = {"value": T / best, "unit": UNIT, "cores": cores, "kind": kind,
                                "sample": "min of %d full block calls of the same workload (T=%d rows, layer 0) after one warm-up" % (done, T)}
        want = fn(xh, np.zeros_like(xh))
        got = torch.zeros_like(xs[0]); block.forward(desc, layers[0], xs[0], got); torch.cuda.synchronize()
        g = got.cpu().numpy()
        line["parity_rel_l2_vs_cpu"] = float(np.sqrt(((g - want) ** 2).sum() / (want ** 2).sum()))

    sampler.stop_flag = True
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
