"""MoE-block benchmark: tokens/s of one Laguna-shaped MoE layer call at a decode batch.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
                    [--workload c1|c2|c3|c4|c5] [--batch T] [--layers L] [--no-sweep]

A step is one pass of the MoE block (route -> top-k -> group-by-expert -> int4
gate/up -> SiLU*up -> int4 down -> combine + shared expert) over one batch of T
synthetic token rows.  Steps cycle over L resident layers and 8 token batches so no
step finds its weights in L2.  N > 1 shards the experts over the ranks (one process
per GPU) with T rows per rank (weak scaling).  Prints one JSON line on rank 0.

At N = 1 the line's headline is the Laguna-shaped layer at decode batch 32; the same
process then measures the other batches of the metric (decode batch 1 and 256, the
4096-token prefill) and reports them in `sweep`, each with its own roofline entry and
end-to-end numbers, and times the reference's own CUDA tier (compiled unmodified for
sm_100a) against this library through the same lag_cuda_moe_group call (`gpu_baseline`).
"""
import argparse
import ctypes as C
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
NB = 8                       # token batches the steps cycle over
HBM_SPEC_GBS = 8000.0        # the part's nominal HBM3e bandwidth, quoted beside the measured copy bandwidth
# DRAM bytes (read + write) of one launch from ncu captures, as a ratio to that launch's algorithmic bytes:
# (workload, rows, stage) -> (ratio, the summary under profiles/ that holds the capture and its command)
NCU_TRAFFIC = {
    ("c2", 32, "q4_gateup"): (776.06 / 776.67, "profiles/q4_tma_c2_batch32.md"),
    ("c2", 32, "q4_down"): (395.97 / 389.0, "profiles/q4_tma_c2_batch32.md"),
    ("c2", 256, "q4_gateup"): ((1097.38 + 8.02) / 1090.52, "profiles/q4_umma_c2_batch256.md"),
    ("c3", 4096, "q4_gateup"): ((1421.16 + 83.80) / 1294.96, "profiles/q4_umma_c3_prefill.md"),
    ("c3", 4096, "q4_down"): ((622.61 + 631.14) / 1358.0, "profiles/q4_umma_c3_prefill.md"),
}


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
    ap.add_argument("--no-sweep", action="store_true", help="N=1: only the headline workload (no other batches, no GPU baseline)")
    ap.add_argument("--umma-terms", type=int, default=0, help="fp16 terms per activation on the tcgen05 path (0 = the library's default)")
    ap.add_argument("--ep-scheme", default="auto", choices=["auto", "replicate", "alltoall"],
                    help="N>1: exchange scheme (auto: replicate up to 256 rows per rank, all-to-all above)")
    ap.add_argument("--ep-python", action="store_true", help="N>1: drive the exchange from Python (three graph replays and two NCCL calls per step) instead of the in-library step")
    ap.add_argument("--no-graph", action="store_true", help="launch the kernels of every step one by one instead of replaying CUDA graphs")
    return ap.parse_args()


def workload_name(cfg, T, world):
    return "%s: D=%d E=%d top%d I=%d shared_I=%d, decode batch %d%s" % (
        cfg.name, cfg.D, cfg.E, cfg.K, cfg.I, cfg.SI, T, " per rank, experts sharded over %d ranks" % world if world > 1 else "")


def load_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


# ---------------------------------------------------------------------------
class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML while the bench runs."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, index, period=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.stop_flag = [], False
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
    # torchrun exports OMP_NUM_THREADS=1 and the reference's thread autotune honours it (c/moe_util.h:79): the CPU
    # arm is meant to use every physical core, so the variable is dropped before the library starts its team.
    os.environ.pop("OMP_NUM_THREADS", None)
    ref = oracle.load_ref()
    laguna_ok = cfg.route_act == 0 and cfg.shared_mode == 1 and cfg.gs == 0 and host.a.get("logit_bias") is None
    if ref is not None:
        ref.omp_autotune()                    # one thread per physical core, c/moe_util.h:78-87
        if ref.threads() < ref.physical_cores():
            ref.set_threads(ref.physical_cores())
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
    """The reference's own CPU path on the host cores, on the global batch of the repo arm (T rows per GPU x N)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from sabrewing_b200 import synth
    world = max(1, args.gpus)
    cfg = synth.CONFIGS[args.workload]
    T = (args.batch or cfg.T) * world
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
            "data": "synthetic", "config": {"workload": workload_name(cfg, args.batch or cfg.T, world), "global_batch": T},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind,
                             "sample": "every step = one full block call of the workload (T=%d rows = the global batch, one layer)" % T},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
def algorithmic_bytes(cfg, T, G):
    """Per-stage algorithmic bytes of one step with G distinct experts selected (weights once, rows in and out)."""
    P, D, I, SI, E = T * cfg.K, cfg.D, cfg.I, cfg.SI, cfg.E
    return {"q4_gateup": G * (I * D + 8 * I) + T * D * 4 + P * I * 4,
            "q4_down": G * (I * D // 2 + 4 * D) + P * I * 4 + P * D * 4,
            "shared_gateup": 2 * SI * D * 2 + T * D * 4 + T * SI * 4,
            "shared_down": SI * D * 2 + T * SI * 4 + T * D * 4,
            "router_logits": E * D * 2 + T * D * 4 + T * E * 4,
            "combine": P * D * 4 + 2 * T * D * 4, "route_topk": 2 * T * E * 4, "dispatch": 3 * P * 4}


def block_bytes(cfg, T, G):
    D, I, SI, E = cfg.D, cfg.I, cfg.SI, cfg.E
    return G * (1.5 * I * D + 8 * I + 4 * D) + (3 * SI * D * 2 if SI else 0) + E * D * 2 + 2 * T * D * 4


def block_flops(cfg, T):
    return T * cfg.K * 6.0 * cfg.I * cfg.D + (T * 6.0 * cfg.SI * cfg.D if cfg.SI else 0.0) + 2.0 * T * cfg.E * cfg.D


def roofline_entry(name, cfg, T, per, G, ms_per_step, peaks):
    """Roofline of the dominant stage (per-stage CUDA events) plus whole-block figures."""
    alg = algorithmic_bytes(cfg, T, G)
    dom = max(per, key=per.get)
    peak = float(peaks.get("hbm_gbs", 6650.0))
    tpeak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    src = "measured (MEASURED_PEAKS.json)" if peaks else "fallback"
    ach = alg[dom] / (per[dom] * 1e-3) / 1e9
    P = T * cfg.K
    flops = {"q4_gateup": 4.0 * P * cfg.I * cfg.D, "q4_down": 2.0 * P * cfg.I * cfg.D}
    tr = NCU_TRAFFIC.get((name, T, dom))
    r = {"bound": "hbm", "kernel": dom, "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
         "peak_source": src, "frac_of_spec_8TBs": ach / HBM_SPEC_GBS,
         "traffic": tr[0] * alg[dom] if tr else None,
         "traffic_source": ("ncu dram read+write bytes of one launch of this workload (%s) as a ratio to that launch's "
                            "algorithmic bytes, times this run's algorithmic bytes" % tr[1]) if tr else None,
         "algorithmic_bytes_per_launch": alg[dom], "kernel_ms": per[dom], "distinct_experts_per_step": G}
    # large groups: the expert GEMMs are bound by the tensor cores, not by HBM
    if dom in flops and flops[dom] / (tpeak * 1e12) > alg[dom] / (peak * 1e9):
        tach = flops[dom] / (per[dom] * 1e-3) / 1e12
        r.update({"bound": "tensor", "achieved": tach, "peak": tpeak, "unit": "TFLOP/s", "frac": tach / tpeak,
                  "algorithmic_flops_per_launch": flops[dom], "hbm_gbs_achieved": ach,
                  "peak_source": ("measured, sustained bf16 (MEASURED_PEAKS.json)" if peaks else "fallback")})
        r.pop("frac_of_spec_8TBs", None)
    exp_ms = per["q4_gateup"] + per["q4_down"]
    extra = {"int4_expert_gbs": G * (1.5 * cfg.I * cfg.D + 8 * cfg.I + 4 * cfg.D) / (exp_ms * 1e-3) / 1e9,
             "block_hbm_frac": block_bytes(cfg, T, G) / (ms_per_step * 1e-3) / 1e9 / peak,
             "block_tensor_frac": block_flops(cfg, T) / (ms_per_step * 1e-3) / 1e12 / tpeak,
             "stage_ms": {k: round(v, 5) for k, v in per.items()}}
    return r, extra


class Single:
    """One single-GPU workload: resident layers, token batches, a block and (optionally) a graph per step pattern."""

    umma_terms = 0           # 0: the library's default

    def __init__(self, name, cfg, T, layers, dev, use_graph=True):
        import numpy as np
        import torch
        from sabrewing_b200 import synth
        from sabrewing_b200.moe_block import MoeBlock, desc_from_config
        self.name, self.cfg, self.T, self.layers, self.dev = name, cfg, T, layers, dev
        self.desc = desc_from_config(cfg)
        self.xs_host = [torch.from_numpy(synth.make_tokens(cfg, T, seed_offset=1000 + i)).pin_memory() for i in range(NB)]
        self.xs = [x.to(dev) for x in self.xs_host]
        self.outs = [torch.zeros_like(x) for x in self.xs]
        self.block = MoeBlock(dev, T, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
        if Single.umma_terms:
            self.block._chk(self.block.lib.sw_moe_set_option(self.block.ctx, 1, Single.umma_terms), "sw_moe_set_option")
        self.graphs = {}
        if use_graph:
            L = len(layers)
            for li in range(L):
                for bi in range(NB):
                    if (li - bi) % np.gcd(L, NB) == 0:          # only the pairs (i % L, i % NB) that occur
                        self.graphs[(li, bi)] = self.block.graph(self.desc, layers[li], self.xs[bi], self.outs[bi])
            torch.cuda.synchronize()

    def step(self, i, use_graph=True):
        li, bi = i % len(self.layers), i % NB
        g = self.graphs.get((li, bi)) if use_graph else None
        if g is not None:
            g.replay()
        else:
            self.block.forward(self.desc, self.layers[li], self.xs[bi], self.outs[bi])

    def timed(self, steps, warmup):
        import torch
        for i in range(warmup):
            self.step(i)
        torch.cuda.synchronize()
        l0 = self.block.lib.sw_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_a = time.perf_counter()
        e0.record()
        for i in range(steps):
            self.step(i)
        e1.record()
        torch.cuda.synchronize()
        t_b = time.perf_counter()
        return e0.elapsed_time(e1), int(self.block.lib.sw_launch_count() - l0), t_a, t_b

    def stages(self, steps):
        """Per-stage ms (CUDA events between the kernels, eager launches) and the mean number of distinct experts."""
        import numpy as np
        import torch
        self.block.profile(True)
        for i in range(min(steps, 500)):
            self.step(i, use_graph=False)
        torch.cuda.synchronize()
        stage_ms, calls = self.block.profile_read()
        self.block.profile(False)
        Gs = []
        for i in range(min(NB * len(self.layers), 16)):
            self.block.route(self.desc, self.layers[i % len(self.layers)], self.xs[i % NB]); Gs.append(self.block.routing()["G"])
        return {k: v / max(calls, 1) for k, v in stage_ms.items()}, float(np.mean(Gs))

    def e2e(self, steps, pinned):
        """sw_moe_forward_host from host rows: H2D of x (and of the residual rows when they are page-locked), the block,
        D2H of the result and a stream sync inside every timed step."""
        import numpy as np
        import torch
        if pinned:
            hx = [x.numpy() for x in self.xs_host]
            keep = [torch.zeros_like(x).pin_memory() for x in self.xs_host]
            ho = [t.numpy() for t in keep]
        else:
            hx = [np.array(x.numpy(), copy=True) for x in self.xs_host]       # ordinary (pageable) allocations
            ho = [np.zeros_like(a) for a in hx]
        n = max(3, min(steps, 200))
        L = len(self.layers)
        for i in range(3):
            self.block.forward_host(self.desc, self.layers[i % L], hx[i % NB], ho[i % NB])
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(n):
            self.block.forward_host(self.desc, self.layers[i % L], hx[i % NB], ho[i % NB])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        nbytes = self.T * self.cfg.D * 4
        return {"value": self.T * n / dt, "unit": UNIT, "h2d_bytes_per_step": (2 if pinned else 1) * nbytes,
                "d2h_bytes_per_step": nbytes, "steps": n,
                "api": "sw_moe_forward_host, page-locked host rows (x up, residual rows up beside the kernels, residual + MoE(x) down; one sync per call)"
                if pinned else "sw_moe_forward_host, pageable host rows (staged through the context's page-locked buffers; MoE(x) down, residual added on the host)"}

    def close(self):
        for g in self.graphs.values():
            g.close()
        self.graphs = {}
        self.block.close()


def make_layers(cfg, dev, n, lo=0, cnt=0, want_host0=False):
    import torch
    from sabrewing_b200 import synth
    from sabrewing_b200.moe_block import MoeLayer
    layers, host0 = [], None
    for li in range(n):
        arrays = synth.make_layer_device(cfg, dev, li)
        if li == 0 and want_host0:
            host0 = host_layer_from(cfg, arrays)
        layers.append(MoeLayer(cfg.D, cfg.I, cfg.SI, arrays, dev, expert_lo=lo, expert_cnt=cnt))
        del arrays
    torch.cuda.empty_cache()
    return layers, host0


def sweep_entry(name, cfg, T, layers, dev, steps, warmup, peaks):
    """One more batch size of the metric, measured like the headline (device-resident, per-stage, end to end)."""
    w = Single(name, cfg, T, layers, dev)
    ms, launches, _, _ = w.timed(steps, warmup)
    per, G = w.stages(steps)
    roof, extra = roofline_entry(name, cfg, T, per, G, ms / steps, peaks)
    e = {"workload": workload_name(cfg, T, 1), "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
         "tokens_per_s": T * steps / (ms * 1e-3), "gpu_launches": launches, "expert_path": w.block.lib.sw_moe_last_path(w.block.ctx),
         "dominant_kernel": roof["kernel"], "frac": roof["frac"], "roofline": roof,
         "block_hbm_frac": extra["block_hbm_frac"], "block_tensor_frac": extra["block_tensor_frac"], "stage_ms": extra["stage_ms"],
         "e2e": w.e2e(steps, True), "e2e_pageable": w.e2e(steps, False)}
    w.close()
    return e


def gpu_baseline(cfg, T, host, x, steps):
    """The reference's own CUDA tier (c/backend_cuda_laguna.cu compiled unmodified for sm_100a) against this library
    through the SAME call, lag_cuda_moe_group (c/backend_cuda_laguna.h:70-75): host routing from the CPU checker,
    pageable host buffers, one blocking call per step, on the same GPU."""
    import numpy as np
    import oracle
    from sabrewing_b200 import capi
    if not os.path.exists(oracle.REF_CUDA_PATH):
        return {"unavailable": "oracle/_ref/libref_cuda_laguna.so was not built (no reference checkout at build time)"}
    orc = oracle.load()
    sel, w = orc.route(host, x, exact=1)
    grp = orc.group(sel, cfg.E)
    ref = C.CDLL(oracle.REF_CUDA_PATH)
    ours = capi.lib()
    vp, ci = C.c_void_p, C.c_int
    ref.lag_cuda_init.restype, ref.lag_cuda_init.argtypes = ci, [ci]
    ref.lag_cuda_upload.restype, ref.lag_cuda_upload.argtypes = vp, [vp, C.c_size_t]
    ref.lag_cuda_free.restype, ref.lag_cuda_free.argtypes = None, [vp]
    ref.lag_cuda_moe_group.restype, ref.lag_cuda_moe_group.argtypes = capi.SIGNATURES["lag_cuda_moe_group"]
    out = {}
    results = {}
    w = np.ascontiguousarray(w, np.float32)
    for tag, lib in (("reference_cuda", ref), ("ours", ours)):
        if lib.lag_cuda_init(0) != 0:
            return {"unavailable": "%s: lag_cuda_init failed" % tag}
        blobs = [lib.lag_cuda_upload(host.a[k].ctypes.data, host.a[k].nbytes) for k in ("gu_q", "gu_s", "dn_q", "dn_s")]
        if not all(blobs):
            return {"unavailable": "%s: upload failed" % tag}
        acc = np.zeros_like(x)

        def call():
            return lib.lag_cuda_moe_group(acc.ctypes.data, x.ctypes.data, blobs[0], blobs[1], blobs[2], blobs[3],
                                          grp["gexp"].ctypes.data, grp["gbeg"].ctypes.data, grp["gcnt"].ctypes.data, grp["G"],
                                          grp["grow"].ctypes.data, grp["rowof"].ctypes.data, w.ctypes.data, T, cfg.K, cfg.I, cfg.D)
        for _ in range(3):
            if call() != 0:
                return {"unavailable": "%s: lag_cuda_moe_group failed" % tag}
        t0 = time.perf_counter()
        for _ in range(steps):
            call()
        dt = time.perf_counter() - t0
        out[tag] = T * steps / dt
        results[tag] = acc.copy()
        for b in blobs:
            lib.lag_cuda_free(b)
    a, b = results["ours"].astype(np.float64), results["reference_cuda"].astype(np.float64)
    return {"value": out["reference_cuda"], "unit": UNIT, "kind": "reference-cuda", "ours_same_call": out["ours"],
            "call": "lag_cuda_moe_group, %s, pageable host buffers, host routing, blocking" % workload_name(cfg, T, 1),
            "steps": steps, "rel_l2_ours_vs_reference_cuda": float(np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-300))),
            "note": "same layer (one of one), same rows every step: the reference's SIMT kernels read the weights of the "
                    "~185 selected experts from HBM each call, as this library does"}


# ---------------------------------------------------------------------------
def run_single(args):
    import numpy as np
    import torch
    from sabrewing_b200 import synth, capi
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    capi.lib()
    peaks = load_peaks()
    cfg = synth.CONFIGS[args.workload]
    T = args.batch or cfg.T
    Single.umma_terms = args.umma_terms
    sampler = ClockSampler(0)
    sampler.start()

    layers, host0 = make_layers(cfg, dev, args.layers, want_host0=not args.no_cpu_baseline)
    w = Single(args.workload, cfg, T, layers, dev, use_graph=not args.no_graph)
    ms, launches, t_a, t_b = w.timed(args.steps, args.warmup)
    clocks = sampler.summary(t_a, t_b)
    line = {"metric": METRIC, "value": T * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 activations x int4 weights (f32 accumulate)", "data": "synthetic",
            "config": {"workload": workload_name(cfg, T, 1), "global_batch": T, "layers_cycled": len(layers),
                       "l2": "inputs larger than L2: steps cycle over %d layers (%.2f GB of expert blobs each per GPU) and %d token batches"
                             % (len(layers), layers[0].expert_bytes() / 1e9, NB),
                       "parallelism": "single", "launch": "cuda graph replay per step" if w.graphs else "one launch per kernel"},
            "clocks": clocks, "gpu_launches": launches}
    per, G = w.stages(args.steps)
    line["roofline"], extra = roofline_entry(args.workload, cfg, T, per, G, ms / args.steps, peaks)
    line.update(extra)
    line["expert_path"] = w.block.lib.sw_moe_last_path(w.block.ctx)
    line["e2e"] = w.e2e(args.steps, True)
    line["e2e_pageable"] = w.e2e(args.steps, False)

    # ---- CPU baseline on the host cores: the reference's own CPU code on the same layer ----
    if host0 is not None:
        kind, cores, fn = cpu_step_fn(cfg, host0)
        xh = w.xs_host[0].numpy()
        best, done = time_cpu(fn, xh, args.cpu_reps)
        line["cpu_baseline"] = {"value": T / best, "unit": UNIT, "cores": cores, "kind": kind,
                                "sample": "min of %d full block calls of the same workload (T=%d rows, layer 0) after one warm-up" % (done, T)}
        want = fn(xh, np.zeros_like(xh))
        got = torch.zeros_like(w.xs[0]); w.block.forward(w.desc, layers[0], w.xs[0], got); torch.cuda.synchronize()
        g = got.cpu().numpy()
        line["parity_rel_l2_vs_cpu"] = float(np.sqrt(((g - want) ** 2).sum() / (want ** 2).sum()))
    w.close()

    # ---- the other batches of the metric, same process ----
    if not args.no_sweep and args.workload == "c2" and T == 32:
        sweep = {}
        try:
            sweep["c2_b1"] = sweep_entry("c2", cfg, 1, layers, dev, max(args.steps, 50), max(args.warmup, 5), peaks)
            sweep["c2_b256"] = sweep_entry("c2", cfg, 256, layers, dev, max(3, min(args.steps, 100)), max(args.warmup, 3), peaks)
        except Exception as e:
            sweep["error"] = str(e)[:200]
        # the reference's CUDA tier on this GPU, through the same C call (weights of layer 0)
        try:
            if host0 is not None:
                line["gpu_baseline"] = gpu_baseline(cfg, T, host0, np.array(w.xs_host[0].numpy(), copy=True), max(3, min(args.steps, 30)))
        except Exception as e:
            line["gpu_baseline"] = {"unavailable": "error: " + str(e)[:160]}
        del layers, w
        torch.cuda.empty_cache()
        try:
            c3 = synth.CONFIGS["c3"]
            l3, _ = make_layers(c3, dev, 2)
            sweep["c3_b4096"] = sweep_entry("c3", c3, c3.T, l3, dev, max(3, min(args.steps, 30)), max(args.warmup, 3), peaks)
            del l3
        except Exception as e:
            sweep["c3_error"] = str(e)[:200]
        line["sweep"] = sweep
    sampler.stop_flag = True
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------
def run_parallel(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from sabrewing_b200 import synth, capi
    from sabrewing_b200.moe_block import MoeBlock, desc_from_config
    from sabrewing_b200.ep import ExpertParallelMoe, shard_range

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    capi.lib()
    peaks = load_peaks()
    cfg = synth.CONFIGS[args.workload]
    T = args.batch or cfg.T
    desc = desc_from_config(cfg)
    lo, cnt = shard_range(cfg.E, world, rank)
    sampler = ClockSampler(local)
    sampler.start()

    layers, _ = make_layers(cfg, dev, args.layers, lo=lo, cnt=cnt)
    xs_host = [torch.from_numpy(synth.make_tokens(cfg, T, seed_offset=1000 + 97 * rank + i)).pin_memory() for i in range(NB)]
    xs = [x.to(dev) for x in xs_host]
    outs = [torch.zeros_like(x) for x in xs]
    block = MoeBlock(dev, T * world, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    scheme = args.ep_scheme if args.ep_scheme != "auto" else ("replicate" if T <= 256 else "alltoall")
    ep = ExpertParallelMoe(block, desc, scheme=scheme)
    native = not args.ep_python
    if native:
        ep.native_init(T, cfg.D, dev)                 # the step is one call into the library, NCCL enqueued there
    # (Python exchange) this rank's kernels of a step as three graphs per (layer, batch) pair; the collectives stay NCCL calls
    if not native and not args.no_graph and scheme == "replicate":
        try:
            for li in range(len(layers)):
                for bi in range(NB):
                    if (li - bi) % np.gcd(len(layers), NB) == 0:
                        ep.prepare(layers[li], xs[bi], outs[bi])
        except Exception as e:                                  # every rank runs the same code: all fall back together
            print("stage capture failed (%s); launching the kernels one by one" % e, file=sys.stderr, flush=True)
            ep._graphs.clear()
        torch.cuda.synchronize()

    def step(i):
        ep.forward(layers[i % len(layers)], xs[i % NB], outs[i % NB])

    def barrier():
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
    t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    clocks = sampler.summary(t_a, t_b)
    line = {"metric": METRIC, "value": T * world * args.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 activations x int4 weights (f32 accumulate)", "data": "synthetic",
            "config": {"workload": workload_name(cfg, T, world), "global_batch": T * world, "layers_cycled": len(layers),
                       "l2": "inputs larger than L2: steps cycle over %d layers (%.2f GB of expert blobs each per GPU) and %d token batches"
                             % (len(layers), layers[0].expert_bytes() / 1e9, NB),
                       "parallelism": "ep%d" % world, "exchange": scheme,
                       "launch": ("one library call per step (sw_ep_forward: kernels and NCCL collectives enqueued by the library)" if native else
                                  "three graph replays and two NCCL calls per step" if ep._graphs else "one launch per kernel")},
            "clocks": clocks, "gpu_launches": int(launches)}

    # ---- where a step's time goes: CUDA events around the five segments (max over ranks of each segment's mean) ----
    try:
        if native:
            seg, nseg = {}, min(args.steps, 50)
            for i in range(nseg):
                ep.native_forward(layers[i % len(layers)], xs[i % NB], outs[i % NB], timed=True)
                torch.cuda.synchronize()
                for k, v in ep.native_segments().items():
                    seg[k] = seg.get(k, 0.0) + v / nseg
        else:
            seg = ep.timed_segments(layers, xs, outs, min(args.steps, 50))
        names = sorted(seg)
        tt = torch.tensor([seg[k] for k in names], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        line["segment_ms"] = {k: round(float(v), 5) for k, v in zip(names, tt.tolist())}
    except Exception as e:
        line["segment_ms"] = {"error": str(e)[:160]}

    # ---- rows and int4 bytes per GPU of one step (imbalance = max / mean rows per GPU) ----
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
        hbm = float(peaks.get("hbm_gbs", 6650.0))
        gbs = [e * per_expert / (line["ms_per_step"] * 1e-3) / 1e9 for e in exps]
        line["expert_parallel"] = {"rows_per_gpu": rows, "distinct_experts_per_gpu": exps,
                                   "imbalance": max(rows) / (sum(rows) / world) if sum(rows) else None,
                                   "int4_gbs_per_gpu": gbs, "hbm_frac_per_gpu": [g / hbm for g in gbs]}
    except Exception as e:                      # a reporting extra: never lose the bench line over it
        line["expert_parallel"] = {"error": str(e)[:120]}

    # ---- end to end: every rank copies its rows in from pinned memory and its result back out each step ----
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

    # ---- strong-scaling reference point: the same GLOBAL batch on one GPU holding all experts (rank 0 alone) ----
    ep.close()
    del ep, block, layers
    torch.cuda.empty_cache()
    barrier()
    if rank == 0:
        try:
            full, _ = make_layers(cfg, dev, 2)
            w1 = Single(args.workload, cfg, T * world, full, dev)
            n1 = max(3, min(args.steps, 50))
            ms1, _, _, _ = w1.timed(n1, 3)
            w1.close()
            line["strong_scaling"] = {"single_gpu_ms_per_step_same_global_batch": ms1 / n1,
                                      "speedup_over_single_gpu": (ms1 / n1) / line["ms_per_step"], "gpus": world,
                                      "note": "one GPU with all experts resident running the global batch of %d rows, same kernels" % (T * world)}
        except Exception as e:
            line["strong_scaling"] = {"error": str(e)[:160]}
    barrier()
    sampler.stop_flag = True
    if rank == 0:
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    elif int(os.environ.get("WORLD_SIZE", "1")) > 1:
        run_parallel(a)
    else:
        run_single(a)
