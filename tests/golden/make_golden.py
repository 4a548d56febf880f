"""Generates tests/golden/*.npz from the reference's own code.

Run where the reference checkout exists (it builds oracle/_ref/ from the
reference sources in place and calls into it):

    python tests/golden/make_golden.py

Each fixture stores the complete inputs of one tiny MoE layer and the outputs the
reference produced for them: `ref_out` = hin + MoE(x) from moe_block()
(c/moe_block.h:18-54) in its exact (double-accumulate) mode, `ref_out_grouped` from
lag_moe_group (c/laguna.c:689-787) where the layer is expressible by the Laguna
glue, and kernel-level outputs of matmul_q4_kb / matmul_f32 / matmul_bf16_k /
softmax_row / moe_topk / quant_row_i4, and (fp4.npz) of matmul_fp4_kb (c/moe_quant.h:259-340)
and the clamped fp4 expert loop (c/deepseek.c:820-842).

    python tests/golden/make_golden.py fp4      # only that fixture
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from sabrewing_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
KEYS = ("router_w", "corr_bias", "logit_bias", "gu_q", "gu_s", "dn_q", "dn_s", "sh_gate", "sh_up", "sh_down")


def host_layer(cfg, a):
    return oracle.HostLayer(cfg.D, cfg.I, cfg.SI, cfg.E, cfg.K, cfg.route_act, cfg.use_corr_bias, cfg.norm_topk,
                            cfg.route_scale, cfg.shared_mode, cfg.gs, **{k: a.get(k) for k in KEYS})


CASES = {
    "laguna_tiny": (synth.scaled(synth.CONFIGS["c2"], D=128, E=16, K=4, I=64, SI=96, T=9, seed=11), 0.02),
    "olmoe_tiny": (synth.scaled(synth.CONFIGS["c1"], D=128, E=8, K=3, I=64, T=5, seed=12), 0.0),
    "zipf_tiny": (synth.scaled(synth.CONFIGS["c3"], D=128, E=32, K=6, I=64, SI=64, T=12, seed=13), 0.01),
    "wide_tiny": (synth.scaled(synth.CONFIGS["c5"], D=160, E=24, K=8, I=96, SI=32, T=7, seed=14), 0.0),
}


def make_fp4(ref):
    """e2m1 codes with ue8m0 exponents around 127 (and the two special bytes 0 and 0xFF)."""
    rng = np.random.default_rng(4242)
    I, O, S = 96, 20, 3
    q = rng.integers(0, 256, (O, I // 2), dtype=np.uint8)
    es = rng.integers(120, 132, (O, I // 32), dtype=np.uint8)
    es[3, 1] = 0; es[7, 0] = 0xFF
    x = rng.standard_normal((S, I), dtype=np.float32)
    k = dict(x=x, q=q, es=es, y_exact=ref.matmul_fp4(x, q, es, 1), y_simd=ref.matmul_fp4(x, q, es, 0))
    # fused experts: E=5 experts, D=64, I=32, K=3 given in a non-sorted order, limit small enough to clamp
    E, D, I2, lim = 5, 64, 32, 3.0
    gu_q = rng.integers(0, 256, (E * 2 * I2, D // 2), dtype=np.uint8)
    gu_es = rng.integers(124, 130, (E * 2 * I2, D // 32), dtype=np.uint8)
    dn_q = rng.integers(0, 256, (E * D, I2 // 2), dtype=np.uint8)
    dn_es = rng.integers(124, 130, (E * D, I2 // 32), dtype=np.uint8)
    xe = rng.standard_normal(D, dtype=np.float32)
    sel = np.array([4, 0, 2], np.int32); w = np.array([0.5, 0.3, 0.2], np.float32)
    k.update(e_x=xe, gu_q=gu_q, gu_es=gu_es, dn_q=dn_q, dn_es=dn_es, sel=sel, w=w, limit=np.float32(lim),
             e_exact=ref.experts_fp4(xe, gu_q, gu_es, dn_q, dn_es, sel, w, I2, D, lim, 1),
             e_simd=ref.experts_fp4(xe, gu_q, gu_es, dn_q, dn_es, sel, w, I2, D, lim, 0))
    np.savez_compressed(os.path.join(HERE, "fp4.npz"), **k)
    print("fp4", sorted(k))


def main():
    oracle.build()
    ref = oracle.load_ref()
    assert ref is not None, "reference checkout not available"
    if sys.argv[1:] == ["fp4"]:
        return make_fp4(ref)
    for name, (cfg, bstd) in CASES.items():
        a = synth.make_layer(cfg, corr_bias_std=bstd)
        x = synth.make_tokens(cfg)
        hin = np.random.default_rng(cfg.seed + 5).standard_normal(x.shape).astype(np.float32)
        L = host_layer(cfg, a)
        out = dict(cfg=np.array([cfg.D, cfg.E, cfg.K, cfg.I, cfg.SI, cfg.route_act, cfg.use_corr_bias, cfg.norm_topk,
                                 cfg.shared_mode, cfg.gs], np.int32),
                   route_scale=np.float32(cfg.route_scale), x=x, hin=hin)
        for k in KEYS:
            if a.get(k) is not None:
                out[k] = a[k]
        out["ref_out"] = ref.moe_block_rows(L, x, hin, exact=1)
        if cfg.route_act == 0 and cfg.shared_mode == 1 and a.get("logit_bias") is None:
            out["ref_out_grouped"] = ref.laguna_moe_rows(L, x, hin, exact=1, group_on=1)
            out["ref_out_pertoken"] = ref.laguna_moe_rows(L, x, hin, exact=1, group_on=0)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
        print(name, {k: v.shape for k, v in out.items() if hasattr(v, "shape") and v.ndim})

    # kernel-level vectors
    rng = np.random.default_rng(99)
    W = rng.standard_normal((24, 96), dtype=np.float32) * np.float32(0.02)
    x = rng.standard_normal((3, 96), dtype=np.float32)
    packed, scale = ref.quant_rows_i4(W)
    Wb = synth.f32_to_bf16(W)
    sc = rng.standard_normal(40).astype(np.float32)
    bias = (rng.standard_normal(40) * 0.1).astype(np.float32)
    k = dict(W=W, x=x, packed=packed, scale=scale,
             q4_exact=ref.matmul_q4(x, packed, scale, 1), q4_simd=ref.matmul_q4(x, packed, scale, 0),
             f32_exact=ref.matmul_f32(x, W, 1), bf16_w=Wb, bf16_exact=ref.matmul_bf16(x, Wb, 1),
             scores=sc, bias=bias, softmax=ref.softmax_row(sc), topk5=ref.topk(sc, None, 0, 5),
             topk5_bias=ref.topk(sc, bias, 1, 5), rms=ref.rmsnorm_rows(x))
    # group-scaled int4 (c/quant.h:167-202): gs=64 with a partial last group, and gs=16
    for gs, I in ((64, 200), (16, 96)):
        Wg = rng.standard_normal((6, I), dtype=np.float32) * np.float32(0.02)
        xg = rng.standard_normal((2, I), dtype=np.float32)
        pq, ps = synth.quant_rows_i4_grouped(Wg, gs)
        k["g%d_x" % gs] = xg; k["g%d_q" % gs] = pq; k["g%d_s" % gs] = ps
        k["g%d_y" % gs] = ref.matmul_i4_grouped(xg, pq, ps, gs)
    np.savez_compressed(os.path.join(HERE, "kernels.npz"), **k)
    print("kernels", sorted(k))
    make_fp4(ref)


if __name__ == "__main__":
    main()
