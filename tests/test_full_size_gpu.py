"""Parity at the UNSCALED benchmark configurations (the shapes, batch sizes and routing policies the headline
numbers are quoted on), through the C-ABI.

Layers are drawn directly in device memory (`synth.make_layer_device`, the generator of the bench) and copied to the
host for the CPU checker, so both sides read the same bytes.  Bars:
  * expert ids in rank order and all five dispatch arrays (gexp, gbeg, gcnt, grow, rowof) bit-exact on ALL rows
    against the checker's exact (double-accumulate) router, combine weights within 5e-7 relative;
  * outputs within 1e-3 relative L2 of the checker's exact f32 path: on all rows where the exact path finishes in
    seconds, else on a fixed subset of >= 64 rows (routing of all rows, experts of the subset through
    `experts_given_routing`, shared expert of the subset);
  * the expert kernels that ran are the ones the configuration is meant to exercise (sw_moe_last_path).
Each case reports the smallest top-k margin it saw: score[k-th] - score[(k+1)-th] of the biased selection scores.
Where that is far above one f32 ulp the bit-exact ids do not hang on a rounding coincidence.
"""
import numpy as np
import pytest
import torch

from conftest import rel_l2, LAYER_KEYS

pytestmark = pytest.mark.gpu

OUT_TOL = 1e-3
W_TOL = 5e-7

# (config, token rows, rows whose outputs are checked (0 = all), expected expert path, fp16 terms on the tcgen05 path)
CASES = [
    ("c1", 32, 0, 2, 2),       # OLMoE-shaped, softmax, no shared expert
    ("c2", 1, 0, 2, 2),        # Laguna-shaped decode batch 1
    ("c2", 32, 0, 2, 2),       # ... batch 32 (the headline)
    ("c2", 256, 0, 3, 2),      # ... batch 256: 10 rows per expert, tcgen05 path in its small-group geometry (32-row chunks)
    ("c2", 256, 0, 3, 1),
    ("c4", 256, 0, 2, 2),      # wide layer, 384 experts, decode batch 256
    ("c3", 4096, 64, 3, 2),    # prefill, Zipf-skewed routing: tcgen05 path, activations as two fp16 terms
    ("c3", 4096, 64, 3, 1),    # ... as one fp16 term (half the tensor work): same ids, output error reported
    ("c5", 1024, 64, 3, 2),    # very large layer, 16 rows per expert on one GPU: tcgen05 path
    ("c5", 1024, 64, 3, 1),
]


def _host_layer(cfg, arrays):
    import oracle
    a = {}
    for k in LAYER_KEYS:
        v = arrays.get(k)
        if v is None:
            a[k] = None
        else:
            v = v.cpu().numpy()
            a[k] = v.view(np.uint16) if v.dtype == np.int16 else v
    return oracle.HostLayer(cfg.D, cfg.I, cfg.SI, cfg.E, cfg.K, cfg.route_act, cfg.use_corr_bias, cfg.norm_topk,
                            cfg.route_scale, cfg.shared_mode, cfg.gs, **a)


def _min_margin(scores, bias, K):
    s = scores + (bias[None, :] if bias is not None else 0.0)
    part = -np.partition(-s, K, axis=1)[:, :K + 1]           # the K+1 largest of every row, unordered
    part.sort(axis=1)
    return float((part[:, 1] - part[:, 0]).min())           # k-th minus (k+1)-th


@pytest.mark.parametrize("name,T,subset,path,terms", CASES)
def test_full_size_config(orc, name, T, subset, path, terms):
    from sabrewing_b200 import synth, capi
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    cfg = synth.CONFIGS[name]
    arrays = synth.make_layer_device(cfg, "cuda:0", 0)
    if cfg.use_corr_bias:                                    # a selection bias that matters, as in the scaled cases
        g = torch.Generator(device="cuda:0"); g.manual_seed(cfg.seed + 11)
        arrays["corr_bias"] = torch.randn(cfg.E, generator=g, device="cuda:0") * 0.01
    host = _host_layer(cfg, arrays)
    layer = MoeLayer(cfg.D, cfg.I, cfg.SI, arrays, "cuda:0")
    del arrays
    desc = desc_from_config(cfg)
    x = synth.make_tokens(cfg, T)
    hin = np.random.default_rng(cfg.seed + 5).standard_normal(x.shape).astype(np.float32)

    blk = MoeBlock("cuda:0", T, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    assert blk.lib.sw_moe_set_option(blk.ctx, capi.OPT_UMMA_TERMS, terms) == 0
    xd = torch.from_numpy(x).cuda(); out = torch.from_numpy(hin).cuda()
    blk.forward(desc, layer, xd, out)
    torch.cuda.synchronize()
    assert blk.status() == 0
    assert blk.lib.sw_moe_last_path(blk.ctx) == path
    got = blk.routing()

    # routing and dispatch: every row, bit for bit
    sel, w, sc = orc.route(host, x, exact=1, want_scores=True)
    margin = _min_margin(sc, host.a.get("corr_bias") if cfg.use_corr_bias else None, cfg.K)
    note = "%s T=%d: min top-k margin %.3e" % (name, T, margin)
    print(note)
    assert np.array_equal(got["sel"], sel), note
    grp = orc.group(sel, cfg.E)
    assert got["G"] == grp["G"], note
    for k in ("gexp", "gbeg", "gcnt", "grow", "rowof"):
        assert np.array_equal(got[k], grp[k]), (k, note)
    werr = float((np.abs(got["w"] - w) / np.abs(w)).max())
    assert werr < W_TOL, (werr, note)

    # outputs
    rows = np.arange(T) if not subset else np.unique(np.linspace(0, T - 1, subset).astype(np.int64))
    xs = np.ascontiguousarray(x[rows])
    want = orc.experts_given_routing(host, xs, sel[rows], w[rows], exact=1) * np.float32(cfg.route_scale)
    if cfg.SI:
        want = want + orc.shared_rows(host, xs, exact=1)
    delta = out.cpu().numpy()[rows] - hin[rows]
    err = rel_l2(delta, want)
    print("%s T=%d: output rel-L2 %.3e on %d rows, path %d, fp16 terms %d" % (name, T, err, len(rows), path, terms))
    assert err < OUT_TOL, (err, note)
    if not subset and T <= 32:
        # the whole block in one call of the checker (residual included), as the scaled cases do
        full = orc.moe_group(host, x, hin, exact=1)
        assert np.array_equal(full["sel"], sel)
        assert rel_l2(out.cpu().numpy() - hin, full["out"] - hin) < OUT_TOL
    blk.close()


def test_device_quantiser_follows_the_reference_rule(orc):
    """The torch quantiser that fills the bench and full-size layers against the checker's quant_row_i4 twin
    (itself bit-equal to the reference's, c/tools/kernel_check.c:27-35): same scale, and codes equal except where
    w/scale sits on a rounding boundary (torch divides, the reference divides too, so in practice all)."""
    from sabrewing_b200 import synth
    cfg = synth.scaled(synth.CONFIGS["c2"], D=512, E=2, K=1, I=128, SI=128)
    # re-create the first expert's gate/up weights exactly as make_layer_device draws them
    g = torch.Generator(device="cuda:0"); g.manual_seed(cfg.seed * 1000003)
    _ = (torch.randn((cfg.E, cfg.D), generator=g, device="cuda:0") * 0.02)
    wdev = torch.randn((2 * cfg.I, cfg.D), generator=g, device="cuda:0") * 0.02
    arrays = synth.make_layer_device(cfg, "cuda:0", 0)
    q_dev = arrays["gu_q"][:2 * cfg.I].cpu().numpy(); s_dev = arrays["gu_s"][:2 * cfg.I].cpu().numpy()
    q_ref, s_ref = orc.quant_rows_i4(wdev.cpu().numpy())
    assert np.array_equal(s_dev, s_ref)
    mism = int((q_dev != q_ref).sum())
    assert mism <= q_ref.size // 100000 + 2, mism
