"""Parity of the CUDA path (through the C-ABI) against the CPU checker and the reference goldens.

Bars: expert ids, weights' order and every dispatch array bit-exact; combine weights
within 2 ulp-level relative error; outputs within 1e-3 relative L2 of the reference's
exact f32 path (the tolerance of the task statement; measured values are ~1e-6).
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import load_golden, synth_case, rel_l2

pytestmark = pytest.mark.gpu

OUT_TOL = 1e-3       # relative L2 bar for outputs
W_TOL = 5e-7         # relative bar for combine weights (f32 ulp level)


def make_block(case, max_tokens=None):
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    cfg = case.cfg
    blk = MoeBlock("cuda:0", max_tokens or max(case.x.shape[0], 1), cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, "cuda:0", gs=cfg.gs)
    return blk, layer, desc_from_config(cfg)


def check_routing(got, want):
    assert np.array_equal(got["sel"], want["sel"])
    assert got["G"] == want["G"]
    for k in ("gexp", "gbeg", "gcnt", "grow", "rowof"):
        assert np.array_equal(got[k], want[k]), k
    werr = np.abs(got["w"] - want["w"])
    assert (werr <= W_TOL * np.abs(want["w"])).all(), werr.max()      # a saturated gate gives exact zeros on both sides


def run_case(case, orc, ref_out=None, path=None):
    blk, layer, desc = make_block(case)
    x = torch.from_numpy(case.x).cuda(); out = torch.from_numpy(case.hin).cuda()
    assert blk.lib.sw_moe_last_path(blk.ctx) == -1
    blk.forward(desc, layer, x, out)
    torch.cuda.synchronize()
    assert blk.status() == 0
    if path is not None:                  # the expert kernels that ran: 0 CUDA cores, 1 mma.sync, 2 TMA, 3 tcgen05
        assert blk.lib.sw_moe_last_path(blk.ctx) == path
    want = orc.moe_group(case.host, case.x, case.hin, exact=1)
    check_routing(blk.routing(), want)
    err = rel_l2(out.cpu().numpy() - case.hin, want["out"] - case.hin)
    assert err < OUT_TOL, err
    if ref_out is not None:
        assert rel_l2(out.cpu().numpy() - case.hin, ref_out - case.hin) < OUT_TOL
    # the host-buffer entry point gives the same bits as the device one
    oh = case.hin.copy()
    blk.forward_host(desc, layer, case.x, oh)
    assert np.array_equal(oh, out.cpu().numpy())
    blk.close()
    return err


@pytest.mark.parametrize("name", ["laguna_tiny", "olmoe_tiny", "zipf_tiny", "wide_tiny"])
def test_golden_fixtures(orc, name):
    case, z = load_golden(name)
    run_case(case, orc, z["ref_out"])


@pytest.mark.parametrize("base,kw,T", [
    ("c1", dict(D=512, I=256), 32),                      # OLMoE-shaped: softmax, no shared
    ("c2", dict(D=1024, I=256, SI=256), 1),              # Laguna-shaped decode batch 1
    ("c2", dict(D=1024, I=256, SI=256), 32),             # ... batch 32
    ("c2", dict(D=512, I=128, SI=128, route_act=2), 8),  # softplus gate variant
    ("c3", dict(D=512, I=128, SI=128), 300),             # Zipf-skewed, ragged group sizes
    ("c4", dict(D=640, I=192), 64),                      # 384 experts, softmax
    ("c5", dict(D=512, I=128, SI=128), 50),              # 512 experts + shared
    ("c2", dict(D=512, E=16, K=4, I=128, SI=128), 40),   # ~10 rows per expert: several passes over a group
    ("c3", dict(D=512, E=16, K=4, I=256, SI=128), 45),   # the same under the Zipf bias: groups from 1 to over 16 rows
    ("c2", dict(D=256, E=8, K=1, I=128, SI=128), 13),    # top-1
    ("c1", dict(D=256, E=8, K=8, I=128), 5),             # every expert selected, softmax
    ("c2", dict(D=384, E=12, K=3, I=128, SI=64), 7),     # D, experts not multiples of 128 / 8
])
def test_scaled_configs(orc, base, kw, T):
    case = synth_case(base, corr_bias_std=0.01, T=T, **kw)
    run_case(case, orc)


@pytest.mark.parametrize("base,kw,T", [
    ("c3", dict(D=512, I=256, SI=128, E=32, K=4), 512),      # Zipf-skewed: groups from a few rows to several 128-row chunks
    ("c5", dict(D=512, I=128, SI=128, E=64, K=8), 160),      # ~20 rows per expert: 32-row tiles
    ("c1", dict(D=256, I=128, E=8, K=2), 700),                # softmax, no shared, 175 rows per expert
])
def test_large_groups_take_the_tensor_memory_path(orc, base, kw, T):
    """Groups averaging >= 8 rows (with I % 128 == 0 and D % 256 == 0) run the tcgen05/TMEM grouped GEMM; same parity bars."""
    case = synth_case(base, corr_bias_std=0.01, T=T, **kw)
    assert T * case.cfg.K >= 16 * case.cfg.E and case.cfg.I % 128 == 0 and case.cfg.D % 256 == 0
    run_case(case, orc, path=3)


@pytest.mark.parametrize("gs,kw", [(64, dict(D=256, I=128, SI=64, E=16, K=4)), (128, dict(D=512, I=256, SI=64, E=16, K=4)),
                                   (64, dict(D=160, I=96, SI=32, E=8, K=2))])       # last: partial final groups
def test_group_scaled_int4(orc, gs, kw):
    """One scale per gs columns (the reference's fmt=4 container, c/quant.h:167-202), checked against the CPU checker."""
    case = synth_case("c2", corr_bias_std=0.01, T=21, gs=gs, **kw)
    run_case(case, orc, path=0)


def test_graph_replay_matches_eager(orc):
    case = synth_case("c2", D=512, E=64, K=6, I=128, SI=128, T=12)
    blk, layer, desc = make_block(case)
    x = torch.from_numpy(case.x).cuda()
    eager = torch.from_numpy(case.hin).cuda(); blk.forward(desc, layer, x, eager)
    out = torch.zeros_like(x)
    g = blk.graph(desc, layer, x, out)          # runs the block twice on `out`
    out.copy_(torch.from_numpy(case.hin).cuda())
    l0 = blk.lib.sw_launch_count()
    g.replay()
    torch.cuda.synchronize()
    assert blk.lib.sw_launch_count() - l0 >= 8   # the replay launched the block's kernels
    assert torch.equal(out, eager)
    check_routing(blk.routing(), orc.moe_group(case.host, case.x, None, exact=1))
    g.close(); blk.close()


def test_f32_router_weights(orc):
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    case = synth_case("c2", D=256, E=64, K=6, I=64, SI=64, T=19)
    cfg = case.cfg
    blk = MoeBlock("cuda:0", 19, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, "cuda:0", router="f32")
    x = torch.from_numpy(case.x).cuda(); out = torch.zeros_like(x)
    blk.forward(desc_from_config(cfg), layer, x, out)
    check_routing(blk.routing(), orc.moe_group(case.host, case.x, None, exact=1))


def test_ties_and_nonfinite_router(orc):
    # zero router weights: every score equal -> ties to the lower id; bias decides selection only
    case = synth_case("c2", D=128, E=32, K=5, I=64, SI=64, T=4)
    case.a["router_w"][:] = 0; case.a["router_bf16"][:] = 0
    case.a["corr_bias"][:] = 0; case.a["corr_bias"][[7, 21]] = 0.25
    run_case(case, orc)
    blk, layer, desc = make_block(case)
    x = torch.from_numpy(case.x).cuda(); x[1, 3] = float("nan")      # poisons every logit of row 1
    blk.route(desc, layer, x)
    r = blk.routing()
    assert r["sel"][0].tolist() == [7, 21, 0, 1, 2]
    assert r["sel"][1].tolist() == [0, 1, 2, 3, 4]                   # degraded selection, c/moe_arch.h:75-86
    assert blk.status() == 0


def test_empty_and_oversized_batches():
    from sabrewing_b200 import capi
    case = synth_case("c1", D=128, E=8, K=2, I=64, T=3)
    blk, layer, desc = make_block(case, max_tokens=4)
    x = torch.zeros((0, 128), device="cuda"); out = torch.zeros((0, 128), device="cuda")
    blk.forward(desc, layer, x, out)                                 # T=0 is a no-op
    x5 = torch.zeros((5, 128), device="cuda")
    with pytest.raises(RuntimeError, match="outside"):
        blk.forward(desc, layer, x5, torch.zeros_like(x5))
    d = desc.c(); d.shared_mode = 2; l = layer.c()
    x3 = torch.zeros((3, 128), device="cuda")
    assert blk.lib.sw_moe_forward(blk.ctx, C.byref(d), C.byref(l), x3.data_ptr(), x3.data_ptr(), 3, None) == -1
    assert "not wired" in capi.last_error()


def test_expert_parallel_shards_sum_to_the_whole(orc):
    """Each shard computes only pairs of its resident experts; the shard sums add up to the routed sum."""
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    case = synth_case("c4", D=256, E=48, K=8, I=96, T=40)
    cfg = case.cfg; desc = desc_from_config(cfg)
    x = torch.from_numpy(case.x).cuda()
    want = orc.moe_group(case.host, case.x, None, exact=1)
    for shards in (1, 2, 4, 8):
        total = torch.zeros_like(x)
        per = cfg.E // shards
        for r in range(shards):
            blk = MoeBlock("cuda:0", 40, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
            layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, "cuda:0", expert_lo=r * per, expert_cnt=per)
            blk.route(desc, layer, x)
            part = torch.empty_like(x)
            blk.experts(desc, layer, x, part)
            total += part
            check_routing(blk.routing(), want)
            blk.close()
        assert rel_l2(total.cpu().numpy(), want["routed"]) < OUT_TOL


# ---- lag_cuda_* drop-in tier: the reference's own GPU self-test bars (c/laguna.c:1565-1662) ----
def _lag():
    from sabrewing_b200 import capi
    l = capi.lib()
    assert l.lag_cuda_init(0) == 0
    return l


def _up(l, a):
    p = l.lag_cuda_upload(a.ctypes.data, a.nbytes)
    assert p
    return p


def test_lag_known_answer_nibbles():
    l = _lag()
    # c/tests/test_backend_cuda.cu:42,105-110, zero-padded to one 32-column unit (nibble 8 = value 0)
    x = np.zeros((1, 32), np.float32); x[0, :4] = [1, -2, 3, -4]
    q = np.full((2, 16), 0x88, np.uint8); q[0, :2] = [0x70, 0xf8]; q[1, :2] = [0xa9, 0xcb]
    s = np.array([1.0, 0.25], np.float32)
    y = np.empty((1, 2), np.float32)
    dq, ds = _up(l, q), _up(l, s)
    assert l.lag_cuda_matmul_q4(y.ctypes.data, x.ctypes.data, dq, ds, 1, 32, 2) == 0
    assert y.tolist() == [[-34.0, -2.5]]
    l.lag_cuda_free(dq); l.lag_cuda_free(ds)


def test_lag_matmuls_match_cpu(orc):
    l = _lag()
    rng = np.random.default_rng(1234)
    I, O = 3072, 2048
    x = (rng.random((3, I), dtype=np.float32) * 2 - 1)
    p = rng.integers(0, 256, (O, I // 2), dtype=np.uint8)
    sc = (0.01 + rng.random(O, dtype=np.float32) * 0.05).astype(np.float32)
    y = np.empty((3, O), np.float32)
    dp, ds = _up(l, p), _up(l, sc)
    assert l.lag_cuda_matmul_q4(y.ctypes.data, x.ctypes.data, dp, ds, 3, I, O) == 0
    yc = orc.matmul_q4(x, p, sc, 1)
    assert (np.abs(y - yc) / (np.abs(yc) + 1e-6)).max() < 1e-3          # the reference's q4 bar
    l.lag_cuda_free(dp); l.lag_cuda_free(ds)
    # bf16 residents
    from sabrewing_b200 import synth
    Wb = synth.f32_to_bf16(rng.random((O, I), dtype=np.float32) * 2 - 1)
    dW = _up(l, Wb)
    assert l.lag_cuda_matmul_bf16(y.ctypes.data, x.ctypes.data, dW, 3, I, O) == 0
    yc = orc.matmul_bf16(x, Wb, 1)
    assert (np.abs(y - yc) / (np.abs(yc) + 1e-6)).max() < 5e-3          # the reference's bf16 bar
    l.lag_cuda_free(dW)
    # int8 residents: [int8 O*I][f32 scale O]
    q8 = rng.integers(-127, 128, (O, I), dtype=np.int8)
    blob = np.concatenate([q8.reshape(-1).view(np.uint8), sc.view(np.uint8)])
    dW = _up(l, blob)
    assert l.lag_cuda_matmul_q8(y.ctypes.data, x.ctypes.data, dW, 3, I, O) == 0
    yc = (x.astype(np.float64) @ q8.astype(np.float64).T) * sc
    assert rel_l2(y, yc) < 1e-5
    l.lag_cuda_free(dW)


def test_lag_fp4_golden_and_selftest_bars(orc):
    """The fp4 pair: committed reference fixtures, then the reference self-test's two cases with its bars
    (c/deepseek.c:1500-1590: matmul max_rel < 1e-3, fused K experts L2rel < 1e-5)."""
    import os
    import conftest
    l = _lag()
    z = np.load(os.path.join(conftest.GOLDEN, "fp4.npz"))
    x, q, es = z["x"], z["q"], z["es"]
    y = np.empty_like(z["y_exact"])
    dq, de = _up(l, q), _up(l, es)
    assert l.lag_cuda_matmul_fp4(y.ctypes.data, x.ctypes.data, dq, de, x.shape[0], x.shape[1], q.shape[0]) == 0
    assert rel_l2(y, z["y_exact"]) < 1e-6
    l.lag_cuda_free(dq); l.lag_cuda_free(de)
    D, I = z["gu_q"].shape[1] * 2, z["dn_q"].shape[1] * 2
    d = [_up(l, z[k]) for k in ("gu_q", "gu_es", "dn_q", "dn_es")]
    out = np.empty(D, np.float32)
    sel = np.ascontiguousarray(z["sel"]); w = np.ascontiguousarray(z["w"])
    assert l.lag_cuda_moe_experts_fp4(out.ctypes.data, z["e_x"].ctypes.data, *d, sel.ctypes.data, w.ctypes.data,
                                      len(sel), I, D, float(z["limit"])) == 0
    assert rel_l2(out, z["e_exact"]) < 1e-5
    for p in d:
        l.lag_cuda_free(p)

    # the reference's self-test shapes: I=2048, D=4096, E=4, K=3, limit 10, exponents 120..131
    rng = np.random.default_rng(1234)
    I, D, E, lim = 2048, 4096, 4, 10.0
    gu = rng.integers(0, 256, (E * 2 * I, D // 2), dtype=np.uint8)
    gue = rng.integers(120, 132, (E * 2 * I, D // 32), dtype=np.uint8)
    dn = rng.integers(0, 256, (E * D, I // 2), dtype=np.uint8)
    dne = rng.integers(120, 132, (E * D, I // 32), dtype=np.uint8)
    x = (rng.random((1, D), dtype=np.float32) * 2 - 1)
    d = [_up(l, a) for a in (gu, gue, dn, dne)]
    got = np.empty((1, 2 * I), np.float32)
    assert l.lag_cuda_matmul_fp4(got.ctypes.data, x.ctypes.data, d[0], d[1], 1, D, 2 * I) == 0
    want = orc.matmul_fp4(x, gu[:2 * I], gue[:2 * I], 1)
    assert (np.abs(got - want) / (np.abs(want) + 1e-6)).max() < 1e-3
    # several rows in one call
    x3 = (rng.random((3, D), dtype=np.float32) * 2 - 1)
    got3 = np.empty((3, 2 * I), np.float32)
    assert l.lag_cuda_matmul_fp4(got3.ctypes.data, x3.ctypes.data, d[0], d[1], 3, D, 2 * I) == 0
    assert rel_l2(got3, orc.matmul_fp4(x3, gu[:2 * I], gue[:2 * I], 1)) < 1e-6
    sel = np.array([0, 2, 3], np.int32); w = np.array([0.5, 0.3, 0.2], np.float32)
    out = np.empty(D, np.float32)
    assert l.lag_cuda_moe_experts_fp4(out.ctypes.data, x.ctypes.data, *d, sel.ctypes.data, w.ctypes.data, 3, I, D, lim) == 0
    want = orc.experts_fp4(x[0], gu, gue, dn, dne, sel, w, I, D, lim, 1)
    assert rel_l2(out, want) < 1e-5
    # K = 0 gives zeros; a width that is not a multiple of 32 is refused
    assert l.lag_cuda_moe_experts_fp4(out.ctypes.data, x.ctypes.data, *d, sel.ctypes.data, w.ctypes.data, 0, I, D, lim) == 0
    assert not out.any()
    assert l.lag_cuda_matmul_fp4(got.ctypes.data, x.ctypes.data, d[0], d[1], 1, D - 16, 8) == -1
    for p in d:
        l.lag_cuda_free(p)


def test_lag_grouped_is_bit_identical_to_per_token(orc):
    """moe_group vs moe_experts on overlapping selections: max|diff| must be exactly 0."""
    l = _lag()
    rng = np.random.default_rng(7)
    D, I, E, S, K = 3072, 1024, 6, 4, 3
    sel = np.array([[0, 1, 2], [1, 2, 3], [0, 2, 4], [2, 3, 5]], np.int32)
    x = (rng.random((S, D), dtype=np.float32) * 2 - 1)
    w = (0.05 + rng.random((S, K), dtype=np.float32) * 0.3).astype(np.float32)
    p13 = rng.integers(0, 256, (E * 2 * I, D // 2), dtype=np.uint8)
    p2 = rng.integers(0, 256, (E * D, I // 2), dtype=np.uint8)
    s13 = (0.01 + rng.random(E * 2 * I, dtype=np.float32) * 0.03).astype(np.float32)
    s2 = (0.01 + rng.random(E * D, dtype=np.float32) * 0.03).astype(np.float32)
    d13, ds13, d2, ds2 = _up(l, p13), _up(l, s13), _up(l, p2), _up(l, s2)
    yref = np.empty((S, D), np.float32); ygrp = np.empty((S, D), np.float32)
    for s in range(S):
        assert l.lag_cuda_moe_experts(yref[s].ctypes.data, x[s].ctypes.data, d13, ds13, d2, ds2,
                                      sel[s].ctypes.data, w[s].ctypes.data, K, I, D) == 0
    g = orc.group(sel, E)
    assert l.lag_cuda_moe_group(ygrp.ctypes.data, x.ctypes.data, d13, ds13, d2, ds2,
                                g["gexp"].ctypes.data, g["gbeg"].ctypes.data, g["gcnt"].ctypes.data, g["G"],
                                g["grow"].ctypes.data, g["rowof"].ctypes.data, w.ctypes.data, S, K, I, D) == 0
    assert np.abs(yref - ygrp).max() == 0.0
    # and both agree with the CPU path
    import oracle
    L = oracle.HostLayer(D, I, 0, E, K, 0, 0, 0, 1.0, 0, 0, gu_q=p13, gu_s=s13, dn_q=p2, dn_s=s2)
    want = orc.experts_given_routing(L, x, sel, w, exact=1)
    assert rel_l2(ygrp, want) < OUT_TOL
    # fused single expert: max|abs| < 1e-3 (the reference's bar for the chained q4->silu->q4)
    y1 = np.empty(D, np.float32)
    assert l.lag_cuda_expert_q4(y1.ctypes.data, x[0].ctypes.data, d13, ds13, d2, ds2, I, D) == 0
    w1 = orc.experts_given_routing(oracle.HostLayer(D, I, 0, E, 1, 0, 0, 0, 1.0, 0, 0, gu_q=p13, gu_s=s13, dn_q=p2, dn_s=s2),
                                   x[:1], np.zeros((1, 1), np.int32), np.ones((1, 1), np.float32), exact=1)
    assert np.abs(y1 - w1[0]).max() < 1e-3
    for d in (d13, ds13, d2, ds2):
        l.lag_cuda_free(d)


def test_lag_rejects_odd_shapes():
    l = _lag()
    y = np.zeros(8, np.float32)
    assert l.lag_cuda_matmul_q4(y.ctypes.data, y.ctypes.data, None, None, 1, 6, 2) == -1   # caller falls back to CPU


def test_shared_stage_ahead_of_finish(orc):
    """sw_moe_shared on a second stream, then finish: same result as the one-call block."""
    case = synth_case("c2", D=512, E=32, K=4, I=128, SI=128, T=24)
    blk, layer, desc = make_block(case)
    x = torch.from_numpy(case.x).cuda()
    want = torch.from_numpy(case.hin).cuda(); blk.forward(desc, layer, x, want)
    out = torch.from_numpy(case.hin).cuda()
    routed = torch.empty_like(x)
    side, cur = torch.cuda.Stream(), torch.cuda.current_stream()
    side.wait_stream(cur)
    with torch.cuda.stream(side):
        blk.shared(desc, layer, x)
    blk.route(desc, layer, x)
    blk.experts(desc, layer, x, routed)
    cur.wait_stream(side)
    blk.finish(desc, layer, x, routed, out)
    torch.cuda.synchronize()
    assert rel_l2(out.cpu().numpy(), want.cpu().numpy()) < 1e-6
    # a finish without a preceding shared() computes the shared expert itself
    out2 = torch.from_numpy(case.hin).cuda()
    blk.finish(desc, layer, x, routed, out2)
    torch.cuda.synchronize()
    assert torch.equal(out2, out)
    blk.close()


def test_forward_host_pinned_and_pageable_agree(orc):
    """forward_host takes page-locked buffers directly (residual uploaded beside the kernels) and stages pageable ones."""
    case = synth_case("c2", D=1024, E=32, K=4, I=128, SI=128, T=64)      # 256 KB of rows: above the copy-stream threshold
    blk, layer, desc = make_block(case)
    want = orc.moe_group(case.host, case.x, case.hin, exact=1)["out"]
    out_pageable = case.hin.copy()
    blk.forward_host(desc, layer, case.x, out_pageable)
    xp = torch.from_numpy(case.x).pin_memory(); op = torch.from_numpy(case.hin.copy()).pin_memory()
    blk.forward_host(desc, layer, xp.numpy(), op.numpy())
    assert rel_l2(out_pageable, want) < 1e-3 and rel_l2(op.numpy(), want) < 1e-3
    assert np.array_equal(op.numpy(), out_pageable)
    blk.close()


def test_stage_capture_replays_like_eager(orc):
    """route + experts and shared + finish recorded with the stage-capture API give the one-call block's result."""
    case = synth_case("c2", D=512, E=32, K=4, I=128, SI=128, T=24)
    blk, layer, desc = make_block(case)
    x = torch.from_numpy(case.x).cuda()
    want = torch.from_numpy(case.hin).cuda(); blk.forward(desc, layer, x, want)
    out = torch.from_numpy(case.hin).cuda()
    routed = torch.empty_like(x)

    def stages(s=None):
        blk.route(desc, layer, x, stream=s); blk.experts(desc, layer, x, routed, stream=s)
        blk.shared(desc, layer, x, stream=s); blk.finish(desc, layer, x, routed, out, stream=s)

    stages()                                       # eager once: set-up work cannot be captured
    torch.cuda.synchronize()
    g = blk.capture(stages)
    out.copy_(torch.from_numpy(case.hin).cuda())
    l0 = blk.lib.sw_launch_count()
    g.replay()
    torch.cuda.synchronize()
    assert blk.lib.sw_launch_count() - l0 >= 8
    assert rel_l2(out.cpu().numpy(), want.cpu().numpy()) < 1e-6
    check_routing(blk.routing(), orc.moe_group(case.host, case.x, None, exact=1))
    g.close(); blk.close()


def test_small_groups_take_the_tma_path_and_odd_widths_the_cuda_cores(orc):
    """Path proof for the decode kernels: widths that are multiples of 128 run k_q4_tma (2); others k_q4_group (0)."""
    run_case(synth_case("c2", corr_bias_std=0.01, T=8, D=512, E=32, K=4, I=128, SI=128), orc, path=2)
    run_case(synth_case("c2", corr_bias_std=0.01, T=8, D=384, E=12, K=3, I=96, SI=64), orc, path=0)


def test_every_kernel_family_on_one_case(orc):
    """The same layer through each expert-kernel family (SW_OPT_EXPERT_PATH): CUDA cores, mma.sync + cp.async,
    mma.sync + TMA, tcgen05; each must report the family that ran and meet the same bars."""
    from sabrewing_b200 import capi
    case = synth_case("c3", corr_bias_std=0.01, T=160, D=512, I=256, SI=128, E=16, K=4)
    want = orc.moe_group(case.host, case.x, case.hin, exact=1)
    for path in (0, 1, 2, 3):
        blk, layer, desc = make_block(case)
        assert blk.lib.sw_moe_set_option(blk.ctx, capi.OPT_EXPERT_PATH, path) == 0
        x = torch.from_numpy(case.x).cuda(); out = torch.from_numpy(case.hin).cuda()
        blk.forward(desc, layer, x, out)
        torch.cuda.synchronize()
        assert blk.status() == 0 and blk.lib.sw_moe_last_path(blk.ctx) == path
        check_routing(blk.routing(), want)
        assert rel_l2(out.cpu().numpy() - case.hin, want["out"] - case.hin) < OUT_TOL, path
        blk.close()


def test_misaligned_weight_blob_is_refused(orc):
    """Every expert kernel reads the int4 blobs 16 bytes at a time: a blob 8 bytes off that alignment is refused with an
    error text before anything is launched."""
    from sabrewing_b200 import capi
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    case = synth_case("c2", corr_bias_std=0.01, T=8, D=512, E=32, K=4, I=128, SI=128)
    cfg = case.cfg
    blk = MoeBlock("cuda:0", 8, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, "cuda:0")
    l = layer.c(); l.gu_q = layer.gu_q.data_ptr() + 8
    d = desc_from_config(cfg).c()
    x = torch.from_numpy(case.x).cuda(); out = torch.zeros_like(x)
    l0 = blk.lib.sw_launch_count()
    assert blk.lib.sw_moe_forward(blk.ctx, C.byref(d), C.byref(l), x.data_ptr(), out.data_ptr(), 8, None) == -1
    assert "16-byte" in capi.last_error() and blk.lib.sw_launch_count() == l0
    lib = _lag()
    y = np.zeros((1, 8), np.float32); xx = np.zeros((1, 64), np.float32)
    assert lib.lag_cuda_matmul_q4(y.ctypes.data, xx.ctypes.data, layer.gu_q.data_ptr() + 8, layer.gu_s.data_ptr(), 1, 64, 8) == -1
    blk.close()


def test_bad_row_pointers_are_refused_before_any_launch():
    """NULL or a column-offset view (not 16-byte aligned) comes back as -1 with a text, not as a device fault."""
    from sabrewing_b200 import capi
    case = synth_case("c2", D=256, E=8, K=2, I=128, SI=128, T=4)
    blk, layer, desc = make_block(case)
    d, l = desc.c(), layer.c()
    buf = torch.zeros(4 * 256 + 8, device="cuda")
    good, off = buf.data_ptr(), buf.data_ptr() + 4
    out = torch.zeros(4 * 256, device="cuda")
    l0 = blk.lib.sw_launch_count()
    assert blk.lib.sw_moe_forward(blk.ctx, C.byref(d), C.byref(l), off, out.data_ptr(), 4, None) == -1
    assert "16-byte" in capi.last_error()
    assert blk.lib.sw_moe_forward(blk.ctx, C.byref(d), C.byref(l), good, None, 4, None) == -1
    assert "null" in capi.last_error()
    assert blk.lib.sw_moe_route(blk.ctx, C.byref(d), C.byref(l), off, 4, None) == -1
    assert blk.lib.sw_launch_count() == l0                                   # nothing was launched
    assert blk.lib.sw_moe_forward(blk.ctx, C.byref(d), C.byref(l), good, out.data_ptr(), 4, None) == 0   # and the context still works
    torch.cuda.synchronize()
    blk.close()


def test_injected_failures_are_clean_errors(orc):
    """Host-side failure injection.  Compute calls: the reference's COLI_GPU_FAIL_AFTER hook and its test
    (c/backend_cuda.cu:684-692, c/tests/test_backend_cuda.cu:93-98): on -> the call reports failure, off -> the same call
    works.  Allocations: the n-th allocation fails, the call returns its error code, what was created so far is released."""
    from sabrewing_b200 import capi
    lib = capi.lib()
    case = synth_case("c2", D=256, E=8, K=2, I=128, SI=128, T=4)
    blk, layer, desc = make_block(case)
    x = torch.from_numpy(case.x).cuda(); out = torch.from_numpy(case.hin).cuda()
    try:
        lib.sw_test_fail_after(0)                                   # every compute call fails
        with pytest.raises(RuntimeError, match="injected"):
            blk.forward(desc, layer, x, out)
        y = np.zeros((1, 8), np.float32)
        assert lib.lag_cuda_matmul_q4(y.ctypes.data, y.ctypes.data, None, None, 1, 64, 8) == -1
        lib.sw_test_fail_after(2)                                   # two calls succeed, the third fails
        blk.route(desc, layer, x); blk.route(desc, layer, x)
        with pytest.raises(RuntimeError, match="injected"):
            blk.route(desc, layer, x)
    finally:
        lib.sw_test_fail_after(-1)
    blk.forward(desc, layer, x, out)                                # off: healthy call right after
    torch.cuda.synchronize()
    want = orc.moe_group(case.host, case.x, case.hin, exact=1)
    assert rel_l2(out.cpu().numpy() - case.hin, want["out"] - case.hin) < OUT_TOL
    blk.close()

    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    try:
        for n in (1, 2, 3):                 # device block, first and second page-locked staging buffer
            lib.sw_test_fail_alloc(n)
            ctx = C.c_void_p()
            assert lib.sw_moe_ctx_create(C.byref(ctx), 0, 64, 32, 4, 1024, 256, 256) == -1
            assert not ctx.value and "failed" in capi.last_error()
        lib.sw_test_fail_alloc(1)
        blob = np.zeros(64, np.uint8)
        assert lib.lag_cuda_upload(blob.ctypes.data, blob.nbytes) is None       # NULL on failure, like the reference
    finally:
        lib.sw_test_fail_alloc(0)
    ctx = C.c_void_p()
    assert lib.sw_moe_ctx_create(C.byref(ctx), 0, 64, 32, 4, 1024, 256, 256) == 0
    lib.sw_moe_ctx_destroy(ctx)
    torch.cuda.synchronize()
    assert abs(torch.cuda.mem_get_info()[0] - free0) < (64 << 20)            # the failed creations leaked no device memory


def test_a_bounded_wait_that_runs_out_reports_and_returns(orc):
    """The give-up path of the kernels' mbarrier waits: a barrier nobody arrives at, a limit of a few thousand polls,
    SW_ST_TIMEOUT in the status word, a clean return, and the context computes correctly afterwards."""
    case = synth_case("c2", D=256, E=8, K=2, I=128, SI=128, T=4)
    blk, layer, desc = make_block(case)
    assert blk.lib.sw_moe_test_wait_timeout(blk.ctx, 4096) == 4
    assert blk.status() == 0                                                  # cleared again by the test entry
    x = torch.from_numpy(case.x).cuda(); out = torch.from_numpy(case.hin).cuda()
    blk.forward(desc, layer, x, out)
    torch.cuda.synchronize()
    want = orc.moe_group(case.host, case.x, case.hin, exact=1)
    assert rel_l2(out.cpu().numpy() - case.hin, want["out"] - case.hin) < OUT_TOL
    blk.close()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_two_devices_in_one_process(orc):
    """Function attributes and occupancy are per device: a second context on another GPU sets its own."""
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    case = synth_case("c3", corr_bias_std=0.01, T=300, D=512, I=256, SI=128, E=16, K=4)      # tcgen05 path: ~200 KB of shared memory
    cfg = case.cfg
    want = orc.moe_group(case.host, case.x, case.hin, exact=1)
    for dev in ("cuda:0", "cuda:1"):
        blk = MoeBlock(dev, 300, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
        layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, dev)
        x = torch.from_numpy(case.x).to(dev); out = torch.from_numpy(case.hin).to(dev)
        with torch.cuda.device(dev):
            blk.forward(desc_from_config(cfg), layer, x, out)
            torch.cuda.synchronize(dev)
        assert blk.status() == 0 and blk.lib.sw_moe_last_path(blk.ctx) == 3
        assert rel_l2(out.cpu().numpy() - case.hin, want["out"] - case.hin) < OUT_TOL
        blk.close()


def test_rmsnorm_and_the_layer_tail_on_a_resident_residual_stream(orc):
    """h += MoE(rmsnorm(h) * w) with h resident on the device (c/laguna.c:1119,1126); the norm alone is the reference's
    rmsnorm_row (c/moe_math.h:58-62) to the last bit on all but double-rounding coincidences."""
    from sabrewing_b200 import capi
    case = synth_case("c2", corr_bias_std=0.01, T=24, D=1024, E=32, K=4, I=256, SI=256)
    cfg = case.cfg
    rng = np.random.default_rng(9)
    h0 = (rng.standard_normal((24, cfg.D)) * 3.0).astype(np.float32)
    wn = (1 + 0.1 * rng.standard_normal(cfg.D)).astype(np.float32)
    xn = orc.rmsnorm_rows(h0, wn, 1e-6)
    lib = capi.lib()
    hd = torch.from_numpy(h0).cuda(); wd = torch.from_numpy(wn).cuda(); yd = torch.empty_like(hd)
    assert lib.sw_rmsnorm(hd.data_ptr(), wd.data_ptr(), yd.data_ptr(), 24, cfg.D, 1e-6, None) == 0
    torch.cuda.synchronize()
    got = yd.cpu().numpy()
    assert (got != xn).mean() < 1e-3 and np.abs(got - xn).max() <= 2.4e-7 * np.abs(xn).max()
    blk, layer, desc = make_block(case)
    blk.forward_norm(desc, layer, hd, wd, 1e-6)
    torch.cuda.synchronize()
    assert blk.status() == 0
    want = orc.moe_group(case.host, xn, h0, exact=1)
    check_routing(blk.routing(), want)
    assert rel_l2(hd.cpu().numpy() - h0, want["out"] - h0) < OUT_TOL
    blk.close()


def test_lag_resident_matmuls_on_tensor_cores(orc):
    """The resident GEMMs either side of the block (c/backend_cuda_laguna.h:32-40): decode-size calls on the f32 kernels
    (element-wise bar of the reference's self-test), batched calls on the tensor cores (mma.sync from 16 rows, tcgen05
    for bf16 from 128)."""
    from sabrewing_b200 import synth
    l = _lag()
    rng = np.random.default_rng(77)
    I, O = 2048, 1536
    p = rng.integers(0, 256, (O, I // 2), dtype=np.uint8)
    sc = (0.01 + rng.random(O, dtype=np.float32) * 0.05).astype(np.float32)
    Wb = synth.f32_to_bf16(rng.random((O, I), dtype=np.float32) * 2 - 1)
    dp, ds, dW = _up(l, p), _up(l, sc), _up(l, Wb)
    for S in (1, 5, 40, 200):
        x = (rng.random((S, I), dtype=np.float32) * 2 - 1)
        y = np.empty((S, O), np.float32)
        assert l.lag_cuda_matmul_q4(y.ctypes.data, x.ctypes.data, dp, ds, S, I, O) == 0
        yc = orc.matmul_q4(x, p, sc, 1)
        assert rel_l2(y, yc) < 1e-5
        assert l.lag_cuda_matmul_bf16(y.ctypes.data, x.ctypes.data, dW, S, I, O) == 0
        yc = orc.matmul_bf16(x, Wb, 1)
        assert rel_l2(y, yc) < 1e-5
    for d in (dp, ds, dW):
        l.lag_cuda_free(d)


def _sigmoid_f32(v):
    v = np.asarray(v, np.float32)
    return (np.float32(1) / (np.float32(1) + np.exp(-v.astype(np.float64)).astype(np.float32))).astype(np.float32)


def test_sigmoid_gated_shared_expert(orc):
    """The qwen35 engine's policy (c/qwen35.c:684-699): out += routed * route_scale + sigmoid(x . g) * shared(x), with the
    gate dot in the exact (double) contract."""
    from sabrewing_b200 import capi
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, MoeDesc
    case = synth_case("c2", corr_bias_std=0.01, T=20, D=512, E=32, K=4, I=128, SI=128)
    cfg = case.cfg
    rng = np.random.default_rng(21)
    case.a["sh_gate_w"] = (rng.standard_normal(cfg.D) * 0.05).astype(np.float32)
    blk = MoeBlock("cuda:0", 20, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, "cuda:0")
    desc = MoeDesc(cfg.E, cfg.K, cfg.route_act, cfg.use_corr_bias, cfg.norm_topk, cfg.route_scale, capi.SHARED_SIGMOID_GATED)
    x = torch.from_numpy(case.x).cuda(); out = torch.from_numpy(case.hin).cuda()
    blk.forward(desc, layer, x, out)
    torch.cuda.synchronize()
    assert blk.status() == 0
    sel, w = orc.route(case.host, case.x, exact=1)
    assert np.array_equal(blk.routing()["sel"], sel)
    routed = orc.experts_given_routing(case.host, case.x, sel, w, exact=1)
    gv = orc.matmul_f32(case.x, case.a["sh_gate_w"].reshape(1, -1), exact=1)[:, 0]
    want = routed * np.float32(cfg.route_scale) + _sigmoid_f32(gv)[:, None] * orc.shared_rows(case.host, case.x, exact=1)
    assert rel_l2(out.cpu().numpy() - case.hin, want) < OUT_TOL
    # the staged calls (shared ahead of finish) give the same rows
    out2 = torch.from_numpy(case.hin).cuda(); r = torch.empty_like(x)
    blk.shared(desc, layer, x); blk.route(desc, layer, x); blk.experts(desc, layer, x, r); blk.finish(desc, layer, x, r, out2)
    torch.cuda.synchronize()
    assert rel_l2(out2.cpu().numpy(), out.cpu().numpy()) < 1e-6
    blk.close()


def test_shared_expert_in_the_routed_weight_pool(orc):
    """The inkling engine's policy (c/inkling.c:1029-1043): the router has one more row (the shared expert's logit); the
    weights are the sigmoids of the K picks and of the shared expert, normalised over all K + 1 and multiplied by
    route_scale * global scale; selection by sigmoid + bias as usual."""
    from sabrewing_b200 import capi, synth
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, MoeDesc
    case = synth_case("c2", corr_bias_std=0.01, T=20, D=512, E=32, K=4, I=128, SI=128)
    cfg = case.cfg
    rng = np.random.default_rng(22)
    extra = synth.f32_to_bf16((rng.standard_normal((1, cfg.D)) * 0.02).astype(np.float32))
    rb = np.concatenate([case.a["router_bf16"], extra]); rw = synth.bf16_to_f32(rb)
    a = dict(case.a); a["router_bf16"] = rb; a["router_w"] = rw; a["route_global_scale"] = 1.5
    blk = MoeBlock("cuda:0", 20, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    layer = MoeLayer(cfg.D, cfg.I, cfg.SI, a, "cuda:0")
    desc = MoeDesc(cfg.E, cfg.K, capi.ROUTE_SIGMOID, 1, 0, 2.5, capi.SHARED_GATED)
    x = torch.from_numpy(case.x).cuda(); out = torch.from_numpy(case.hin).cuda()
    blk.forward(desc, layer, x, out)
    torch.cuda.synchronize()
    assert blk.status() == 0
    # restatement: exact logits of all E + 1 rows, sigmoid, top-K of score + bias over the E experts, pooled weights
    sc = _sigmoid_f32(orc.matmul_f32(case.x, rw, exact=1))
    sel = np.stack([orc.topk(sc[t, :cfg.E].copy(), case.a["corr_bias"], 1, cfg.K) for t in range(20)])
    w = np.take_along_axis(sc[:, :cfg.E], sel, axis=1).astype(np.float32)
    ws = sc[:, cfg.E]
    sm = np.zeros(20, np.float32)
    for k in range(cfg.K):
        sm = (sm + w[:, k]).astype(np.float32)
    sm = (sm + ws).astype(np.float32)
    f = (np.float32(np.float32(2.5) * np.float32(1.5)) / sm).astype(np.float32)
    wn = (w * f[:, None]).astype(np.float32); wsn = (ws * f).astype(np.float32)
    got = blk.routing(want_scores=True)
    assert np.array_equal(got["sel"], sel)
    assert (np.abs(got["w"] - wn) / np.abs(wn)).max() < W_TOL
    assert np.array_equal(got["scores"], sc[:, :cfg.E])
    routed = orc.experts_given_routing(case.host, case.x, sel, wn, exact=1)
    want = routed + wsn[:, None] * orc.shared_rows(case.host, case.x, exact=1)
    assert rel_l2(out.cpu().numpy() - case.hin, want) < OUT_TOL
    blk.close()


def test_activation_scales_far_from_one(orc):
    """The tensor-core expert kernels carry activations as fp16 pairs.  Every token row is divided by a power of two on
    its way in (largest magnitude in [1, 2)), the gate is multiplied back before SiLU and SiLU(gate)*up travels divided
    by the square, so the bar holds at any input scale on every kernel family: here 1e-6 ... 1e6 times the usual size,
    where plain fp16 pairs would flush to zero or overflow."""
    from sabrewing_b200 import capi
    base = synth_case("c3", corr_bias_std=0.01, T=160, D=512, I=256, SI=128, E=16, K=4)
    for scale in (1e-6, 1e-4, 1e4, 1e6):
        case = synth_case("c3", corr_bias_std=0.01, T=160, D=512, I=256, SI=128, E=16, K=4)
        case.x[:] = base.x * np.float32(scale)
        case.x[7] *= np.float32(1e-3)                          # rows of one batch at different scales
        case.x[11] = 0.0                                       # and a row of zeros
        case.hin[:] = 0.0                                      # no residual: a tiny MoE(x) must not drown in its rounding
        want = orc.moe_group(case.host, case.x, case.hin, exact=1)
        for path in (0, 1, 2, 3):
            blk, layer, desc = make_block(case)
            assert blk.lib.sw_moe_set_option(blk.ctx, capi.OPT_EXPERT_PATH, path) == 0
            x = torch.from_numpy(case.x).cuda(); out = torch.from_numpy(case.hin).cuda()
            blk.forward(desc, layer, x, out)
            torch.cuda.synchronize()
            assert blk.status() == 0 and blk.lib.sw_moe_last_path(blk.ctx) == path, (scale, path)
            check_routing(blk.routing(), want)
            got = out.cpu().numpy() - case.hin
            ref = want["out"] - case.hin
            assert rel_l2(got, ref) < OUT_TOL, (scale, path, rel_l2(got, ref))
            # per row too: a small row must not hide behind the large ones
            for r in (0, 7, 11):
                nr = np.linalg.norm(ref[r])
                assert np.linalg.norm(got[r] - ref[r]) <= OUT_TOL * max(nr, 1e-30) + 0.0, (scale, path, r)
            blk.close()


def test_shapes_around_the_kernels_tile_sizes(orc):
    """Shapes chosen to land on the edges of today's kernels: top-k of every width the combine step treats differently
    (1 ... 16: full rounds of 8 or 16 plus a last round of exactly the remaining width), token counts on both sides of the
    tiled router (128 rows, tiles of 64 x 64 with ragged last tiles in both directions), expert counts that are not a
    multiple of 64 or 32, pair counts on the many-CTA dispatch, the softmax and the sigmoid gate.  Bit-exact routing and
    dispatch, outputs inside the bar."""
    shapes = [
        # base, T, E, K, D, I, SI
        ("c2", 3, 24, 1, 256, 128, 128),
        ("c1", 5, 40, 2, 256, 128, 0),
        ("c2", 70, 96, 3, 512, 128, 128),
        ("c1", 130, 72, 5, 256, 256, 0),
        ("c2", 129, 100, 7, 512, 128, 128),
        ("c1", 200, 130, 9, 256, 128, 0),
        ("c2", 64, 48, 12, 256, 128, 128),
        ("c1", 33, 64, 16, 512, 128, 0),
        ("c2", 257, 200, 16, 256, 128, 128),
        # more than 16384 pairs: the many-CTA dispatch, with a ragged last segment and expert counts off every power of two
        ("c1", 2100, 100, 8, 256, 128, 0),
        ("c2", 1701, 130, 10, 256, 128, 128),
    ]
    for base, T, E, K, D, I, SI in shapes:
        case = synth_case(base, corr_bias_std=0.01 if base == "c2" else 0.0, T=T, E=E, K=K, D=D, I=I, SI=SI)
        run_case(case, orc)
