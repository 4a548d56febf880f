"""The CPU checker against the reference's golden vectors and compiled code (no GPU)."""
import numpy as np
import pytest

from conftest import load_golden, synth_case, rel_l2

GOLDEN_CASES = ["laguna_tiny", "olmoe_tiny", "zipf_tiny", "wide_tiny"]


def test_known_answer_nibbles(orc):
    # c/tests/test_backend_cuda.cu:42,105-110: rows [-8,-1,0,7] and [1,2,3,4], low nibble first
    x = np.array([[1, -2, 3, -4]], np.float32)
    q4 = np.array([[0x70, 0xf8], [0xa9, 0xcb]], np.uint8)
    s4 = np.array([1.0, 0.25], np.float32)
    for exact in (0, 1):
        assert orc.matmul_q4(x, q4, s4, exact).tolist() == [[-34.0, -2.5]]


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_block_matches_reference_golden(orc, name):
    case, z = load_golden(name)
    rows = orc.moe_rows(case.host, case.x, case.hin, exact=1)
    grp = orc.moe_group(case.host, case.x, case.hin, exact=1)
    assert np.array_equal(rows, z["ref_out"])          # bit-exact vs moe_block()
    assert np.array_equal(grp["out"], z["ref_out"])    # grouping changes no bit
    if "ref_out_grouped" in z.files:
        assert np.array_equal(grp["out"], z["ref_out_grouped"])   # vs lag_moe_group
        assert np.array_equal(rows, z["ref_out_pertoken"])
    # the float-accumulate port stays within float noise of the exact contract
    assert rel_l2(orc.moe_group(case.host, case.x, case.hin, exact=0)["out"], z["ref_out"]) < 1e-5


def test_kernel_goldens(orc):
    z = np.load(__import__("os").path.join(__import__("conftest").GOLDEN, "kernels.npz"))
    p, s = orc.quant_rows_i4(z["W"])
    assert np.array_equal(p, z["packed"]) and np.array_equal(s, z["scale"])
    assert np.array_equal(orc.matmul_q4(z["x"], z["packed"], z["scale"], 1), z["q4_exact"])
    assert rel_l2(orc.matmul_q4(z["x"], z["packed"], z["scale"], 0), z["q4_simd"]) < 1e-5
    assert np.array_equal(orc.matmul_f32(z["x"], z["W"], 1), z["f32_exact"])
    assert np.array_equal(orc.matmul_bf16(z["x"], z["bf16_w"], 1), z["bf16_exact"])
    assert np.array_equal(orc.softmax_row(z["scores"]), z["softmax"])
    assert np.array_equal(orc.topk(z["scores"], None, 0, 5), z["topk5"])
    assert np.array_equal(orc.topk(z["scores"], z["bias"], 1, 5), z["topk5_bias"])
    assert np.array_equal(orc.rmsnorm_rows(z["x"]), z["rms"])
    for gs in (64, 16):
        y = orc.matmul_i4_grouped(z["g%d_x" % gs], z["g%d_q" % gs], z["g%d_s" % gs], gs, exact=0)
        yd = orc.matmul_i4_grouped(z["g%d_x" % gs], z["g%d_q" % gs], z["g%d_s" % gs], gs, exact=1)
        assert rel_l2(y, z["g%d_y" % gs]) < 1e-5 and rel_l2(yd, z["g%d_y" % gs]) < 1e-5


def test_numpy_quantiser_matches_c(orc):
    from sabrewing_b200 import synth
    rng = np.random.default_rng(3)
    W = rng.standard_normal((50, 256), dtype=np.float32) * np.float32(0.02)
    W[7] = 0                                   # all-zero row hits the 1e-12 scale floor
    W[8, 3] = 1e-13
    p, s = synth.quant_rows_i4(W); pc, sc = orc.quant_rows_i4(W)
    assert np.array_equal(p, pc) and np.array_equal(s, sc)


def test_topk_ties_and_nonfinite(orc):
    E, K = 12, 4
    flat = np.full(E, 0.5, np.float32)
    assert orc.topk(flat, None, 0, K).tolist() == [0, 1, 2, 3]          # ties -> lower id
    bias = np.zeros(E, np.float32); bias[9] = 0.1; bias[4] = 0.1
    assert orc.topk(flat, bias, 1, K).tolist() == [4, 9, 0, 1]          # bias drives selection
    assert orc.topk(flat, bias, 0, K).tolist() == [0, 1, 2, 3]          # ...only when enabled
    nan = np.full(E, np.nan, np.float32)
    assert orc.topk(nan, None, 0, K).tolist() == [0, 1, 2, 3]           # degraded selection (c/moe_arch.h:75-86)
    mixed = nan.copy(); mixed[5] = 0.1; mixed[2] = 0.2
    assert orc.topk(mixed, None, 0, K).tolist() == [2, 5, 0, 1]


def test_group_is_stable_counting_sort(orc):
    rng = np.random.default_rng(4)
    S, K, E = 37, 5, 11
    sel = np.stack([rng.permutation(E)[:K] for _ in range(S)]).astype(np.int32)
    sel[:, :] = np.where(sel == 3, 4 if False else sel, sel)
    g = orc.group(sel, E)
    flat = sel.reshape(-1)
    order = np.argsort(flat, kind="stable")
    assert np.array_equal(g["grow"], (order // K).astype(np.int32))
    assert np.array_equal(g["rowof"][order], np.arange(S * K, dtype=np.int32))
    present = np.unique(flat)
    assert np.array_equal(g["gexp"], present.astype(np.int32))
    assert np.array_equal(g["gcnt"], np.bincount(flat, minlength=E)[present].astype(np.int32))
    assert np.array_equal(g["gbeg"], np.concatenate([[0], np.cumsum(g["gcnt"])[:-1]]).astype(np.int32))


def test_empty_expert_groups_are_skipped(orc):
    sel = np.array([[5, 1], [5, 9]], np.int32)
    g = orc.group(sel, 12)
    assert g["G"] == 3 and g["gexp"].tolist() == [1, 5, 9] and g["gcnt"].tolist() == [1, 2, 1]
    assert g["grow"].tolist() == [0, 0, 1, 1] and g["rowof"].tolist() == [1, 0, 2, 3]

def test_fp4_goldens(orc, ref):
    """fp4 products against fixtures made by the compiled reference (matmul_fp4_kb, the clamped expert loop)."""
    z = np.load(__import__("os").path.join(__import__("conftest").GOLDEN, "fp4.npz"))
    assert np.array_equal(orc.matmul_fp4(z["x"], z["q"], z["es"], 1), z["y_exact"])
    assert rel_l2(orc.matmul_fp4(z["x"], z["q"], z["es"], 0), z["y_exact"]) < 1e-6
    assert rel_l2(z["y_simd"], z["y_exact"]) < 1e-6
    I, D = z["dn_q"].shape[1] * 2, z["gu_q"].shape[1] * 2
    args = (z["e_x"], z["gu_q"], z["gu_es"], z["dn_q"], z["dn_es"], z["sel"], z["w"], I, D, float(z["limit"]))
    assert np.array_equal(orc.experts_fp4(*args, 1), z["e_exact"])
    assert rel_l2(orc.experts_fp4(*args, 0), z["e_exact"]) < 1e-5
    # the fixture really clamps: without the limit the result differs
    assert rel_l2(orc.experts_fp4(*args[:-1], 1e30, 1), z["e_exact"]) > 1e-3
    # ue8m0 special bytes: 0xFF contributes nothing, 0 is 2^-127
    y = orc.matmul_fp4(z["x"], z["q"], z["es"], 1)
    es2 = z["es"].copy(); es2[7, :] = 0xFF
    assert np.all(orc.matmul_fp4(z["x"], z["q"], es2, 1)[:, 7] == 0) and np.all(np.isfinite(y))
    if ref is not None:
        assert np.array_equal(ref.matmul_fp4(z["x"], z["q"], z["es"], 1), z["y_exact"])
        assert np.array_equal(ref.experts_fp4(*args, 1), z["e_exact"])


@pytest.mark.parametrize("base,kw", [
    ("c2", dict(D=256, E=32, K=6, I=128, SI=64, T=21)),
    ("c1", dict(D=192, E=16, K=4, I=96, T=17)),
    ("c3", dict(D=256, E=64, K=10, I=64, SI=64, T=40)),
])
def test_restatement_matches_compiled_reference(orc, ref, base, kw):
    if ref is None:
        pytest.skip("compiled reference not present (oracle/_ref)")
    case = synth_case(base, corr_bias_std=0.01, **kw)
    want = ref.moe_block_rows(case.host, case.x, case.hin, exact=1)
    assert np.array_equal(orc.moe_rows(case.host, case.x, case.hin, exact=1), want)
    assert np.array_equal(orc.moe_group(case.host, case.x, case.hin, exact=1)["out"], want)
    if case.cfg.route_act == 0 and case.cfg.shared_mode == 1 and case.a["logit_bias"] is None:
        assert np.array_equal(ref.laguna_moe_rows(case.host, case.x, case.hin, 1, 1), want)
    # the reference's timed default (AVX-512 f32) stays within 1e-5 of its exact mode
    assert rel_l2(ref.moe_block_rows(case.host, case.x, case.hin, exact=0), want) < 1e-5


def test_softplus_gate_restatement(orc):
    # no reference router uses softplus; the restatement applies c/moe_math.h:54 as the gate
    case = synth_case("c2", D=128, E=16, K=4, I=64, SI=64, T=6, route_act=2)
    sel, w, sc = orc.route(case.host, case.x, exact=1, want_scores=True)
    logits = orc.matmul_f32(case.x, case.a["router_w"], 1)
    want = np.log1p(np.exp(logits.astype(np.float64)))
    assert np.allclose(sc, want, rtol=1e-6)
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)
