"""The allocation-free routing entry point against the regular one (collected last on purpose).

sw_moe_route_static serves hosts that cannot allocate device memory when they need a routing
decision (every free byte already belongs to their expert cache, or an allocation's device-wide
synchronisation is not acceptable).  Its working memory is a fixed array inside the library, so
the checks here are: same ids and weights as sw_moe_route, on two calls in a row that reuse the
array, and a clear refusal beyond the stated limits.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import synth_case

pytestmark = pytest.mark.gpu


def _route_both(case, T):
    from sabrewing_b200 import capi
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    cfg = case.cfg
    lib = capi.lib()
    layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, "cuda:0")
    desc = desc_from_config(cfg)
    x = torch.from_numpy(case.x[:T].copy()).cuda()
    blk = MoeBlock("cuda:0", T, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    blk.route(desc, layer, x)
    want = blk.routing()
    sel = torch.full((T, cfg.K), -1, dtype=torch.int32, device="cuda")
    w = torch.zeros((T, cfg.K), dtype=torch.float32, device="cuda")
    d, l = desc.c(), layer.c()
    rc = lib.sw_moe_route_static(C.byref(d), C.byref(l), x.data_ptr(), T, sel.data_ptr(), w.data_ptr(), None)
    assert rc == 0, capi.last_error()
    torch.cuda.synchronize()
    blk.close()
    return want, sel.cpu().numpy(), w.cpu().numpy()


def test_static_route_matches_regular_route_twice_in_a_row(orc):
    # two different layers back to back: the second call finds the first call's leftovers in the array
    for base, kw, T in (("c2", dict(D=1024, I=256, SI=256), 5), ("c1", dict(D=512, I=256), 8), ("c2", dict(D=1024, I=256, SI=256), 1)):
        case = synth_case(base, corr_bias_std=0.01, T=8, **kw)
        want, sel, w = _route_both(case, T)
        assert np.array_equal(sel, want["sel"])
        assert np.abs(w - want["w"]).max() <= 5e-7 * np.abs(want["w"]).max()
        # and against the CPU checker directly: ids bit-exact, weights at f32 rounding level
        osel, ow = orc.route(case.host, case.x[:T].copy(), exact=1)
        assert np.array_equal(sel, osel)
        assert (np.abs(w - ow) / np.abs(ow)).max() < 5e-7


def test_static_route_back_to_back_on_one_stream_without_a_sync(orc):
    """Two calls with different layers queued on the same non-default stream, nothing between them: the second call's
    ticket reset and launch are ordered behind the first by the stream alone.  Covers the f32 router and the softplus gate."""
    from sabrewing_b200 import capi
    from sabrewing_b200.moe_block import MoeLayer, desc_from_config
    lib = capi.lib()
    ca = synth_case("c2", corr_bias_std=0.01, T=8, D=1024, I=256, SI=256, route_act=2)       # softplus gate
    cb = synth_case("c1", corr_bias_std=0.0, T=6, D=512, I=256)                             # softmax
    la = MoeLayer(ca.cfg.D, ca.cfg.I, ca.cfg.SI, ca.a, "cuda:0", router="f32")
    lb = MoeLayer(cb.cfg.D, cb.cfg.I, cb.cfg.SI, cb.a, "cuda:0")
    xa = torch.from_numpy(ca.x).cuda(); xb = torch.from_numpy(cb.x).cuda()
    sa = torch.full((8, ca.cfg.K), -1, dtype=torch.int32, device="cuda"); wa = torch.zeros((8, ca.cfg.K), device="cuda")
    sb = torch.full((6, cb.cfg.K), -1, dtype=torch.int32, device="cuda"); wb = torch.zeros((6, cb.cfg.K), device="cuda")
    da, dla, db, dlb = desc_from_config(ca.cfg).c(), la.c(), desc_from_config(cb.cfg).c(), lb.c()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    h = C.c_void_p(st.cuda_stream)
    assert lib.sw_moe_route_static(C.byref(da), C.byref(dla), xa.data_ptr(), 8, sa.data_ptr(), wa.data_ptr(), h) == 0, capi.last_error()
    assert lib.sw_moe_route_static(C.byref(db), C.byref(dlb), xb.data_ptr(), 6, sb.data_ptr(), wb.data_ptr(), h) == 0, capi.last_error()
    st.synchronize()
    for case, sel, w in ((ca, sa, wa), (cb, sb, wb)):
        osel, ow = orc.route(case.host, case.x, exact=1)
        assert np.array_equal(sel.cpu().numpy(), osel)
        assert (np.abs(w.cpu().numpy() - ow) / np.abs(ow)).max() < 5e-7


def test_static_route_rejects_sizes_beyond_its_array():
    from sabrewing_b200 import capi
    from sabrewing_b200.moe_block import MoeLayer, desc_from_config
    case = synth_case("c1", D=512, I=256, T=9)
    cfg = case.cfg
    layer = MoeLayer(cfg.D, cfg.I, cfg.SI, case.a, "cuda:0")
    d, l = desc_from_config(cfg).c(), layer.c()
    x = torch.from_numpy(case.x).cuda()
    sel = torch.zeros((9, cfg.K), dtype=torch.int32, device="cuda"); w = torch.zeros((9, cfg.K), device="cuda")
    lib = capi.lib()
    assert lib.sw_moe_route_static(C.byref(d), C.byref(l), x.data_ptr(), 9, sel.data_ptr(), w.data_ptr(), None) == -1
    assert "T outside" in capi.last_error()
    d.n_experts = 1024
    assert lib.sw_moe_route_static(C.byref(d), C.byref(l), x.data_ptr(), 4, sel.data_ptr(), w.data_ptr(), None) == -1
    assert "n_experts" in capi.last_error()
    d.n_experts = cfg.E
    for bad_d in (8192 + 32, 500):              # wider than the array's rows; not a multiple of 32
        l.D = bad_d
        assert lib.sw_moe_route_static(C.byref(d), C.byref(l), x.data_ptr(), 4, sel.data_ptr(), w.data_ptr(), None) == -1
        assert "D must be" in capi.last_error()
    l.D = cfg.D
    assert lib.sw_moe_route_static(C.byref(d), C.byref(l), x.data_ptr() + 4, 4, sel.data_ptr(), w.data_ptr(), None) == -1
    assert "16-byte" in capi.last_error()
