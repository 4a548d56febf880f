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


def test_static_route_matches_regular_route_twice_in_a_row():
    # two different layers back to back: the second call finds the first call's leftovers in the array
    for base, kw, T in (("c2", dict(D=1024, I=256, SI=256), 5), ("c1", dict(D=512, I=256), 8), ("c2", dict(D=1024, I=256, SI=256), 1)):
        case = synth_case(base, corr_bias_std=0.01, T=8, **kw)
        want, sel, w = _route_both(case, T)
        assert np.array_equal(sel, want["sel"])
        assert np.abs(w - want["w"]).max() <= 5e-7 * np.abs(want["w"]).max()


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
