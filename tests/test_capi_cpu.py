"""The C-ABI library loads and exports every symbol include/sabrewing_b200.h declares (no GPU)."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "sabrewing_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b((?:lag_cuda|sw)_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from sabrewing_b200 import build, capi
    build.build()
    l = capi.lib()
    names = declared_symbols()
    assert len(names) >= 20
    for n in names:
        assert hasattr(l, n), n
        assert n in capi.SIGNATURES, "binding missing for " + n
    assert sorted(capi.SIGNATURES) == names


def test_glm_boundary_symbols_are_exported():
    """Every coli_cuda_* entry point include/sabrewing_b200_glm.h declares is exported by the library."""
    from sabrewing_b200 import build, capi
    build.build()
    text = open(os.path.join(ROOT, "include", "sabrewing_b200_glm.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = sorted(set(re.findall(r"\b(coli_cuda_[a-z0-9_]+)\s*\(", text)))
    assert len(names) >= 30
    l = C.CDLL(capi.LIB_PATH)
    for n in names:
        assert hasattr(l, n), n
    # without a device the set-up reports failure (0) and the engine keeps its CPU path
    import torch
    if not torch.cuda.is_available():
        assert l.coli_cuda_init((C.c_int * 1)(0), 1) == 0
        assert l.coli_cuda_device_count() == 0


def test_struct_layouts_match_reference_descriptor():
    from sabrewing_b200 import capi
    # MoeDesc (c/moe_arch.h:33-41): 5 ints, float, enum -> 28 bytes, fields in this order
    assert [f[0] for f in capi.SwMoeDesc._fields_] == ["n_experts", "topk", "route_act", "use_corr_bias",
                                                     "norm_topk", "route_scale", "shared_mode"]
    assert C.sizeof(capi.SwMoeDesc) == 28
    assert C.sizeof(capi.SwMoeLayer) == 16 + 10 * 8 + 16 + 16   # 4 ints, 10 pointers, 3 ints + padding, pointer, float + padding


def test_calls_fail_cleanly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    from sabrewing_b200 import capi
    l = capi.lib()
    assert l.lag_cuda_init(0) == -1                    # reference convention: -1, caller falls back
    assert l.lag_cuda_upload(None, 16) is None         # NULL on failure
    ctx = C.c_void_p()
    assert l.sw_moe_ctx_create(C.byref(ctx), 0, 4, 8, 2, 64, 64, 0) == -1
    assert capi.last_error() != ""
    assert l.sw_moe_ctx_create(C.byref(ctx), 0, 4, 100000, 2, 64, 64, 0) == -1   # limit check comes first
    assert "bad limits" in capi.last_error()


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    from sabrewing_b200 import capi
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        capi.lib()


def test_host_selftest_of_per_device_setup_and_map_cache():
    """Function attributes / occupancy are cached per device and the tensor-map cache is keyed by device too."""
    from sabrewing_b200 import capi
    assert capi.lib().sw_selftest_host() == 0


def _layer(**kw):
    from sabrewing_b200 import capi
    base = dict(D=128, I=64, SI=0, router_dtype=capi.DTYPE_BF16, router_w=0x1000, corr_bias=None, logit_bias=None,
                gu_q=0x2000, gu_s=0x3000, dn_q=0x4000, dn_s=0x5000, sh_gate=None, sh_up=None, sh_down=None,
                expert_lo=0, expert_cnt=0, gs=0, sh_gate_w=None, route_global_scale=0.0)
    base.update(kw)
    return capi.SwMoeLayer(*[base[f[0]] for f in capi.SwMoeLayer._fields_])


def test_validate_refuses_null_and_misaligned_buffers_without_a_device():
    """Return codes only: nothing is launched (the pointers are never dereferenced)."""
    from sabrewing_b200 import capi
    l = capi.lib()
    d = capi.SwMoeDesc(8, 2, 0, 0, 0, 1.0, 0)
    ok = _layer()
    assert l.sw_moe_validate(C.byref(d), C.byref(ok), 0x10000, 0x20000) == 0
    assert l.sw_moe_validate(C.byref(d), C.byref(ok), None, 0x20000) == -1 and "null" in capi.last_error()
    assert l.sw_moe_validate(C.byref(d), C.byref(ok), 0x10004, 0x20000) == -1 and "16-byte" in capi.last_error()   # a column-offset view
    assert l.sw_moe_validate(C.byref(d), C.byref(ok), 0x10000, 0x20008) == -1
    bad = _layer(router_w=0x1008)
    assert l.sw_moe_validate(C.byref(d), C.byref(bad), 0x10000, 0x20000) == -1 and "aligned" in capi.last_error()
    bad = _layer(gu_s=0x3004)
    assert l.sw_moe_validate(C.byref(d), C.byref(bad), 0x10000, 0x20000) == -1
    bad = _layer(dn_q=None)
    assert l.sw_moe_validate(C.byref(d), C.byref(bad), 0x10000, 0x20000) == -1 and "missing" in capi.last_error()
    d2 = capi.SwMoeDesc(8, 2, 0, 0, 0, 1.0, 1)           # shared expert asked for, weights absent
    assert l.sw_moe_validate(C.byref(d2), C.byref(_layer(SI=64)), 0x10000, 0x20000) == -1
    # the allocation-free routing entry checks its buffers before it touches CUDA
    sel = 0x30000
    assert l.sw_moe_route_static(C.byref(d), C.byref(ok), 0x10004, 2, sel, sel, None) == -1 and "16-byte" in capi.last_error()
    assert l.sw_moe_route_static(C.byref(d), C.byref(_layer(router_w=0x1002)), 0x10000, 2, sel, sel, None) == -1
    assert l.sw_moe_route_static(C.byref(d), C.byref(ok), 0x10000, 2, 0x30002, sel, None) == -1
    assert l.sw_moe_route_static(C.byref(d), C.byref(ok), None, 2, sel, sel, None) == -1 and "null" in capi.last_error()
