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


def test_struct_layouts_match_reference_descriptor():
    from sabrewing_b200 import capi
    # MoeDesc (c/moe_arch.h:33-41): 5 ints, float, enum -> 28 bytes, fields in this order
    assert [f[0] for f in capi.SwMoeDesc._fields_] == ["n_experts", "topk", "route_act", "use_corr_bias",
                                                     "norm_topk", "route_scale", "shared_mode"]
    assert C.sizeof(capi.SwMoeDesc) == 28
    assert C.sizeof(capi.SwMoeLayer) == 16 + 10 * 8 + 16      # 4 ints, 10 pointers, 3 ints + padding


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
