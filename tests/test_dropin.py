"""The reference's own engine program as the caller of this library.

`oracle/Makefile dropin` compiles the reference's laguna.c with -DCOLI_CUDA where it lies and links it against
libsabrewing_b200.so in place of the reference's backend_cuda_laguna.o (the link line of a maintainer who swaps the
backend, c/Makefile:199-200,295-296).  The CPU part checks the link; the GPU part runs the reference's GPU
acceptance test, `LAG_CUDA_TEST=1 ./laguna` (c/laguna.c:1555-1665,1673), against this library: bf16 and int4
matmuls and the fused int4 expert within the reference's bars, grouped experts BIT-identical to the per-token path.
"""
import os
import re
import subprocess

import pytest


def _binary():
    import oracle
    if not os.path.exists(oracle.DROPIN_PATH):
        if oracle.reference_dir() is None:
            pytest.skip("no reference checkout and no prebuilt oracle/_ref/laguna_dropin")
        from sabrewing_b200 import build
        build.build()
        oracle.build()
    return oracle.DROPIN_PATH


def test_reference_engine_links_against_this_library_with_nothing_unresolved():
    from sabrewing_b200 import capi
    exe = _binary()
    undef = subprocess.run(["nm", "-D", "--undefined-only", exe], check=True, capture_output=True, text=True).stdout
    wanted = sorted(set(re.findall(r"\b(lag_cuda_[a-z0-9_]+)", undef)))
    assert len(wanted) >= 9, wanted                       # every lag_cuda_* call laguna.c makes
    defined = subprocess.run(["nm", "-D", "--defined-only", capi.LIB_PATH], check=True, capture_output=True, text=True).stdout
    have = set(re.findall(r"\b(lag_cuda_[a-z0-9_]+)", defined))
    assert set(wanted) <= have, sorted(set(wanted) - have)
    ldd = subprocess.run(["ldd", exe], check=True, capture_output=True, text=True).stdout
    assert "libsabrewing_b200.so" in ldd and "not found" not in ldd, ldd


@pytest.mark.gpu
def test_reference_gpu_selftest_passes_against_this_library():
    exe = _binary()
    env = dict(os.environ, LAG_CUDA_TEST="1", GPU_DEV="0")
    r = subprocess.run([exe], env=env, capture_output=True, text=True, timeout=600)
    lines = [l for l in r.stdout.splitlines() if l.startswith("[cuda-test]")]
    assert r.returncode == 0, r.stdout + r.stderr
    assert len(lines) == 5, r.stdout + r.stderr               # bf16, q4, fused expert, grouped, summary
    for l in lines[:3]:
        assert l.rstrip().endswith("OK"), l
    assert lines[3].rstrip().endswith("BIT-IDENTICAL"), lines[3]
    assert lines[4].rstrip().endswith("ALL PASS"), lines[4]
    print("\n".join(lines))
