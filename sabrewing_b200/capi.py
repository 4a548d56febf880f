"""ctypes binding of libsabrewing_b200.so (include/sabrewing_b200.h).

The library is the product; this module only declares its C signatures.  There is
no CPU fallback: if the shared library is missing the import of `lib()` raises.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsabrewing_b200.so")

ROUTE_SIGMOID, ROUTE_SOFTMAX, ROUTE_SOFTPLUS = 0, 1, 2
SHARED_NONE, SHARED_UNSCALED, SHARED_GATED, SHARED_SIGMOID_GATED = 0, 1, 3, 4
DTYPE_F32, DTYPE_BF16 = 0, 1
OPT_UMMA_TERMS, OPT_EXPERT_PATH = 1, 2
EP_REPLICATE, EP_ALLTOALL = 0, 1


class SwMoeDesc(C.Structure):
    """Field-for-field MoeDesc of the reference (c/moe_arch.h:33-41)."""
    _fields_ = [("n_experts", C.c_int), ("topk", C.c_int), ("route_act", C.c_int),
                ("use_corr_bias", C.c_int), ("norm_topk", C.c_int), ("route_scale", C.c_float),
                ("shared_mode", C.c_int)]


class SwMoeLayer(C.Structure):
    _fields_ = [("D", C.c_int), ("I", C.c_int), ("SI", C.c_int), ("router_dtype", C.c_int),
                ("router_w", C.c_void_p), ("corr_bias", C.c_void_p), ("logit_bias", C.c_void_p),
                ("gu_q", C.c_void_p), ("gu_s", C.c_void_p), ("dn_q", C.c_void_p), ("dn_s", C.c_void_p),
                ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p),
                ("expert_lo", C.c_int), ("expert_cnt", C.c_int), ("gs", C.c_int),
                ("sh_gate_w", C.c_void_p), ("route_global_scale", C.c_float)]


# name -> (restype, argtypes); every symbol include/sabrewing_b200.h declares
_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
_pd, _pl = C.POINTER(SwMoeDesc), C.POINTER(SwMoeLayer)
SIGNATURES = {
    "lag_cuda_init": (_i, [_i]),
    "lag_cuda_free_bytes": (_sz, []),
    "lag_cuda_total_bytes": (_sz, []),
    "lag_cuda_upload": (_vp, [_vp, _sz]),
    "lag_cuda_free": (None, [_vp]),
    "lag_cuda_matmul_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "lag_cuda_matmul_q8": (_i, [_vp, _vp, _vp, _i, _i, _i]),
    "lag_cuda_matmul_q4": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "lag_cuda_expert_q4": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "lag_cuda_moe_experts": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i]),
    "lag_cuda_moe_group": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _vp, _vp, _vp, _i, _i, _i, _i]),
    "lag_cuda_matmul_fp4": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i]),
    "lag_cuda_moe_experts_fp4": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, C.c_float]),
    "sw_moe_ctx_create": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _i, _i, _i]),
    "sw_moe_ctx_destroy": (None, [_vp]),
    "sw_moe_forward": (_i, [_vp, _pd, _pl, _vp, _vp, _i, _vp]),
    "sw_moe_forward_host": (_i, [_vp, _pd, _pl, _vp, _vp, _i]),
    "sw_moe_forward_norm": (_i, [_vp, _pd, _pl, _vp, _vp, _f, _i, _vp]),
    "sw_rmsnorm": (_i, [_vp, _vp, _vp, _i, _i, _f, _vp]),
    "sw_moe_graph_create": (_i, [_vp, _pd, _pl, _vp, _vp, _i, C.POINTER(_vp)]),
    "sw_moe_graph_launch": (_i, [_vp, _vp]),
    "sw_moe_graph_destroy": (None, [_vp]),
    "sw_moe_route": (_i, [_vp, _pd, _pl, _vp, _i, _vp]),
    "sw_moe_experts": (_i, [_vp, _pd, _pl, _vp, _vp, _i, _vp]),
    "sw_moe_finish": (_i, [_vp, _pd, _pl, _vp, _vp, _vp, _i, _vp]),
    "sw_moe_shared": (_i, [_vp, _pd, _pl, _vp, _i, _vp]),
    "sw_moe_experts_routed": (_i, [_vp, _pd, _pl, _vp, _vp, _vp, _vp, _i, _vp]),
    "sw_ep_unique_id": (_i, [_vp]),
    "sw_ep_create": (_i, [C.POINTER(_vp), _vp, _vp, _i, _i, _i, _i, _i]),
    "sw_ep_destroy": (None, [_vp]),
    "sw_ep_forward": (_i, [_vp, _pd, _pl, _vp, _vp, _i, _i, _i, _vp]),
    "sw_ep_segments": (_i, [_vp, C.POINTER(C.c_float), _i]),
    "sw_moe_capture_stream": (_vp, [_vp]),
    "sw_moe_capture_begin": (_i, [_vp]),
    "sw_moe_capture_end": (_i, [_vp, C.POINTER(_vp)]),
    "sw_layer_load": (_i, [C.c_char_p, _i, _i, _i, _i, _pl, C.POINTER(_i), C.POINTER(_vp)]),
    "sw_layer_free": (None, [_vp]),
    "sw_moe_route_static": (_i, [_pd, _pl, _vp, _i, _vp, _vp, _vp]),
    "sw_moe_get_routing": (_i, [_vp, _vp, _vp, _vp, C.POINTER(_i), _vp, _vp, _vp, _vp, _vp]),
    "sw_moe_status": (_i, [_vp]),
    "sw_moe_last_path": (_i, [_vp]),
    "sw_moe_set_option": (_i, [_vp, _i, _i]),
    "sw_moe_validate": (_i, [_pd, _pl, _vp, _vp]),
    "sw_test_fail_after": (None, [_i]),
    "sw_test_fail_alloc": (None, [_i]),
    "sw_moe_test_wait_timeout": (_i, [_vp, _i]),
    "sw_selftest_host": (_i, []),
    "sw_moe_profile": (_i, [_vp, _i]),
    "sw_moe_profile_read": (_i, [_vp, C.POINTER(C.c_float), C.POINTER(_i)]),
    "sw_moe_stage_count": (_i, []),
    "sw_moe_stage_name": (C.c_char_p, [_i]),
    "sw_launch_count": (C.c_longlong, []),
    "sw_last_error": (C.c_char_p, []),
}

_lib = None


def lib():
    """The loaded shared library with typed entry points; raises if it was never built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s is missing: run `python -m sabrewing_b200.build` (nvcc, sm_100a). "
                               "There is no CPU fallback." % LIB_PATH)
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def last_error():
    return lib().sw_last_error().decode("utf-8", "replace")
