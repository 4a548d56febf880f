"""CPU checker for the MoE-block hot path.  TEST INFRASTRUCTURE ONLY.

`oracle.load()` gives ctypes access to the C restatement (moe_oracle.c);
`oracle.load_ref()` to the reference's own code compiled in place (ref_shim.c),
or None when that library was never built.  Only tests, the smoke check and the
bench's CPU-baseline / reference arm import this package; the shipped library and
the `sabrewing_b200` package never do.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

ROUTE_SIGMOID, ROUTE_SOFTMAX = 0, 1
SHARED_NONE, SHARED_UNSCALED = 0, 1


class Layer(C.Structure):
    """Mirror of OrcLayer / RefLayer (moe_oracle.c, ref_shim.c)."""
    _fields_ = [
        ("D", C.c_int), ("I", C.c_int), ("SI", C.c_int), ("E", C.c_int), ("K", C.c_int),
        ("route_act", C.c_int), ("use_corr_bias", C.c_int), ("norm_topk", C.c_int),
        ("route_scale", C.c_float), ("shared_mode", C.c_int), ("gs", C.c_int),
        ("router_w", C.c_void_p), ("corr_bias", C.c_void_p), ("logit_bias", C.c_void_p),
        ("gu_q", C.c_void_p), ("gu_s", C.c_void_p), ("dn_q", C.c_void_p), ("dn_s", C.c_void_p),
        ("sh_gate", C.c_void_p), ("sh_up", C.c_void_p), ("sh_down", C.c_void_p),
    ]


def _cpu_flags():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def isa_level():
    """'v4' when the host can run the AVX-512 build, else 'v3'."""
    need = {"avx512f", "avx512bw", "avx512cd", "avx512dq", "avx512vl"}
    return "v4" if need <= _cpu_flags() else "v3"


def reference_dir():
    """The c/ directory of the reference checkout: $SABREWING_REF, else ../reference/c beside this repository.

    None when neither holds laguna.c (the compiled reference under _ref/ is then used as shipped)."""
    cands = [os.environ.get("SABREWING_REF"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference", "c")]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "laguna.c")):
            return c
    return None


def build(ref_dir=None):
    """Compile the restatement; with a reference checkout at hand also the in-place reference builds:
    the CPU path (ref), the reference engine linked against this repository's library (dropin) and the
    reference's CUDA tier for sm_100a (refcuda).  An explicit ref_dir that does not exist is an error."""
    subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
    if ref_dir is None:
        ref_dir = reference_dir()
        if ref_dir is None:
            return
    elif not os.path.isfile(os.path.join(ref_dir, "laguna.c")):
        raise FileNotFoundError("no reference checkout at %r (set SABREWING_REF=<checkout>/c)" % ref_dir)
    subprocess.run(["make", "-C", _HERE, "ref", "REF=" + ref_dir], check=True, capture_output=True)
    swlib = os.path.join(os.path.dirname(_HERE), "sabrewing_b200", "libsabrewing_b200.so")
    if os.path.exists(swlib):
        subprocess.run(["make", "-C", _HERE, "dropin", "REF=" + ref_dir], check=True, capture_output=True)
    if os.path.exists("/usr/local/cuda/bin/nvcc") or os.environ.get("NVCC"):
        subprocess.run(["make", "-C", _HERE, "refcuda", "REF=" + ref_dir], check=True, capture_output=True)


DROPIN_PATH = os.path.join(_HERE, "_ref", "laguna_dropin")
REF_CUDA_PATH = os.path.join(_HERE, "_ref", "libref_cuda_laguna.so")


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


_F = C.POINTER(C.c_float)
_I = C.POINTER(C.c_int)
_vp = C.c_void_p


class _Lib:
    """Thin typed wrapper; `prefix` is 'orc_' or 'ref_'."""

    def __init__(self, path, prefix):
        self.path, self.prefix = path, prefix
        self.lib = C.CDLL(path)

    def fn(self, name):
        return getattr(self.lib, self.prefix + name)

    # ---- kernels -------------------------------------------------------------
    def matmul_f32(self, x, W, exact=1):
        S, I = x.shape; O = W.shape[0]
        y = np.empty((S, O), np.float32)
        f = self.fn("matmul_f32"); f.restype = None
        f(_ptr(y), _ptr(x), _ptr(W), C.c_int(S), C.c_int(I), C.c_int(O), C.c_int(exact))
        return y

    def matmul_bf16(self, x, W, exact=1):
        S, I = x.shape; O = W.shape[0]
        y = np.empty((S, O), np.float32)
        f = self.fn("matmul_bf16"); f.restype = None
        f(_ptr(y), _ptr(x), _ptr(W), C.c_int(S), C.c_int(I), C.c_int(O), C.c_int(exact))
        return y

    def matmul_q4(self, x, packed, scale, exact=1):
        S, I = x.shape; O = packed.shape[0]
        y = np.empty((S, O), np.float32)
        f = self.fn("matmul_q4"); f.restype = None
        f(_ptr(y), _ptr(x), _ptr(packed), _ptr(scale), C.c_int(S), C.c_int(I), C.c_int(O), C.c_int(exact))
        return y

    def matmul_fp4(self, x, packed, es, exact=1):
        """y[S,O] for e2m1 codes `packed` [O, I/2] and ue8m0 exponents `es` [O, I/32]."""
        S, I = x.shape; O = packed.shape[0]
        y = np.empty((S, O), np.float32)
        f = self.fn("matmul_fp4"); f.restype = None
        f(_ptr(y), _ptr(x), _ptr(packed), _ptr(es), C.c_int(S), C.c_int(I), C.c_int(O), C.c_int(exact))
        return y

    def experts_fp4(self, x, gu_q, gu_es, dn_q, dn_es, sel, w, I, D, limit, exact=1):
        """out[D] = sum_a w[a] * fp4 expert sel[a] of one token x[D] with the clamped SwiGLU."""
        out = np.empty(D, np.float32); h = np.empty(2 * I + D, np.float32)
        sel = np.ascontiguousarray(sel, np.int32); w = np.ascontiguousarray(w, np.float32)
        f = self.fn("experts_fp4"); f.restype = None
        f(_ptr(out), _ptr(x), _ptr(gu_q), _ptr(gu_es), _ptr(dn_q), _ptr(dn_es), _ptr(sel), _ptr(w),
          C.c_int(len(sel)), C.c_int(I), C.c_int(D), C.c_float(limit), C.c_int(exact), _ptr(h))
        return out

    def matmul_i4_grouped(self, x, q4, scale, gs, exact=0):
        S, I = x.shape; O = q4.shape[0]
        y = np.empty((S, O), np.float32)
        f = self.fn("matmul_i4_grouped"); f.restype = None
        if self.prefix == "ref_":
            f(_ptr(y), _ptr(x), _ptr(q4), _ptr(scale), C.c_int(S), C.c_int(I), C.c_int(O), C.c_int(gs))
        else:
            f(_ptr(y), _ptr(x), _ptr(q4), _ptr(scale), C.c_int(S), C.c_int(I), C.c_int(O), C.c_int(gs), C.c_int(exact))
        return y

    def quant_rows_i4(self, w):
        rows, I = w.shape
        packed = np.empty((rows, I // 2), np.uint8); scale = np.empty(rows, np.float32)
        f = self.fn("quant_rows_i4"); f.restype = None
        f(_ptr(w), C.c_int(rows), C.c_int(I), _ptr(packed), _ptr(scale))
        return packed, scale

    def softmax_row(self, x):
        y = np.array(x, np.float32, copy=True)
        f = self.fn("softmax_row"); f.restype = None
        f(_ptr(y), C.c_int(y.size))
        return y

    def topk(self, score, bias, use_bias, K):
        sel = np.full(K, -1, np.int32)
        f = self.fn("topk"); f.restype = None
        f(_ptr(score), _ptr(bias), C.c_int(use_bias), C.c_int(score.size), C.c_int(K), _ptr(sel))
        return sel

    def rmsnorm_rows(self, x, w=None, eps=1e-6):
        S, D = x.shape
        out = np.empty_like(x)
        if w is None and self.prefix == "ref_":
            w = np.ones(D, np.float32)
        f = self.fn("rmsnorm_rows"); f.restype = None
        f(_ptr(out), _ptr(x), _ptr(w), C.c_int(S), C.c_int(D), C.c_float(eps))
        return out

    def set_threads(self, n):
        f = self.fn("set_threads"); f.restype = None; f(C.c_int(n))

    def threads(self):
        f = self.fn("threads"); f.restype = C.c_int; return f()


class Oracle(_Lib):
    def __init__(self, path):
        super().__init__(path, "orc_")

    def route(self, layer, x, exact=1, want_scores=False):
        S = x.shape[0]; K = layer.c.K; E = layer.c.E
        sel = np.empty((S, K), np.int32); w = np.empty((S, K), np.float32)
        sc = np.empty((S, E), np.float32) if want_scores else None
        f = self.fn("route"); f.restype = None
        f(C.byref(layer.c), _ptr(x), C.c_int(S), C.c_int(exact), _ptr(sel), _ptr(w), _ptr(sc))
        return (sel, w, sc) if want_scores else (sel, w)

    def group(self, sel, E):
        S, K = sel.shape; T = S * K
        gexp = np.empty(E, np.int32); gbeg = np.empty(E, np.int32); gcnt = np.empty(E, np.int32)
        grow = np.empty(T, np.int32); rowof = np.empty(T, np.int32)
        f = self.fn("group"); f.restype = C.c_int
        G = f(_ptr(sel), C.c_int(S), C.c_int(K), C.c_int(E), _ptr(gexp), _ptr(gbeg), _ptr(gcnt), _ptr(grow), _ptr(rowof))
        return dict(G=G, gexp=gexp[:G].copy(), gbeg=gbeg[:G].copy(), gcnt=gcnt[:G].copy(), grow=grow, rowof=rowof)

    def moe_rows(self, layer, x, hin=None, exact=1):
        S, D = x.shape
        h = np.zeros((S, D), np.float32) if hin is None else np.array(hin, np.float32, copy=True)
        f = self.fn("moe_rows"); f.restype = None
        f(C.byref(layer.c), _ptr(x), _ptr(h), C.c_int(S), C.c_int(exact))
        return h

    def moe_group(self, layer, x, hin=None, exact=1):
        """Returns dict: out, sel, w, G, gexp, gbeg, gcnt, grow, rowof, routed."""
        S, D = x.shape; K = layer.c.K; E = layer.c.E; T = S * K
        h = np.zeros((S, D), np.float32) if hin is None else np.array(hin, np.float32, copy=True)
        sel = np.empty((S, K), np.int32); w = np.empty((S, K), np.float32)
        G = C.c_int(0)
        gexp = np.empty(E, np.int32); gbeg = np.empty(E, np.int32); gcnt = np.empty(E, np.int32)
        grow = np.empty(T, np.int32); rowof = np.empty(T, np.int32)
        routed = np.empty((S, D), np.float32)
        f = self.fn("moe_group"); f.restype = None
        f(C.byref(layer.c), _ptr(x), _ptr(h), C.c_int(S), C.c_int(exact), _ptr(sel), _ptr(w), C.byref(G),
          _ptr(gexp), _ptr(gbeg), _ptr(gcnt), _ptr(grow), _ptr(rowof), _ptr(routed))
        g = G.value
        return dict(out=h, sel=sel, w=w, G=g, gexp=gexp[:g].copy(), gbeg=gbeg[:g].copy(), gcnt=gcnt[:g].copy(),
                    grow=grow, rowof=rowof, routed=routed)

    def experts_given_routing(self, layer, x, sel, w, exact=1):
        S, D = x.shape
        routed = np.empty((S, D), np.float32)
        sel = np.ascontiguousarray(sel, np.int32); w = np.ascontiguousarray(w, np.float32)
        f = self.fn("experts_given_routing"); f.restype = None
        f(C.byref(layer.c), _ptr(x), C.c_int(S), _ptr(sel), _ptr(w), _ptr(routed), C.c_int(exact))
        return routed

    def shared_rows(self, layer, x, exact=1):
        S, D = x.shape
        so = np.empty((S, D), np.float32)
        f = self.fn("shared_rows"); f.restype = None
        f(C.byref(layer.c), _ptr(x), C.c_int(S), _ptr(so), C.c_int(exact))
        return so


class Reference(_Lib):
    """The reference's own code (compiled in place from its sources)."""

    def __init__(self, path):
        super().__init__(path, "ref_")

    def laguna_moe_rows(self, layer, x, hin=None, exact=1, group_on=1):
        S, D = x.shape
        h = np.zeros((S, D), np.float32) if hin is None else np.array(hin, np.float32, copy=True)
        f = self.fn("laguna_moe_rows"); f.restype = C.c_int
        rc = f(C.byref(layer.c), _ptr(x), _ptr(h), C.c_int(S), C.c_int(exact), C.c_int(group_on))
        if rc != 0:
            raise ValueError("layer is not expressible by the Laguna engine glue")
        return h

    def moe_block_rows(self, layer, x, hin=None, exact=1):
        S, D = x.shape
        h = np.zeros((S, D), np.float32) if hin is None else np.array(hin, np.float32, copy=True)
        f = self.fn("moe_block_rows"); f.restype = C.c_int
        rc = f(C.byref(layer.c), _ptr(x), _ptr(h), C.c_int(S), C.c_int(exact))
        if rc != 0:
            raise ValueError("layer is not expressible by moe_block hooks")
        return h

    def omp_autotune(self):
        f = self.fn("omp_autotune"); f.restype = None; f()

    def physical_cores(self):
        f = self.fn("physical_cores"); f.restype = C.c_int; return f()

    def has_avx512(self):
        f = self.fn("has_avx512"); f.restype = C.c_int; return bool(f())


class HostLayer:
    """Keeps the numpy arrays of one layer alive next to the C struct that points at them.

    `arrays` keys: router_w f32 [E,D]; corr_bias/logit_bias f32 [E] or None;
    gu_q u8 [E*2I, D/2], gu_s f32; dn_q u8 [E*D, I/2], dn_s f32;
    sh_gate/sh_up u16 [SI,D], sh_down u16 [D,SI] or None.
    """

    def __init__(self, D, I, SI, E, K, route_act, use_corr_bias, norm_topk, route_scale, shared_mode, gs=0, **arrays):
        self.a = {k: (None if v is None else np.ascontiguousarray(v)) for k, v in arrays.items()}
        g = self.a.get
        self.c = Layer(D, I, SI, E, K, route_act, use_corr_bias, norm_topk, route_scale, shared_mode, gs,
                       _ptr(g("router_w")), _ptr(g("corr_bias")), _ptr(g("logit_bias")),
                       _ptr(g("gu_q")), _ptr(g("gu_s")), _ptr(g("dn_q")), _ptr(g("dn_s")),
                       _ptr(g("sh_gate")), _ptr(g("sh_up")), _ptr(g("sh_down")))


_cache = {}


def load():
    """The C restatement; built on first use (gcc is part of the toolchain)."""
    if "orc" not in _cache:
        path = os.path.join(_HERE, "liboracle_%s.so" % isa_level())
        if not os.path.exists(path):
            subprocess.run(["make", "-C", _HERE, "all"], check=True, capture_output=True)
        _cache["orc"] = Oracle(path)
    return _cache["orc"]


def load_ref():
    """The compiled reference, or None when oracle/_ref/ holds no library."""
    if "ref" not in _cache:
        path = os.path.join(_HERE, "_ref", "libref_%s.so" % isa_level())
        _cache["ref"] = Reference(path) if os.path.exists(path) else None
    return _cache["ref"]
