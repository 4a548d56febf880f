"""Host-side mirror of the reference's MoE-block interface over the C-ABI.

`MoeDesc` carries the reference's descriptor fields (c/moe_arch.h:33-41); `MoeLayer`
holds what the reference's hooks reach through engine state (router weights,
correction bias, int4 expert container, bf16 shared expert; c/moe_arch.h:45-55,
c/laguna.c:572-617) as device tensors.  `MoeBlock.forward(x, out)` is
`out += MoE(x)` exactly like moe_block()/lag_moe_rows() (c/moe_block.h:18-54,
c/laguna.c:805-823).  torch is used for device memory and streams only.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import capi


@dataclass
class MoeDesc:
    n_experts: int
    topk: int
    route_act: int = capi.ROUTE_SIGMOID
    use_corr_bias: int = 0
    norm_topk: int = 0
    route_scale: float = 1.0
    shared_mode: int = capi.SHARED_NONE

    def c(self):
        return capi.SwMoeDesc(self.n_experts, self.topk, self.route_act, self.use_corr_bias,
                              self.norm_topk, self.route_scale, self.shared_mode)


def desc_from_config(cfg):
    return MoeDesc(cfg.E, cfg.K, cfg.route_act, cfg.use_corr_bias, cfg.norm_topk, cfg.route_scale, cfg.shared_mode)


def _dev(t, device, dtype=None):
    if t is None:
        return None
    if isinstance(t, np.ndarray):
        if t.dtype == np.uint16:
            t = torch.from_numpy(t.view(np.int16))
        else:
            t = torch.from_numpy(t)
    t = t.to(device)
    if dtype is not None:
        t = t.to(dtype)
    return t.contiguous()


class MoeLayer:
    """Device-resident weights of one layer (optionally one expert-parallel shard of it)."""

    def __init__(self, D, I, SI, arrays, device, router="bf16", expert_lo=0, expert_cnt=0, n_experts=None, gs=0):
        a = arrays
        self.D, self.I, self.SI, self.gs = D, I, SI, gs
        self.device = torch.device(device)
        if router == "bf16":
            self.router_w = _dev(a["router_bf16"], device); self.router_dtype = capi.DTYPE_BF16
        else:
            self.router_w = _dev(a["router_w"], device, torch.float32); self.router_dtype = capi.DTYPE_F32
        self.corr_bias = _dev(a.get("corr_bias"), device)
        self.logit_bias = _dev(a.get("logit_bias"), device)
        self.expert_lo, self.expert_cnt = expert_lo, expert_cnt
        gu_q, gu_s, dn_q, dn_s = a["gu_q"], a["gu_s"], a["dn_q"], a["dn_s"]
        if expert_cnt > 0:       # keep only the rows of the resident experts (scales are [rows] or [rows, groups])
            lo, hi = expert_lo, expert_lo + expert_cnt
            gu_q, gu_s = gu_q[lo * 2 * I:hi * 2 * I], gu_s[lo * 2 * I:hi * 2 * I]
            dn_q, dn_s = dn_q[lo * D:hi * D], dn_s[lo * D:hi * D]
        self.gu_q, self.gu_s = _dev(gu_q, device), _dev(gu_s, device)
        self.dn_q, self.dn_s = _dev(dn_q, device), _dev(dn_s, device)
        self.sh_gate, self.sh_up, self.sh_down = (_dev(a.get(k), device) for k in ("sh_gate", "sh_up", "sh_down"))
        self.sh_gate_w = _dev(a.get("sh_gate_w"), device)                 # qwen35-style one-row gate of the shared expert
        self.route_global_scale = float(a.get("route_global_scale", 0.0) or 0.0)

    @staticmethod
    def _p(t):
        return None if t is None else t.data_ptr()

    def c(self):
        p = self._p
        return capi.SwMoeLayer(self.D, self.I, self.SI, self.router_dtype, p(self.router_w), p(self.corr_bias),
                               p(self.logit_bias), p(self.gu_q), p(self.gu_s), p(self.dn_q), p(self.dn_s),
                               p(self.sh_gate), p(self.sh_up), p(self.sh_down), self.expert_lo, self.expert_cnt, self.gs,
                               p(self.sh_gate_w), self.route_global_scale)

    def expert_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.gu_q, self.gu_s, self.dn_q, self.dn_s))


class _RawStream:
    """A CUDA stream handle with the attribute the block's stream arguments read."""

    def __init__(self, handle):
        self.cuda_stream = handle


class MoeGraph:
    """A captured block call; replay() launches it on a stream."""

    def __init__(self, block, handle, last, keep):
        self.block, self.handle, self._last, self._keep = block, handle, last, keep

    def replay(self, stream=None):
        b = self.block
        b._last = self._last
        b._chk(b.lib.sw_moe_graph_launch(self.handle, b._stream(stream)), "sw_moe_graph_launch")

    def close(self):
        if self.handle:
            self.block.lib.sw_moe_graph_destroy(self.handle)
            self.handle = C.c_void_p()


class MoeBlock:
    """One scratch context; run any layer whose sizes fit the limits given here."""

    def __init__(self, device, max_tokens, n_experts, topk, D, I, SI=0):
        self.lib = capi.lib()
        self.device = torch.device(device)
        idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.ctx = C.c_void_p()
        rc = self.lib.sw_moe_ctx_create(C.byref(self.ctx), idx, max_tokens, n_experts, topk, D, I, SI)
        if rc != 0:
            raise RuntimeError("sw_moe_ctx_create: " + capi.last_error())
        self.limits = (max_tokens, n_experts, topk, D, I, SI)
        self._last = None

    def close(self):
        if self.ctx:
            self.lib.sw_moe_ctx_destroy(self.ctx)
            self.ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _stream(self, stream):
        if stream is None:
            stream = torch.cuda.current_stream(self.device)
        return C.c_void_p(stream.cuda_stream)

    def _chk(self, rc, what):
        if rc != 0:
            raise RuntimeError("%s: %s" % (what, capi.last_error()))

    def forward(self, desc, layer, x, out, stream=None):
        """out[T,D] += MoE(x[T,D]); x, out f32 device tensors; asynchronous on `stream`."""
        assert x.is_cuda and out.is_cuda and x.dtype == torch.float32 and out.dtype == torch.float32
        assert x.is_contiguous() and out.is_contiguous() and x.shape == out.shape
        T = x.shape[0]
        d, l = desc.c(), layer.c()
        self._last = (T, desc.topk, desc.n_experts)
        self._chk(self.lib.sw_moe_forward(self.ctx, C.byref(d), C.byref(l), x.data_ptr(), out.data_ptr(), T,
                                          self._stream(stream)), "sw_moe_forward")
        return out

    def forward_norm(self, desc, layer, h, norm_w, eps, stream=None):
        """h[T,D] += MoE(rmsnorm(h) * norm_w): the layer tail with the residual stream on the device (c/laguna.c:1119,1126)."""
        d, l = desc.c(), layer.c()
        self._last = (h.shape[0], desc.topk, desc.n_experts)
        self._chk(self.lib.sw_moe_forward_norm(self.ctx, C.byref(d), C.byref(l), h.data_ptr(), norm_w.data_ptr(), eps, h.shape[0],
                                               self._stream(stream)), "sw_moe_forward_norm")
        return h

    def graph(self, desc, layer, x, out):
        """Capture forward(desc, layer, x, out) into a CUDA graph (runs the block twice on `out` while doing so)."""
        d, l = desc.c(), layer.c()
        g = C.c_void_p()
        self._chk(self.lib.sw_moe_graph_create(self.ctx, C.byref(d), C.byref(l), x.data_ptr(), out.data_ptr(), x.shape[0],
                                               C.byref(g)), "sw_moe_graph_create")
        return MoeGraph(self, g, (x.shape[0], desc.topk, desc.n_experts), (layer, x, out))

    def forward_host(self, desc, layer, x_host, out_host):
        """Same through host numpy buffers (H2D, block, D2H, sync); out_host updated in place."""
        assert x_host.dtype == np.float32 and out_host.dtype == np.float32
        assert x_host.flags.c_contiguous and out_host.flags.c_contiguous and x_host.shape == out_host.shape
        T = x_host.shape[0]
        d, l = desc.c(), layer.c()
        self._last = (T, desc.topk, desc.n_experts)
        self._chk(self.lib.sw_moe_forward_host(self.ctx, C.byref(d), C.byref(l), x_host.ctypes.data,
                                               out_host.ctypes.data, T), "sw_moe_forward_host")
        return out_host

    def route(self, desc, layer, x, stream=None):
        T = x.shape[0]
        d, l = desc.c(), layer.c()
        self._last = (T, desc.topk, desc.n_experts)
        self._chk(self.lib.sw_moe_route(self.ctx, C.byref(d), C.byref(l), x.data_ptr(), T, self._stream(stream)),
                  "sw_moe_route")

    def experts(self, desc, layer, x, routed, stream=None):
        d, l = desc.c(), layer.c()
        self._chk(self.lib.sw_moe_experts(self.ctx, C.byref(d), C.byref(l), x.data_ptr(), routed.data_ptr(),
                                          x.shape[0], self._stream(stream)), "sw_moe_experts")
        return routed

    def experts_routed(self, desc, layer, x, sel, w, routed, stream=None):
        """routed = weighted sum over the resident experts for routing given by the caller (sel int32 [T,K] with -1 =
        no expert, w f32 [T,K]; device tensors)."""
        d, l = desc.c(), layer.c()
        self._last = (x.shape[0], desc.topk, desc.n_experts)
        self._chk(self.lib.sw_moe_experts_routed(self.ctx, C.byref(d), C.byref(l), x.data_ptr(), sel.data_ptr(), w.data_ptr(),
                                                 routed.data_ptr(), x.shape[0], self._stream(stream)), "sw_moe_experts_routed")
        return routed

    def shared(self, desc, layer, x, stream=None):
        """The shared expert of x ahead of time; the next finish() with as many rows uses it."""
        d, l = desc.c(), layer.c()
        self._chk(self.lib.sw_moe_shared(self.ctx, C.byref(d), C.byref(l), x.data_ptr(), x.shape[0], self._stream(stream)),
                  "sw_moe_shared")

    def finish(self, desc, layer, x, routed, out, stream=None):
        d, l = desc.c(), layer.c()
        self._chk(self.lib.sw_moe_finish(self.ctx, C.byref(d), C.byref(l), x.data_ptr(), routed.data_ptr(),
                                         out.data_ptr(), x.shape[0], self._stream(stream)), "sw_moe_finish")
        return out

    def capture(self, fn, keep=()):
        """Record the stage calls `fn(stream)` makes (route / experts / shared / finish with that stream) into a
        MoeGraph.  fn must already have run once eagerly with the same arguments."""
        self._chk(self.lib.sw_moe_capture_begin(self.ctx), "sw_moe_capture_begin")
        cs = _RawStream(self.lib.sw_moe_capture_stream(self.ctx))
        h = C.c_void_p()
        try:
            fn(cs)
        finally:
            rc = self.lib.sw_moe_capture_end(self.ctx, C.byref(h))
        self._chk(rc, "sw_moe_capture_end")
        return MoeGraph(self, h, self._last, keep)

    def routing(self, want_scores=False):
        """Host copies of the last routing: sel, w, G, gexp, gbeg, gcnt, grow, rowof (c/laguna.c:709-723)."""
        T, K, E = self._last
        sel = np.empty((T, K), np.int32); w = np.empty((T, K), np.float32)
        sc = np.empty((T, E), np.float32) if want_scores else None
        G = C.c_int(0)
        gexp = np.empty(E, np.int32); gbeg = np.empty(E, np.int32); gcnt = np.empty(E, np.int32)
        grow = np.empty(T * K, np.int32); rowof = np.empty(T * K, np.int32)
        p = lambda a: None if a is None else a.ctypes.data
        self._chk(self.lib.sw_moe_get_routing(self.ctx, p(sel), p(w), p(sc), C.byref(G), p(gexp), p(gbeg), p(gcnt),
                                              p(grow), p(rowof)), "sw_moe_get_routing")
        g = G.value
        r = dict(sel=sel, w=w, G=g, gexp=gexp[:g].copy(), gbeg=gbeg[:g].copy(), gcnt=gcnt[:g].copy(),
                 grow=grow, rowof=rowof)
        if want_scores:
            r["scores"] = sc
        return r

    def profile(self, enable=True):
        """Start (or stop) per-stage CUDA-event timing of forward(); see profile_read()."""
        self._chk(self.lib.sw_moe_profile(self.ctx, 1 if enable else 0), "sw_moe_profile")

    def profile_read(self):
        """{stage name: total ms}, calls recorded since profile(True)."""
        n = self.lib.sw_moe_stage_count()
        ms = (C.c_float * n)(); calls = C.c_int(0)
        self._chk(self.lib.sw_moe_profile_read(self.ctx, ms, C.byref(calls)), "sw_moe_profile_read")
        return {self.lib.sw_moe_stage_name(i).decode(): float(ms[i]) for i in range(n)}, calls.value

    def status(self):
        return self.lib.sw_moe_status(self.ctx)
