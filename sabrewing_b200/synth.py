"""Seeded synthetic MoE layers with the shapes, dtypes and value distributions of the
benchmark configurations (real checkpoints are not available offline).

Host generation (`make_layer`) is numpy-only and is what the parity tests use, so the
CPU checker and the GPU read the same bytes.  `make_layer_device` draws the same
distributions with torch directly in device memory for the full-size bench layers
(the int4 container produced there obeys the same per-row rule: scale = max|w|/7,
q = clamp(rint(w/scale), -8, 7), byte = (lo+8) | (hi+8)<<4; reference
c/tools/kernel_check.c:27-35).
"""
from dataclasses import dataclass, replace

import numpy as np

ROUTE_SIGMOID, ROUTE_SOFTMAX, ROUTE_SOFTPLUS = 0, 1, 2
SHARED_NONE, SHARED_UNSCALED = 0, 1


@dataclass(frozen=True)
class MoeConfig:
    name: str
    D: int
    E: int
    K: int
    I: int
    SI: int
    route_act: int
    use_corr_bias: int
    norm_topk: int
    route_scale: float
    shared_mode: int
    T: int
    seed: int
    zipf: float = 0.0       # >0: add ln(p_e), p_e ~ rank^-zipf, to the router logits
    gs: int = 0             # 0: one scale per row; >0: one scale per gs inputs


# The five benchmark configurations (shapes from the benchmark description; the
# sigmoid gate for the Laguna-shaped layers follows the reference engine,
# c/laguna.c:701,819, route_scale 2.5 its default).
CONFIGS = {
    "c1": MoeConfig("c1", 2048, 64, 8, 1024, 0, ROUTE_SOFTMAX, 0, 0, 1.0, SHARED_NONE, 32, 0),
    "c2": MoeConfig("c2", 4096, 256, 10, 1024, 1024, ROUTE_SIGMOID, 1, 1, 2.5, SHARED_UNSCALED, 32, 1),
    "c3": MoeConfig("c3", 4096, 256, 10, 1024, 1024, ROUTE_SIGMOID, 1, 1, 2.5, SHARED_UNSCALED, 4096, 2, zipf=1.1),
    "c4": MoeConfig("c4", 5120, 384, 8, 1536, 0, ROUTE_SOFTMAX, 0, 0, 1.0, SHARED_NONE, 256, 3),
    "c5": MoeConfig("c5", 7168, 512, 8, 2048, 2048, ROUTE_SOFTMAX, 0, 0, 1.0, SHARED_UNSCALED, 1024, 4),
    # the same layer with Zipf(1.1)-skewed routing (the benchmark runs the very large layer both ways)
    "c5z": MoeConfig("c5z", 7168, 512, 8, 2048, 2048, ROUTE_SOFTMAX, 0, 0, 1.0, SHARED_UNSCALED, 1024, 4, zipf=1.1),
}


def scaled(cfg, **kw):
    """A smaller layer with the same routing policy (for tests the CPU checker finishes fast)."""
    return replace(cfg, **kw)


def f32_to_bf16(a):
    """Round-to-nearest-even f32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = u + (np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1)))
    return (r >> np.uint32(16)).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def quant_rows_i4(w):
    """Per-row int4 (nibble-8) quantiser; numpy twin of the reference C rule."""
    w = np.ascontiguousarray(w, np.float32)
    mx = np.abs(w).max(axis=1)
    s = (mx / np.float32(7.0)).astype(np.float32)
    s = np.maximum(s, np.float32(1e-12))
    q = np.rint(w / s[:, None]).astype(np.int32)
    q = np.clip(q, -8, 7) + 8
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    return packed, s


def quant_rows_i4_grouped(w, gs):
    """Group-scaled int4 (one scale per gs inputs; layout of c/quant.h:167-202)."""
    w = np.ascontiguousarray(w, np.float32)
    O, I = w.shape
    ng = (I + gs - 1) // gs
    pad = ng * gs - I
    wp = np.pad(w, ((0, 0), (0, pad))).reshape(O, ng, gs)
    s = np.maximum((np.abs(wp).max(axis=2) / np.float32(7.0)).astype(np.float32), np.float32(1e-12))
    q = np.clip(np.rint(wp / s[:, :, None]).astype(np.int32), -8, 7).reshape(O, ng * gs)[:, :I] + 8
    if I % 2:
        q = np.pad(q, ((0, 0), (0, 1)))
    packed = (q[:, 0::2] | (q[:, 1::2] << 4)).astype(np.uint8)
    return packed, s


def rmsnorm_rows(x, eps=1e-6):
    """Unit-weight RMSNorm, sum of squares in double (reference c/moe_math.h:58-62)."""
    x = np.ascontiguousarray(x, np.float32)
    ss = (x.astype(np.float64) ** 2).sum(axis=1)
    inv = (np.float32(1.0) / np.sqrt((ss / x.shape[1]).astype(np.float32) + np.float32(eps))).astype(np.float32)
    return (x * inv[:, None]).astype(np.float32)


def zipf_logit_bias(E, s, rng):
    ranks = rng.permutation(E) + 1
    p = ranks.astype(np.float64) ** (-s)
    p /= p.sum()
    return np.log(p).astype(np.float32)


def make_layer(cfg, corr_bias_std=0.0):
    """Host arrays of one layer.  Returns a dict of numpy arrays (see oracle.HostLayer)."""
    rng = np.random.default_rng(cfg.seed)
    D, E, I, SI = cfg.D, cfg.E, cfg.I, cfg.SI
    a = {}
    rb = f32_to_bf16(rng.standard_normal((E, D), dtype=np.float32) * np.float32(0.02))
    a["router_bf16"] = rb
    a["router_w"] = bf16_to_f32(rb)
    a["corr_bias"] = None
    if cfg.use_corr_bias:
        a["corr_bias"] = (rng.standard_normal(E).astype(np.float32) * np.float32(corr_bias_std)).astype(np.float32)
    a["logit_bias"] = zipf_logit_bias(E, cfg.zipf, rng) if cfg.zipf > 0 else None
    quant = quant_rows_i4 if cfg.gs == 0 else (lambda w: quant_rows_i4_grouped(w, cfg.gs))
    gq, gsc, dq, dsc = [], [], [], []
    for _ in range(E):
        p, s = quant(rng.standard_normal((2 * I, D), dtype=np.float32) * np.float32(0.02)); gq.append(p); gsc.append(s)
        p, s = quant(rng.standard_normal((D, I), dtype=np.float32) * np.float32(0.02)); dq.append(p); dsc.append(s)
    a["gu_q"] = np.concatenate(gq); a["gu_s"] = np.concatenate(gsc)
    a["dn_q"] = np.concatenate(dq); a["dn_s"] = np.concatenate(dsc)
    if cfg.shared_mode != SHARED_NONE:
        a["sh_gate"] = f32_to_bf16(rng.standard_normal((SI, D), dtype=np.float32) * np.float32(0.02))
        a["sh_up"] = f32_to_bf16(rng.standard_normal((SI, D), dtype=np.float32) * np.float32(0.02))
        a["sh_down"] = f32_to_bf16(rng.standard_normal((D, SI), dtype=np.float32) * np.float32(0.02))
    else:
        a["sh_gate"] = a["sh_up"] = a["sh_down"] = None
    return a


def make_tokens(cfg, T=None, seed_offset=1000):
    """N(0,1) activations after a unit-weight RMSNorm, f32 [T, D]."""
    rng = np.random.default_rng(cfg.seed + seed_offset)
    T = cfg.T if T is None else T
    return rmsnorm_rows(rng.standard_normal((T, cfg.D), dtype=np.float32))


def make_layer_device(cfg, device, layer_index=0):
    """Same distributions drawn with torch directly in device memory (full-size bench layers).

    Returns a dict of torch tensors with the keys of `make_layer` (router_bf16 as
    torch.bfloat16 bits in int16, int4 blobs as uint8).
    """
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(cfg.seed * 1000003 + layer_index)
    D, E, I, SI = cfg.D, cfg.E, cfg.I, cfg.SI
    out = {}
    rw = (torch.randn((E, D), generator=g, device=device) * 0.02).to(torch.bfloat16)
    out["router_bf16"] = rw.view(torch.int16)
    out["router_w"] = rw.float()
    out["corr_bias"] = torch.zeros(E, device=device) if cfg.use_corr_bias else None
    if cfg.zipf > 0:
        rng = np.random.default_rng(cfg.seed + 77 + layer_index)
        out["logit_bias"] = torch.from_numpy(zipf_logit_bias(E, cfg.zipf, rng)).to(device)
    else:
        out["logit_bias"] = None

    seven = torch.full((), 7.0, dtype=torch.float32, device=device)

    def quant_dev(rows, cols, nrep):
        q = torch.empty((nrep * rows, cols // 2), dtype=torch.uint8, device=device)
        s = torch.empty((nrep * rows,), dtype=torch.float32, device=device)
        for e in range(nrep):
            w = torch.randn((rows, cols), generator=g, device=device) * 0.02
            # tensor / tensor: a true division (torch turns a division by a Python scalar into a multiplication by
            # its reciprocal, which is one ulp off the reference's max|w| / 7.0f on some rows)
            sc = (w.abs().amax(dim=1) / seven).clamp_min(1e-12)
            v = torch.round(w / sc[:, None]).clamp_(-8, 7).to(torch.int32) + 8
            q[e * rows:(e + 1) * rows] = (v[:, 0::2] | (v[:, 1::2] << 4)).to(torch.uint8)
            s[e * rows:(e + 1) * rows] = sc
        return q, s

    out["gu_q"], out["gu_s"] = quant_dev(2 * I, D, E)
    out["dn_q"], out["dn_s"] = quant_dev(D, I, E)
    if cfg.shared_mode != SHARED_NONE:
        for k, shp in (("sh_gate", (SI, D)), ("sh_up", (SI, D)), ("sh_down", (D, SI))):
            out[k] = (torch.randn(shp, generator=g, device=device) * 0.02).to(torch.bfloat16).view(torch.int16)
    else:
        out["sh_gate"] = out["sh_up"] = out["sh_down"] = None
    return out
