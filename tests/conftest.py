import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
LAYER_KEYS = ("router_w", "corr_bias", "logit_bias", "gu_q", "gu_s", "dn_q", "dn_s", "sh_gate", "sh_up", "sh_down")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


class Case:
    """One layer + tokens: host arrays, the oracle's view of them, and the config."""

    def __init__(self, cfg, arrays, x, hin=None):
        import oracle
        from sabrewing_b200 import synth
        self.cfg, self.a, self.x = cfg, arrays, np.ascontiguousarray(x, np.float32)
        self.hin = np.zeros_like(self.x) if hin is None else np.ascontiguousarray(hin, np.float32)
        if "router_bf16" not in arrays:
            arrays["router_bf16"] = synth.f32_to_bf16(arrays["router_w"])
        self.host = oracle.HostLayer(cfg.D, cfg.I, cfg.SI, cfg.E, cfg.K, cfg.route_act, cfg.use_corr_bias,
                                     cfg.norm_topk, cfg.route_scale, cfg.shared_mode, cfg.gs,
                                     **{k: arrays.get(k) for k in LAYER_KEYS})


def load_golden(name):
    from sabrewing_b200 import synth
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    D, E, K, I, SI, act, ucb, norm, shm, gs = [int(v) for v in z["cfg"]]
    cfg = synth.MoeConfig(name, D, E, K, I, SI, act, ucb, norm, float(z["route_scale"]), shm, z["x"].shape[0], 0, gs=gs)
    arrays = {k: (z[k] if k in z.files else None) for k in LAYER_KEYS}
    return Case(cfg, arrays, z["x"], z["hin"]), z


def synth_case(base, corr_bias_std=0.0, T=None, **kw):
    from sabrewing_b200 import synth
    cfg = synth.scaled(synth.CONFIGS[base], **kw)
    a = synth.make_layer(cfg, corr_bias_std=corr_bias_std)
    x = synth.make_tokens(cfg, T)
    hin = np.random.default_rng(cfg.seed + 5).standard_normal(x.shape).astype(np.float32)
    return Case(cfg, a, x, hin)


def rel_l2(a, b):
    a = np.asarray(a, np.float64); b = np.asarray(b, np.float64)
    return float(np.sqrt(((a - b) ** 2).sum() / max((b ** 2).sum(), 1e-300)))


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle.load()


@pytest.fixture(scope="session")
def ref():
    import oracle
    return oracle.load_ref()
