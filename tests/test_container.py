"""The int4 container: the converter's quantiser and file layout (CPU), and the loader that reads a layer from the
file straight into device memory (GPU).  Layout and names follow the reference's container (docs/laguna.md:34-42,
c/tools/convert_laguna_int4.py:49-59, c/laguna.c:410-446)."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import synth_case, rel_l2


def test_converter_quantiser_matches_the_reference_rule(orc):
    from sabrewing_b200 import convert
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((64, 256)) * 0.02).astype(np.float32)
    q, s = convert.quant_int4_rows(w)
    qr, sr = orc.quant_rows_i4(w)                 # bit-equal to the reference's quant_row_i4 (floor 1e-12 instead of 1e-8)
    assert np.array_equal(s, sr) and np.array_equal(q, qr)
    z = np.zeros((2, 8), np.float32)
    assert convert.quant_int4_rows(z)[1].tolist() == [np.float32(1e-8)] * 2       # the converter's floor


def test_container_file_is_plain_safetensors(tmp_path):
    """The writer's output is read back by the stock safetensors package: names, dtypes, shapes and bytes."""
    from safetensors import safe_open
    from sabrewing_b200 import convert
    case = synth_case("c2", corr_bias_std=0.01, T=2, D=128, E=4, K=2, I=64, SI=64)
    a = case.a
    path = str(tmp_path / "layer3.safetensors")
    convert.write_safetensors(path, convert.layer_tensors(3, a["router_w"], a["corr_bias"], a["gu_q"], a["gu_s"], a["dn_q"], a["dn_s"],
                                                          a["sh_gate"], a["sh_up"], a["sh_down"]))
    with safe_open(path, framework="np") as f:
        names = set(f.keys())
        p = "model.layers.3.mlp."
        assert {p + "gate.weight", p + "experts.e_score_correction_bias", p + "experts.gate_up_proj", p + "experts.gate_up_proj.qs",
                p + "experts.down_proj", p + "experts.down_proj.qs", p + "shared_expert.gate_proj.weight"} <= names
        assert np.array_equal(f.get_tensor(p + "experts.gate_up_proj"), a["gu_q"])
        assert np.array_equal(f.get_tensor(p + "experts.down_proj.qs"), a["dn_s"])
        assert f.get_slice(p + "gate.weight").get_shape() == [4, 128]


def test_convert_layer_fuses_gate_and_up_rows_per_expert(tmp_path, orc):
    from safetensors import safe_open
    from sabrewing_b200 import convert
    rng = np.random.default_rng(5)
    E, D, I = 3, 64, 32
    experts = [tuple((rng.standard_normal(s) * 0.02).astype(np.float32) for s in ((I, D), (I, D), (D, I))) for _ in range(E)]
    path = str(tmp_path / "l0.safetensors")
    convert.convert_layer(path, 0, rng.standard_normal((E, D)).astype(np.float32), None, experts)
    with safe_open(path, framework="np") as f:
        gu = f.get_tensor("model.layers.0.mlp.experts.gate_up_proj"); gs = f.get_tensor("model.layers.0.mlp.experts.gate_up_proj.qs")
        assert gu.shape == (E * 2 * I, D // 2)
        for e, (g, u, d) in enumerate(experts):                 # gate rows then up rows of expert e start at row e*2I
            q, s = orc.quant_rows_i4(np.concatenate([g, u]))
            assert np.array_equal(gu[e * 2 * I:(e + 1) * 2 * I], q) and np.array_equal(gs[e * 2 * I:(e + 1) * 2 * I], s)


@pytest.mark.gpu
def test_loader_reads_a_layer_into_device_memory(tmp_path, orc):
    import torch
    from sabrewing_b200 import capi, convert
    from sabrewing_b200.moe_block import MoeBlock, MoeLayer, desc_from_config
    case = synth_case("c2", corr_bias_std=0.01, T=16, D=512, E=16, K=4, I=128, SI=128)
    cfg, a = case.cfg, case.a
    os.makedirs(tmp_path / "snap")
    # two files, as a sharded snapshot: layer 7 in one, an unrelated layer in the other
    convert.write_safetensors(str(tmp_path / "snap" / "model-00001.safetensors"),
                              convert.layer_tensors(2, a["router_w"], None, a["gu_q"], a["gu_s"], a["dn_q"], a["dn_s"]))
    convert.write_safetensors(str(tmp_path / "snap" / "model-00002.safetensors"),
                              convert.layer_tensors(7, a["router_w"], a["corr_bias"], a["gu_q"], a["gu_s"], a["dn_q"], a["dn_s"],
                                                    a["sh_gate"], a["sh_up"], a["sh_down"]))
    lib = capi.lib()
    layer = capi.SwMoeLayer(); h = C.c_void_p(); ne = C.c_int(0)
    assert lib.sw_layer_load(str(tmp_path / "snap").encode(), 7, 0, 0, 0, C.byref(layer), C.byref(ne), C.byref(h)) == 0, capi.last_error()
    assert (ne.value, layer.D, layer.I, layer.SI, layer.router_dtype) == (cfg.E, cfg.D, cfg.I, cfg.SI, capi.DTYPE_F32)
    blk = MoeBlock("cuda:0", 16, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    d = desc_from_config(cfg).c()
    x = torch.from_numpy(case.x).cuda(); out = torch.from_numpy(case.hin).cuda()
    assert lib.sw_moe_forward(blk.ctx, C.byref(d), C.byref(layer), x.data_ptr(), out.data_ptr(), 16, None) == 0, capi.last_error()
    torch.cuda.synchronize()
    # same bits as the layer uploaded from the arrays (f32 router)
    ref_layer = MoeLayer(cfg.D, cfg.I, cfg.SI, a, "cuda:0", router="f32")
    out2 = torch.from_numpy(case.hin).cuda()
    blk.forward(desc_from_config(cfg), ref_layer, x, out2)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
    want = orc.moe_group(case.host, case.x, case.hin, exact=1)
    assert rel_l2(out.cpu().numpy() - case.hin, want["out"] - case.hin) < 1e-3
    # an expert-parallel shard: only the rows of experts [4, 12)
    shard = capi.SwMoeLayer(); hs = C.c_void_p()
    assert lib.sw_layer_load(str(tmp_path / "snap" / "model-00002.safetensors").encode(), 7, 0, 4, 8, C.byref(shard), None, C.byref(hs)) == 0
    assert (shard.expert_lo, shard.expert_cnt) == (4, 8)
    # the shard through the block: its partial sums equal those of the same shard uploaded from the arrays
    blk2 = MoeBlock("cuda:0", 16, cfg.E, cfg.K, cfg.D, cfg.I, cfg.SI)
    routed_shard = torch.empty_like(x); routed_ref = torch.empty_like(x)
    assert lib.sw_moe_route(blk2.ctx, C.byref(d), C.byref(shard), x.data_ptr(), 16, None) == 0
    assert lib.sw_moe_experts(blk2.ctx, C.byref(d), C.byref(shard), x.data_ptr(), routed_shard.data_ptr(), 16, None) == 0
    ref_shard = MoeLayer(cfg.D, cfg.I, cfg.SI, a, "cuda:0", router="f32", expert_lo=4, expert_cnt=8)
    blk2.route(desc_from_config(cfg), ref_shard, x); blk2.experts(desc_from_config(cfg), ref_shard, x, routed_ref)
    torch.cuda.synchronize()
    assert torch.equal(routed_shard, routed_ref)
    # refusals: a layer the files do not hold, a path that does not exist
    bad = capi.SwMoeLayer(); hb = C.c_void_p()
    assert lib.sw_layer_load(str(tmp_path / "snap").encode(), 9, 0, 0, 0, C.byref(bad), None, C.byref(hb)) == -1 and "missing" in capi.last_error()
    assert lib.sw_layer_load(str(tmp_path / "nope").encode(), 7, 0, 0, 0, C.byref(bad), None, C.byref(hb)) == -1
    assert lib.sw_layer_load(str(tmp_path / "snap").encode(), 7, 0, 10, 8, C.byref(bad), None, C.byref(hb)) == -1 and "outside" in capi.last_error()
    blk.close(); blk2.close()
    lib.sw_layer_free(h); lib.sw_layer_free(hs)
