"""Writer of the reference's Laguna int4 container (one MoE layer per call), for conversion and for tests.

Counterpart of c/tools/convert_laguna_int4.py: routed experts are quantised per row to packed int4 (low nibble = even
column, +8 offset, scale = max|w| / 7 with the converter's floor of 1e-8) and fused per layer -- `experts.gate_up_proj`
[E*2I, D/2] with each expert's gate rows followed by its up rows, `experts.down_proj` [E*D, I/2], each with a `.qs`
array of f32 row scales; router weight and e_score_correction_bias stay f32; the shared expert is bf16.  The file is
plain safetensors: 8-byte little-endian header length, JSON header, raw bytes (written here without any dependency).
"""
import json
import struct

import numpy as np


def quant_int4_rows(w):
    """f32 [O, I] -> (packed u8 [O, I/2], f32 scales [O]); numpy twin of the reference converter's rule."""
    w = np.ascontiguousarray(w, np.float32)
    s = np.abs(w).max(axis=1, keepdims=True) / np.float32(7.0)
    s[s < 1e-8] = 1e-8
    q = np.clip(np.rint(w / s), -8, 7).astype(np.int32)
    lo = (q[:, 0::2] + 8).astype(np.uint8)
    hi = (q[:, 1::2] + 8).astype(np.uint8)
    return (lo | (hi << 4)), s[:, 0].astype(np.float32)


_DT = {np.dtype(np.uint8): "U8", np.dtype(np.float32): "F32", np.dtype(np.int32): "I32"}


def write_safetensors(path, tensors):
    """tensors: name -> numpy array, or (numpy uint16 array, "BF16") for bf16 bit patterns."""
    header, blobs, off = {}, [], 0
    for name, t in tensors.items():
        if isinstance(t, tuple):
            arr, dt = np.ascontiguousarray(t[0], np.uint16), t[1]
        else:
            arr = np.ascontiguousarray(t); dt = _DT[arr.dtype]
        b = arr.tobytes()
        header[name] = {"dtype": dt, "shape": list(arr.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b); off += len(b)
    h = json.dumps(header, separators=(",", ":")).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h))); f.write(h)
        for b in blobs:
            f.write(b)


def layer_tensors(layer_index, router_w, corr_bias, gu_q, gu_s, dn_q, dn_s, sh_gate=None, sh_up=None, sh_down=None):
    """Names of one layer as c/laguna.c:410-446 reads them; the int4 arrays are already in container form."""
    p = "model.layers.%d.mlp." % layer_index
    t = {p + "gate.weight": np.asarray(router_w, np.float32),
         p + "experts.gate_up_proj": gu_q, p + "experts.gate_up_proj.qs": np.asarray(gu_s, np.float32),
         p + "experts.down_proj": dn_q, p + "experts.down_proj.qs": np.asarray(dn_s, np.float32)}
    if corr_bias is not None:
        t[p + "experts.e_score_correction_bias"] = np.asarray(corr_bias, np.float32)
    if sh_gate is not None:
        t[p + "shared_expert.gate_proj.weight"] = (sh_gate, "BF16")
        t[p + "shared_expert.up_proj.weight"] = (sh_up, "BF16")
        t[p + "shared_expert.down_proj.weight"] = (sh_down, "BF16")
    return t


def convert_layer(path, layer_index, router_w, corr_bias, experts, shared=None):
    """experts: list of (gate [I,D], up [I,D], down [D,I]) f32 arrays of one layer; shared: (gate, up, down) as bf16 bit
    patterns (uint16) or None.  Quantises, fuses and writes the layer's container file."""
    gq, gs, dq, ds = [], [], [], []
    for g, u, d in experts:
        q, s = quant_int4_rows(np.concatenate([g, u], axis=0)); gq.append(q); gs.append(s)
        q, s = quant_int4_rows(d); dq.append(q); ds.append(s)
    sh = shared or (None, None, None)
    write_safetensors(path, layer_tensors(layer_index, router_w, corr_bias, np.concatenate(gq), np.concatenate(gs),
                                          np.concatenate(dq), np.concatenate(ds), *sh))
