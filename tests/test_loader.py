"""The weight loader on the host (no GPU): safetensors shards written here with numpy are read back through the native
reader (iq_st_*) and assembled with the reference's rules (Loader/Safetensors.swift, Loader/Quant.swift,
Layers/Linear.swift:104-183, :599-610; the cases follow FormatTests.swift)."""
import json
import os
import struct

import numpy as np
import pytest

from ingot_b200 import capi, loader, synth
from oracle import qref


def write_safetensors(path, tensors, metadata=None, pad_header_to=None):
    """tensors: name -> (dtype string, numpy array whose bytes are the payload, shape)."""
    header, blobs, off = {}, [], 0
    if metadata is not None:
        header["__metadata__"] = metadata
    for name, (dt, arr, shape) in tensors.items():
        raw = np.ascontiguousarray(arr).tobytes()
        header[name] = {"dtype": dt, "shape": list(shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    js = json.dumps(header).encode()
    if pad_header_to is not None:
        js += b" " * (pad_header_to - len(js))
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(js)))
        f.write(js)
        for b in blobs:
            f.write(b)


def affine_layer(rng, prefix, N, K, bits, experts=None, gs=64):
    w, s, b = synth.affine_np(rng, N, K, bits, experts or 1, gs)
    if experts is None:
        w, s, b = w[0], s[0], b[0]
    return {prefix + ".weight": ("U32", w, w.shape), prefix + ".scales": ("BF16", s, s.shape),
            prefix + ".biases": ("BF16", b, b.shape)}, (w, s, b)


@pytest.fixture()
def pack(tmp_path):
    """Two shards with an index, a config with per-path overrides, one tensor at an odd offset."""
    rng = np.random.default_rng(5)
    t0, raw = {}, {}
    for name, (N, K, bits) in {"model.layers.0.attn.qkv": (96, 256, 8), "model.layers.0.attn.ab": (32, 256, 4),
                               "model.layers.0.mlp.gate_proj": (128, 256, 4), "model.layers.0.mlp.up_proj": (64, 256, 4)}.items():
        d, r = affine_layer(rng, name, N, K, bits)
        t0.update(d)
        raw[name] = r
    t0["model.norm.weight"] = ("F32", np.arange(7, dtype=np.float32), (7,))
    t0["odd"] = ("U8", np.arange(5, dtype=np.uint8), (5,))  # makes what follows unaligned
    t0["after_odd"] = ("F32", np.array([1.5, -2.0], dtype=np.float32), (2,))
    t1 = {}
    d, r = affine_layer(rng, "language_model.model.layers.1.mlp.experts.gate_proj", 64, 128, 4, experts=4)
    t1.update(d)
    raw["experts"] = r
    mw = rng.integers(0, 2**32, size=(2, 32, 8), dtype=np.uint64).astype(np.uint32)
    ms = (127 + rng.integers(-8, 1, size=(2, 32, 2))).astype(np.uint8)
    t1["language_model.model.layers.1.mlp.experts.up_proj.weight"] = ("U32", mw, mw.shape)
    t1["language_model.model.layers.1.mlp.experts.up_proj.scales"] = ("U8", ms, ms.shape)
    t1["vision_tower.layers.1.x"] = ("F16", np.zeros(4, dtype=np.float16), (4,))
    write_safetensors(tmp_path / "model-00001-of-00002.safetensors", t0, metadata={"format": "mlx", "nested": {"a": [1, 2.5, None]}})
    write_safetensors(tmp_path / "model-00002-of-00002.safetensors", t1)
    wm = {k: "model-00001-of-00002.safetensors" for k in t0}
    wm.update({k: "model-00002-of-00002.safetensors" for k in t1})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": wm}))
    cfg = {"hidden_size": 256, "quantization": {
        "group_size": 64, "bits": 4, "model.layers.0.attn.qkv": {"group_size": 64, "bits": 8},
        "language_model.model.layers.1.mlp.experts.up_proj": {"group_size": 32, "bits": 4, "mode": "mxfp4"}}}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    return tmp_path, raw, (mw, ms)


def test_header_table_shards_and_bytes(pack):
    d, raw, _ = pack
    st = loader.SafetensorsStore(str(d))
    assert len(st.tensors) == 4 * 3 + 3 + 3 + 2 + 1
    t = st.info("model.norm.weight")
    assert (t.dtype, t.shape, t.shard, t.byte_count) == ("F32", (7,), 0, 28)
    assert np.array_equal(st.array(t), np.arange(7, dtype=np.float32))
    a = st.info("after_odd")
    assert st.alignment(a) % 2 == 1 or st.alignment(a) < 4   # sits right after 5 odd bytes
    assert np.array_equal(st.array(a), np.array([1.5, -2.0], dtype=np.float32))
    w = st.info("model.layers.0.attn.qkv.weight")
    assert np.array_equal(st.array(w), raw["model.layers.0.attn.qkv"][0])
    e = st.info("language_model.model.layers.1.mlp.experts.gate_proj.scales")
    assert e.shard == 1 and e.shape == (4, 64, 2)
    with pytest.raises(loader.SafetensorsError) as ex:
        st.info("nope")
    assert ex.value.kind == "missing"
    st.close()


def test_layer_prefix_prefers_the_language_model(pack):
    d, _, _ = pack
    st = loader.SafetensorsStore(str(d))
    assert st.layer_prefix(0) == "model.layers.0."
    assert st.layer_prefix(1) == "language_model.model.layers.1."   # not the vision tower's layers.1.
    with pytest.raises(loader.SafetensorsError):
        st.layer_prefix(7)
    assert loader.SafetensorsStore.preferred_prefix({"b.layers.0.", "a.layers.0.", "x.language_model.layers.0."}) == \
        "x.language_model.layers.0."


def test_quantized_linear_reads_bits_from_shapes_and_checks_the_config(pack):
    d, _, _ = pack
    st = loader.SafetensorsStore(str(d))
    cfg = loader.ModelConfig.from_file(str(d / "config.json"))
    q = loader.QuantizedLinear(st, "model.layers.0.attn.qkv", cfg)
    assert (q.params.bits, q.params.group_size, q.out_features, q.in_features, q.experts) == (8, 64, 96, 256, 1)
    q = loader.QuantizedLinear(st, "language_model.model.layers.1.mlp.experts.gate_proj", cfg)
    assert (q.params.bits, q.experts, q.out_features, q.in_features) == (4, 4, 64, 128)
    # an MXFP4 layer is a load error unless the caller has MXFP4 kernels for it (the MoE experts)
    with pytest.raises(loader.SafetensorsError) as ex:
        loader.QuantizedLinear(st, "language_model.model.layers.1.mlp.experts.up_proj", cfg)
    assert "mxfp4" in str(ex.value)
    q = loader.QuantizedLinear(st, "language_model.model.layers.1.mlp.experts.up_proj", cfg, mxfp4=True)
    assert q.is_mxfp4 and (q.experts, q.out_features, q.in_features) == (2, 32, 64)
    # the config says 8 bits for a path whose shapes say 4
    bad = loader.ModelConfig({"quantization": {"group_size": 64, "bits": 8}})
    with pytest.raises(loader.SafetensorsError) as ex:
        loader.QuantizedLinear(st, "model.layers.0.attn.ab", bad)
    assert "config says 8 bits, the shapes say 4" in str(ex.value)
    # an override without `mode` is affine even when the default is mxfp4
    c2 = loader.ModelConfig({"quantization": {"group_size": 32, "bits": 4, "mode": "mxfp4", "r": {"group_size": 64, "bits": 8}}})
    assert c2.quant("r").mode == "affine" and c2.quant("other").mode == "mxfp4"


def test_concat_same_bits_with_zero_padding(pack):
    d, raw, _ = pack
    st = loader.SafetensorsStore(str(d))
    cfg = loader.ModelConfig.from_file(str(d / "config.json"))
    h = loader.dense_q(st, cfg, ["model.layers.0.mlp.gate_proj", "model.layers.0.mlp.up_proj"], pad_to=128)
    assert (h.N, h.K, h.bits, h.gs) == (256, 256, 4, 64)
    g, u = raw["model.layers.0.mlp.gate_proj"], raw["model.layers.0.mlp.up_proj"]
    assert np.array_equal(h.w[:128], g[0]) and np.array_equal(h.w[128:192], u[0]) and not h.w[192:].any()
    assert np.array_equal(h.s[:128], g[1]) and np.array_equal(h.b[128:192], u[2]) and not h.s[192:].any()


def test_mixed_4_and_8_bits_concatenate_at_8_bits_losslessly(pack):
    """A 4-bit piece beside an 8-bit one: codes x 16, scales / 16, biases as they are; every weight keeps its value
    bit for bit (Linear.swift:118-176; FormatTests.swift)."""
    d, raw, _ = pack
    st = loader.SafetensorsStore(str(d))
    cfg = loader.ModelConfig.from_file(str(d / "config.json"))
    h = loader.dense_q(st, cfg, ["model.layers.0.attn.qkv", "model.layers.0.attn.ab"])
    assert (h.N, h.K, h.bits) == (128, 256, 8)
    q8, q4 = raw["model.layers.0.attn.qkv"], raw["model.layers.0.attn.ab"]
    assert np.array_equal(h.w[:96], q8[0]) and np.array_equal(h.s[:96], q8[1])
    codes4 = qref.unpack_q(q4[0], 4)
    assert np.array_equal(qref.unpack_q(h.w[96:], 8), codes4 * 16)
    assert np.array_equal(qref.dequant_affine(h.w[96:], h.s[96:], h.b[96:], 8), qref.dequant_affine(q4[0], q4[1], q4[2], 4))


def test_widen_words_known_answer():
    """The word 0x76543210 holds the values 0..7, low nibble first; widened they are 0x00, 0x10, .. 0x70."""
    src = np.array([0x76543210, 0xFEDCBA98], dtype=np.uint32)
    dst = np.zeros(4, dtype=np.uint32)
    capi.lib().iq_widen4to8_words(src.ctypes.data, dst.ctypes.data, 2)
    assert dst.tolist() == [0x30201000, 0x70605040, 0xB0A09080, 0xF0E0D0C0]
    s = np.array([0x3C00, 0x4080, 0x0000], dtype=np.uint16)  # bf16 0.0078125, 4.0, 0
    out = np.zeros(3, dtype=np.uint16)
    capi.lib().iq_scales_div16_bf16(s.ctypes.data, out.ctypes.data, 3)
    assert out.tolist() == [0x3A00, 0x3E80, 0x0000]


def test_stacked_experts_and_mxfp4(pack):
    d, raw, (mw, ms) = pack
    st = loader.SafetensorsStore(str(d))
    cfg = loader.ModelConfig.from_file(str(d / "config.json"))
    w, s, b, l = loader.stacked_experts(st, cfg, "language_model.model.layers.1.mlp.experts.gate_proj")
    assert np.array_equal(w, raw["experts"][0]) and np.array_equal(s, raw["experts"][1]) and np.array_equal(b, raw["experts"][2])
    w, s, b, l = loader.stacked_experts(st, cfg, "language_model.model.layers.1.mlp.experts.up_proj")
    assert l.is_mxfp4 and b is None and np.array_equal(w, mw) and np.array_equal(s, ms)


def test_malformed_files_are_format_errors(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(loader.SafetensorsError) as ex:
        loader.SafetensorsStore(str(tmp_path))
    assert ex.value.kind == "format" and "too short" in str(ex.value)
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(loader.SafetensorsError) as ex:
        loader.SafetensorsStore(str(tmp_path))
    assert "header out of range" in str(ex.value)
    js = json.dumps({"t": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(js)) + js + b"\x00" * 8)
    with pytest.raises(loader.SafetensorsError) as ex:
        loader.SafetensorsStore(str(tmp_path))
    assert "inconsistent size in t" in str(ex.value)
    # a shape whose element count wraps 64 bits ([2^32, 2^32] -> 0 elements) must not pass for an empty tensor
    for shape in ([2**32, 2**32], [2**62, 4], [2**40, 2**22, 2]):
        js = json.dumps({"t": {"dtype": "F32", "shape": shape, "data_offsets": [0, 0]}}).encode()
        p.write_bytes(struct.pack("<Q", len(js)) + js + b"\x00" * 8)
        with pytest.raises(loader.SafetensorsError) as ex:
            loader.SafetensorsStore(str(tmp_path))
        assert ex.value.kind == "format" and "inconsistent size in t" in str(ex.value)
    js = json.dumps({"t": {"dtype": "F64", "shape": [1], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(js)) + js + b"\x00" * 8)
    with pytest.raises(loader.SafetensorsError) as ex:
        loader.SafetensorsStore(str(tmp_path))
    assert "malformed entry: t" in str(ex.value)
    os.remove(p)
    with pytest.raises(loader.SafetensorsError) as ex:
        loader.SafetensorsStore(str(tmp_path))
    assert ex.value.kind == "io"


def test_groups_of_32_and_6_bits_load_as_they_are(tmp_path):
    """A 4-bit matrix with groups of 32 (from its config entry) and a 6-bit one (bits read off the shapes: 6 K / 32 words
    per row): the host arrays are the checkpoint's, and dequantise to the same weights. Groups of 32 with 8 bits, which
    no kernel takes, are refused (Layers/Linear.swift:58-63)."""
    rng = np.random.default_rng(32)
    t, raw = {}, {}
    for name, (N, K, bits, gs) in {"m.q32": (48, 256, 4, 32), "m.head6": (64, 128, 6, 64), "m.bad": (16, 128, 8, 32)}.items():
        d, r = affine_layer(rng, name, N, K, bits, gs=gs)
        t.update(d)
        raw[name] = r
    write_safetensors(tmp_path / "model.safetensors", t)
    cfg = loader.ModelConfig({"quantization": {"group_size": 64, "bits": 4, "m.q32": {"group_size": 32, "bits": 4},
                                               "m.head6": {"group_size": 64, "bits": 6},
                                               "m.bad": {"group_size": 32, "bits": 8}}})
    st = loader.SafetensorsStore(str(tmp_path))
    h = loader.dense_q(st, cfg, ["m.q32"])
    assert (h.N, h.K, h.bits, h.gs) == (48, 256, 4, 32) and h.s.shape == (48, 8)
    w, s, b = raw["m.q32"]
    assert np.array_equal(qref.dequant_affine(h.w, h.s, h.b, 4, 32), qref.dequant_affine(w, s, b, 4, 32))
    h6 = loader.dense_q(st, cfg, ["m.head6"])
    assert (h6.N, h6.K, h6.bits, h6.gs) == (64, 128, 6, 64) and h6.w.shape == (64, 24)
    w, s, b = raw["m.head6"]
    assert np.array_equal(h6.w, w) and np.array_equal(qref.dequant_affine(h6.w, h6.s, h6.b, 6), qref.dequant_affine(w, s, b, 6))
    with pytest.raises(loader.SafetensorsError):
        loader.dense_q(st, cfg, ["m.bad"])
