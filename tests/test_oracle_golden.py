"""The CPU oracle against the reference's own known-answer vectors (tests/golden/*.json, extracted from the reference's
test sources by tests/golden/make_golden.py). No GPU."""
import json
import os

import numpy as np
import pytest

from oracle import qref

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    with open(os.path.join(GOLD, name)) as f:
        return json.load(f)


def test_nibble_order_kat():
    f = load("format_kat.json")
    assert qref.pack_q(np.array(f["pack4_in"]), 4).tolist() == f["pack4_out"] == [0x87654321]
    assert qref.unpack_q(np.array(f["pack4_out"], dtype=np.uint32), 4).tolist() == f["pack4_in"]


def test_affine_dequant_kat():
    f = load("format_kat.json")
    N, K = f["N"], f["K"]
    q = np.array(f["codes"]).reshape(N, K)
    w = qref.pack_q(q, 4)
    s = qref.f32_to_bf16(np.array(f["scales"], dtype=np.float32)).reshape(N, K // 64)
    b = qref.f32_to_bf16(np.array(f["biases"], dtype=np.float32)).reshape(N, K // 64)
    got = qref.dequant_affine(w, s, b, 4).reshape(-1)
    assert (got == np.array(f["expected"], dtype=np.float32)).all()


@pytest.mark.parametrize("bits", [4, 6, 8])
def test_pack_unpack_roundtrip(bits):
    rng = np.random.default_rng(bits)
    q = rng.integers(0, 1 << bits, size=(3, 5, 64))
    assert (qref.unpack_q(qref.pack_q(q, bits), bits) == q).all()


def test_6bit_stream_matches_the_scalar_rule():
    """Value j of a 6-bit row sits in bits 6j.. of one little-endian stream, crossing word boundaries
    (unpackQ, Loader/Quant.swift:126-136; the generator of Tests/IngotTests/KernelHarness.swift:150-172)."""
    rng = np.random.default_rng(66)
    q = rng.integers(0, 64, size=128)
    row = qref.pack_q(q, 6)
    assert row.shape == (24,)
    for j in range(128):
        bit = 6 * j
        w, o = bit // 32, bit % 32
        v = int(row[w]) >> o
        if o + 6 > 32:
            v |= int(row[w + 1]) << (32 - o)
        assert v & 63 == q[j]
    by = row.view(np.uint8)  # the harness sets bit p of byte p / 8
    for j in (0, 5, 21, 127):
        for bit in range(6):
            p_ = 6 * j + bit
            assert ((int(by[p_ // 8]) >> (p_ % 8)) & 1) == ((int(q[j]) >> bit) & 1)


def test_bf16_rne():
    # ties go to even: 1 + 2^-8 is halfway between 1 and 1 + 2^-7
    f = np.array([1.0 + 2.0**-8, 1.0 + 3 * 2.0**-8, -0.0, 3.140625], dtype=np.float32)
    r = qref.round_bf16(f)
    assert r.tolist() == [1.0, 1.0 + 2.0**-6, -0.0, 3.140625]


def test_mxfp4_kat_bit_exact():
    g = load("mxfp4_kat.json")
    w = np.array(g["words"], dtype=np.uint32).reshape(g["rows"], g["cols"] // 8)
    s = np.array(g["scales"], dtype=np.uint8).reshape(g["rows"], g["cols"] // 32)
    v = qref.dequant_mxfp4(w, s).reshape(-1)
    assert (v.view(np.uint32) == np.array(g["value_bits"], dtype=np.uint32)).all()  # the sign of zero included
    assert qref.E2M1.tolist() == g["e2m1"]
    assert qref.e8m0_to_f32(np.array([116, 135], dtype=np.uint8)).tolist() == [2.0**-11, 256.0]
    assert np.isnan(qref.e8m0_to_f32(np.array([255], dtype=np.uint8))[0])


def test_swiglu_oai_kat():
    o = load("swiglu_oai_kat.json")
    g = np.repeat(np.array(o["g"], dtype=np.float32), len(o["u"]))
    u = np.tile(np.array(o["u"], dtype=np.float32), len(o["g"]))
    y = qref.swiglu_oai(g, u, o["limit"])
    want = np.array(o["y"])
    assert (np.abs(y - want) <= o["tol"] * np.maximum(1, np.abs(want))).all()


def dense_weights(inds, w, E):
    out = np.zeros((inds.shape[0], E), dtype=np.float32)
    for r in range(inds.shape[0]):
        for i, v in zip(inds[r], w[r]):
            out[r, int(i)] += v
    return out


@pytest.mark.parametrize("case", load("router_vectors.json")["cases"], ids=lambda c: c["name"])
def test_router_vectors(case):
    """Selection and weights against mlx-lm's routers (rows 2.. as in the reference: rows 0-1 carry exact ties that
    mlx-lm's argpartition breaks either way) and the lower-index rule on the tied rows."""
    E, K, B = case["experts"], case["topK"], case["rows"]
    lg = np.array(case["logits"], dtype=np.float32).reshape(B, E)
    inds, w = qref.route(lg, K, logit_bias=case.get("logitBias"), select_bias=case["bias"],
                         sigmoid=case["score"] == "sigmoid", scale=case["scale"], eps=case["eps"],
                         per_expert_scale=case.get("perExpertScale"))
    dense = dense_weights(inds, w, E)
    mlx = np.array(case["weights"], dtype=np.float32).reshape(B, E)
    assert ((dense[2:] != 0) == (mlx[2:] != 0)).all()
    assert qref.max_rel(dense[2:], mlx[2:]) <= 1e-5
    # rows 0-1: K-1 clear winners at (7e) % E, then the lower index of the tied pair
    for r, (a, b) in enumerate([(E // 4 + 1, 3 * E // 4 - 1), (E // 2 + 3, E // 2 - 5)]):
        assert sorted(inds[r, : K - 1].tolist()) == sorted((7 * e) % E for e in range(1, K))
        assert inds[r, K - 1] == min(a, b)


def test_route_ties_e512_k10():
    """Constructed logits of the reference's moe-route-e512 case (KernelCaseTests.swift:454-472): nine clear winners and
    an exact tie for the 10th place between experts 301 and 450; 301 wins."""
    E, K = 512, 10
    lg = np.full((1, E), -3, dtype=np.float32)
    for e in [5, 17, 33, 64, 100, 200, 255, 256, 511]:
        lg[0, e] = 5
    lg[0, 301] = lg[0, 450] = 2
    inds, w = qref.route(lg, K)
    assert inds[0].tolist() == [5, 17, 33, 64, 100, 200, 255, 256, 511, 301]
    ex = np.exp(np.array([0] * 9 + [-3], dtype=np.float32))
    assert np.allclose(w[0], ex / ex.sum(), rtol=1e-6)


def test_route_all_minus_inf_and_nan():
    lg = np.full((1, 32), -np.inf, dtype=np.float32)
    inds, _ = qref.route(lg, 4)
    assert inds[0].tolist() == [0, 1, 2, 3]
    lg = np.zeros((1, 32), dtype=np.float32)
    lg[0, 3] = np.nan
    lg[0, 5] = 1
    inds, _ = qref.route(lg, 3)
    assert inds[0].tolist() == [5, 0, 1]


def test_group_pairs_is_a_bijection():
    rng = np.random.default_rng(1)
    inds = rng.integers(0, 32, size=(50, 4)).astype(np.uint32)
    offsets, row_map, pos = qref.group_pairs(inds, 32)
    assert sorted(row_map.tolist()) == list(range(200))
    assert (pos[row_map] == np.arange(200)).all()
    flat = inds.reshape(-1)
    for e in range(32):
        seg = row_map[offsets[e]:offsets[e + 1]]
        assert (flat[seg] == e).all() and (np.diff(seg.astype(np.int64)) > 0).all()


def test_moe_block_equals_full_softmax_form():
    """The engine's weights (softmax over the chosen logits) equal ref/moe_ref.py's softmax -> top-k -> renormalise."""
    rng = np.random.default_rng(2)
    lg = rng.normal(size=(16, 64)).astype(np.float32)
    inds, w = qref.route(lg, 8)
    p = np.exp(lg - lg.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    order = np.argsort(-p, axis=1, kind="stable")[:, :8]
    sc = np.take_along_axis(p, order, 1)
    sc /= sc.sum(1, keepdims=True)
    assert (order == inds).all() and np.allclose(sc, w, rtol=1e-5)
