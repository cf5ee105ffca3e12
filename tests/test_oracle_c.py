"""The C restatement (oracle/c/qoracle.c, the timed CPU baseline) against the numpy oracle. No GPU."""
import numpy as np
import pytest

from ingot_b200 import synth
from oracle import cref, qref


@pytest.mark.parametrize("bits", [4, 8])
def test_qmm_affine(bits):
    rng = np.random.default_rng(bits)
    w, s, b = synth.affine_np(rng, 96, 320, bits)
    x = synth.activations_np(rng, 5, 320)
    y, _ = cref.qmm(x, w[0], s[0], b[0], "affine", bits, 64)
    assert qref.max_rel(y, qref.qmm_affine(x, w[0], s[0], b[0], bits)) <= 1e-5


@pytest.mark.parametrize("bits,group", [(4, 32), (6, 64)])
def test_qmm_affine_other_formats(bits, group):
    """Groups of 32 and the 6-bit bit stream, the formats of the reference's q4-g32 and lfm-qmv6 kernel cases."""
    rng = np.random.default_rng(10 * bits + group)
    w, s, b = synth.affine_np(rng, 48, 256, bits, 1, group)
    x = synth.activations_np(rng, 3, 256)
    y, _ = cref.qmm(x, w[0], s[0], b[0], "affine", bits, group)
    assert qref.max_rel(y, qref.qmm_affine(x, w[0], s[0], b[0], bits, group)) <= 1e-5


def test_qmm_mxfp4():
    rng = np.random.default_rng(7)
    w, s = synth.mxfp4_np(rng, 64, 288)
    x = synth.activations_np(rng, 4, 288)
    y, _ = cref.qmm(x, w[0], s[0], None, "mxfp4", 4, 32)
    assert qref.max_rel(y, qref.matmul_t(x, qref.dequant_mxfp4(w[0], s[0]))) <= 1e-5


def test_route_and_moe():
    rng = np.random.default_rng(3)
    E, K, D, I, T = 32, 4, 256, 128, 9
    g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
    x = synth.activations_np(rng, T, D)
    lg = qref.router_logits(x, synth.router_np(rng, E, D))
    inds, wts = qref.route(lg, K)
    ic, wc = cref.route(lg, E, K)
    assert (ic == inds).all() and np.abs(wc - wts).max() <= 1e-6
    deq = lambda t, e: qref.dequant_affine(t[0][e], t[1][e], t[2][e], 4)
    yr = qref.moe_ffn(x, inds, wts, lambda e: (deq(g, e), deq(u, e), deq(d, e)))
    yc, _ = cref.moe_ffn(x, inds, wts, g, u, d, "affine")
    assert qref.max_rel(yc, yr) <= 1e-4


def test_moe_mxfp4_with_biases():
    rng = np.random.default_rng(4)
    E, K, D, I, T = 32, 4, 192, 192, 6
    g, u, d = synth.mxfp4_np(rng, I, D, E), synth.mxfp4_np(rng, I, D, E), synth.mxfp4_np(rng, D, I, E)
    x = synth.activations_np(rng, T, D)
    bg, bu, bd = (synth.round_bf16(rng.normal(0, 0.01, size=(E, n)).astype(np.float32)) for n in (I, I, D))
    lg = qref.router_logits(x, synth.router_np(rng, E, D))
    inds, wts = qref.route(lg, K)
    deq = lambda t, e: qref.dequant_mxfp4(t[0][e], t[1][e])
    yr = qref.moe_ffn(x, inds, wts, lambda e: (deq(g, e), deq(u, e), deq(d, e)), act="swiglu_oai", biases=(bg, bu, bd))
    yc, _ = cref.moe_ffn(x, inds, wts, g + (None,), u + (None,), d + (None,), "mxfp4", act="swiglu_oai", biases=(bg, bu, bd))
    assert qref.max_rel(yc, yr) <= 1e-4
