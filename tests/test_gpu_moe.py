"""MoE layer (iq_moe_* through MoELayer) against the CPU oracle: routing indices bit-exact, weights 1e-5, outputs within
the tolerance. Mirrors the reference's MoE and router kernel cases (Tests/IngotTests/KernelCaseMoE.swift:45-114,
KernelCaseRouter.swift:110-141, KernelCaseGptOss.swift:13-65, KernelCaseMXFP4.swift:49-134)."""
import json
import os

import numpy as np
import pytest
import torch

from ingot_b200 import capi, synth
from ingot_b200.moe import MoELayer, RouterSpec
from oracle import qref
from gpu_util import TOL, x_tensor

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def build_layer(rng, device, E, K, D, I, fmt="affine", act="silu", biases=False, router_bias=False, max_tokens=16,
                expert_lo=0, expert_count=None):
    host = {}
    if fmt == "affine":
        g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
        mk = lambda t, lo, hi: synth.dense_q_affine(t[0][lo:hi], t[1][lo:hi], t[2][lo:hi], 4, device)
        host["deq"] = lambda t, e: qref.dequant_affine(t[0][e], t[1][e], t[2][e], 4)
    else:
        g, u, d = synth.mxfp4_np(rng, I, D, E), synth.mxfp4_np(rng, I, D, E), synth.mxfp4_np(rng, D, I, E)
        mk = lambda t, lo, hi: synth.dense_q_mxfp4(t[0][lo:hi], t[1][lo:hi], device)
        host["deq"] = lambda t, e: qref.dequant_mxfp4(t[0][e], t[1][e])
    host["g"], host["u"], host["d"] = g, u, d
    wr = synth.router_np(rng, E, D)
    host["router"] = wr
    lo = expert_lo
    hi = lo + (expert_count if expert_count is not None else E)
    bt = {}
    if biases:
        host["biases"] = tuple(synth.round_bf16(rng.normal(0, 0.01, size=(E, n)).astype(np.float32)) for n in (I, I, D))
        bt = dict(zip(("gate_bias", "up_bias", "down_bias"),
                      (torch.from_numpy(b[lo:hi].copy()).to(device) for b in host["biases"])))
    else:
        host["biases"] = None
    lb = None
    if router_bias:
        host["router_bias"] = rng.uniform(-1, 1, size=E).astype(np.float32)
        lb = torch.from_numpy(host["router_bias"]).to(device)
    else:
        host["router_bias"] = None
    layer = MoELayer(RouterSpec(E, K, logit_bias=lb), synth.bf16_values_tensor(wr, device), mk(g, lo, hi), mk(u, lo, hi),
                     mk(d, lo, hi), act=act, max_tokens=max_tokens, expert_lo=lo, **bt)
    host["weights"] = lambda e: (host["deq"](g, e), host["deq"](u, e), host["deq"](d, e))
    return layer, host


def check_layer(layer, host, x, T, act, tol=TOL, half_gu=False):
    dev = layer.device
    xt = x_tensor(x, dev)
    out = torch.zeros(T, layer.D, dtype=torch.float32, device=dev)
    layer.encode(xt, out, T)
    assert capi.context(0).device_status() == 0
    v = layer.views(T)
    logits = qref.router_logits(x, host["router"])
    inds, wts = qref.route(logits, layer.router.top_k, logit_bias=host["router_bias"])
    # The logits of the chosen experts are the correctly rounded dot products, bit for bit. So are all the others,
    # except with many tokens and a bf16 router, where logits that cannot reach the top k stay at their tensor-core
    # value (within the kernel's error bound, far below 2e-2 here).
    got_logits = v["logits"][:, : layer.router.experts].cpu().numpy()
    pick = inds.astype(np.int64)
    assert np.array_equal(np.take_along_axis(got_logits, pick, axis=1), np.take_along_axis(logits, pick, axis=1)), \
        "router logits of the chosen experts differ"
    if T <= 64 or layer.router.experts % 64 != 0:
        assert np.array_equal(got_logits, logits), "router logits differ"
    else:
        assert np.abs(got_logits - logits).max() <= 2e-2
    assert np.array_equal(v["inds"].cpu().numpy().astype(np.uint32), inds), "routing indices differ"
    assert qref.max_rel(v["wts"].cpu().numpy(), wts) <= 1e-5
    # permutation: a bijection, grouped by expert in ascending pair order
    offsets, row_map, pos = qref.group_pairs(inds, layer.router.experts)
    assert np.array_equal(v["offsets"].cpu().numpy().astype(np.uint32), offsets)
    assert np.array_equal(v["row_map"].cpu().numpy().astype(np.uint32), row_map)
    assert np.array_equal(v["pos"].cpu().numpy().astype(np.uint32), pos)
    ref = qref.moe_ffn(x, inds, wts, host["weights"], act=act, biases=host["biases"], half_gu=half_gu)
    err = qref.max_rel(out.cpu().numpy(), ref)
    assert err <= tol, err
    return out


@pytest.mark.parametrize("T", [1, 2, 5, 16, 64, 300, 1000, 2150, 2500, 3500])
def test_moe_small_affine(cuda_device, T):
    rng = np.random.default_rng(T)
    layer, host = build_layer(rng, cuda_device, 32, 4, 256, 128, max_tokens=T)
    check_layer(layer, host, synth.activations_np(rng, T, 256), T, "silu")


@pytest.mark.parametrize("T", [1, 7, 40, 2100, 2600])
def test_moe_small_mxfp4_gptoss_style(cuda_device, T):
    """gpt-oss style: MXFP4 experts, expert biases, clamped swiglu_oai, router bias, hidden 576 (not a multiple of 128)."""
    rng = np.random.default_rng(50 + T)
    layer, host = build_layer(rng, cuda_device, 32, 4, 576, 192, fmt="mxfp4", act="swiglu_oai", biases=True,
                              router_bias=True, max_tokens=T)
    check_layer(layer, host, synth.activations_np(rng, T, 576), T, "swiglu_oai")


@pytest.mark.parametrize("T", [1, 8, 16, 64, 100, 256, 512])
def test_moe_c2_configuration(cuda_device, T):
    """128 experts, top-8, d_model 2048, d_ff 768, 4-bit g64, bf16 router ~ N(0, 0.02), x ~ N(0, 1), seed 0. The token
    counts walk the decode tile kernels (8-row tiles with one and two live row sets, 16-row tiles) and the first size of
    the grouped GEMM."""
    rng = np.random.default_rng(0)
    layer, host = build_layer(rng, cuda_device, 128, 8, 2048, 768, max_tokens=T)
    check_layer(layer, host, synth.activations_np(rng, T, 2048), T, "silu")


def test_moe_c2_layer_at_the_benchmarked_size(cuda_device):
    """The layer the 48-layer stack is made of, at the benchmark's 4096 prefill tokens (32,768 routed rows: the chunked
    counting sort, 256-row tiles, the single-accumulator gate/up path): logits, indices, weights and the whole permutation
    against the oracle in full, the outputs on 32 sampled tokens."""
    rng = np.random.default_rng(4096)
    T, E, K, D, I = 4096, 128, 8, 2048, 768
    layer, host = build_layer(rng, cuda_device, E, K, D, I, max_tokens=T)
    x = synth.activations_np(rng, T, D)
    out = torch.zeros(T, D, dtype=torch.float32, device=cuda_device)
    layer.encode(x_tensor(x, cuda_device), out, T)
    assert capi.context(0).device_status() == 0
    v = layer.views(T)
    logits = qref.router_logits(x, host["router"])
    inds, wts = qref.route(logits, K)
    assert np.array_equal(v["inds"].cpu().numpy().astype(np.uint32), inds), "routing indices differ"
    assert qref.max_rel(v["wts"].cpu().numpy(), wts) <= 1e-5
    offsets, row_map, pos = qref.group_pairs(inds, E)
    assert np.array_equal(v["offsets"].cpu().numpy().astype(np.uint32), offsets)
    assert np.array_equal(v["row_map"].cpu().numpy().astype(np.uint32), row_map)
    assert np.array_equal(v["pos"].cpu().numpy().astype(np.uint32), pos)
    sel = np.sort(rng.choice(T, size=32, replace=False))
    ref = qref.moe_ffn(x[sel], inds[sel], wts[sel], host["weights"])
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    err = qref.max_rel(got[sel], ref)
    assert err <= TOL, err


@pytest.mark.parametrize("T", [1, 256])
def test_moe_c3_configuration(cuda_device, T):
    """32 experts, top-4, d_model = d_ff = 2880, MXFP4, expert biases, clamped SwiGLU."""
    rng = np.random.default_rng(0)
    layer, host = build_layer(rng, cuda_device, 32, 4, 2880, 2880, fmt="mxfp4", act="swiglu_oai", biases=True,
                              max_tokens=T)
    check_layer(layer, host, synth.activations_np(rng, T, 2880), T, "swiglu_oai")


def router_cases():
    with open(os.path.join(GOLD, "router_vectors.json")) as f:
        return json.load(f)["cases"]


@pytest.mark.parametrize("case", router_cases(), ids=lambda c: c["name"])
def test_route_kernel_against_mlx_lm_vectors(cuda_device, case):
    """The route kernel on the reference's router vectors (logits at the stride padded to 64): indices bit-exact against
    the CPU rule, weights 1e-5, chosen sets and weights against mlx-lm on rows 2.. (KernelCaseRouter.swift:110-141)."""
    rng = np.random.default_rng(1)
    E, K, B = case["experts"], case["topK"], case["rows"]
    lb = case.get("logitBias")
    pes = case.get("perExpertScale")
    sig = case["score"] == "sigmoid"
    sb = case.get("bias") if sig else None  # sigmoid families: the bias only steers the selection
    dev_f32 = lambda v: None if v is None else torch.tensor(v, dtype=torch.float32, device=cuda_device)
    g, u, d = synth.affine_np(rng, 64, 128, 4, E), synth.affine_np(rng, 64, 128, 4, E), synth.affine_np(rng, 128, 64, 4, E)
    mk = lambda t: synth.dense_q_affine(t[0], t[1], t[2], 4, cuda_device)
    spec = RouterSpec(E, K, scale=case["scale"], logit_bias=dev_f32(lb), per_expert_scale=dev_f32(pes),
                      score=case["score"], select_bias=dev_f32(sb), eps=case["eps"] if sig else 0.0)
    layer = MoELayer(spec, synth.bf16_values_tensor(synth.router_np(rng, E, 128), cuda_device), mk(g), mk(u), mk(d))
    ld = (E + 63) // 64 * 64
    lg = np.array(case["logits"], dtype=np.float32).reshape(B, E)
    padded = np.zeros((B, ld), dtype=np.float32)
    padded[:, :E] = lg
    inds, wts = layer.route(torch.from_numpy(padded).to(cuda_device), B)
    torch.cuda.synchronize()
    ri, rw = qref.route(lg, K, logit_bias=lb, scale=case["scale"], per_expert_scale=pes, sigmoid=sig, select_bias=sb,
                        eps=case["eps"] if sig else 0.0)
    assert np.array_equal(inds.cpu().numpy().astype(np.uint32), ri)
    assert qref.max_rel(wts.cpu().numpy(), rw) <= 1e-5
    dense = np.zeros((B, E), dtype=np.float32)
    gi, gw = inds.cpu().numpy(), wts.cpu().numpy()
    for r in range(B):
        for k in range(K):
            dense[r, gi[r, k]] += gw[r, k]
    mlx = np.array(case["weights"], dtype=np.float32).reshape(B, E)
    assert ((dense[2:] != 0) == (mlx[2:] != 0)).all()
    assert qref.max_rel(dense[2:], mlx[2:]) <= 1e-5


def test_route_kernel_ties_e512_k10_and_edge_rows(cuda_device):
    rng = np.random.default_rng(2)
    E, K = 512, 10
    g, u, d = synth.affine_np(rng, 64, 128, 4, E), synth.affine_np(rng, 64, 128, 4, E), synth.affine_np(rng, 128, 64, 4, E)
    mk = lambda t: synth.dense_q_affine(t[0], t[1], t[2], 4, cuda_device)
    layer = MoELayer(RouterSpec(E, K), synth.bf16_values_tensor(synth.router_np(rng, E, 128), cuda_device), mk(g), mk(u), mk(d))
    lg = rng.uniform(-4, 4, size=(12, E)).astype(np.float32)
    lg[0, :] = -3
    for e in [5, 17, 33, 64, 100, 200, 255, 256, 511]:
        lg[0, e] = 5
    lg[0, 301] = lg[0, 450] = 2          # exact tie for the 10th place: 301 wins
    lg[1, :] = -np.inf                   # nothing to choose from: indices 0..9
    lg[2, 7] = np.nan                    # NaN counts as -inf
    inds, wts = layer.route(torch.from_numpy(lg).to(cuda_device), 12)
    torch.cuda.synchronize()
    ri, rw = qref.route(lg, K)
    got = inds.cpu().numpy().astype(np.uint32)
    assert np.array_equal(got, ri)
    assert got[0].tolist() == [5, 17, 33, 64, 100, 200, 255, 256, 511, 301]
    assert got[1].tolist() == list(range(10))
    ok = np.ones(12, dtype=bool)
    ok[1] = False  # weights of the all -inf row are NaN on both sides
    assert qref.max_rel(wts.cpu().numpy()[ok], rw[ok]) <= 1e-5


def tensor_router_layer(rng, device, wr, K, T):
    E, D = wr.shape
    I = 64
    g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
    mk = lambda t: synth.dense_q_affine(t[0], t[1], t[2], 4, device)
    return MoELayer(RouterSpec(E, K), synth.bf16_values_tensor(wr, device), mk(g), mk(u), mk(d), max_tokens=T)


def test_tensor_router_error_bound_and_exact_selection(cuda_device):
    """Many tokens, bf16 router, bf16 activations: the logits come from the tensor cores, then the route kernel recomputes
    exactly every logit within twice the error bound of the k-th largest. The approximate logits must sit far inside the
    bound the kernel assumes (K * 2^-21 * ||x|| * max||w||); indices, the chosen logits and the weights must be what
    float64 logits give."""
    rng = np.random.default_rng(77)
    E, K, D, T = 128, 8, 2048, 1024
    wr = synth.router_np(rng, E, D)
    layer = tensor_router_layer(rng, cuda_device, wr, K, T)
    x = synth.activations_np(rng, T, D)
    xt = x_tensor(x, cuda_device)
    out = torch.zeros(T, D, dtype=torch.float32, device=cuda_device)
    layer.encode(xt, out, T, only="router")
    torch.cuda.synchronize()
    approx = layer.views(T)["logits"][:, :E].cpu().numpy().copy()
    exact = qref.router_logits(x, wr)
    bound = D * 2.0 ** -21 * np.linalg.norm(wr, axis=1).max() * np.linalg.norm(x, axis=1)  # per token
    worst = (np.abs(approx - exact).max(axis=1) / bound).max()
    assert worst <= 1 / 8, f"tensor-core logits use {worst:.3f} of the assumed error bound"
    assert not np.array_equal(approx, exact)  # (they really are the approximate ones)
    layer.encode(xt, out, T, only="route")
    assert capi.context(0).device_status() == 0
    v = layer.views(T)
    inds, wts = qref.route(exact, K)
    assert np.array_equal(v["inds"].cpu().numpy().astype(np.uint32), inds)
    assert qref.max_rel(v["wts"].cpu().numpy(), wts) <= 1e-5
    pick = inds.astype(np.int64)
    refined = v["logits"][:, :E].cpu().numpy()
    assert np.array_equal(np.take_along_axis(refined, pick, axis=1), np.take_along_axis(exact, pick, axis=1))


def test_tensor_router_near_ties_at_the_boundary(cuda_device):
    """Adversarial margins: the 128 experts are 64 pairs whose rows differ by one bf16 ulp in one weight, and x is tiny at
    that position, so the two logits of a pair differ by a few fp32 ulps at most (or tie). With top-7 the boundary between
    the 7th and the 8th place falls inside a pair for every token: only the exact recomputation (and the lower-index
    rule on ties) can give the oracle's indices."""
    rng = np.random.default_rng(78)
    E, K, D, T = 128, 7, 2048, 512
    base = synth.router_np(rng, E // 2, D)
    wr = np.repeat(base, 2, axis=0)
    k0 = 1000
    bits = synth.to_bf16_bits(wr[1::2, k0])
    wr[1::2, k0] = synth.bf16_bits_to_f32((bits + 1).astype(np.uint16))  # one ulp up in the odd rows
    x = synth.activations_np(rng, T, D)
    x[:, k0] = synth.round_bf16((2.0 ** -rng.integers(8, 13, size=T)).astype(np.float32) * rng.choice([-1.0, 1.0], size=T).astype(np.float32))
    exact = qref.router_logits(x, wr)
    gap = np.abs(exact[:, 0::2] - exact[:, 1::2])
    ulp = np.spacing(np.abs(exact[:, 0::2]).astype(np.float32))
    assert (gap <= 8 * ulp).mean() > 0.8 and (gap == 0).any() and (gap > 0).any()  # a few ulps apart, some exact ties
    layer = tensor_router_layer(rng, cuda_device, wr, K, T)
    out = torch.zeros(T, D, dtype=torch.float32, device=cuda_device)
    layer.encode(x_tensor(x, cuda_device), out, T, only=("router", "route"))
    assert capi.context(0).device_status() == 0
    inds, wts = qref.route(exact, K)
    got = layer.views(T)["inds"].cpu().numpy().astype(np.uint32)
    assert np.array_equal(got, inds)
    # the boundary really splits a pair: the 7th choice's partner is the runner-up that was left out
    assert ((inds[:, -1] ^ 1)[:, None] != inds).all(axis=1).mean() > 0.9


@pytest.mark.parametrize("T", [3, 200])
def test_router_8bit_affine(cuda_device, T):
    """A router stored as 8-bit affine codes (MoE.swift:258-273 keeps the router quantized when the checkpoint does): the
    logits are the float64 dot products with the fp32 weights s*q + b, bit for bit, through both router kernels."""
    rng = np.random.default_rng(70 + T)
    E, K, D, I = 64, 4, 256, 128
    g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
    mk = lambda t: synth.dense_q_affine(t[0], t[1], t[2], 4, cuda_device)
    rw, rs, rb = synth.affine_np(rng, E, D, 8)
    dev_t = lambda a, dt: torch.from_numpy(a[0].view(dt).copy()).to(cuda_device)
    layer = MoELayer(RouterSpec(E, K), dev_t(rw, np.int32), mk(g), mk(u), mk(d), max_tokens=T,
                     router_scales=dev_t(rs, np.int16).view(torch.bfloat16), router_biases=dev_t(rb, np.int16).view(torch.bfloat16))
    x = synth.activations_np(rng, T, D)
    xt = x_tensor(x, cuda_device)
    out = torch.zeros(T, D, dtype=torch.float32, device=cuda_device)
    layer.encode(xt, out, T, only=("router", "route"))
    torch.cuda.synchronize()
    v = layer.views(T)
    wr = qref.dequant_affine(rw[0], rs[0], rb[0], 8)
    logits = qref.router_logits(x, wr)
    assert np.array_equal(v["logits"][:, :E].cpu().numpy(), logits)
    inds, _ = qref.route(logits, K)
    assert np.array_equal(v["inds"].cpu().numpy().astype(np.uint32), inds)


@pytest.mark.parametrize("act", ["gelu", "relu2"])
@pytest.mark.parametrize("T", [3, 40, 700])
def test_moe_other_activations(cuda_device, act, T):
    """GELU (tanh form) gate and relu^2 without gate (qmm.metal:9-31 ACT 1 and 3) through the decode tiles (int8 and fp16
    GEMV kernels) and the tcgen05 grouped GEMM."""
    rng = np.random.default_rng(90 + T)
    layer, host = build_layer(rng, cuda_device, 32, 2, 2048, 128, act=act, max_tokens=T)
    check_layer(layer, host, synth.activations_np(rng, T, 2048), T, act)


@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("T", [1, 19, 300])
def test_moe_shared_expert(cuda_device, T, gated):
    """A shared expert of its own width beside the routed experts, with its 8-bit sigmoid gate or weight 1
    (MoE.swift:140-154; KernelCaseMoE.swift:45-114): GEMV tiles for few tokens, the tcgen05 path for many."""
    rng = np.random.default_rng(300 + T)
    E, K, D, I, IS = 32, 4, 256, 128, 192
    sg, su, sd = synth.affine_np(rng, IS, D, 4), synth.affine_np(rng, IS, D, 4), synth.affine_np(rng, D, IS, 4)
    gw = synth.affine_np(rng, 1, D, 8)
    mk = lambda t, bits: synth.dense_q_affine(t[0], t[1], t[2], bits, cuda_device)
    g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
    wr = synth.router_np(rng, E, D)
    layer = MoELayer(RouterSpec(E, K), synth.bf16_values_tensor(wr, cuda_device), mk(g, 4), mk(u, 4), mk(d, 4), max_tokens=T,
                     shared=(mk(sg, 4), mk(su, 4), mk(sd, 4)), shared_gate=mk(gw, 8) if gated else None)
    x = synth.activations_np(rng, T, D)
    out = torch.zeros(T, D, dtype=torch.float32, device=cuda_device)
    layer.encode(x_tensor(x, cuda_device), out, T)
    torch.cuda.synchronize()
    assert capi.context(0).device_status() == 0
    deq = lambda t, e=0, bits=4: qref.dequant_affine(t[0][e], t[1][e], t[2][e], bits)
    inds, wts = qref.route(qref.router_logits(x, wr), K)
    ref = qref.moe_ffn(x, inds, wts, lambda e: (deq(g, e), deq(u, e), deq(d, e)))
    ref = ref + qref.shared_expert(x, deq(sg), deq(su), deq(sd), deq(gw, 0, 8)[0] if gated else None)
    assert qref.max_rel(out.cpu().numpy(), ref) <= TOL


def test_moe_load_guards(cuda_device):
    """Shapes the reference refuses at load (MoE.swift:186-219) come back as named errors."""
    rng = np.random.default_rng(3)
    with pytest.raises(capi.IngotError) as e:
        build_layer(rng, cuda_device, 48, 4, 256, 128)  # experts not a multiple of 32
    assert e.value.status == -2
    with pytest.raises(capi.IngotError):
        build_layer(rng, cuda_device, 32, 4, 256, 96)  # d_ff not a multiple of 64


def test_moe_pieces_and_external_routing(cuda_device):
    """`only:` runs single pieces on what earlier pieces left in the scratch; routing set by the caller is honoured."""
    rng = np.random.default_rng(4)
    T = 24
    layer, host = build_layer(rng, cuda_device, 32, 4, 256, 128, max_tokens=T)
    x = synth.activations_np(rng, T, 256)
    xt = x_tensor(x, cuda_device)
    full = torch.zeros(T, 256, dtype=torch.float32, device=cuda_device)
    layer.encode(xt, full, T)
    torch.cuda.synchronize()
    out = torch.zeros_like(full)
    for piece in ("router", "route", "group", "gateup", "down", "combine"):
        layer.encode(xt, out, T, only=piece)
    torch.cuda.synchronize()
    assert torch.equal(out, full)
    # accumulate into a residual
    res = torch.ones_like(full)
    layer.encode(xt, res, T, accumulate=True)
    torch.cuda.synchronize()
    assert torch.allclose(res - 1, full, atol=1e-5)
    # routing chosen by hand
    inds = torch.from_numpy(np.stack([rng.permutation(32)[:4] for _ in range(T)]).astype(np.int32)).to(cuda_device)
    wts = torch.from_numpy(rng.uniform(0.1, 1, size=(T, 4)).astype(np.float32)).to(cuda_device)
    layer.set_external_routing(inds, wts)
    layer.encode(xt, out, T)
    torch.cuda.synchronize()
    layer.set_external_routing(None, None)
    ref = qref.moe_ffn(x, inds.cpu().numpy().astype(np.uint32), wts.cpu().numpy(), host["weights"])
    assert qref.max_rel(out.cpu().numpy(), ref) <= TOL
