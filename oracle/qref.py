"""CPU oracle of ingot's quantized-matmul path (numpy). TEST INFRASTRUCTURE ONLY.

This module restates, in fp32/fp64 numpy, what the reference engine's quantized linear and MoE operators compute.
It is the checker for the CUDA kernels: only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it. The library proper never does (it fails loudly when its CUDA extension is missing).

Sources restated here (paths inside the reference project):
  * weight formats, bf16 conversions, pack/unpack, CPU dequantisation: Sources/Ingot/Loader/Quant.swift:4-12,119-202
  * nibble-order and dequant known answers: Tests/IngotTests/FormatTests.swift:39-70
  * MXFP4 known answers: Tests/IngotTests/KernelCaseMXFP4.swift:141-182 (generator ref/mxfp4_ref.py:16-18)
  * router rule (top-k, ties to the lower index, weights): Tests/IngotTests/KernelCaseRouter.swift:57-80,
    Sources/Ingot/Shaders/qmm_nax_moe.metal:57-94
  * fp32 "truth" MoE block: ref/moe_ref.py:107-136; CPU MoE with given routing, h rounding, biases:
    Tests/IngotTests/KernelHarness.swift:720-766
  * activations: Sources/Ingot/Shaders/qmm.metal:17-31, Tests/IngotTests/KernelHarness.swift:176-188
  * error metric: Tests/IngotTests/KernelHarness.swift:39-47

The arithmetic itself is defined by MLX (ml-explore/mlx, `quantized.h`, `fp_quantized.h`) and mlx-lm 0.32.2, neither
vendored in the reference; parity is pinned on the reference's own golden vectors (tests/golden/*.json). The affine
qmv/qmm/gather_qmm *outputs* have no stored vectors in the reference (its tests draw random tensors): for those the
oracle is pinned only through the dequantisation known answers plus the matmul definition.
"""
from __future__ import annotations

import numpy as np

# ----------------------------------------------------------------------------------------------------------------
# bf16 / fp16 helpers


def bf16_to_f32(u16: np.ndarray) -> np.ndarray:
    """bf16 bit patterns (uint16) -> float32 (Quant.swift:119: bits << 16)."""
    return (np.asarray(u16, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def f32_to_bf16(f: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns with round-to-nearest-even (Quant.swift:121-125). NaN is not handled, as there."""
    u = np.ascontiguousarray(f, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint16)


def round_bf16(f: np.ndarray) -> np.ndarray:
    return bf16_to_f32(f32_to_bf16(f))


def round_f16(f: np.ndarray) -> np.ndarray:
    return np.asarray(f, dtype=np.float32).astype(np.float16).astype(np.float32)


# ----------------------------------------------------------------------------------------------------------------
# packing (Quant.swift:129-147)


def pack_q(q: np.ndarray, bits: int) -> np.ndarray:
    """Pack integer codes [..., K] into uint32 [..., K*bits/32]; value j sits in bits [bits*j, bits*j+bits) of the row
    (for widths that do not divide 32 the row is one little-endian bit stream, Quant.swift:126-136)."""
    if 32 % bits != 0:
        q = np.asarray(q, dtype=np.uint8) & np.uint8((1 << bits) - 1)
        assert (q.shape[-1] * bits) % 32 == 0
        b = np.unpackbits(q[..., None], axis=-1, bitorder="little")[..., :bits]
        by = np.packbits(b.reshape(*q.shape[:-1], -1), axis=-1, bitorder="little")
        return np.ascontiguousarray(by).view(np.uint32)
    per = 32 // bits
    q = np.asarray(q, dtype=np.uint32) & np.uint32((1 << bits) - 1)
    assert q.shape[-1] % per == 0
    q = q.reshape(*q.shape[:-1], q.shape[-1] // per, per)
    sh = (np.arange(per, dtype=np.uint32) * np.uint32(bits)).astype(np.uint32)
    return np.bitwise_or.reduce(q << sh, axis=-1).astype(np.uint32)


def unpack_q(w: np.ndarray, bits: int) -> np.ndarray:
    """uint32 [..., W] -> codes uint32 [..., W*32/bits] (inverse of pack_q)."""
    if 32 % bits != 0:
        by = np.ascontiguousarray(np.asarray(w, dtype=np.uint32)).view(np.uint8)
        b = np.unpackbits(by, axis=-1, bitorder="little").reshape(*by.shape[:-1], -1, bits)
        return np.packbits(b, axis=-1, bitorder="little")[..., 0].astype(np.uint32)
    per = 32 // bits
    w = np.asarray(w, dtype=np.uint32)
    sh = (np.arange(per, dtype=np.uint32) * np.uint32(bits)).astype(np.uint32)
    q = (w[..., None] >> sh) & np.uint32((1 << bits) - 1)
    return q.reshape(*w.shape[:-1], w.shape[-1] * per)


# ----------------------------------------------------------------------------------------------------------------
# MXFP4 element / scale decode (Quant.swift:190-202)

E2M1 = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6], dtype=np.float32)


def e8m0_to_f32(s: np.ndarray) -> np.ndarray:
    s = np.asarray(s, dtype=np.uint8)
    out = np.ldexp(np.float32(1), s.astype(np.int32) - 127).astype(np.float32)
    return np.where(s == 255, np.float32(np.nan), out)


# ----------------------------------------------------------------------------------------------------------------
# dequantisation (Quant.swift:162-188)


def dequant_affine(w: np.ndarray, scales: np.ndarray, biases: np.ndarray, bits: int, group: int = 64) -> np.ndarray:
    """w uint32 [..., N, K*bits/32], scales/biases bf16 bits [..., N, K/group] -> float32 [..., N, K]: s*q + b."""
    q = unpack_q(w, bits).astype(np.float32)
    s = np.repeat(bf16_to_f32(scales), group, axis=-1)
    b = np.repeat(bf16_to_f32(biases), group, axis=-1)
    assert q.shape == s.shape, (q.shape, s.shape)
    return (s * q + b).astype(np.float32)


def dequant_mxfp4(w: np.ndarray, scales_u8: np.ndarray) -> np.ndarray:
    """w uint32 [..., N, K/8] (e2m1 nibbles, low nibble first), scales uint8 e8m0 [..., N, K/32] -> float32."""
    q = unpack_q(w, 4)
    v = E2M1[q]
    s = np.repeat(e8m0_to_f32(scales_u8), 32, axis=-1)
    return (s * v).astype(np.float32)


# ----------------------------------------------------------------------------------------------------------------
# matmul


def matmul_t(x: np.ndarray, wf: np.ndarray) -> np.ndarray:
    """Y[M,N] = X[M,K] · W[N,K]^T with a float64 accumulator, returned as float32 (the fp32 reference value)."""
    return (np.asarray(x, dtype=np.float64) @ np.asarray(wf, dtype=np.float64).T).astype(np.float32)


def qmm_affine(x, w, scales, biases, bits, group=64):
    return matmul_t(x, dequant_affine(w, scales, biases, bits, group))


# ----------------------------------------------------------------------------------------------------------------
# activations (qmm.metal:17-31; KernelHarness.swift:176-188)


def silu_glu(g, u):
    g = np.asarray(g, dtype=np.float32)
    return (g / (np.float32(1) + np.exp(-g)) * np.asarray(u, dtype=np.float32)).astype(np.float32)


def swiglu_oai(g, u, limit: float = 7.0, alpha: float = 1.702):
    g = np.minimum(np.asarray(g, dtype=np.float32), np.float32(limit))
    u = np.clip(np.asarray(u, dtype=np.float32), np.float32(-limit), np.float32(limit))
    return ((u + np.float32(1)) * (g / (np.float32(1) + np.exp(np.float32(-alpha) * g)))).astype(np.float32)


def gelu_glu(g, u):
    """GELU (tanh form, mlx-lm nn.gelu_approx) gate: 0.5 g (1 + tanh z) u, z = sqrt(2/pi) (g + 0.044715 g^3), written as
    g sigmoid(2z) u like the reference (qmm.metal:11-13, 21-23)."""
    g = np.asarray(g, dtype=np.float32)
    z2 = (np.float32(1.5957691216057308) * (g + np.float32(0.044715) * g * g * g)).astype(np.float32)
    with np.errstate(over="ignore"):
        return (g / (np.float32(1) + np.exp(-z2)) * np.asarray(u, dtype=np.float32)).astype(np.float32)


def relu2(g, u):
    """Nemotron-H's relu^2 without gate (qmm.metal:15-16, 24-26): max(u, 0)^2; g is ignored."""
    r = np.maximum(np.asarray(u, dtype=np.float32), np.float32(0))
    return (r * r).astype(np.float32)


ACTS = {"silu": silu_glu, "swiglu_oai": swiglu_oai, "gelu": gelu_glu, "relu2": relu2}

# ----------------------------------------------------------------------------------------------------------------
# router


def router_logits(x: np.ndarray, wr: np.ndarray) -> np.ndarray:
    """fp32 logits defined as the correctly rounded dot product (float64 accumulation, one rounding to float32).

    x [T, D] and wr [E, D] hold values exactly representable in fp32 (bf16/fp16 inputs), so every product is exact in
    float64 and the sum does not depend on the order at fp32 resolution. The CUDA router accumulates in float64 for
    the same reason: it makes the top-k indices reproducible bit for bit."""
    return (np.asarray(x, dtype=np.float64) @ np.asarray(wr, dtype=np.float64).T).astype(np.float32)


def route(logits: np.ndarray, top_k: int, *, logit_bias=None, select_bias=None, sigmoid: bool = False,
          scale: float = 1.0, eps: float = 0.0, per_expert_scale=None):
    """The engine's routing rule (KernelCaseRouter.swift:57-80): returns (inds uint32 [T,k], wts float32 [T,k]).

    Top-k by score (+ selection bias), descending, ties to the lower index, NaN treated as -inf; weights from the
    unbiased scores: softmax over the chosen logits (exp(l - l_top1) / sum) or sigmoid p / (sum p + eps); then
    x scale and x per-expert scale. A router linear bias (`logit_bias`) is part of the logits."""
    l = np.array(logits, dtype=np.float32, copy=True)
    T, E = l.shape
    if logit_bias is not None:
        l = (l + np.asarray(logit_bias, dtype=np.float32)[None, :]).astype(np.float32)
    if sigmoid:
        # the fp32 score is the correctly rounded sigmoid (evaluated in float64): independent of an exp implementation
        with np.errstate(over="ignore"):
            p = (1.0 / (1.0 + np.exp(-l.astype(np.float64)))).astype(np.float32)
    else:
        p = l
    sel = p if select_bias is None else (p + np.asarray(select_bias, dtype=np.float32)[None, :]).astype(np.float32)
    sel = np.where(np.isnan(sel), np.float32(-np.inf), sel)
    # stable argsort of -sel keeps the lower index first among equal scores
    order = np.argsort(-sel.astype(np.float64), axis=1, kind="stable")[:, :top_k]
    inds = order.astype(np.uint32)
    top = np.take_along_axis(p, order, axis=1)
    if sigmoid:
        w = top.copy()
        s = np.zeros(T, dtype=np.float32)
        for k in range(top_k):  # sequential fp32 sum, k order
            s = (s + w[:, k]).astype(np.float32)
        s = (s + np.float32(eps)).astype(np.float32)
        w = (w / s[:, None]).astype(np.float32)
    else:
        ex = np.exp((top - top[:, :1]).astype(np.float32)).astype(np.float32)
        s = np.zeros(T, dtype=np.float32)
        for k in range(top_k):
            s = (s + ex[:, k]).astype(np.float32)
        w = (ex / s[:, None]).astype(np.float32)
    w = (w * np.float32(scale)).astype(np.float32)
    if per_expert_scale is not None:
        w = (w * np.asarray(per_expert_scale, dtype=np.float32)[order]).astype(np.float32)
    return inds, w


def group_pairs(inds: np.ndarray, n_experts: int):
    """Token->expert permutation (moe_group, qmm_nax_moe.metal:139-217) with the order inside an expert fixed to
    ascending pair id (the reference leaves it to its atomics and declares it irrelevant).

    Returns offsets [E+1], row_map [P] (sorted position -> pair id), pos [P] (pair id -> sorted position)."""
    flat = np.asarray(inds, dtype=np.int64).reshape(-1)
    row_map = np.argsort(flat, kind="stable").astype(np.uint32)
    counts = np.bincount(flat, minlength=n_experts)
    offsets = np.zeros(n_experts + 1, dtype=np.uint32)
    offsets[1:] = np.cumsum(counts)
    pos = np.empty_like(row_map)
    pos[row_map] = np.arange(flat.size, dtype=np.uint32)
    return offsets, row_map, pos


# ----------------------------------------------------------------------------------------------------------------
# MoE FFN


def moe_ffn(x: np.ndarray, inds: np.ndarray, wts: np.ndarray, expert_weights, *, act: str = "silu",
            limit: float = 7.0, biases=None, half_gu: bool = False, round_h: bool = True) -> np.ndarray:
    """MoE layer with the routing given (KernelHarness.swift:720-766):
    y[t] = sum_k w[t,k] * (down_e(h) + bd_e), h = half(act(gate_e x + bg_e, up_e x + bu_e)).

    expert_weights(e) -> (gate [I,D], up [I,D], down [D,I]) float32, called only for experts some row picks.
    biases = (bg [E,I], bu [E,I], bd [E,D]) or None. half_gu rounds gate and up to half before the activation (the
    reference's prefill kernels); round_h rounds h to half (both decode and prefill kernels do)."""
    x = np.asarray(x, dtype=np.float32)
    T, D = x.shape
    K = inds.shape[1]
    y = np.zeros((T, D), dtype=np.float64)
    flat = np.asarray(inds, dtype=np.int64).reshape(-1)
    wf = np.asarray(wts, dtype=np.float32).reshape(-1)
    for e in np.unique(flat):
        hits = np.nonzero(flat == e)[0]
        gate, up, down = expert_weights(int(e))
        xs = x[hits // K]
        g = matmul_t(xs, gate)
        u = matmul_t(xs, up)
        if biases is not None:
            g = (g + biases[0][e][None, :]).astype(np.float32)
            u = (u + biases[1][e][None, :]).astype(np.float32)
        if half_gu:
            g, u = round_f16(g), round_f16(u)
        h = ACTS[act](g, u) if act != "swiglu_oai" else swiglu_oai(g, u, limit)
        if round_h:
            h = round_f16(h)
        o = matmul_t(h, down)
        if biases is not None:
            o = (o + biases[2][e][None, :]).astype(np.float32)
        np.add.at(y, hits // K, wf[hits, None].astype(np.float64) * o.astype(np.float64))
    return y.astype(np.float32)


def shared_expert(x, gate, up, down, gate_w=None, *, act: str = "silu", round_h: bool = True):
    """The shared expert's contribution (MoE.swift:140-154; verify.metal:262-281): w_s * down(half(act(gate x, up x))) with
    w_s = sigmoid(x . gate_w) per token, or 1 without a gate tensor. gate/up [I_s, D], down [D, I_s], gate_w [D]."""
    x = np.asarray(x, dtype=np.float32)
    h = ACTS[act](matmul_t(x, gate), matmul_t(x, up))
    if round_h:
        h = round_f16(h)
    y = matmul_t(h, down)
    if gate_w is None:
        return y
    logit = (x.astype(np.float64) @ np.asarray(gate_w, dtype=np.float64)).astype(np.float32)
    with np.errstate(over="ignore"):
        w = (1.0 / (1.0 + np.exp(-logit.astype(np.float64)))).astype(np.float32)
    return (w[:, None] * y).astype(np.float32)


def moe_block(x, router_w, top_k, expert_weights, *, router_bias=None, **kw):
    """Router + MoE FFN: returns (y, inds, wts, logits). Equals ref/moe_ref.py:107-136 without its shared expert:
    softmax over all experts, top-k, renormalise == softmax over the top-k logits (the engine's form)."""
    logits = router_logits(x, router_w)
    inds, wts = route(logits, top_k, logit_bias=router_bias)
    return moe_ffn(x, inds, wts, expert_weights, **kw), inds, wts, logits


def rmsnorm(r: np.ndarray, eps: float = 1e-6) -> np.ndarray:
    """Unit-weight RMSNorm in fp32 (verify.metal:503-523), the input normalisation of the layer stack."""
    r = np.asarray(r, dtype=np.float32)
    ms = (r.astype(np.float64) ** 2).mean(axis=-1, keepdims=True)
    return (r / np.sqrt(ms + eps)).astype(np.float32)


# ----------------------------------------------------------------------------------------------------------------
# error metric (KernelHarness.swift:39-47)


def max_rel(got: np.ndarray, ref: np.ndarray) -> float:
    """max|got - ref| / max|ref|; NaN anywhere in `got` gives infinity."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    if np.isnan(got).any():
        return float("inf")
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


# ----------------------------------------------------------------------------------------------------------------
# sampling candidates


def topk64(row: np.ndarray, temperature: float, k: int = 64):
    """The sampler's candidates of one row of logits (TopK64Tests.swift:44-63): the logits x >= -FLT_MAX by value
    descending, ties to the lower id, padded with (0xFFFFFFFF, -FLT_MAX); the row maximum; Z = sum exp((x - max) / T)
    in float64."""
    row = np.asarray(row, dtype=np.float32)
    fmax = np.float32(np.finfo(np.float32).max)
    cand = np.nonzero(row >= -fmax)[0]
    order = cand[np.lexsort((cand, -row[cand].astype(np.float64)))][:k]
    ids = np.full(k, 0xFFFFFFFF, dtype=np.uint32)
    vals = np.full(k, -fmax, dtype=np.float32)
    ids[: len(order)] = order
    vals[: len(order)] = row[order]
    with np.errstate(invalid="ignore", over="ignore"):
        mx = np.float32(np.nanmax(row)) if row.size else np.float32(-np.inf)
        z = float(np.sum(np.exp((row.astype(np.float64) - float(mx)) / temperature)))
    return ids, vals, mx, z


def argmax_rows(x: np.ndarray) -> np.ndarray:
    """Index of the largest value of each row, ties to the lower index (verify.metal:525-547)."""
    return np.argmax(np.asarray(x, dtype=np.float32), axis=1).astype(np.uint32)


# ----------------------------------------------------------------------------------------------------------------
# Formats whose kernels are not built yet. PARITY UNPINNED: the reference stores no vectors for them (its tests draw
# random tensors and compare with the CPU code restated below); what pins these functions is the algebra checked in
# tests/test_oracle_formats.py (H H = n I, the rotation against an explicit Hadamard matrix, the embedding's inverse).


def fwht(v: np.ndarray) -> np.ndarray:
    """Unnormalised Sylvester Walsh-Hadamard transform over the last axis (a power of two), float32 arithmetic in the
    order of the reference's butterfly (Tests/IngotTests/KernelHarness.swift:196-210)."""
    v = np.array(v, dtype=np.float32, copy=True)
    n = v.shape[-1]
    assert n & (n - 1) == 0
    h = 1
    while h < n:
        w = v.reshape(*v.shape[:-1], n // (2 * h), 2, h)
        a, b = w[..., 0, :].copy(), w[..., 1, :].copy()
        w[..., 0, :] = a + b
        w[..., 1, :] = a - b
        h *= 2
    return v


def rotate_input(x: np.ndarray, signs: np.ndarray, block: int = 1024) -> np.ndarray:
    """The ternary layers' input rotation: x <- H_1024(x * signs) / 32 per block of 1024 inputs, rounded to fp16
    (had_rows_h, Shaders/xc_tern.metal:29-40; CPU.rotate, KernelHarness.swift:212-224)."""
    x = np.asarray(x, dtype=np.float32)
    rows, K = x.shape
    assert K % block == 0
    v = (x * np.asarray(signs, dtype=np.float32)[None, :]).reshape(rows, K // block, block)
    return round_f16((fwht(v) / np.float32(np.sqrt(block))).reshape(rows, K))


def dequant_ternary(w: np.ndarray, scales_f16: np.ndarray) -> np.ndarray:
    """2-bit codes q in {0, 1, 2}, sixteen per word low bits first, w = (q - 1) * s with one fp16 scale per group of 128
    (Syn.ternary, KernelHarness.swift:125-148; embed_rows_t, xc_tern.metal:56-61). w uint32 [N, K/16], scales float16
    [N, K/128] -> float32 [N, K]."""
    q = unpack_q(w, 2).astype(np.float32) - np.float32(1)
    s = np.repeat(np.asarray(scales_f16, dtype=np.float16).astype(np.float32), 128, axis=-1)
    assert q.shape == s.shape, (q.shape, s.shape)
    return q * s


def embed_ternary(w: np.ndarray, scales_f16: np.ndarray, signs: np.ndarray, tokens, block: int = 1024) -> np.ndarray:
    """Rows of a ternary table back in the un-rotated basis: H_1024(row) / 32 * signs per block (embed_rows_t,
    xc_tern.metal:44-65; the bonsai-embed case, KernelCaseTests.swift:133-155)."""
    rows = dequant_ternary(w, scales_f16)[np.asarray(tokens, dtype=np.int64)]
    T, K = rows.shape
    v = fwht(rows.reshape(T, K // block, block)) / np.float32(np.sqrt(block))
    return v.reshape(T, K) * np.asarray(signs, dtype=np.float32)[None, :]


def quant_i8_rows(a: np.ndarray):
    """Symmetric int8 per row: scale max|a| / 127 (1 for a zero row), round half to even, clamp to +-127
    (CPU.quantI8, KernelHarness.swift:250-255). Returns (values as float32, scales)."""
    a = np.asarray(a, dtype=np.float32)
    amax = np.abs(a).max(axis=1)
    sc = np.where(amax > 0, amax / np.float32(127), np.float32(1)).astype(np.float32)
    q = np.clip(np.rint(a / sc[:, None]), -127, 127).astype(np.float32)
    return q, sc


def w8a8_emulated(x: np.ndarray, wf: np.ndarray, lb: int) -> np.ndarray:
    """The lossy prefill GEMM of the serving path, emulated: unnormalised Hadamard of n = 32 * 2^lb per contiguous block of
    x and of W, int8 per row, Y = (Xq Wq^T) sx sw / n (CPU.w8a8, KernelHarness.swift:225-248; the kernel case takes
    lb = 3 when K / 32 is a multiple of 32, else 0: KernelCaseTests.swift:645)."""
    x = np.asarray(x, dtype=np.float32)
    wf = np.asarray(wf, dtype=np.float32)
    n = 32 << lb
    K = x.shape[1]
    assert K % n == 0 and wf.shape[1] == K
    rot = lambda a: fwht(a.reshape(a.shape[0], K // n, n)).reshape(a.shape[0], K)
    xq, sx = quant_i8_rows(rot(x))
    wq, sw = quant_i8_rows(rot(wf))
    y = (xq.astype(np.float64) @ wq.astype(np.float64).T).astype(np.float32)
    return y * sx[:, None] * sw[None, :] / np.float32(n)


def w8a8_ternary_emulated(xr: np.ndarray, w: np.ndarray, scales_f16: np.ndarray) -> np.ndarray:
    """The ternary layers' W8A8 prefill GEMM, emulated (the bonsai-int8 kernel case,
    Tests/IngotTests/KernelCaseFlashNextI8.swift:155-213): `xr` is the already rotated input (rotate_input); it goes to
    int8 per row; a weight row goes to int8 with ONE scale, s_row = max_g |s_g| / 127, as t * round(|s_g| / s_row) with
    t the ternary digit; Y = (Xq Wq^T) sx sw. w uint32 [N, K/16], scales float16 [N, K/128]."""
    xq, sx = quant_i8_rows(np.asarray(xr, dtype=np.float32))
    t = unpack_q(w, 2).astype(np.float32) - np.float32(1)
    sg = np.abs(np.asarray(scales_f16, dtype=np.float16).astype(np.float32))
    gmax = sg.max(axis=1)
    srow = np.where(gmax > 0, gmax / np.float32(127), np.float32(1)).astype(np.float32)
    qg = np.rint(sg / srow[:, None]).astype(np.float32)
    sign = np.sign(np.asarray(scales_f16, dtype=np.float16).astype(np.float32))
    wq = t * np.repeat(qg * sign, 128, axis=1)
    y = (xq.astype(np.float64) @ wq.astype(np.float64).T).astype(np.float32)
    return y * sx[:, None] * srow[None, :]
