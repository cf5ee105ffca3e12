"""Seeded synthetic tensors with the shapes and value distributions of the benchmark configurations.

Small cases are drawn with numpy (`*_np`, host arrays that the tests also hand to the CPU oracle); full-size cases
are drawn directly on the device with torch's generator (`*_cuda`) so that nothing large crosses PCIe.

Distributions: affine codes uniform over all code values; scale ~ U(0.002, 0.02) rounded to bf16; bias =
bf16(-2^(bits-1) * scale + N(0, 0.001)); activations ~ N(0, 1); router bf16 ~ N(0, 0.02); MXFP4 codes uniform over the
16 e2m1 values, e8m0 scale 127 + e with e uniform in [-8, 0], expert biases ~ N(0, 0.01) rounded to bf16.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .linear import DenseQ


# ---- bf16 helpers (host) -----------------------------------------------------------------------------------------------
def to_bf16_bits(f: np.ndarray) -> np.ndarray:
    """float32 array -> bf16 bit patterns (uint16), round to nearest even."""
    t = torch.from_numpy(np.ascontiguousarray(f, dtype=np.float32)).to(torch.bfloat16)
    return t.view(torch.int16).numpy().view(np.uint16).copy()


def bf16_bits_to_f32(u: np.ndarray) -> np.ndarray:
    return (u.astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_bf16(f: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(to_bf16_bits(f))


# ---- numpy generators ---------------------------------------------------------------------------------------------
def affine_np(rng: np.random.Generator, N: int, K: int, bits: int, experts: int = 1, group: int = 64):
    """Returns (w uint32 [E, N, K*bits/32], scales uint16 bf16 bits [E, N, K/group], biases likewise)."""
    words = K * bits // 32
    w = rng.integers(0, 2**32, size=(experts, N, words), dtype=np.uint64).astype(np.uint32)
    s = to_bf16_bits(rng.uniform(0.002, 0.02, size=(experts, N, K // group)).astype(np.float32))
    sf = bf16_bits_to_f32(s)
    b = to_bf16_bits((-(2 ** (bits - 1)) * sf + rng.normal(0, 0.001, size=sf.shape)).astype(np.float32))
    return w, s, b


def mxfp4_np(rng: np.random.Generator, N: int, K: int, experts: int = 1):
    """Returns (w uint32 [E, N, K/8] of e2m1 codes, scales uint8 e8m0 [E, N, K/32])."""
    w = rng.integers(0, 2**32, size=(experts, N, K // 8), dtype=np.uint64).astype(np.uint32)
    s = (127 + rng.integers(-8, 1, size=(experts, N, K // 32))).astype(np.uint8)
    return w, s


def ternary_np(rng: np.random.Generator, N: int, K: int):
    """The rotated ternary format as the reference's tests draw it (Syn.ternary, KernelHarness.swift:125-148): codes q in
    {0, 1, 2} sixteen per word, one fp16 scale in [0.01, 0.04) per group of 128, and the rotation's signs.
    Returns (w uint32 [N, K/16], scales float16 [N, K/128], signs float32 [K])."""
    q = rng.integers(0, 3, size=(N, K), dtype=np.uint64)
    sh = (2 * (np.arange(K, dtype=np.uint64) % 16))[None, :]
    w = (q << sh).reshape(N, K // 16, 16).sum(axis=2).astype(np.uint32)
    scales = (0.01 + 0.03 * rng.random(size=(N, K // 128))).astype(np.float16)
    signs = np.where(rng.integers(0, 2, size=K) == 0, 1.0, -1.0).astype(np.float32)
    return w, scales, signs


def activations_np(rng: np.random.Generator, rows: int, K: int) -> np.ndarray:
    """x ~ N(0, 1) rounded to bf16, returned as float32 values."""
    return round_bf16(rng.normal(0, 1, size=(rows, K)).astype(np.float32))


def router_np(rng: np.random.Generator, E: int, D: int) -> np.ndarray:
    return round_bf16(rng.normal(0, 0.02, size=(E, D)).astype(np.float32))


# ---- upload ----------------------------------------------------------------------------------------------------------
def _u32_tensor(a: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int32).copy()).to(device)


def _bf16_tensor(bits: np.ndarray, device) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).to(device).view(torch.bfloat16)


def bf16_values_tensor(f: np.ndarray, device) -> torch.Tensor:
    """float32 values that are exactly bf16 -> bf16 device tensor."""
    return torch.from_numpy(np.ascontiguousarray(f, dtype=np.float32)).to(device).to(torch.bfloat16)


def dense_q_affine(w: np.ndarray, s: np.ndarray, b: np.ndarray, bits: int, device, group: int = 64) -> DenseQ:
    E, N, words = w.shape
    K = words * 32 // bits
    return DenseQ(_u32_tensor(w, device), _bf16_tensor(s, device), _bf16_tensor(b, device), N, K, bits, group, "affine", E)


def dense_q_ternary(w: np.ndarray, scales: np.ndarray, signs: np.ndarray, device) -> DenseQ:
    N, K = w.shape[0], w.shape[1] * 16
    m = DenseQ(torch.from_numpy(w.view(np.int32).copy()).to(device), torch.from_numpy(scales.copy()).to(device), None, N, K, 2,
               128, "affine")
    m.set_hadamard(torch.from_numpy(signs.copy()).to(device))
    return m


def dense_q_mxfp4(w: np.ndarray, s: np.ndarray, device) -> DenseQ:
    E, N, words = w.shape
    return DenseQ(_u32_tensor(w, device), torch.from_numpy(s.copy()).to(device), None, N, words * 8, 4, 32, "mxfp4", E)


# ---- device generators (full-size benchmark tensors) -----------------------------------------------------------------
def affine_cuda(gen: torch.Generator, N: int, K: int, bits: int, experts: int = 1, group: int = 64) -> DenseQ:
    dev = gen.device
    words = K * bits // 32
    w = torch.randint(-2**31, 2**31 - 1, (experts, N, words), dtype=torch.int32, device=dev, generator=gen)
    s = (0.002 + 0.018 * torch.rand((experts, N, K // group), device=dev, generator=gen)).to(torch.bfloat16)
    b = (-(2 ** (bits - 1)) * s.float() + 0.001 * torch.randn(s.shape, device=dev, generator=gen)).to(torch.bfloat16)
    return DenseQ(w, s, b, N, K, bits, group, "affine", experts)


def mxfp4_cuda(gen: torch.Generator, N: int, K: int, experts: int = 1) -> DenseQ:
    dev = gen.device
    w = torch.randint(-2**31, 2**31 - 1, (experts, N, K // 8), dtype=torch.int32, device=dev, generator=gen)
    s = (127 + torch.randint(-8, 1, (experts, N, K // 32), device=dev, generator=gen)).to(torch.uint8)
    return DenseQ(w, s, None, N, K, 4, 32, "mxfp4", experts)


def activations_cuda(gen: torch.Generator, rows: int, K: int, dtype=torch.bfloat16) -> torch.Tensor:
    return torch.randn((rows, K), device=gen.device, generator=gen).to(dtype)


def router_cuda(gen: torch.Generator, E: int, D: int) -> torch.Tensor:
    return (0.02 * torch.randn((E, D), device=gen.device, generator=gen)).to(torch.bfloat16)
