"""Helpers of the GPU parity tests: seeded tensors on the host for the oracle, the same bytes on the device."""
import numpy as np
import torch

from ingot_b200 import synth
from oracle import qref

TOL = 1e-3  # max|gpu - ref| / max|ref| against the fp32 CPU oracle, asserted on fp32 outputs


def affine_case(rng, N, K, bits, device, experts=1, group=64):
    w, s, b = synth.affine_np(rng, N, K, bits, experts, group)
    return synth.dense_q_affine(w, s, b, bits, device, group), (w, s, b)


def mxfp4_case(rng, N, K, device, experts=1):
    w, s = synth.mxfp4_np(rng, N, K, experts)
    return synth.dense_q_mxfp4(w, s, device), (w, s)


def x_tensor(x_np, device, dtype=torch.bfloat16):
    return torch.from_numpy(x_np).to(device).to(dtype)


def deq(host, bits=4, e=0, group=64):
    if len(host) == 3:
        return qref.dequant_affine(host[0][e], host[1][e], host[2][e], bits, group)
    return qref.dequant_mxfp4(host[0][e], host[1][e])


def bf16_rne(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16)
