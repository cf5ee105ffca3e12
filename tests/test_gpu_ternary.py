"""The rotated ternary format (2-bit codes, groups of 128, fp16 scale, w = (q - 1) * s, inputs rotated by a blockwise
Hadamard transform): rotation, decode GEMV, prefill GEMM and embedding against the CPU oracle. Mirrors the reference's
bonsai-qmv, bonsai-prefill and bonsai-embed kernel cases (Tests/IngotTests/KernelCaseTests.swift:97-155), with their
shapes and their 1e-4 bound."""
import numpy as np
import pytest
import torch

from ingot_b200 import capi, synth
from ingot_b200.linear import VQMV
from oracle import qref
from gpu_util import x_tensor

pytestmark = pytest.mark.gpu
TERN_TOL = 1e-4  # the reference's bound for these kernels (.maxRel(1e-4))


def case(rng, N, K, device):
    w, s, signs = synth.ternary_np(rng, N, K)
    return synth.dense_q_ternary(w, s, signs, device), qref.dequant_ternary(w, s), signs, (w, s)


def half_activations(rng, rows, K):
    return qref.round_f16(rng.normal(0, 1, size=(rows, K)).astype(np.float32))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_rotation_is_the_cpu_rule_bit_for_bit(cuda_device, dtype):
    """H_1024(x * signs) / 32 per block, fp32 butterflies in the reference's order, rounded once to half."""
    rng = np.random.default_rng(1)
    m, _, signs, _ = case(rng, 16, 3072, cuda_device)
    x = synth.activations_np(rng, 5, 3072) if dtype != torch.float32 else rng.normal(0, 1, size=(5, 3072)).astype(np.float32)
    if dtype == torch.float16:
        x = qref.round_f16(x)
    got = m.encode_rotate(x_tensor(x, cuda_device, dtype), 5)[:5].float().cpu().numpy()
    assert np.array_equal(got, qref.rotate_input(x, signs))


@pytest.mark.parametrize("N,K,rows", [(64, 2048, 16), (64, 2048, 5), (32, 9216, 16), (128, 1024, 1)])
def test_ternary_qmv(cuda_device, N, K, rows):
    rng = np.random.default_rng(N + K + rows)
    m, wf, signs, _ = case(rng, N, K, cuda_device)
    x = half_activations(rng, rows, K)
    y = torch.zeros(rows, N, dtype=torch.float32, device=cuda_device)
    VQMV.encode(x_tensor(x, cuda_device, torch.float16), m, y, rows)
    torch.cuda.synchronize()
    ref = qref.matmul_t(qref.rotate_input(x, signs), wf)
    err = qref.max_rel(y.cpu().numpy(), ref)
    assert err <= TERN_TOL, err


def test_ternary_qmv_row_invariance_accumulate_prefix(cuda_device):
    rng = np.random.default_rng(7)
    N, K = 64, 2048
    m, wf, signs, _ = case(rng, N, K, cuda_device)
    x = half_activations(rng, 16, K)
    xt = x_tensor(x, cuda_device, torch.float16)
    full = torch.zeros(16, N, dtype=torch.float32, device=cuda_device)
    VQMV.encode(xt, m, full, 16)
    for i in (0, 4, 8, 15):  # a row alone, and among i + 1: the same bits (KernelCaseTests.swift:113)
        alone = torch.zeros(1, N, dtype=torch.float32, device=cuda_device)
        VQMV.encode(xt[i:i + 1].contiguous(), m, alone, 1)
        part = torch.zeros(i + 1, N, dtype=torch.float32, device=cuda_device)
        VQMV.encode(xt[: i + 1].contiguous(), m, part, i + 1)
        torch.cuda.synchronize()
        assert torch.equal(alone[0], full[i]) and torch.equal(part[i], full[i])
    ref = qref.matmul_t(qref.rotate_input(x, signs), wf)
    y0 = torch.from_numpy(rng.normal(size=(16, N)).astype(np.float32)).to(cuda_device)
    y = y0.clone()
    VQMV.encode(xt, m, y, 16, accumulate=True)
    yp = torch.full((16, N), -1.0, dtype=torch.float32, device=cuda_device)
    VQMV.encode(xt, m, yp, 16, n_prefix=32)
    torch.cuda.synchronize()
    assert qref.max_rel((y - y0).cpu().numpy(), ref) <= TERN_TOL
    assert qref.max_rel(yp[:, :32].cpu().numpy(), ref[:, :32]) <= TERN_TOL and (yp[:, 32:] == -1.0).all()


@pytest.mark.parametrize("M,N,K", [(64, 64, 2048), (64, 128, 4096), (320, 256, 1024)])
def test_ternary_prefill_gemm(cuda_device, M, N, K):
    """The tcgen05 GEMM with the ternary dequantiser, after the input rotation (bonsai-prefill)."""
    rng = np.random.default_rng(M + N + K)
    m, wf, signs, _ = case(rng, N, K, cuda_device)
    x = half_activations(rng, M, K)
    y = torch.zeros(M, N, dtype=torch.float32, device=cuda_device)
    m.encode_qmm_f32(x_tensor(x, cuda_device, torch.float16), y, M)
    assert capi.context(0).device_status() == 0
    ref = qref.matmul_t(qref.rotate_input(x, signs), wf)
    err = qref.max_rel(y.cpu().numpy(), ref)
    assert err <= TERN_TOL, err


def test_ternary_unpacked_codes_bit_exact(cuda_device):
    """Scale 1 and one-hot rotated inputs read the codes back: (q - 1) exactly, through the GEMV and the GEMM."""
    rng = np.random.default_rng(9)
    N, K = 64, 1024
    w, _, signs = synth.ternary_np(rng, N, K)
    s = np.ones((N, K // 128), dtype=np.float16)
    m = synth.dense_q_ternary(w, s, signs, cuda_device)
    m.had = None  # feed the kernels directly: no rotation
    codes = qref.unpack_q(w, 2).astype(np.float32) - 1
    eye = torch.eye(K, dtype=torch.float16, device=cuda_device)
    for r0 in (0, 512, 1008):
        y = torch.zeros(16, N, dtype=torch.float32, device=cuda_device)
        VQMV.encode(eye[r0:r0 + 16].contiguous(), m, y, 16)
        torch.cuda.synchronize()
        assert np.array_equal(y.cpu().numpy().T, codes[:, r0:r0 + 16])
    y = torch.zeros(K, N, dtype=torch.float32, device=cuda_device)
    m.encode_qmm_f32(eye, y, K)
    assert capi.context(0).device_status() == 0
    assert np.array_equal(y.cpu().numpy().T, codes)


def test_ternary_embedding(cuda_device):
    """Rows of a ternary table back in the un-rotated basis (bonsai-embed: V = 40, K = 2048, six tokens)."""
    rng = np.random.default_rng(11)
    V, K = 40, 2048
    m, _, signs, (w, s) = case(rng, V, K, cuda_device)
    tok = [3, 0, 39, 17, 17, 8]
    tt = torch.tensor(tok, dtype=torch.int32, device=cuda_device)
    of = torch.zeros(6, K, dtype=torch.float32, device=cuda_device)
    oh = torch.zeros(6, K, dtype=torch.float16, device=cuda_device)
    m.encode_embed(tt, 6, out_f=of, out_h=oh)
    torch.cuda.synchronize()
    ref = qref.embed_ternary(w, s, signs, tok)
    assert qref.max_rel(of.cpu().numpy(), ref) <= 1e-6
    assert torch.equal(oh, of.to(torch.float16))


def test_ternary_guards(cuda_device):
    rng = np.random.default_rng(12)
    m, _, _, _ = case(rng, 64, 1024, cuda_device)
    x = torch.zeros(2, 1024, dtype=torch.bfloat16, device=cuda_device)
    y = torch.zeros(2, 64, dtype=torch.float32, device=cuda_device)
    m.had = None
    with pytest.raises(capi.IngotError) as e:  # the kernel takes the rotation's fp16 output
        VQMV.encode(x, m, y, 2)
    assert e.value.status == -1
