"""Rotated W8A8 prefill GEMM (iq_qmm_w8a8 through DenseQ.encode_qmm_i8) against the CPU emulation of the same arithmetic
and against the exact product. Mirrors the reference's int8-serve kernel case
(Tests/IngotTests/KernelCaseTests.swift:623-661): its shapes, its activations with a few outlier channels, its bounds
(relative RMS error 2e-3 against the emulation, 5e-2 against the exact one)."""
import numpy as np
import pytest
import torch

from ingot_b200 import capi, synth
from oracle import qref
from gpu_util import affine_case, deq, x_tensor

pytestmark = pytest.mark.gpu


def rel_rms(got, ref):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return float(np.sqrt(((got - ref) ** 2).sum() / max((ref ** 2).sum(), 1e-300)))


@pytest.mark.parametrize("K,N,M,group", [(2048, 256, 64, 64), (1536, 256, 64, 64), (9216, 256, 64, 64), (2048, 384, 320, 64),
                                         (1024, 128, 64, 32)])
def test_w8a8_against_emulation_and_exact(cuda_device, K, N, M, group):
    rng = np.random.default_rng(K + N + M)
    m, host = affine_case(rng, N, K, 4, cuda_device, group=group)
    wf = deq(host, 4, group=group)
    x = rng.normal(0, 1, size=(M, K)).astype(np.float32)
    for ch in (7, 300, K - 5):  # a few outlier channels: what the rotation is for
        x[:, ch] *= 20
    x = qref.round_f16(x)
    y = torch.zeros(M, N, dtype=torch.float32, device=cuda_device)
    m.encode_qmm_i8(x_tensor(x, cuda_device, torch.float16), y, M)
    assert capi.context(0).device_status() == 0
    got = y.cpu().numpy()
    lb = 3 if (K // 32) % 32 == 0 else 0
    e_emul = rel_rms(got, qref.w8a8_emulated(x, wf, lb))
    e_exact = rel_rms(got, qref.matmul_t(x, wf))
    assert e_emul <= 2e-3, e_emul
    assert e_exact <= 5e-2, e_exact


def test_w8a8_outputs_accumulate_and_guards(cuda_device):
    rng = np.random.default_rng(5)
    M, N, K = 128, 128, 1024
    m, host = affine_case(rng, N, K, 4, cuda_device)
    x = synth.activations_np(rng, M, K)
    xt = x_tensor(x, cuda_device)  # bf16 activations
    y = torch.zeros(M, N, dtype=torch.float32, device=cuda_device)
    m.encode_qmm_i8(xt, y, M)
    ref = qref.w8a8_emulated(x, deq(host, 4), 3)
    assert rel_rms(y.cpu().numpy(), ref) <= 2e-3
    yb = torch.zeros(M, N, dtype=torch.bfloat16, device=cuda_device)
    m.encode_qmm_i8(xt, yb, M)
    y0 = torch.ones(M, N, dtype=torch.float32, device=cuda_device)
    m.encode_qmm_i8(xt, y0, M, accumulate=True)
    torch.cuda.synchronize()
    assert torch.equal(yb, y.to(torch.bfloat16))
    assert torch.allclose(y0 - 1, y, atol=1e-4)
    m8, _ = affine_case(rng, N, K, 8, cuda_device)
    with pytest.raises(capi.IngotError) as e:  # 8-bit layers go through the exact GEMM (DenseQ.int8OK)
        m8.encode_qmm_i8(xt, y, M)
    assert e.value.status == -2
    with pytest.raises(capi.IngotError):
        m.encode_qmm_i8(xt[:96], y, 96)  # rows % 64


@pytest.mark.parametrize("N,K", [(128, 2048), (128, 9216)])
def test_w8a8_ternary_against_emulation_and_exact(cuda_device, N, K):
    """The reference's bonsai-int8 kernel case (Tests/IngotTests/KernelCaseFlashNextI8.swift:155-213): its shapes (K = 9216
    is nine Hadamard blocks), its bounds (relative RMS 2e-3 against the emulation, 3e-2 against the exact product), the
    half output, the accumulated output, and a 64-row chunk giving the same bits alone as inside 128 rows."""
    rng = np.random.default_rng(N + K)
    M = 128
    w, s, signs = synth.ternary_np(rng, N, K)
    m = synth.dense_q_ternary(w, s, signs, cuda_device)
    x = qref.round_f16(rng.normal(0, 1, size=(M, K)).astype(np.float32))
    xr = qref.rotate_input(x, signs)
    emu = qref.w8a8_ternary_emulated(xr, w, s)
    exact = qref.matmul_t(xr, qref.dequant_ternary(w, s))
    scratch = torch.empty(m.qmm_i8_scratch_bytes(M), dtype=torch.uint8, device=cuda_device)

    def run(rows, r0, acc=None, half=False):
        xt = x_tensor(x[r0:r0 + rows], cuda_device, torch.float16)
        if acc is not None:
            y = torch.from_numpy(acc.copy()).to(cuda_device)
        else:
            y = torch.zeros(rows, N, dtype=torch.float16 if half else torch.float32, device=cuda_device)
        m.encode_qmm_i8(xt, y, rows, accumulate=acc is not None, scratch=scratch)
        torch.cuda.synchronize()
        return y.float().cpu().numpy()

    y = run(M, 0)
    assert rel_rms(y, emu) <= 2e-3
    assert rel_rms(y, exact) <= 3e-2
    yh = run(M, 0, half=True)
    assert qref.max_rel(yh, qref.round_f16(y)) <= 2e-3
    base = rng.normal(0, 1, size=(M, N)).astype(np.float32)
    assert qref.max_rel(run(M, 0, acc=base), base + y) <= 1e-4
    both = np.concatenate([run(64, 0), run(64, 64)], axis=0)
    assert np.array_equal(both.view(np.uint32), y.view(np.uint32))
