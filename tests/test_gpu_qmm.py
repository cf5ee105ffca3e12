"""Prefill GEMM on the tcgen05 tensor cores (iq_qmm through DenseQ.encode_qmm_f32) against the CPU oracle. Mirrors the
reference's qmm kernel cases (Tests/IngotTests/KernelCaseG32.swift:44-78, KernelCaseMixedBits.swift:98-121)."""
import numpy as np
import pytest
import torch

from ingot_b200 import capi, synth
from ingot_b200.linear import VQMV
from oracle import qref
from gpu_util import TOL, affine_case, deq, mxfp4_case, x_tensor

pytestmark = pytest.mark.gpu


def run_qmm(m, x, rows, y_dtype=torch.float32, accumulate=False, y=None):
    ws = torch.empty(max(m.qmm_workspace_bytes(rows, x.dtype), 256), dtype=torch.uint8, device=x.device)
    if y is None:
        y = torch.zeros(rows, m.N, dtype=y_dtype, device=x.device)
    m.encode_qmm_f32(x, y, rows, accumulate=accumulate, workspace=ws)
    assert capi.context(0).device_status() == 0  # synchronises; no bounded wait gave up
    return y


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,N,K", [(64, 128, 64), (64, 64, 128), (128, 256, 512), (192, 192, 256), (256, 128, 2048),
                                   (320, 384, 1024), (512, 512, 4096)])
def test_qmm_affine_matches_oracle(cuda_device, bits, M, N, K):
    rng = np.random.default_rng(100 * bits + M + N + K)
    m, host = affine_case(rng, N, K, bits, cuda_device)
    x = synth.activations_np(rng, M, K)
    y = run_qmm(m, x_tensor(x, cuda_device), M)
    ref = qref.matmul_t(x, deq(host, bits))
    err = qref.max_rel(y.cpu().numpy(), ref)
    assert err <= TOL, err


def test_qmm_outputs_and_accumulate(cuda_device):
    rng = np.random.default_rng(21)
    M, N, K = 128, 256, 512
    m, host = affine_case(rng, N, K, 4, cuda_device)
    xh = synth.activations_np(rng, M, K)
    ref = qref.matmul_t(xh, deq(host, 4))
    x = x_tensor(xh, cuda_device)
    y32 = run_qmm(m, x, M)
    # half / bf16 outputs are the rounding of the kernel's own fp32 result (the reference loosens half outputs to 2e-3,
    # KernelCaseG32.swift:77)
    assert torch.equal(run_qmm(m, x, M, torch.float16), y32.to(torch.float16))
    assert torch.equal(run_qmm(m, x, M, torch.bfloat16), y32.to(torch.bfloat16))
    y0 = torch.from_numpy(rng.normal(size=(M, N)).astype(np.float32)).to(cuda_device)
    y = run_qmm(m, x, M, accumulate=True, y=y0.clone())
    assert qref.max_rel((y - y0).cpu().numpy(), ref) <= TOL
    # fp16 activations are used in place (no conversion pass), fp32 activations are converted
    for dt in (torch.float16, torch.float32):
        assert qref.max_rel(run_qmm(m, x_tensor(xh, cuda_device, dt), M).cpu().numpy(), ref) <= TOL


def test_qmm_mxfp4(cuda_device):
    rng = np.random.default_rng(22)
    M, N, K = 128, 192, 576
    m, host = mxfp4_case(rng, N, K, cuda_device)
    x = synth.activations_np(rng, M, K)
    y = run_qmm(m, x_tensor(x, cuda_device), M)
    assert qref.max_rel(y.cpu().numpy(), qref.matmul_t(x, deq(host))) <= TOL


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,N,K", [(512, 14336, 4096), (2048, 14336, 4096), (512, 4096, 14336), (2048, 4096, 14336)])
def test_qmm_prefill_configuration(cuda_device, bits, M, N, K):
    """The prefill configuration at full size: the oracle on 192 sampled output features, and agreement with the decode
    GEMV kernel (itself checked against the oracle) on 16 sampled token rows over every output feature."""
    rng = np.random.default_rng(bits + M + N)
    m, host = affine_case(rng, N, K, bits, cuda_device)
    x = synth.activations_np(rng, M, K)
    xt = x_tensor(x, cuda_device)
    y = run_qmm(m, xt, M)
    sel = np.sort(rng.choice(N, size=192, replace=False))
    wf = qref.dequant_affine(host[0][0][sel], host[1][0][sel], host[2][0][sel], bits)
    ref = qref.matmul_t(x, wf)
    err = qref.max_rel(y[:, torch.from_numpy(sel).to(cuda_device)].cpu().numpy(), ref)
    assert err <= TOL, err
    rows = torch.from_numpy(np.sort(rng.choice(M, size=16, replace=False))).to(cuda_device)
    yv = torch.zeros(16, N, dtype=torch.float32, device=cuda_device)
    VQMV.encode(xt[rows].contiguous(), m, yv, 16)
    torch.cuda.synchronize()
    scale = float(yv.abs().max())
    assert float((y[rows] - yv).abs().max()) / scale <= TOL


def test_qmm_rejects_what_the_reference_rejects(cuda_device):
    rng = np.random.default_rng(23)
    m, _ = affine_case(rng, 128, 128, 4, cuda_device)
    x = torch.zeros(96, 128, dtype=torch.float16, device=cuda_device)
    y = torch.zeros(96, 128, dtype=torch.float32, device=cuda_device)
    with pytest.raises(capi.IngotError) as e:
        m.encode_qmm_f32(x, y, 96)  # rows % 64 (Linear.swift:695)
    assert e.value.status == -1
    xb = torch.zeros(64, 128, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(capi.IngotError) as e:
        m.encode_qmm_f32(xb, y, 64)  # bf16 activations need the conversion workspace
    assert e.value.status == -4
