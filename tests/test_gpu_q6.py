"""6-bit affine weights (MLX bit-stream packing, groups of 64): the decode GEMV of a tied lm_head and its embedding
rows, against the CPU oracle. Mirrors the reference's lfm-qmv6 kernel case (Tests/IngotTests/KernelCaseTests.swift:216-240):
1 and 16 rows within 1e-4, a row that does not depend on the others or on the row count, embedding rows."""
import numpy as np
import pytest
import torch

from ingot_b200 import capi, synth
from ingot_b200.linear import VQMV
from oracle import qref
from gpu_util import affine_case, deq, x_tensor

pytestmark = pytest.mark.gpu
TOL6 = 1e-4  # the reference's bound for this kernel (its 4-bit cases take 1e-3)


def qmv(m, x, rows, y_dtype=torch.float32, **kw):
    y = torch.zeros(rows, kw.pop("n_out", m.N), dtype=y_dtype, device=x.device)
    VQMV.encode(x, m, y, rows, **kw)
    torch.cuda.synchronize()
    return y


# 4752 and 4800 rows: 297 and 300 blocks of 16 over two CTAs per SM leave blocks over, which are cut into K slices
@pytest.mark.parametrize("N,K,rows", [(128, 2048, 1), (128, 2048, 16), (512, 4096, 5), (4752, 2048, 3), (4800, 2048, 9),
                                      (16, 4096, 8)])
def test_qmv6_matches_oracle(cuda_device, N, K, rows):
    rng = np.random.default_rng(600 + N + K + rows)
    m, host = affine_case(rng, N, K, 6, cuda_device)
    x = synth.activations_np(rng, rows, K)
    y = qmv(m, x_tensor(x, cuda_device), rows)
    err = qref.max_rel(y.cpu().numpy(), qref.matmul_t(x, deq(host, 6)))
    assert err <= TOL6, err
    assert capi.context(0).device_status() == 0


def test_qmv6_unpacks_codes_exactly(cuda_device):
    """Scale 1, bias 0 and a one-hot input per row: the output is the code itself, for every position of the stream."""
    rng = np.random.default_rng(61)
    N, K = 32, 2048
    q = rng.integers(0, 64, size=(1, N, K))
    w = qref.pack_q(q, 6)
    one = synth.to_bf16_bits(np.ones((1, N, K // 64), dtype=np.float32))
    zero = synth.to_bf16_bits(np.zeros((1, N, K // 64), dtype=np.float32))
    m = synth.dense_q_affine(w, one, zero, 6, cuda_device)
    for r0 in range(0, K, 16 * 8):  # every eighth block of sixteen inputs, plus the stream's last
        x = torch.zeros(16, K, dtype=torch.float16, device=cuda_device)
        x[torch.arange(16), r0 + torch.arange(16)] = 1.0
        y = qmv(m, x, 16)
        assert np.array_equal(y.cpu().numpy().T, q[0][:, r0:r0 + 16].astype(np.float32))
    x = torch.zeros(16, K, dtype=torch.float16, device=cuda_device)
    x[torch.arange(16), K - 16 + torch.arange(16)] = 1.0
    assert np.array_equal(qmv(m, x, 16).cpu().numpy().T, q[0][:, K - 16:].astype(np.float32))


def test_qmv6_row_invariance_outputs_and_prefix(cuda_device):
    rng = np.random.default_rng(62)
    N, K = 4752, 2048
    m, host = affine_case(rng, N, K, 6, cuda_device)
    xh = synth.activations_np(rng, 16, K)
    x = x_tensor(xh, cuda_device)
    full = qmv(m, x, 16)
    for i in (0, 3, 7, 8, 15):
        assert torch.equal(qmv(m, x[: i + 1].contiguous(), i + 1)[i], full[i])
        assert torch.equal(qmv(m, x[i:i + 1].contiguous(), 1)[0], full[i])
    # half and bf16 outputs are the rounding of the fp32 result; accumulate adds to what is there
    assert torch.equal(qmv(m, x, 16, torch.float16), full.to(torch.float16))
    assert torch.equal(qmv(m, x, 16, torch.bfloat16), full.to(torch.bfloat16))
    y0 = torch.from_numpy(rng.normal(size=(16, N)).astype(np.float32)).to(cuda_device)
    y = y0.clone()
    VQMV.encode(x, m, y, 16, accumulate=True)
    torch.cuda.synchronize()
    assert torch.equal(y, y0 + full)
    ref = qref.matmul_t(xh, deq(host, 6))
    yp = torch.full((4, 64), -1.0, dtype=torch.float32, device=cuda_device)
    VQMV.encode(x, m, yp, 4, n_prefix=64)
    torch.cuda.synchronize()
    assert qref.max_rel(yp.cpu().numpy(), ref[:4, :64]) <= TOL6
    for dt in (torch.float16, torch.float32):
        assert qref.max_rel(qmv(m, x_tensor(xh, cuda_device, dt), 16).cpu().numpy(), ref) <= TOL6


def test_q6_rejections(cuda_device):
    rng = np.random.default_rng(63)
    m, _ = affine_case(rng, 64, 512, 6, cuda_device)  # k is not a multiple of 2048
    x = torch.zeros(1, 512, dtype=torch.bfloat16, device=cuda_device)
    y = torch.zeros(1, 64, dtype=torch.float32, device=cuda_device)
    with pytest.raises(capi.IngotError):
        VQMV.encode(x, m, y, 1)
    m2, _ = affine_case(rng, 64, 2048, 6, cuda_device)
    with pytest.raises(capi.IngotError):  # no 6-bit prefill GEMM
        m2.encode_qmm_f32(torch.zeros(64, 2048, dtype=torch.float16, device=cuda_device),
                          torch.zeros(64, 64, dtype=torch.float32, device=cuda_device), 64,
                          workspace=torch.empty(256, dtype=torch.uint8, device=cuda_device))


def test_embed_rows_6bit_exact(cuda_device):
    rng = np.random.default_rng(64)
    V, K = 128, 2048
    m, host = affine_case(rng, V, K, 6, cuda_device)
    w = deq(host, 6)
    tok = torch.tensor([5, 127, 0, 64], dtype=torch.int32, device=cuda_device)
    of = torch.zeros(4, K, dtype=torch.float32, device=cuda_device)
    oh = torch.zeros(4, K, dtype=torch.float16, device=cuda_device)
    m.encode_embed(tok, 4, of, oh)
    torch.cuda.synchronize()
    ref = w[[5, 127, 0, 64]]
    assert np.array_equal(of.cpu().numpy(), ref)
    assert np.array_equal(oh.cpu().numpy(), qref.round_f16(ref).astype(np.float16))
