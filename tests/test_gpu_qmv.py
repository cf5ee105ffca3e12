"""Decode GEMV (iq_qmv through VQMV.encode) against the CPU oracle. Mirrors the reference's qmv kernel cases
(Tests/IngotTests/KernelCaseG32.swift:21-78, KernelCaseMixedBits.swift:73-121, KernelCaseTests.swift:68-86,614-621)."""
import numpy as np
import pytest
import torch

from ingot_b200 import capi, synth
from ingot_b200.linear import VQMV
from oracle import qref
from gpu_util import TOL, affine_case, deq, mxfp4_case, x_tensor

pytestmark = pytest.mark.gpu


def run(m, x, rows, y_dtype=torch.float32, **kw):
    y = torch.zeros(rows, kw.pop("n_out", m.N), dtype=y_dtype, device=x.device)
    VQMV.encode(x, m, y, rows, **kw)
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("N,K", [(16, 64), (64, 128), (256, 512), (1024, 4096), (80, 2880)])
@pytest.mark.parametrize("rows", [1, 3, 8, 9, 16])
def test_qmv_affine_matches_oracle(cuda_device, bits, N, K, rows):
    rng = np.random.default_rng(1000 * bits + N + K + rows)
    m, host = affine_case(rng, N, K, bits, cuda_device)
    x = synth.activations_np(rng, rows, K)
    y = run(m, x_tensor(x, cuda_device), rows)
    ref = qref.matmul_t(x, deq(host, bits))
    assert qref.max_rel(y.cpu().numpy(), ref) <= TOL


def test_qmv_c0_shape_seed0(cuda_device):
    """The decode configuration itself: x bf16 [1, 4096], W [14336, 4096] 4-bit g64, seed 0."""
    rng = np.random.default_rng(0)
    m, host = affine_case(rng, 14336, 4096, 4, cuda_device)
    x = synth.activations_np(rng, 1, 4096)
    xt = x_tensor(x, cuda_device)
    y = run(m, xt, 1)
    ref = qref.matmul_t(x, deq(host, 4))
    err = qref.max_rel(y.cpu().numpy(), ref)
    assert err <= TOL, err
    # bf16 output = round-to-nearest-even of the kernel's own fp32 result
    yb = run(m, xt, 1, y_dtype=torch.bfloat16)
    assert torch.equal(yb, y.to(torch.bfloat16))


def test_qmv_down_projection_shape(cuda_device):
    rng = np.random.default_rng(5)
    m, host = affine_case(rng, 4096, 14336, 4, cuda_device)
    x = synth.activations_np(rng, 2, 14336)
    y = run(m, x_tensor(x, cuda_device), 2)
    assert qref.max_rel(y.cpu().numpy(), qref.matmul_t(x, deq(host, 4))) <= TOL


@pytest.mark.parametrize("N,K,rows", [(64, 64, 1), (2880, 2880, 1), (576, 192, 7), (128, 2880, 16)])
def test_qmv_mxfp4_matches_oracle(cuda_device, N, K, rows):
    rng = np.random.default_rng(N + K + rows)
    m, host = mxfp4_case(rng, N, K, cuda_device)
    x = synth.activations_np(rng, rows, K)
    y = run(m, x_tensor(x, cuda_device), rows)
    assert qref.max_rel(y.cpu().numpy(), qref.matmul_t(x, deq(host))) <= TOL


def test_qmv_mxfp4_golden_codes(cuda_device):
    """One-hot activations read the dequantised weights back: the reference's MXFP4 known-answer vector, bit for bit."""
    import json, os
    g = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "mxfp4_kat.json")))
    w = np.zeros((1, 16, 8), dtype=np.uint32)
    s = np.full((1, 16, 2), 127, dtype=np.uint8)
    w[0, :2] = np.array(g["words"], dtype=np.uint32).reshape(2, 8)
    s[0, :2] = np.array(g["scales"], dtype=np.uint8).reshape(2, 2)
    m = synth.dense_q_mxfp4(w, s, cuda_device)
    x = torch.eye(64, dtype=torch.float16, device=cuda_device)
    want = np.array(g["values"], dtype=np.float32).reshape(2, 64)
    for r0 in range(0, 64, 16):
        y = run(m, x[r0:r0 + 16].contiguous(), 16)
        got = y[:, :2].cpu().numpy().T  # [2, 16]
        assert np.array_equal(got, want[:, r0:r0 + 16])


@pytest.mark.parametrize("bits", [4, 8])
def test_qmv_unpacked_codes_bit_exact(cuda_device, bits):
    """With scale 1 and bias 0, one-hot activations return the codes themselves: unpacking is bit-exact."""
    rng = np.random.default_rng(bits)
    N, K = 32, 128
    q = rng.integers(0, 1 << bits, size=(1, N, K))
    w = qref.pack_q(q, bits)
    one = synth.to_bf16_bits(np.ones((1, N, K // 64), dtype=np.float32))
    zero = synth.to_bf16_bits(np.zeros((1, N, K // 64), dtype=np.float32))
    m = synth.dense_q_affine(w, one, zero, bits, cuda_device)
    x = torch.eye(K, dtype=torch.float16, device=cuda_device)
    for r0 in range(0, K, 16):
        y = run(m, x[r0:r0 + 16].contiguous(), 16)
        assert np.array_equal(y.cpu().numpy().T, q[0][:, r0:r0 + 16].astype(np.float32))


def test_qmv_row_invariance(cuda_device):
    """Row i gives the same bits alone, with i + 1 rows and with 16 rows and other neighbours."""
    rng = np.random.default_rng(11)
    m, _ = affine_case(rng, 512, 2048, 4, cuda_device)
    x = x_tensor(synth.activations_np(rng, 16, 2048), cuda_device)
    full = run(m, x, 16)
    for i in (0, 3, 7, 8, 15):
        part = run(m, x[: i + 1].contiguous(), i + 1)
        assert torch.equal(part[i], full[i])
        alone = run(m, x[i:i + 1].contiguous(), 1)
        assert torch.equal(alone[0], full[i])


@pytest.mark.parametrize("bits", [4, 8])
def test_qmv_tail_split_parity_and_row_invariance(cuda_device, bits):
    """A matrix whose 16-row blocks do not divide over the CTAs (304 blocks on 148 SMs x 2: eight left over, cut into K
    slices): parity with the oracle, the same bits for a row alone, among 4, 7 and 16, and on a second call."""
    rng = np.random.default_rng(21 + bits)
    N, K = 4864, 2048
    m, host = affine_case(rng, N, K, bits, cuda_device)
    x = synth.activations_np(rng, 16, K)
    xt = x_tensor(x, cuda_device)
    full = run(m, xt, 16)
    assert qref.max_rel(full.cpu().numpy(), qref.matmul_t(x, deq(host, bits))) <= TOL
    again = run(m, xt, 16)
    assert torch.equal(full, again)
    for rows in (1, 4, 7):
        part = run(m, xt[:rows].contiguous(), rows)
        assert torch.equal(part, full[:rows])
    alone = run(m, xt[9:10].contiguous(), 1)
    assert torch.equal(alone[0], full[9])


def test_qmv_strides_accumulate_prefix_dtypes(cuda_device):
    rng = np.random.default_rng(12)
    N, K, rows = 256, 512, 5
    m, host = affine_case(rng, N, K, 4, cuda_device)
    xh = synth.activations_np(rng, rows, K)
    ref = qref.matmul_t(xh, deq(host, 4))
    # padded row strides
    xp = torch.zeros(rows, K + 64, dtype=torch.bfloat16, device=cuda_device)
    xp[:, :K] = x_tensor(xh, cuda_device)
    yp = torch.full((rows, N + 48), 7.0, dtype=torch.float32, device=cuda_device)
    VQMV.encode(xp, m, yp, rows)
    torch.cuda.synchronize()
    assert qref.max_rel(yp[:, :N].cpu().numpy(), ref) <= TOL
    assert (yp[:, N:] == 7.0).all()
    # accumulate
    y0 = torch.from_numpy(rng.normal(size=(rows, N)).astype(np.float32)).to(cuda_device)
    y = y0.clone()
    VQMV.encode(x_tensor(xh, cuda_device), m, y, rows, accumulate=True)
    torch.cuda.synchronize()
    assert qref.max_rel((y - y0).cpu().numpy(), ref) <= TOL
    # n_prefix: only the first rows of W
    y = torch.full((rows, N), -1.0, dtype=torch.float32, device=cuda_device)
    VQMV.encode(x_tensor(xh, cuda_device), m, y, rows, n_prefix=64)
    torch.cuda.synchronize()
    assert qref.max_rel(y[:, :64].cpu().numpy(), ref[:, :64]) <= TOL and (y[:, 64:] == -1.0).all()
    # fp16 and fp32 activations
    for dt in (torch.float16, torch.float32):
        y = run(m, x_tensor(xh, cuda_device, dt), rows)
        assert qref.max_rel(y.cpu().numpy(), ref) <= TOL


def test_qmv_rejects_what_the_reference_rejects(cuda_device):
    rng = np.random.default_rng(13)
    m, _ = affine_case(rng, 64, 128, 4, cuda_device)
    x = torch.zeros(17, 128, dtype=torch.bfloat16, device=cuda_device)
    y = torch.zeros(17, 64, dtype=torch.float32, device=cuda_device)
    with pytest.raises(capi.IngotError) as e:
        VQMV.encode(x, m, y, 17)  # rows <= 16 (Linear.swift precondition)
    assert e.value.status == -1
    with pytest.raises(capi.IngotError):
        VQMV.encode(x, m, y, 4, n_prefix=24)


def test_qmv_negative_control(cuda_device):
    """A perturbed input must make the parity check fail (the reference's --perturb controls)."""
    rng = np.random.default_rng(14)
    m, host = affine_case(rng, 64, 256, 4, cuda_device)
    x = synth.activations_np(rng, 1, 256)
    w2 = host[0].copy()
    w2[0, 5, 3] ^= 0x000000F0
    ref_bad = qref.matmul_t(x, qref.dequant_affine(w2[0], host[1][0], host[2][0], 4))
    y = run(m, x_tensor(x, cuda_device), 1)
    assert qref.max_rel(y.cpu().numpy(), ref_bad) > TOL


def int8_path_case(rng, device, N=256, K=2048, bits=4):
    """A matrix the int8 tensor-core GEMV takes (K a multiple of 2048): its activations go through 14-bit block fixed
    point per group of 64, which the cases below stress."""
    m, host = affine_case(rng, N, K, bits, device)
    return m, qref.dequant_affine(host[0][0], host[1][0], host[2][0], bits)


@pytest.mark.parametrize("bits", [4, 8])
def test_qmv_int8_path_outlier_per_group(cuda_device, bits):
    """One activation of about 1e3 in every group of 64 among values ~ N(0, 1): the group's fixed-point step follows the
    outlier. The result stays inside the bound against the fp32 oracle."""
    rng = np.random.default_rng(31 + bits)
    m, wf = int8_path_case(rng, cuda_device, bits=bits)
    x = synth.activations_np(rng, 3, 2048)
    for g in range(2048 // 64):
        x[:, g * 64 + rng.integers(0, 64)] = np.float32(1000.0) * rng.choice([-1.0, 1.0])
    x = synth.round_bf16(x)
    y = run(m, x_tensor(x, cuda_device), 3)
    assert qref.max_rel(y.cpu().numpy(), qref.matmul_t(x, wf)) <= TOL


def test_qmv_int8_path_wide_dynamic_range_fp32(cuda_device):
    """fp32 activations whose groups span 2^-20 .. 2^20 in magnitude (each group at its own scale), and one group of
    values that are subnormal in half precision: the per-group exponent carries the range."""
    rng = np.random.default_rng(33)
    m, wf = int8_path_case(rng, cuda_device)
    x = rng.normal(0, 1, size=(2, 2048)).astype(np.float32)
    for g in range(32):
        x[:, g * 64:(g + 1) * 64] *= np.float32(2.0) ** rng.integers(-20, 21)
    x[:, 5 * 64:6 * 64] = rng.normal(0, 1, size=(2, 64)).astype(np.float32) * np.float32(3e-8)  # below fp16's normal range
    y = run(m, torch.from_numpy(x).to(cuda_device), 2)
    assert qref.max_rel(y.cpu().numpy(), qref.matmul_t(x, wf)) <= TOL
    # a row that is tiny everywhere keeps its relative accuracy (nothing is flushed at these magnitudes)
    xs = (rng.normal(0, 1, size=(1, 2048)) * 1e-6).astype(np.float32)
    ys = run(m, torch.from_numpy(xs).to(cuda_device), 1)
    assert qref.max_rel(ys.cpu().numpy(), qref.matmul_t(xs, wf)) <= TOL


@pytest.mark.parametrize("bad", [float("nan"), float("inf"), -float("inf")])
@pytest.mark.parametrize("K", [2048, 512])
def test_qmv_non_finite_activations_propagate(cuda_device, bad, K):
    """A NaN or an infinity in x must not come out as a finite number, on the int8 path (K = 2048) as on the fp16 one
    (K = 512), as in the reference's fp32 product; rows without one are untouched."""
    rng = np.random.default_rng(35)
    m, host = affine_case(rng, 64, K, 4, cuda_device)
    x = synth.activations_np(rng, 3, K)
    x[1, 77] = bad
    y = run(m, x_tensor(x, cuda_device), 3).cpu().numpy()
    ref = qref.matmul_t(x[[0, 2]], deq(host, 4))
    assert not np.isfinite(y[1]).any()
    assert qref.max_rel(y[[0, 2]], ref) <= TOL
