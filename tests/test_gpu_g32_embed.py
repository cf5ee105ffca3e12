"""4-bit affine matrices with groups of 32 (decode GEMV, prefill GEMM, dense FFN) and the embedding gather, against the
CPU oracle. Mirrors the reference's q4-g32 kernel case (Tests/IngotTests/KernelCaseG32.swift:12-93): the group index is
k / 32 and the scale stride K / 32 on every path, rows do not depend on their neighbours, embedding rows are exact."""
import numpy as np
import pytest
import torch

from ingot_b200 import capi, synth
from ingot_b200.linear import DenseMLP, DenseQ, VQMV
from oracle import qref
from gpu_util import TOL, affine_case, deq, x_tensor

pytestmark = pytest.mark.gpu


def qmv(m, x, rows, **kw):
    y = torch.zeros(rows, kw.pop("n_out", m.N), dtype=torch.float32, device=x.device)
    VQMV.encode(x, m, y, rows, **kw)
    torch.cuda.synchronize()
    return y


def qmm(m, x, rows, y_dtype=torch.float32, accumulate=False, y=None):
    ws = torch.empty(max(m.qmm_workspace_bytes(rows, x.dtype), 256), dtype=torch.uint8, device=x.device)
    if y is None:
        y = torch.zeros(rows, m.N, dtype=y_dtype, device=x.device)
    m.encode_qmm_f32(x, y, rows, accumulate=accumulate, workspace=ws)
    assert capi.context(0).device_status() == 0
    return y


@pytest.mark.parametrize("N,K,rows", [(64, 2048, 16), (48, 2048, 5), (32, 1536, 1), (256, 5120, 9), (4096, 4096, 1)])
def test_qmv_g32_matches_oracle(cuda_device, N, K, rows):
    rng = np.random.default_rng(32 + N + K + rows)
    m, host = affine_case(rng, N, K, 4, cuda_device, group=32)
    x = synth.activations_np(rng, rows, K)
    y = qmv(m, x_tensor(x, cuda_device), rows)
    assert qref.max_rel(y.cpu().numpy(), qref.matmul_t(x, deq(host, 4, group=32))) <= TOL


def test_qmv_g32_prefix_dtypes_and_row_invariance(cuda_device):
    rng = np.random.default_rng(33)
    N, K, rows = 64, 2048, 6
    m, host = affine_case(rng, N, K, 4, cuda_device, group=32)
    xh = synth.activations_np(rng, rows, K)
    ref = qref.matmul_t(xh, deq(host, 4, group=32))
    y = torch.full((rows, 32), -1.0, dtype=torch.float32, device=cuda_device)
    VQMV.encode(x_tensor(xh, cuda_device), m, y, rows, n_prefix=32)
    torch.cuda.synchronize()
    assert qref.max_rel(y.cpu().numpy(), ref[:, :32]) <= TOL
    for dt in (torch.float16, torch.float32):
        assert qref.max_rel(qmv(m, x_tensor(xh, cuda_device, dt), rows).cpu().numpy(), ref) <= TOL
    mi, _ = affine_case(rng, 256, 2048, 4, cuda_device, group=32)
    x = x_tensor(synth.activations_np(rng, 16, 2048), cuda_device)
    full = qmv(mi, x, 16)
    for i in (0, 4, 8, 15):
        assert torch.equal(qmv(mi, x[: i + 1].contiguous(), i + 1)[i], full[i])
        assert torch.equal(qmv(mi, x[i:i + 1].contiguous(), 1)[0], full[i])


def test_qmv_g32_unpacks_codes_exactly(cuda_device):
    """Scale 1 / bias 0 in one group and scale 2 / bias 1 in the next: an identity input returns the codes, so a wrong
    group index (k / 64 instead of k / 32) or nibble order shows up exactly."""
    rng = np.random.default_rng(34)
    N, K = 32, 128
    q = rng.integers(0, 16, size=(1, N, K))
    w = qref.pack_q(q, 4)
    sc = np.tile(np.array([1.0, 2.0], dtype=np.float32), (1, N, K // 64))
    bi = np.tile(np.array([0.0, 1.0], dtype=np.float32), (1, N, K // 64))
    m = synth.dense_q_affine(w, synth.to_bf16_bits(sc), synth.to_bf16_bits(bi), 4, cuda_device, 32)
    want = (q[0] * np.repeat(sc[0], 32, axis=1) + np.repeat(bi[0], 32, axis=1)).astype(np.float32)
    x = torch.eye(K, dtype=torch.float16, device=cuda_device)
    for r0 in range(0, K, 16):
        y = qmv(m, x[r0:r0 + 16].contiguous(), 16)
        assert np.array_equal(y.cpu().numpy().T, want[:, r0:r0 + 16])


@pytest.mark.parametrize("M,N,K", [(64, 128, 2048), (64, 256, 4096), (320, 384, 1024), (512, 1024, 4096)])
def test_qmm_g32_matches_oracle(cuda_device, M, N, K):
    rng = np.random.default_rng(35 + M + N + K)
    m, host = affine_case(rng, N, K, 4, cuda_device, group=32)
    xh = synth.activations_np(rng, M, K)
    ref = qref.matmul_t(xh, deq(host, 4, group=32))
    x = x_tensor(xh, cuda_device)
    y32 = qmm(m, x, M)
    assert qref.max_rel(y32.cpu().numpy(), ref) <= TOL
    assert torch.equal(qmm(m, x, M, torch.float16), y32.to(torch.float16))
    y0 = torch.from_numpy(rng.normal(size=(M, N)).astype(np.float32)).to(cuda_device)
    ya = qmm(m, x, M, accumulate=True, y=y0.clone())
    assert qref.max_rel((ya - y0).cpu().numpy(), ref) <= TOL


@pytest.mark.parametrize("group", [64, 32])
@pytest.mark.parametrize("rows", [3, 128])
def test_dense_ffn(cuda_device, rows, group):
    """Dense gated FFN (gate|up concatenated by rows, then down) with groups of 64 and of 32: decode rows through the
    fused GEMV, prefill rows through the GEMMs."""
    rng = np.random.default_rng(36 + rows + group)
    D, F = 512, 1024
    gu, hgu = affine_case(rng, 2 * F, D, 4, cuda_device, group=group)
    dn, hdn = affine_case(rng, D, F, 4, cuda_device, group=group)
    xh = synth.activations_np(rng, rows, D)
    wgu = deq(hgu, 4, group=group)
    g, u = qref.matmul_t(xh, wgu[:F]), qref.matmul_t(xh, wgu[F:])
    h = qref.round_f16(qref.silu_glu(g, u))
    ref = qref.matmul_t(h, deq(hdn, 4, group=group))
    out = torch.zeros(rows, D, dtype=torch.float32, device=cuda_device)
    DenseMLP(gu, dn).encode(x_tensor(xh, cuda_device), out, rows)
    torch.cuda.synchronize()
    assert qref.max_rel(out.cpu().numpy(), ref) <= 2 * TOL  # h is rounded to fp16 on both sides, from sums in other orders


@pytest.mark.parametrize("act", ["silu", "gelu", "relu2", "swiglu_oai"])
@pytest.mark.parametrize("rows", [5, 320])
def test_dense_ffn_activations(cuda_device, rows, act):
    """The four gated activations of the reference's dswiglu (Shaders/yy_model.metal:187-227) through the dense FFN:
    decode rows on the fused GEMV, prefill rows on the tcgen05 GEMM whose epilogue applies the activation to the gate and
    up tiles of one stage (no fp32 gate|up round trip)."""
    from ingot_b200 import capi
    rng = np.random.default_rng(50 + rows)
    D, F = 512, 768
    gu, hgu = affine_case(rng, 2 * F, D, 4, cuda_device)
    dn, hdn = affine_case(rng, D, F, 4, cuda_device)
    xh = synth.activations_np(rng, rows, D)
    wgu = deq(hgu, 4)
    g, u = qref.matmul_t(xh, wgu[:F]), qref.matmul_t(xh, wgu[F:])
    h = qref.round_f16(qref.swiglu_oai(g, u, 7.0) if act == "swiglu_oai" else qref.ACTS[act](g, u))
    ref = qref.matmul_t(h, deq(hdn, 4))
    out = torch.zeros(rows, D, dtype=torch.float32, device=cuda_device)
    DenseMLP(gu, dn, act=act).encode(x_tensor(xh, cuda_device), out, rows)
    assert capi.context(0).device_status() == 0
    assert qref.max_rel(out.cpu().numpy(), ref) <= 2 * TOL


def test_moe_rejects_g32_experts(cuda_device):
    from ingot_b200.moe import MoELayer, RouterSpec
    rng = np.random.default_rng(37)
    E, D, F = 32, 128, 64
    g, _ = affine_case(rng, F, D, 4, cuda_device, experts=E, group=32)
    u, _ = affine_case(rng, F, D, 4, cuda_device, experts=E, group=32)
    d, _ = affine_case(rng, D, F, 4, cuda_device, experts=E, group=32)
    router = torch.zeros(E, D, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(capi.IngotError):
        MoELayer(RouterSpec(E, 2), router, g, u, d)


# ---- embedding -------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("bits,group", [(4, 64), (4, 32), (8, 64)])
def test_embed_rows_exact(cuda_device, bits, group):
    rng = np.random.default_rng(40 + bits + group)
    V, K = 40, 2048
    tok = np.array([3, 0, 39, 17, 17, 8], dtype=np.int32)
    m, host = affine_case(rng, V, K, bits, cuda_device, group=group)
    w = deq(host, bits, group=group)
    of = torch.full((len(tok), K), 9.0, dtype=torch.float32, device=cuda_device)
    oh = torch.full((len(tok), K), 9.0, dtype=torch.float16, device=cuda_device)
    m.encode_embed(torch.from_numpy(tok).to(cuda_device), len(tok), of, oh)
    torch.cuda.synchronize()
    ref = w[tok]
    assert np.array_equal(of.cpu().numpy(), ref)
    assert np.array_equal(oh.cpu().numpy(), qref.round_f16(ref).astype(np.float16))


def test_embed_rows_single_output_stride_and_range(cuda_device):
    rng = np.random.default_rng(44)
    V, K = 100, 320
    m, host = affine_case(rng, V, K, 4, cuda_device)
    w = deq(host, 4)
    tok = torch.tensor([99, 100, 5, 7], dtype=torch.int32, device=cuda_device)  # 100 is outside the table: a zero row
    buf = torch.full((4, K + 64), 5.0, dtype=torch.float16, device=cuda_device)
    m.encode_embed(tok, 4, out_h=buf)
    torch.cuda.synchronize()
    ref = qref.round_f16(w[[99, 0, 5, 7]]).astype(np.float16)
    ref[1] = 0
    assert np.array_equal(buf[:, :K].cpu().numpy(), ref) and (buf[:, K:] == 5.0).all()
    of = torch.zeros(4, K, dtype=torch.float32, device=cuda_device)
    m.encode_embed(tok, 4, out_f=of)
    torch.cuda.synchronize()
    assert np.array_equal(of[2:].cpu().numpy(), w[[5, 7]])
    with pytest.raises(ValueError):
        m.encode_embed(tok, 4)


def test_embed_rows_bf16_table(cuda_device):
    rng = np.random.default_rng(45)
    V, K = 64, 256
    t = torch.from_numpy(rng.normal(size=(V, K)).astype(np.float32)).to(cuda_device).to(torch.bfloat16)
    m = DenseQ(t, None, None, V, K, 16)
    tok = torch.tensor([63, 1, 1, 30], dtype=torch.int32, device=cuda_device)
    of = torch.zeros(4, K, dtype=torch.float32, device=cuda_device)
    oh = torch.zeros(4, K, dtype=torch.float16, device=cuda_device)
    m.encode_embed(tok, 4, of, oh)
    torch.cuda.synchronize()
    want = t[tok.long()].float()
    assert torch.equal(of, want) and torch.equal(oh, want.to(torch.float16))
