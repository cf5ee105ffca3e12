"""argmax_rows and TopK64 against the CPU rule, on the reference's shapes (Tests/IngotTests/TopK64Tests.swift:14-36, :68-86):
candidates bit for bit (ids and values), the maximum exact, Z to 1e-5; and the decode tail: lm_head GEMV then arg-max."""
import numpy as np
import pytest
import torch

from ingot_b200 import sampling, synth
from ingot_b200.linear import VQMV
from oracle import qref
from gpu_util import x_tensor

pytestmark = pytest.mark.gpu


def logits(shape, V, rows, seed):
    rng = np.random.default_rng(seed)
    u = rng.random((rows, V), dtype=np.float32)
    r = np.arange(rows, dtype=np.float32)[:, None]
    i = np.arange(V, dtype=np.float32)[None, :]
    if shape == "random":
        return (u * 30 - 15).astype(np.float32)
    if shape == "ties":
        return (np.floor(u * 12) * 0.5).astype(np.float32)   # 12 levels: many ties at the cut
    if shape == "ascending":
        return (i * np.float32(1e-3) + r).astype(np.float32)
    if shape == "descending":
        return (-i * np.float32(1e-3) - r).astype(np.float32)
    x = (u * 8).astype(np.float32)
    x[u < 0.5] = -np.inf
    return x


def check(x, temps):
    rows, V = x.shape
    dev = torch.device("cuda", 0)
    tk = sampling.TopK64(rows, V, dev)
    xt = torch.from_numpy(x).to(dev)
    idx, val, z = tk.encode(xt, rows, temps)
    am = sampling.argmax_rows(xt, rows)
    torch.cuda.synchronize()
    idx, val, z, am = idx.cpu().numpy().astype(np.uint32), val.cpu().numpy(), z.cpu().numpy(), am.cpu().numpy().astype(np.uint32)
    assert np.array_equal(am, qref.argmax_rows(x))
    for r in range(rows):
        wi, wv, mx, Z = qref.topk64(x[r], temps[r if len(temps) > 1 else 0])
        assert np.array_equal(idx[r], wi), f"row {r}: ids"
        assert np.array_equal(val[r].view(np.uint32), wv.view(np.uint32)), f"row {r}: values"
        assert z[r, 0] == mx
        assert abs(float(z[r, 1]) / Z - 1) < 1e-5


@pytest.mark.parametrize("shape", ["random", "ties", "ascending", "descending", "negInf"])
def test_candidates_match_full_sort(cuda_device, shape):
    for V, rows in [(262144, 1), (151936, 3), (3000, 2), (100, 1), (40, 2), (7, 1)]:
        check(logits(shape, V, rows, V), [0.7])


def test_each_row_its_own_temperature(cuda_device):
    check(logits("random", 50000, 4, 9), [0.3, 1.0, 1.5, 0.8])


def test_signed_zeros_tie_and_keep_their_bits(cuda_device):
    x = np.full((1, 200), -1.0, dtype=np.float32)
    x[0, 5] = 0.0
    x[0, 3] = -0.0
    x[0, 9] = 0.0
    check(x, [1.0])


def test_lm_head_then_argmax(cuda_device):
    """The decode tail: a 151,936-row 4-bit lm_head through the GEMV, then the arg-max of the kernel's own logits."""
    rng = np.random.default_rng(4)
    N, K = 151936, 2048
    w, s, b = synth.affine_np(rng, N, K, 4)
    m = synth.dense_q_affine(w, s, b, 4, cuda_device)
    x = synth.activations_np(rng, 2, K)
    y = torch.zeros(2, N, dtype=torch.float32, device=cuda_device)
    VQMV.encode(x_tensor(x, cuda_device), m, y, 2)
    am = sampling.argmax_rows(y, 2)
    torch.cuda.synchronize()
    assert np.array_equal(am.cpu().numpy().astype(np.uint32), qref.argmax_rows(y.cpu().numpy()))
    ref = qref.matmul_t(x, qref.dequant_affine(w[0], s[0], b[0], 4))
    assert qref.max_rel(y.cpu().numpy(), ref) <= 1e-3
