"""The oracle's restatements of the formats whose kernels are still to come (ternary with the Hadamard input rotation,
the emulated W8A8 prefill GEMM), checked through what the mathematics fixes: the reference stores no vectors for them.
No GPU."""
import numpy as np
import scipy.linalg

from oracle import qref


def test_fwht_is_the_sylvester_hadamard_matrix():
    rng = np.random.default_rng(1)
    for n in (2, 32, 1024):
        v = rng.normal(size=(3, n)).astype(np.float32)
        H = scipy.linalg.hadamard(n).astype(np.float64)
        assert np.allclose(qref.fwht(v), v.astype(np.float64) @ H.T, rtol=1e-5, atol=1e-4)
    e = np.eye(32, dtype=np.float32)
    assert np.array_equal(qref.fwht(qref.fwht(e)), 32 * e)  # H H = n I, exactly on small integers


def test_rotation_keeps_the_product_and_the_embedding_undoes_it():
    """x . w = rotate(x) . w' when w' holds the rotated weights: with R = H D / 32 (D the signs) orthogonal,
    (R x) . (R w) = x . w; and the embedding returns D H w' / 32 = R^T w'."""
    rng = np.random.default_rng(2)
    K, N = 2048, 24
    signs = np.where(rng.integers(0, 2, size=K) == 0, 1.0, -1.0).astype(np.float32)
    q = rng.integers(0, 3, size=(N, K))
    w = qref.pack_q(q, 2)
    s = (0.01 + 0.03 * rng.random(size=(N, K // 128))).astype(np.float16)
    wf = qref.dequant_ternary(w, s)
    assert wf.shape == (N, K) and set(np.unique(np.sign(wf))) <= {-1.0, 0.0, 1.0}
    assert np.array_equal(wf[3, 130], (np.float32(q[3, 130]) - 1) * np.float32(s[3, 1]))
    x = qref.round_f16(rng.normal(size=(5, K)).astype(np.float32))
    xr = qref.rotate_input(x, signs)
    # the un-rotated rows of the table, then the product in the original basis
    back = qref.embed_ternary(w, s, signs, np.arange(N))
    y_rot = qref.matmul_t(xr, wf)
    y_orig = qref.matmul_t(x, back)
    assert qref.max_rel(y_rot, y_orig) <= 2e-3  # xr is rounded to fp16
    # norms are kept (R is orthogonal)
    assert np.allclose(np.linalg.norm(xr, axis=1), np.linalg.norm(x, axis=1), rtol=1e-3)


def test_w8a8_emulation_is_close_to_the_exact_product_and_exact_on_integers():
    rng = np.random.default_rng(3)
    M, N, K = 16, 32, 2048
    x = rng.normal(size=(M, K)).astype(np.float32)
    x[:, [7, 300, K - 5]] *= 20  # the outlier channels the rotation is for
    wf = rng.normal(scale=0.05, size=(N, K)).astype(np.float32)
    ref = x.astype(np.float64) @ wf.astype(np.float64).T
    for lb in (0, 3):
        y = qref.w8a8_emulated(x, wf, lb)
        rms = np.sqrt(np.mean((y - ref) ** 2)) / np.sqrt(np.mean(ref ** 2))
        assert rms <= 0.05, (lb, rms)  # the reference's bound against the exact product (KernelCaseTests.swift:655)
    q, sc = qref.quant_i8_rows(np.array([[0.5, -1.5, 2.5, 127.0], [0, 0, 0, 0]], dtype=np.float32))
    assert q.tolist() == [[0.0, -2.0, 2.0, 127.0], [0, 0, 0, 0]] and sc.tolist() == [1.0, 1.0]  # ties to even


def test_w8a8_ternary_emulation_follows_its_definition():
    """One scale per weight row (max group scale / 127), codes t * rint(s_g / s_row), int8 rows of the rotated input:
    a hand case, and the lossy product stays within the reference's 3e-2 of the exact one
    (Tests/IngotTests/KernelCaseFlashNextI8.swift:180-200)."""
    rng = np.random.default_rng(5)
    N, K = 4, 256
    codes = rng.integers(0, 3, size=(N, K)).astype(np.uint32)
    w = np.zeros((N, K // 16), dtype=np.uint32)
    for j in range(16):
        w |= codes[:, j::16] << np.uint32(2 * j)
    s = np.array([[0.5, 0.25], [1.0, 1.0], [0.125, 0.5], [0.75, 0.375]], dtype=np.float16)
    xr = qref.round_f16(rng.normal(0, 1, size=(3, K)).astype(np.float32))
    y = qref.w8a8_ternary_emulated(xr, w, s)
    xq, sx = qref.quant_i8_rows(xr)
    t = codes.astype(np.float32) - 1
    for n in range(N):
        srow = np.float32(s[n].astype(np.float32).max() / np.float32(127))
        qg = np.rint(s[n].astype(np.float32) / srow)
        wq = t[n] * np.repeat(qg, 128)
        ref = (xq @ wq) * sx * srow
        assert np.allclose(y[:, n], ref, rtol=1e-6, atol=1e-6)
    exact = qref.matmul_t(xr, qref.dequant_ternary(w, s))
    assert np.sqrt(((y - exact) ** 2).sum() / (exact ** 2).sum()) <= 3e-2
