"""Column-split dense linear (iq_linear_colsplit): rank r holds output features [r*N/G, (r+1)*N/G), every rank ends up
with the whole y. On one GPU the ranks are emulated in one process, one after the other, with the flag barriers left out
(kernels that wait for one another may only run on separate GPUs); with two or more GPUs the real exchange runs in child
processes. The reference has no multi-GPU path; a shard is the row range its nPrefix / row-concatenation code addresses
(Layers/Linear.swift:107-183, 350-366), and the parity bar is the one of its qmv / qmm kernel cases."""
import ctypes as C
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from ingot_b200 import capi, ep, synth
from oracle import qref
from gpu_util import TOL, x_tensor

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {torch.float32: capi.IQ_F32, torch.float16: capi.IQ_F16, torch.bfloat16: capi.IQ_BF16}


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,N,K,bits,rows,y_dtype", [
    (2, 256, 512, 4, 1, torch.float32), (4, 512, 2048, 4, 5, torch.float32), (8, 1024, 2048, 8, 16, torch.float32),
    (2, 1024, 512, 4, 192, torch.float32),   # GEMM path, slices above the single-kernel exchange's size
    (4, 512, 256, 4, 64, torch.bfloat16),    # GEMM path, small slices, bf16 output
])
def test_colsplit_emulated_on_one_gpu(cuda_device, world, N, K, bits, rows, y_dtype):
    rng = np.random.default_rng(world + N + rows)
    w, s, b = synth.affine_np(rng, N, K, bits)
    full = synth.dense_q_affine(w, s, b, bits, cuda_device)
    x = synth.activations_np(rng, rows, K)
    xt = x_tensor(x, cuda_device)
    ref = qref.matmul_t(x, qref.dequant_affine(w[0], s[0], b[0], bits))
    ctx = capi.context(cuda_device.index or 0)
    ys = [torch.full((rows, N), 7.0, dtype=y_dtype, device=cuda_device) for _ in range(world)]
    flags = [torch.zeros(64, dtype=torch.int32, device=cuda_device) for _ in range(world)]
    arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    handles, shards = [], [ep.shard_rows(full, r, world) for r in range(world)]
    try:
        for r in range(world):
            h = C.c_void_p()
            ctx.check(capi.lib().iq_colsplit_create(ctx.handle, r, world, N, rows, DT[y_dtype], arr(ys), arr(flags), C.byref(h)))
            handles.append(h)
        for rep in range(2):  # a second pass over the same buffers
            for r in range(world):
                n = C.c_size_t()
                q = shards[r].qlinear()
                ctx.check(capi.lib().iq_linear_colsplit_workspace_bytes(handles[r], C.byref(q), rows, DT[xt.dtype], C.byref(n)))
                ws = torch.empty(max(n.value, 256), dtype=torch.uint8, device=cuda_device)
                ctx.check(capi.lib().iq_linear_colsplit(handles[r], 0, xt.data_ptr(), DT[xt.dtype], xt.stride(0), C.byref(q),
                                                        rows, capi.IQ_FLAG_NO_BARRIER, ws.data_ptr(), ws.numel()))
                torch.cuda.synchronize()
            assert ctx.device_status() == 0
            for r in range(world):
                tol = TOL if y_dtype == torch.float32 else 8e-3  # bf16 output: half an ulp of the output type
                assert qref.max_rel(ys[r].float().cpu().numpy(), ref) <= tol
                assert torch.equal(ys[r], ys[0])  # every rank holds the same bits
    finally:
        for h in handles:
            capi.lib().iq_colsplit_destroy(h)


def test_colsplit_guards(cuda_device):
    ctx = capi.context(cuda_device.index or 0)
    y = torch.zeros(4, 96, dtype=torch.float32, device=cuda_device)
    fl = torch.zeros(64, dtype=torch.int32, device=cuda_device)
    arr = lambda t, n: (C.c_void_p * n)(*[t.data_ptr()] * n)
    h = C.c_void_p()
    # 96 output features do not make four shards of whole 16-row blocks
    assert capi.lib().iq_colsplit_create(ctx.handle, 0, 4, 96, 4, capi.IQ_F32, arr(y, 4), arr(fl, 4), C.byref(h)) == -1
    assert capi.lib().iq_colsplit_create(ctx.handle, 0, 9, 144, 4, capi.IQ_F32, arr(y, 9), arr(fl, 9), C.byref(h)) == -1
    ctx.check(capi.lib().iq_colsplit_create(ctx.handle, 0, 2, 96, 4, capi.IQ_F32, arr(y, 2), arr(fl, 2), C.byref(h)))
    try:
        rng = np.random.default_rng(1)
        m = synth.dense_q_affine(*synth.affine_np(rng, 64, 128, 4), 4, cuda_device)  # 64 rows, the shard must have 48
        x = torch.zeros(4, 128, dtype=torch.bfloat16, device=cuda_device)
        q = m.qlinear()
        st = capi.lib().iq_linear_colsplit(h, 0, x.data_ptr(), capi.IQ_BF16, 128, C.byref(q), 1, 0, 0, 0)
        assert st == -1 and b"shard" in capi.lib().iq_last_error(ctx.handle)
        assert capi.lib().iq_linear_colsplit(h, 0, x.data_ptr(), capi.IQ_BF16, 128, C.byref(q), 5, 0, 0, 0) == -1  # rows > max
    finally:
        capi.lib().iq_colsplit_destroy(h)


def test_peer_wait_times_out_and_reports(cuda_device):
    """A rank whose peer never arrives: the flag barrier's bounded wait runs out (nothing ever sets the peer's flag), the
    kernel returns, iq_ctx_status reports IQ_ERR_TIMEOUT once, and the context goes on working. The bound is a context
    setting, shortened here to about a millisecond."""
    ctx = capi.context(cuda_device.index or 0)
    rng = np.random.default_rng(2)
    N, K = 64, 128
    w, s, b = synth.affine_np(rng, N, K, 4)
    full = synth.dense_q_affine(w, s, b, 4, cuda_device)
    shard = ep.shard_rows(full, 0, 2)
    ys = [torch.zeros(1, N, dtype=torch.float32, device=cuda_device) for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device=cuda_device) for _ in range(2)]
    arr = lambda ts: (C.c_void_p * 2)(*[t.data_ptr() for t in ts])
    h = C.c_void_p()
    ctx.check(capi.lib().iq_colsplit_create(ctx.handle, 0, 2, N, 1, capi.IQ_F32, arr(ys), arr(flags), C.byref(h)))
    x = synth.activations_np(rng, 1, K)
    xt = x_tensor(x, cuda_device)
    ctx.set_wait_cycles(2_000_000)
    try:
        q = shard.qlinear()
        ctx.check(capi.lib().iq_linear_colsplit(h, 0, xt.data_ptr(), capi.IQ_BF16, K, C.byref(q), 1, 0, 0, 0))  # rank 1 never calls
        assert ctx.device_status() == -6     # IQ_ERR_TIMEOUT, and the kernel came back
        assert ctx.device_status() == 0      # the word is cleared when read
        # the expert-parallel barrier takes the same bound
        hep = C.c_void_p()
        bufs = [torch.zeros(4096, dtype=torch.uint8, device=cuda_device) for _ in range(2)]
        ctx.check(capi.lib().iq_ep_create(ctx.handle, 0, 2, 32, 8, arr(bufs), arr(bufs), arr(flags), arr(bufs), C.byref(hep)))
        ctx.check(capi.lib().iq_ep_barrier(hep, 0, 0))
        assert ctx.device_status() == -6
        capi.lib().iq_ep_destroy(hep)
    finally:
        ctx.set_wait_cycles(4_000_000_000)
        capi.lib().iq_colsplit_destroy(h)
    # the context still works: rank 0's slice was computed before the barrier gave up
    ref = qref.matmul_t(x, qref.dequant_affine(w[0][:32], s[0][:32], b[0][:32], 4))
    assert qref.max_rel(ys[0][:, :32].cpu().numpy(), ref) <= TOL


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["device", "nccl"])
def test_colsplit_ranks(exchange):
    """The exchange between real GPUs (as many as the box has, up to 8), eager and replayed from a CUDA graph, decode and
    prefill row counts, against the CPU oracle."""
    n = min(torch.cuda.device_count(), 8)
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "colsplit_child.py"), exchange]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "COLSPLIT_OK" in r.stdout
