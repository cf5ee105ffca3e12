"""Expert-parallel pieces on the GPU. On one GPU the ranks are emulated in one process, one after the other, with the
all-to-all done by copies (no kernel waits on another); with two or more GPUs the NCCL path runs in child processes."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest
import torch

from ingot_b200 import ep, synth
from ingot_b200.moe import MoELayer, RouterSpec
from oracle import qref
from gpu_util import TOL, x_tensor

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def make_layers(rng, device, E, K, D, I, world, max_tokens):
    g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
    wr = synth.router_np(rng, E, D)
    per = E // world
    layers = []
    for r in range(world):
        lo, hi = r * per, (r + 1) * per
        mk = lambda t: synth.dense_q_affine(t[0][lo:hi], t[1][lo:hi], t[2][lo:hi], 4, device)
        layers.append(MoELayer(RouterSpec(E, K), synth.bf16_values_tensor(wr, device), mk(g), mk(u), mk(d),
                               expert_lo=lo, max_tokens=max_tokens))
    deq = lambda t, e: qref.dequant_affine(t[0][e], t[1][e], t[2][e], 4)
    return layers, wr, (lambda e: (deq(g, e), deq(u, e), deq(d, e)))


@pytest.mark.parametrize("world,T", [(2, 6), (4, 37), (2, 128)])
def test_ep_pieces_emulated_on_one_gpu(cuda_device, world, T):
    rng = np.random.default_rng(world * 100 + T)
    E, K, D, I = 32, 4, 256, 128
    layers, wr, weights = make_layers(rng, cuda_device, E, K, D, I, world, T)
    x = synth.activations_np(rng, T, D)
    slices = [ep.token_slice(r, world, T) for r in range(world)]
    xs = [x_tensor(x[lo:lo + n], cuda_device) for lo, n in slices]
    outs = [torch.zeros(n, D, dtype=torch.float32, device=cuda_device) for _, n in slices]
    counts_all = torch.zeros(world, E, dtype=torch.int32, device=cuda_device)
    send_rows = []
    for r, (lo, n) in enumerate(slices):
        layers[r].encode(xs[r], outs[r], n, only=("router", "route", "group"))
        off = layers[r].views(n)["offsets"]
        counts_all[r] = off[1:] - off[:-1]
        rows = torch.zeros(n * K, D, dtype=torch.float16, device=cuda_device)
        layers[r].pack_rows(xs[r], rows, n)
        send_rows.append(rows)
    torch.cuda.synchronize()
    ca = counts_all.cpu().numpy()
    plans = [ep.plan_exchange(ca, r) for r in range(world)]
    send_off = [np.concatenate([[0], np.cumsum(p[0])]) for p in plans]
    back = [torch.zeros(s.shape, dtype=torch.float32, device=cuda_device) for s in send_rows]
    for r in range(world):  # owner r
        recv = plans[r][1]
        R = sum(recv)
        buf = torch.zeros(max(R, 1), D, dtype=torch.float16, device=cuda_device)
        o = 0
        for s in range(world):
            buf[o:o + recv[s]] = send_rows[s][send_off[s][r]:send_off[s][r + 1]]
            o += recv[s]
        yd = torch.zeros(max(R, 1), D, dtype=torch.float32, device=cuda_device)
        ws = torch.empty(layers[r].experts_workspace_bytes(max(R, 1), world), dtype=torch.uint8, device=cuda_device)
        layers[r].experts(buf, R, counts_all, world, yd, ws)
        torch.cuda.synchronize()
        o = 0
        for s in range(world):
            back[s][send_off[s][r]:send_off[s][r + 1]] = yd[o:o + recv[s]]
            o += recv[s]
    for r, (lo, n) in enumerate(slices):
        layers[r].combine_rows(back[r], outs[r], n)
    torch.cuda.synchronize()
    got = torch.cat(outs).cpu().numpy()
    inds, wts = qref.route(qref.router_logits(x, wr), K)
    ref = qref.moe_ffn(x, inds, wts, weights)
    # the expert outputs cross the "wire" as fp32
    assert qref.max_rel(got, ref) <= TOL


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ep_nccl_two_ranks():
    """Two ranks over NCCL: the expert-parallel layer equals the single-GPU layer on the same tokens."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "ep_nccl_child.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "EP_OK" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ep_device_exchange():
    """The exchange done by the library's own kernels over peer memory (no host synchronisation), eager and from a CUDA
    graph, on as many GPUs as the box has (2, 4 or 8)."""
    n = min(torch.cuda.device_count(), 8)
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "ep_device_child.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "EPDX_OK" in r.stdout
