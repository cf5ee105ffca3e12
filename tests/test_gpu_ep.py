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


@pytest.mark.parametrize("world,T,region", [(2, 6, 0), (4, 37, 0), (2, 128, 0), (4, 37, 64), (2, 128, 300)])
def test_ep_pieces_emulated_on_one_gpu(cuda_device, world, T, region):
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
        # packed: the sources' rows follow each other; regions: source s starts at row s * region
        starts = [s * region for s in range(world)] if region else list(np.concatenate([[0], np.cumsum(recv)])[:world])
        cap = world * region if region else max(R, 1)
        buf = torch.zeros(cap, D, dtype=torch.float16, device=cuda_device)
        for s in range(world):
            buf[starts[s]:starts[s] + recv[s]] = send_rows[s][send_off[s][r]:send_off[s][r + 1]]
        yd = torch.zeros(cap, D, dtype=torch.float32, device=cuda_device)
        ws = torch.empty(layers[r].experts_workspace_bytes(cap, world), dtype=torch.uint8, device=cuda_device)
        layers[r].experts(buf, R, counts_all, world, yd, ws, region_rows=region)
        torch.cuda.synchronize()
        for s in range(world):
            back[s][send_off[s][r]:send_off[s][r + 1]] = yd[starts[s]:starts[s] + recv[s]]
    for r, (lo, n) in enumerate(slices):
        layers[r].combine_rows(back[r], outs[r], n)
    torch.cuda.synchronize()
    got = torch.cat(outs).cpu().numpy()
    inds, wts = qref.route(qref.router_logits(x, wr), K)
    ref = qref.moe_ffn(x, inds, wts, weights)
    # the expert outputs cross the "wire" as fp32
    assert qref.max_rel(got, ref) <= TOL


@pytest.mark.parametrize("world,T,yd_dtype,fused", [(2, 6, torch.float32, False), (4, 37, torch.float32, True),
                                                    (4, 150, torch.float16, False), (8, 64, torch.float32, True),
                                                    (2, 150, torch.float16, True), (2, 200, torch.float32, True)])
def test_ep_device_pieces_emulated_on_one_gpu(cuda_device, world, T, yd_dtype, fused):
    """The kernels of the device-side exchange (rows and counts pushed into per-source regions, plan, return) with every
    rank's buffers on one GPU and the ranks run one after the other. The flag barrier is left out: its kernels wait for
    one another and may only run on separate GPUs; the plan is built by the stand-alone entry point instead."""
    import ctypes as C

    from ingot_b200 import capi
    rng = np.random.default_rng(world * 1000 + T)
    E, K, D, I = 32, 4, 256, 128
    layers, wr, weights = make_layers(rng, cuda_device, E, K, D, I, world, T)
    x = synth.activations_np(rng, T, D)
    slices = [ep.token_slice(r, world, T) for r in range(world)]
    region = max(n for _, n in slices) * K
    cap = world * region
    mk = lambda shape, dt: [torch.zeros(shape, dtype=dt, device=cuda_device) for _ in range(world)]
    recv, back = mk((cap, D), torch.float16), mk((region, D), yd_dtype)
    flags, counts = mk((64,), torch.int32), mk((world, E), torch.int32)
    ctx = capi.context(cuda_device.index or 0)
    arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    eps = []
    for r in range(world):
        h = C.c_void_p()
        ctx.check(capi.lib().iq_ep_create(ctx.handle, r, world, E, region, arr(recv), arr(back), arr(flags), arr(counts),
                                          C.byref(h)))
        eps.append(h)
    xs = [x_tensor(x[lo:lo + n], cuda_device) for lo, n in slices]
    outs = [torch.zeros(n, D, dtype=torch.float32, device=cuda_device) for _, n in slices]
    dt = {torch.float32: capi.IQ_F32, torch.float16: capi.IQ_F16, torch.bfloat16: capi.IQ_BF16}
    try:
        for rep in range(2):  # a second pass over the same buffers: nothing may depend on their being zeroed
            for r, (lo, n) in enumerate(slices):
                layers[r].encode(xs[r], outs[r], n, only=("router", "route", "group"))
                v = layers[r].views(n)
                ctx.check(capi.lib().iq_ep_pack_push(eps[r], 0, xs[r].data_ptr(), dt[xs[r].dtype], xs[r].stride(0), n, K, D,
                                                     v["inds"].data_ptr(), v["pos"].data_ptr(), v["offsets"].data_ptr()))
            for r in range(world):
                ctx.check(capi.lib().iq_ep_plan(eps[r], 0))
                yd = torch.zeros(cap, D, dtype=yd_dtype, device=cuda_device)
                ws = torch.empty(layers[r].experts_workspace_bytes(cap, world), dtype=torch.uint8, device=cuda_device)
                if fused and rep == 0:  # the experts' kernels store through a table of row addresses
                    table = torch.zeros(cap, dtype=torch.int64, device=cuda_device)
                    ctx.check(capi.lib().iq_ep_return_rows(eps[r], 0, dt[yd_dtype], D, table.data_ptr()))
                    layers[r].experts(recv[r], min(cap, T * K), counts[r], world, yd, ws, region_rows=region, yd_rows=table)
                elif fused and world == 2:  # the same order as an index: the experts fetch the rows where they arrived
                    table = torch.full((cap,), -1, dtype=torch.int64, device=cuda_device)
                    index = torch.full((cap,), -1, dtype=torch.int32, device=cuda_device)
                    merged = C.c_void_p()
                    ctx.check(capi.lib().iq_ep_index(eps[r], 0, D, dt[yd_dtype], index.data_ptr(), table.data_ptr(),
                                                     C.byref(merged)))
                    layers[r].experts_indexed(recv[r], index, min(cap, T * K), merged.value, yd, ws, yd_rows=table)
                elif fused:  # the same with the rows gathered expert-major first
                    table = torch.full((cap,), -1, dtype=torch.int64, device=cuda_device)
                    xc = torch.zeros(cap, D, dtype=torch.float16, device=cuda_device)
                    merged = C.c_void_p()
                    ctx.check(capi.lib().iq_ep_compact(eps[r], 0, recv[r].data_ptr(), D, dt[yd_dtype], xc.data_ptr(),
                                                       table.data_ptr(), C.byref(merged)))
                    layers[r].experts(xc, min(cap, T * K), merged.value, 1, yd, ws, yd_rows=table)
                else:
                    layers[r].experts(recv[r], min(cap, T * K), counts[r], world, yd, ws, region_rows=region)
                    ctx.check(capi.lib().iq_ep_return_push(eps[r], 0, yd.data_ptr(), dt[yd_dtype], D))
                torch.cuda.synchronize()
            for r, (lo, n) in enumerate(slices):
                layers[r].combine_rows(back[r], outs[r], n)
            torch.cuda.synchronize()
            got = torch.cat(outs).cpu().numpy()
            inds, wts = qref.route(qref.router_logits(x, wr), K)
            ref = qref.moe_ffn(x, inds, wts, weights)
            assert qref.max_rel(got, ref) <= TOL
            for c in counts[1:]:
                assert torch.equal(c, counts[0])
    finally:
        for h in eps:
            capi.lib().iq_ep_destroy(h)


@pytest.mark.parametrize("world,T,yd_dtype", [(2, 6, torch.float32), (4, 37, torch.float16), (8, 64, torch.float32),
                                              (2, 200, torch.float16), (4, 150, torch.float32)])
def test_ep_token_dispatch_emulated_on_one_gpu(cuda_device, world, T, yd_dtype):
    """The dispatch that sends every token row once per destination rank (iq_ep_pack_push_tokens: the rows in a token
    layout, the token of every routed pair beside them) and the index built from it (iq_ep_index_tokens), with every
    rank's buffers on one GPU and the ranks run one after the other; two passes over the same buffers."""
    import ctypes as C

    from ingot_b200 import capi
    rng = np.random.default_rng(world * 977 + T)
    E, K, D, I = 32, 4, 256, 128
    layers, wr, weights = make_layers(rng, cuda_device, E, K, D, I, world, T)
    x = synth.activations_np(rng, T, D)
    slices = [ep.token_slice(r, world, T) for r in range(world)]
    tok_rows = max(n for _, n in slices)
    region = tok_rows * K
    cap = world * region
    mk = lambda shape, dt: [torch.zeros(shape, dtype=dt, device=cuda_device) for _ in range(world)]
    recv, back = mk((cap, D), torch.float16), mk((region, D), yd_dtype)
    flags, counts = mk((64,), torch.int32), mk((world, E), torch.int32)
    ctx = capi.context(cuda_device.index or 0)
    arr = lambda ts: (C.c_void_p * world)(*[t.data_ptr() for t in ts])
    eps = []
    for r in range(world):
        h = C.c_void_p()
        ctx.check(capi.lib().iq_ep_create(ctx.handle, r, world, E, region, arr(recv), arr(back), arr(flags), arr(counts),
                                          C.byref(h)))
        eps.append(h)
    xs = [x_tensor(x[lo:lo + n], cuda_device) for lo, n in slices]
    outs = [torch.zeros(n, D, dtype=torch.float32, device=cuda_device) for _, n in slices]
    dt = {torch.float32: capi.IQ_F32, torch.float16: capi.IQ_F16, torch.bfloat16: capi.IQ_BF16}
    try:
        for rep in range(2):
            for r, (lo, n) in enumerate(slices):
                layers[r].encode(xs[r], outs[r], n, only=("router", "route", "group"))
                v = layers[r].views(n)
                ctx.check(capi.lib().iq_ep_pack_push_tokens(eps[r], 0, xs[r].data_ptr(), dt[xs[r].dtype], xs[r].stride(0), n, K,
                                                            D, v["inds"].data_ptr(), v["pos"].data_ptr(),
                                                            v["offsets"].data_ptr(), tok_rows))
            for r in range(world):
                ctx.check(capi.lib().iq_ep_plan(eps[r], 0))
                yd = torch.zeros(cap, D, dtype=yd_dtype, device=cuda_device)
                ws = torch.empty(layers[r].experts_workspace_bytes(cap, world), dtype=torch.uint8, device=cuda_device)
                table = torch.full((cap,), -1, dtype=torch.int64, device=cuda_device)
                index = torch.full((cap,), -1, dtype=torch.int32, device=cuda_device)
                merged = C.c_void_p()
                ctx.check(capi.lib().iq_ep_index_tokens(eps[r], 0, D, dt[yd_dtype], tok_rows, index.data_ptr(), table.data_ptr(),
                                                        C.byref(merged)))
                layers[r].experts_indexed(recv[r], index, min(cap, T * K), merged.value, yd, ws, yd_rows=table)
                torch.cuda.synchronize()
                total = int(counts[r].to(torch.int64)[:, r * (E // world):(r + 1) * (E // world)].sum().item())
                idx = index[:total].cpu().numpy()
                assert idx.min() >= 0 and idx.max() < world * tok_rows, "a row index outside the token layout"
            for r, (lo, n) in enumerate(slices):
                layers[r].combine_rows(back[r], outs[r], n)
            torch.cuda.synchronize()
            got = torch.cat(outs).cpu().numpy()
            inds, wts = qref.route(qref.router_logits(x, wr), K)
            ref = qref.moe_ffn(x, inds, wts, weights)
            assert qref.max_rel(got, ref) <= TOL
    finally:
        for h in eps:
            capi.lib().iq_ep_destroy(h)


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
@pytest.mark.parametrize("ret", ["f32", "f16", "f16,copy", "f16,compact", "f16,pairs"])
def test_ep_device_exchange(ret):
    """The exchange done by the library's own kernels over peer memory (no host synchronisation), eager and from a CUDA
    graph, on as many GPUs as the box has (2, 4 or 8)."""
    n = min(torch.cuda.device_count(), 8)
    n = 8 if n >= 8 else (4 if n >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr",
           "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "ep_device_child.py")] + ret.split(",")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "EPDX_OK" in r.stdout
