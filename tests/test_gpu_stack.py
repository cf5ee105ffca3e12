"""The layer skeleton of the benchmark stack (fp32 residual, unit RMSNorm, r += MoE(RMSNorm(r)); ModelRound.swift:194-221
of the reference): the normalisation kernel against the oracle, every layer's update against the oracle on the layer's
own normalised input, and MoEStack.forward against the same steps taken one by one."""
import numpy as np
import pytest
import torch

from ingot_b200 import ep, synth
from ingot_b200.moe import MoELayer, RouterSpec
from oracle import qref
from gpu_util import TOL

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_rmsnorm_matches_oracle(cuda_device, dtype):
    rng = np.random.default_rng(2)
    x = (rng.normal(0, 3, size=(37, 512))).astype(np.float32)
    xt = torch.from_numpy(x).to(cuda_device)
    out = torch.zeros(37, 512, dtype=dtype, device=cuda_device)
    ep.rmsnorm(xt, out, 37)
    torch.cuda.synchronize()
    ref = qref.rmsnorm(x, eps=1e-6)
    tol = {torch.float32: 1e-6, torch.float16: 1e-3, torch.bfloat16: 8e-3}[dtype]   # half an ulp of the output type
    assert qref.max_rel(out.float().cpu().numpy(), ref) <= tol


@pytest.mark.parametrize("T", [5, 300])
def test_stack_layers_against_oracle(cuda_device, T):
    rng = np.random.default_rng(40 + T)
    E, K, D, I, L = 32, 4, 256, 128, 3
    layers, hosts = [], []
    for _ in range(L):
        g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
        wr = synth.router_np(rng, E, D)
        mk = lambda t: synth.dense_q_affine(t[0], t[1], t[2], 4, cuda_device)
        layers.append(MoELayer(RouterSpec(E, K), synth.bf16_values_tensor(wr, cuda_device), mk(g), mk(u), mk(d), max_tokens=T))
        hosts.append((g, u, d, wr))
    stack = ep.MoEStack([ep.ExpertParallelMoE(l, None, T, 1) for l in layers], T)
    r0 = rng.normal(0, 1, size=(T, D)).astype(np.float32)
    r = torch.from_numpy(r0).to(cuda_device)
    xn = torch.zeros(T, D, dtype=torch.bfloat16, device=cuda_device)
    deq = lambda t, e: qref.dequant_affine(t[0][e], t[1][e], t[2][e], 4)
    for l, (g, u, d, wr) in zip(layers, hosts):
        before = r.cpu().numpy().copy()
        ep.rmsnorm(r, xn, T)
        l.encode(xn, r, T, accumulate=True)
        torch.cuda.synchronize()
        xh = xn.float().cpu().numpy()
        assert qref.max_rel(xh, qref.rmsnorm(before, eps=1e-6)) <= 8e-3
        inds, wts = qref.route(qref.router_logits(xh, wr), K)
        assert np.array_equal(l.views(T)["inds"].cpu().numpy().astype(np.uint32), inds)
        want = before + qref.moe_ffn(xh, inds, wts, lambda e: (deq(g, e), deq(u, e), deq(d, e)))
        assert qref.max_rel(r.cpu().numpy() - before, want - before) <= TOL
    # the stack helper takes exactly these steps
    r2 = torch.from_numpy(r0).to(cuda_device)
    stack.forward(r2, T)
    torch.cuda.synchronize()
    assert torch.equal(r2, r)


@pytest.mark.parametrize("T", [64, 4096])
def test_stack_at_the_benchmarked_sizes(cuda_device, T):
    """Two layers of the benchmark's stack at its own layer shape (128 experts, top-8, d_model 2048, d_ff 768) and token
    counts (decode batch 64, prefill 4096): every layer's routing in full and its update on 32 sampled tokens against
    the oracle, on the layer's own normalised input."""
    rng = np.random.default_rng(7 + T)
    E, K, D, I, L = 128, 8, 2048, 768, 2
    layers, hosts = [], []
    for li in range(L):
        g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
        wr = synth.router_np(rng, E, D)
        mk = lambda t: synth.dense_q_affine(t[0], t[1], t[2], 4, cuda_device)
        layer = MoELayer(RouterSpec(E, K), synth.bf16_values_tensor(wr, cuda_device), mk(g), mk(u), mk(d),
                         max_tokens=T if li == 0 else 1)
        if li > 0:
            layer.share_scratch(layers[0])
        layers.append(layer)
        hosts.append((g, u, d, wr))
    r0 = rng.normal(0, 1, size=(T, D)).astype(np.float32)
    r = torch.from_numpy(r0).to(cuda_device)
    xn = torch.zeros(T, D, dtype=torch.bfloat16, device=cuda_device)
    deq = lambda t, e: qref.dequant_affine(t[0][e], t[1][e], t[2][e], 4)
    sel = np.sort(rng.choice(T, size=min(T, 32), replace=False))
    for l, (g, u, d, wr) in zip(layers, hosts):
        before = r.cpu().numpy().copy()
        ep.rmsnorm(r, xn, T)
        l.encode(xn, r, T, accumulate=True)
        torch.cuda.synchronize()
        xh = xn.float().cpu().numpy()
        inds, wts = qref.route(qref.router_logits(xh, wr), K)
        assert np.array_equal(l.views(T)["inds"].cpu().numpy().astype(np.uint32), inds)
        upd = qref.moe_ffn(xh[sel], inds[sel], wts[sel], lambda e: (deq(g, e), deq(u, e), deq(d, e)))
        assert qref.max_rel(r.cpu().numpy()[sel] - before[sel], upd) <= TOL
    stack = ep.MoEStack([ep.ExpertParallelMoE(l, None, T, 1) for l in layers], T)
    r2 = torch.from_numpy(r0).to(cuda_device)
    stack.forward(r2, T)
    torch.cuda.synchronize()
    assert torch.equal(r2, r)
