"""Child of tests/test_gpu_ep.py::test_ep_device_exchange (run under torch.distributed.run, one rank per GPU): the
device-side exchange (peer stores + flag barrier), eagerly and replayed from a CUDA graph, against the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ingot_b200 import capi, ep, synth  # noqa: E402
from ingot_b200.moe import MoELayer, RouterSpec  # noqa: E402
from oracle import qref  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl")
    rng = np.random.default_rng(11)
    E, K, D, I, T = 32, 4, 256, 128, 391  # enough rows per expert for the tensor-core kernels
    g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
    wr = synth.router_np(rng, E, D)
    x = synth.activations_np(rng, T, D)
    lo, per = ep.expert_range(rank, world, E)
    mk = lambda t: synth.dense_q_affine(t[0][lo:lo + per], t[1][lo:lo + per], t[2][lo:lo + per], 4, dev)
    tl, tn = ep.token_slice(rank, world, T)
    layer = MoELayer(RouterSpec(E, K), synth.bf16_values_tensor(wr, dev), mk(g), mk(u), mk(d), expert_lo=lo, max_tokens=tn)
    tmax = -(-T // world)  # the region size must be the same on every rank
    yd_dtype = torch.float16 if "f16" in sys.argv[1:] else torch.float32
    epl = ep.ExpertParallelMoE(layer, None, tn, T * K)
    dx = ep.DeviceExchange(E, K, D, tmax, yd_dtype, dev, fused_return=False if "copy" in sys.argv[1:] else ("compact" if "compact" in sys.argv[1:] else ("pairs" if "pairs" in sys.argv[1:] else True)))
    epl.use_device_exchange(dx)
    xt = torch.from_numpy(x[tl:tl + tn]).to(dev).to(torch.bfloat16)
    out = torch.zeros(tn, D, dtype=torch.float32, device=dev)
    inds, wts = qref.route(qref.router_logits(x, wr), K)
    deq = lambda t, e: qref.dequant_affine(t[0][e], t[1][e], t[2][e], 4)
    ref = qref.moe_ffn(x, inds, wts, lambda e: (deq(g, e), deq(u, e), deq(d, e)))[tl:tl + tn]
    errs = []
    dist.barrier()
    for _ in range(2):
        out.zero_()
        epl.encode(xt, out, tn)
        torch.cuda.synchronize()
        errs.append(qref.max_rel(out.cpu().numpy(), ref))
    # the same layer captured in a CUDA graph and replayed three times
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr, stream=s):
            epl.encode(xt, out, tn)
    torch.cuda.synchronize()
    dist.barrier()
    for _ in range(3):
        out.zero_()
        gr.replay()
        torch.cuda.synchronize()
        errs.append(qref.max_rel(out.cpu().numpy(), ref))
    status = capi.context(local).device_status()
    ok = torch.tensor([1 if (max(errs) <= 1e-3 and status == 0) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    dist.barrier()
    if rank == 0:
        print("EPDX_OK" if int(ok.item()) == 1 else f"EPDX_FAIL errs={errs} status={status}")
    code = 0 if int(ok.item()) == 1 else 1
    dist.destroy_process_group()
    sys.exit(code)


if __name__ == "__main__":
    main()
