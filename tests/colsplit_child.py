"""Child of tests/test_gpu_colsplit.py::test_colsplit_ranks (run under torch.distributed.run, one rank per GPU): the
column-split linear with the device-side exchange (peer stores + flag barrier) or the NCCL all-gather, eagerly and
replayed from a CUDA graph, for decode and prefill row counts, against the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from ingot_b200 import capi, ep, synth  # noqa: E402
from oracle import qref  # noqa: E402


def main():
    exchange = sys.argv[1] if len(sys.argv) > 1 else "device"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rng = np.random.default_rng(3)  # the same tensors on every rank
    N, K, max_rows = 2048, 2048, 128
    w, s, b = synth.affine_np(rng, N, K, 4)
    ws, ss, bs = ep.shard_tensors(w, s, b, rank, world, N)
    per = N // world
    shard = synth.dense_q_affine(ws.reshape(1, per, -1), ss.reshape(1, per, -1), bs.reshape(1, per, -1), 4, dev)
    lin = ep.ColumnSplitLinear(shard, N, None, max_rows, exchange=exchange)
    wf = qref.dequant_affine(w[0], s[0], b[0], 4)
    errs = []
    dist.barrier()
    for rows in (1, 16, 128):
        x = synth.activations_np(rng, rows, K)
        xt = torch.from_numpy(x).to(dev).to(torch.bfloat16)
        ref = qref.matmul_t(x, wf)
        for _ in range(2):
            y = lin.encode(xt, rows)
            torch.cuda.synchronize()
            errs.append(qref.max_rel(y[:rows].float().cpu().numpy(), ref))
        if exchange == "device":  # the same call captured in a CUDA graph and replayed
            st = torch.cuda.Stream()
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=st):
                    lin.encode(xt, rows)
            torch.cuda.synchronize()
            dist.barrier()
            for _ in range(3):
                lin.y.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                gr.replay()
                torch.cuda.synchronize()
                errs.append(qref.max_rel(lin.y[:rows].float().cpu().numpy(), ref))
    status = capi.context(local).device_status()
    ok = torch.tensor([1 if (max(errs) <= 1e-3 and status == 0) else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    dist.barrier()
    if rank == 0:
        print("COLSPLIT_OK" if int(ok.item()) == 1 else f"COLSPLIT_FAIL errs={errs} status={status}")
    code = 0 if int(ok.item()) == 1 else 1
    lin.close()
    dist.destroy_process_group()
    sys.exit(code)


if __name__ == "__main__":
    main()
