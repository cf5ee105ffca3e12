#!/usr/bin/env python3
"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py --gpus N --steps K --warmup W          (N > 1: launched by torch.distributed.run, one rank per GPU)
    python bench.py --impl reference --gpus N --steps K --warmup W

Headline workload (`config.workload`): the 48-layer stack of the MoE FFN configuration (128 experts, top-8, d_model
2048, expert d_ff 768, 4-bit g64, SiLU-SwiGLU, bf16 router ~ N(0, 0.02), per layer r += MoE(RMSNorm(r)) on an fp32
residual), prefill of 4096 tokens, seeded synthetic weights and activations. One step = one pass of the 4096 tokens
through the 48 layers. With N GPUs the experts are sharded 128/N per GPU and the tokens 4096/N per rank (total work
fixed: "strong" scaling); `value` is whole-job tokens/s. The same JSON line carries the other two parts of the
metric: `qmv` (decode GEMV x[1,4096] · W[14336,4096]ᵀ 4-bit, HBM GB/s) and `qmm` (prefill GEMM M=2048, TFLOP/s), each
with its own roofline fraction, plus `decode` (the stack at batch 64).

`--impl reference` times the reference's CPU path: ingot has only a Metal implementation, so the CPU path is the C
restatement under oracle/ of its fp32 semantics ("port"), run with all host threads on a bounded sample of the same
workload (one layer of the stack per step).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

E, TOPK, D, I = 128, 8, 2048, 768
LAYERS = 48
PREFILL_TOKENS = 4096
DECODE_TOKENS = 64


def measured_peaks():
    """Roofline denominators: the driver's measurement on this pool if present, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def profiled_traffic(filename: str):
    """DRAM bytes (read + write) of one launch as an ncu capture recorded them: the `traffic_bytes_per_launch:` line of a
    summary under profiles/. Returns (bytes or None, "profiles/<file>" or None); a missing file or line gives None, so a
    number never outlives the summary it came from."""
    import re

    path = os.path.join(ROOT, "profiles", filename)
    try:
        with open(path) as f:
            m = re.search(r"traffic_bytes_per_launch:\s*(\d+)", f.read())
    except OSError:
        return None, None
    return (int(m.group(1)), "profiles/" + filename) if m else (None, None)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [v.strip() for v in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------------
# GPU arm


def RETURN_DTYPE(torch):
    """Element type of the expert outputs on the way back to the tokens' ranks (N > 1). fp16 is what the reference
    stores between its down projection and its combine for affine experts (yd, MoEPrefill.swift:159-160)."""
    return torch.float16


def build_stack(torch, dev, rank: int, world: int, max_local_tokens: int, layers: int):
    """The stack's weights, seeded per layer and identical whatever the number of ranks: every rank draws the full
    expert tensors of a layer on its device and keeps its own contiguous slice."""
    from ingot_b200 import ep, synth
    from ingot_b200.linear import DenseQ
    from ingot_b200.moe import MoELayer, RouterSpec

    lo, per = ep.expert_range(rank, world, E)
    out, first, first_ep = [], None, None
    for li in range(layers):
        gen = torch.Generator(device=dev)
        gen.manual_seed(li)
        router = synth.router_cuda(gen, E, D)
        mats = []
        for (n, k) in ((I, D), (I, D), (D, I)):
            full = synth.affine_cuda(gen, n, k, 4, E)
            mats.append(DenseQ(full.w[lo:lo + per].clone(), full.s[lo:lo + per].clone(), full.b[lo:lo + per].clone(), n, k,
                               4, 64, "affine", per))
            del full
        layer = MoELayer(RouterSpec(E, TOPK), router, mats[0], mats[1], mats[2], expert_lo=lo,
                         max_tokens=max_local_tokens if first is None else 1)
        if first is None:
            first = layer
        else:
            layer.share_scratch(first)
        epl = ep.ExpertParallelMoE(layer, None, max_local_tokens, PREFILL_TOKENS * TOPK if world > 1 else 1, shared=first_ep)
        if first_ep is None:
            first_ep = epl
            if world > 1:  # rows move by the library's own peer stores; nothing in a layer touches the host
                dx = ep.DeviceExchange(E, TOPK, D, max_local_tokens, RETURN_DTYPE(torch), dev)
        if world > 1:
            epl.use_device_exchange(dx)
        out.append(epl)
    return ep.MoEStack(out, max_local_tokens)


def time_steps(torch, dist, world, fn, steps, warmup, drain=None):
    """W untimed + K timed calls of fn between barriers, CUDA events on the current stream, max over ranks (ms/step).
    drain: called after the last timed step and before the closing timestamp (work that fn left on other streams)."""
    for _ in range(warmup):
        fn()
    if drain is not None:
        drain()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    if drain is not None:
        drain()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def graph_time_us(torch, fn, n_in_graph: int, reps: int = 20, dist=None, world: int = 1) -> float:
    """Average device time of one call of fn(i): n_in_graph calls captured into a CUDA graph and replayed, which takes
    the host's launch cost out of a microsecond-scale kernel's timing. With world > 1 every rank makes the same calls
    (kernels that meet at a barrier included) and the result is the maximum over the ranks."""
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(n_in_graph):
                fn(i)
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / (reps * n_in_graph) * 1e3
    if world > 1:
        t = torch.tensor([us], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item())
    return us


def count_own_kernels(graph):
    """Kernel nodes of a captured CUDA graph, and how many of them are this library's kernels (namespace iq in the
    mangled name): the launches one replay makes. Returns (own or None when names cannot be read, all kernel nodes), or
    (None, None) when the graph cannot be inspected."""
    try:
        from cuda.bindings import driver as drv

        raw = graph.raw_cuda_graph()
        g = drv.CUgraph(int(raw))
        err, _, n = drv.cuGraphGetNodes(g, 0)
        if int(err) != 0 or n == 0:
            return None, None
        err, nodes, n = drv.cuGraphGetNodes(g, n)
        own = total = named = 0
        for node in nodes[:n]:
            err, ty = drv.cuGraphNodeGetType(node)
            if int(err) != 0 or ty != drv.CUgraphNodeType.CU_GRAPH_NODE_TYPE_KERNEL:
                continue
            total += 1
            try:
                err, prm = drv.cuGraphKernelNodeGetParams(node)
                err2, name = drv.cuFuncGetName(prm.func) if int(err) == 0 else (1, b"")
                if int(err2) == 0 and name:
                    named += 1
                    if b"2iq" in name or b"iq::" in name:
                        own += 1
            except Exception:
                pass
        return (own if named == total else None), total
    except Exception:
        return None, None


def capture(torch, fn):
    """Captures fn() (kernel launches only, no host synchronisation) into a CUDA graph and returns the graph: the step
    then costs one launch on the host, which is what a serving loop does with a fixed-shape step."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph(keep_graph=True)  # the graph stays inspectable (launch count)
        except TypeError:
            g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            fn()
        try:
            g.instantiate()
        except Exception:
            pass  # already instantiated at the end of the capture
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    return g


def bench_qmv(torch, dev, peaks):
    """Decode GEMV: x bf16 [1, 4096], W [14336, 4096] 4-bit g64; eight distinct weight copies (264 MB > L2) in rotation."""
    from ingot_b200 import synth
    from ingot_b200.linear import VQMV

    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    N, K = 14336, 4096
    ms = [synth.affine_cuda(gen, N, K, 4) for _ in range(8)]
    x = synth.activations_cuda(gen, 1, K)
    y = torch.zeros(1, N, dtype=torch.bfloat16, device=dev)
    us = graph_time_us(torch, lambda i: VQMV.encode(x, ms[i % 8], y, 1), 64)
    nbytes = ms[0].weight_bytes() + K * 2 + N * 2  # codes + scales + biases + x + y = 33,067,008 B
    gbs = nbytes / us / 1e3
    qmv_traffic, qmv_traffic_src = profiled_traffic("qmv_imma_c0_14336x4096.md")
    return {"workload": "qmv x[1,4096] W[14336,4096] 4-bit g64, bf16 in/out", "us_per_call": round(us, 3),
            "bytes_per_call": nbytes, "gbs": round(gbs, 1),
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(gbs / peaks["hbm_gbs"], 4), "frac_of_8TBs_nominal": round(gbs / 8000.0, 4),
                         "traffic": qmv_traffic, "traffic_source": qmv_traffic_src, "peak_source": peaks["source"]},
            "l2": "8 weight copies in rotation (264 MB > 126 MB L2)", "timing": "CUDA graph of 64 calls, CUDA events",
            "lm_head": [{k: r[k] for k in ("workload", "us_per_call", "gbs")} | {"frac": r["roofline"]["frac"]}
                        for r in (bench_qmv_shape(torch, dev, peaks, 128000, 2048, b) for b in (4, 6, 8))]}


def bench_qmv_shape(torch, dev, peaks, N, K, bits, rows=1):
    """Decode GEMV of another shape (an lm_head: `--only qmv --qmv-shape 128000,2048,4`): enough weight copies in
    rotation to exceed L2, fp32 logits out."""
    from ingot_b200 import synth
    from ingot_b200.linear import VQMV

    gen = torch.Generator(device=dev)
    gen.manual_seed(2)
    one = N * (K * bits // 8 + K // 64 * 4)
    copies = max(2, -(-300_000_000 // one))
    ms = [synth.affine_cuda(gen, N, K, bits) for _ in range(copies)]
    x = synth.activations_cuda(gen, rows, K)
    y = torch.zeros(rows, N, dtype=torch.float32, device=dev)
    us = graph_time_us(torch, lambda i: VQMV.encode(x, ms[i % copies], y, rows), 4 * copies)
    nbytes = ms[0].weight_bytes() + rows * K * 2 + rows * N * 4
    gbs = nbytes / us / 1e3
    return {"workload": f"qmv x[{rows},{K}] W[{N},{K}] {bits}-bit g64, bf16 in, fp32 out", "us_per_call": round(us, 3),
            "bytes_per_call": nbytes, "gbs": round(gbs, 1),
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": round(gbs / peaks["hbm_gbs"], 4), "traffic": None, "peak_source": peaks["source"]},
            "l2": f"{copies} weight copies in rotation ({copies * one // 1000000} MB > 126 MB L2)",
            "timing": f"CUDA graph of {4 * copies} calls, CUDA events"}


def bench_qmm(torch, dev, peaks):
    """Prefill GEMM: x bf16 [M, 4096], W [14336, 4096], 4- and 8-bit, and the transposed down projection."""
    from ingot_b200 import synth

    gen = torch.Generator(device=dev)
    gen.manual_seed(1)
    res = []
    for (M, N, K, bits) in ((2048, 14336, 4096, 4), (512, 14336, 4096, 4), (2048, 14336, 4096, 8), (2048, 4096, 14336, 4)):
        ws_ = [synth.affine_cuda(gen, N, K, bits) for _ in range(3)]  # three copies: > L2 together with x and y
        x = synth.activations_cuda(gen, M, K)
        y = torch.zeros(M, N, dtype=torch.bfloat16, device=dev)
        wk = torch.empty(max(ws_[0].qmm_workspace_bytes(M, x.dtype), 256), dtype=torch.uint8, device=dev)
        us = graph_time_us(torch, lambda i: ws_[i % 3].encode_qmm_f32(x, y, M, workspace=wk), 6, reps=5)
        tf = 2.0 * M * N * K / us / 1e6
        res.append({"M": M, "N": N, "K": K, "bits": bits, "us_per_call": round(us, 1), "tflops": round(tf, 1),
                    "frac_burst": round(tf / peaks["bf16_tflops"], 4),
                    "frac_sustained": round(tf / peaks["bf16_tflops_sustained"], 4)})
        del ws_
    head = res[0]
    return {"workload": "qmm x[2048,4096] W[14336,4096] 4-bit g64, bf16 in/out (includes the bf16->fp16 pass)",
            "tflops": head["tflops"],
            "roofline": {"bound": "tensor", "achieved": head["tflops"], "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": head["frac_burst"], "traffic": None, "peak_source": peaks["source"]},
            "cases": res}


def layer0_host_weights(torch, dev):
    """The first layer's full tensors (all 128 experts) as the stack draws them (seed 0), on the host, for the checker."""
    import numpy as np

    from ingot_b200 import synth

    gen = torch.Generator(device=dev)
    gen.manual_seed(0)
    router = synth.router_cuda(gen, E, D).float().cpu().numpy()
    mats = []
    for (n, k) in ((I, D), (I, D), (D, I)):
        full = synth.affine_cuda(gen, n, k, 4, E)
        mats.append((full.w.cpu().numpy().view(np.uint32), full.s.view(torch.int16).cpu().numpy().view(np.uint16),
                     full.b.view(torch.int16).cpu().numpy().view(np.uint16)))
        del full
    return router, mats


def parity_check(torch, dist, dev, stack, r0_dev, t_n, world, return_dtype):
    """Before anything is timed: the stack's first layer on this rank's tokens against the CPU oracle (the checker, never
    the thing measured). Routing indices of every token bit for bit against oracle.qref.route; the layer's update on
    32 sampled tokens against the C oracle's MoE FFN within 1e-3 (max|d| / max|ref|). Worst rank reported."""
    import numpy as np

    from ingot_b200 import ep
    from oracle import cref, qref

    l0 = stack.layers[0]
    r = r0_dev.clone()
    before = r.cpu().numpy().copy()
    ep.rmsnorm(r, stack.xn, t_n)
    l0.encode(stack.xn, r, t_n, accumulate=True)
    torch.cuda.synchronize()
    xn = stack.xn[:t_n].float().cpu().numpy()
    got_inds = l0.layer.views(t_n)["inds"].cpu().numpy().astype(np.uint32)
    upd = r.cpu().numpy() - before
    router, mats = layer0_host_weights(torch, dev)
    inds, wts = qref.route(qref.router_logits(xn, router), TOPK)
    inds_exact = bool(np.array_equal(got_inds, inds))
    rng = np.random.default_rng(99)
    sel = np.sort(rng.choice(t_n, size=min(32, t_n), replace=False))
    cref.set_threads(max(1, cref.host_threads() // max(world, 1)))
    ref, _ = cref.moe_ffn(xn[sel], inds[sel], wts[sel], mats[0], mats[1], mats[2], "affine")
    max_rel = float(qref.max_rel(upd[sel], ref))
    if world > 1:
        t = torch.tensor([max_rel, 0.0 if inds_exact else 1.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        max_rel, inds_exact = float(t[0].item()), bool(t[1].item() == 0.0)
    return {"max_rel": round(max_rel, 7), "tolerance": 1e-3, "inds_exact": inds_exact, "sampled_tokens_per_rank": int(len(sel)),
            "layer": "first layer of the stack, this rank's tokens, against oracle/ (C + numpy restatement)",
            "return_dtype": {torch.float16: "f16", torch.float32: "f32"}[return_dtype] if world > 1 else "n/a"}


def piece_times(torch, dist, world, stack, r, t_n):
    """Device time of every piece of one layer (the first), each captured eight times in a CUDA graph of its own and
    replayed, max over ranks; the pieces run on the state a full forward pass left behind."""
    l0 = stack.layers[0]
    L, xn = l0.layer, stack.xn
    from ingot_b200 import ep

    stack.forward(r.clone(), t_n)
    torch.cuda.synchronize()
    tm = lambda fn: round(graph_time_us(torch, lambda i: fn(), 8, reps=5, dist=dist, world=world), 2)
    out = {"norm": tm(lambda: ep.rmsnorm(r, xn, t_n)),
           "router": tm(lambda: L.encode(xn, r, t_n, only="router")),
           "route": tm(lambda: L.encode(xn, r, t_n, only="route")),
           "group": tm(lambda: L.encode(xn, r, t_n, only="group"))}
    if world == 1:
        out["gateup"] = tm(lambda: L.encode(xn, r, t_n, only="gateup"))
        out["down"] = tm(lambda: L.encode(xn, r, t_n, only="down"))
        out["combine"] = tm(lambda: L.encode(xn, r, t_n, only="combine"))
        return out
    dx, b, k = l0.dx, l0.buf, L.router.top_k
    v = L.views(t_n)
    by_token = dx.fused_return is True  # every token row once per destination rank
    out["pack_push"] = tm(lambda: (dx.pack_push_tokens if by_token else dx.pack_push)(xn, t_n, k, v["inds"], v["pos"],
                                                                                       v["offsets"]))
    out["barrier_plan"] = tm(lambda: dx.barrier(then_plan=True))
    merged = [None]

    def index():
        merged[0] = (dx.index_tokens if by_token else dx.index)(b["index_dx"], b["rows_dx"])

    out["index"] = tm(index)
    out["experts_gateup_down_return"] = tm(lambda: L.experts_indexed(dx.recv, b["index_dx"], min(t_n * k, dx.max_rows), merged[0],
                                                                    b["yd_dx"], b["ws_dx"], yd_rows=b["rows_dx"]))
    out["barrier"] = tm(lambda: dx.barrier())
    out["combine"] = tm(lambda: L.combine_rows(dx.back, r, t_n, accumulate=True))
    return out


def bench_colsplit(torch, dist, dev, rank, world, peaks):
    """The column-split dense linear over the ranks: x[1, 4096] . W[14336, 4096]^T 4-bit (us per call, whole y on every
    rank) and x[2048, 4096] (TFLOP/s per GPU and in total), with the library's own peer-store exchange (calls captured
    in a CUDA graph), and the same kernels with a host-launched NCCL all-gather for comparison. Every rank draws its own
    shard; enough shard copies rotate to exceed L2."""
    from ingot_b200 import ep, synth

    N, K = 14336, 4096
    lo, per = ep.column_shard(rank, world, N)
    gen = torch.Generator(device=dev)
    gen.manual_seed(100 + rank)
    one = per * (K // 2 + K // 64 * 4)
    copies = max(2, -(-300_000_000 // one))
    shards = [synth.affine_cuda(gen, per, K, 4) for _ in range(copies)]
    res = {"workload": f"W[14336,4096] 4-bit g64 split {world} ways by output features ({per} per GPU), y fp32 on every rank",
           "l2": f"{copies} shard copies in rotation ({copies * one // 1000000} MB per GPU)"}
    for tag, M in (("decode", 1), ("prefill", 2048)):
        x = synth.activations_cuda(gen, M, K)
        entry = {"rows": M}
        for exchange in ("device", "nccl"):
            try:
                lin = ep.ColumnSplitLinear(shards[0], N, None, M, exchange=exchange)

                def call(i):
                    lin.shard = shards[i % copies]
                    lin.encode(x, M)

                if exchange == "device":
                    n_graph = 4 * copies if M == 1 else 4
                    us = graph_time_us(torch, call, n_graph, reps=5 if M == 1 else 3, dist=dist, world=world)
                else:  # the library collective is launched by the host, call by call, as a caller would
                    n_calls = 50 if M == 1 else 8
                    us = time_steps(torch, dist, world, lambda: [call(i) for i in range(n_calls)], 3, 1) * 1e3 / n_calls
                entry[exchange + "_us"] = round(us, 2)
                lin.close()
                del lin
            except Exception as exc:  # the comparison arm must not take the bench down
                entry[exchange + "_us"] = None
                entry[exchange + "_error"] = repr(exc)[:200]
        us = entry.get("device_us")
        if us:
            if M == 1:
                gb = (one + K * 2 + N * 4) / us / 1e3  # per GPU: its shard + x in, the whole y out
                entry["gbs_per_gpu"] = round(gb, 1)
                entry["frac_hbm_per_gpu"] = round(gb / peaks["hbm_gbs"], 4)
            else:
                tf = 2.0 * M * N * K / us / 1e6
                entry["tflops_total"] = round(tf, 1)
                entry["tflops_per_gpu"] = round(tf / world, 1)
                entry["frac_burst_per_gpu"] = round(tf / world / peaks["bf16_tflops"], 4)
                entry["allgather_bytes_per_gpu"] = int(M * per * 4 * (world - 1))
        res[tag] = entry
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist

    from ingot_b200 import ep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N > 1 with torch.distributed.run")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    T = args.tokens
    t_lo, t_n = ep.token_slice(rank, world, T)
    d_lo, d_n = ep.token_slice(rank, world, DECODE_TOKENS)
    stack = build_stack(torch, dev, rank, world, max(t_n, 1), args.layers)

    gen = torch.Generator(device="cpu")
    gen.manual_seed(1234)
    r0_host = torch.randn(T, D, generator=gen)                     # residual r0 ~ N(0, 1), the same on every rank
    r0_pinned = r0_host[t_lo:t_lo + t_n].contiguous().pin_memory()
    r0_dev = r0_pinned.to(dev)
    r = torch.empty_like(r0_dev)
    out_pinned = torch.empty_like(r0_pinned).pin_memory()

    # parity first: nothing below is worth a number if the layer differs from the oracle
    parity = None
    if args.layers > 0 and not args.no_parity:
        if world > 1:
            dist.barrier()
        parity = parity_check(torch, dist, dev, stack, r0_dev, t_n, world, RETURN_DTYPE(torch))

    def step_eager():
        r.copy_(r0_dev)
        stack.forward(r, t_n)

    # no host synchronisation inside a step, on one GPU or many: one CUDA graph per step
    if world > 1:
        dist.barrier()
    step_graph = capture(torch, step_eager)
    fwd_graph = capture(torch, lambda: stack.forward(r, t_n))
    own_launches, all_launches = count_own_kernels(step_graph)

    def step():
        step_graph.replay()

    # End to end: host buffers in, host buffer out, through the public API a caller drives. Every step copies its input
    # from pinned host memory and reads its result back; as a serving loop would, the copies run on streams of their own,
    # so step i + 1's input arrives while step i computes and step i's result leaves while step i + 1 computes. The host
    # waits for a step's result one step later.
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
    stage = [torch.empty_like(r0_dev) for _ in range(2)]   # inputs as they arrive
    result = [torch.empty_like(r0_dev) for _ in range(2)]  # results waiting for their copy out
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_taken = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    e2e_state = {"i": 0}

    def fetch(b):  # host -> device copy of one step's input into staging buffer b
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(ev_taken[b])
            stage[b].copy_(r0_pinned, non_blocking=True)
            ev_in[b].record(copy_in)

    def step_e2e():
        i = e2e_state["i"]
        b = i % 2
        cur = torch.cuda.current_stream()
        if i == 0:
            fetch(b)
        fetch(1 - b)  # the next step's input, while this step computes
        cur.wait_event(ev_in[b])
        r.copy_(stage[b])
        ev_taken[b].record(cur)
        fwd_graph.replay()
        cur.wait_event(ev_out[b])  # the copy out of two steps ago has left this buffer
        result[b].copy_(r)
        ev_done[b].record(cur)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(ev_done[b])
            out_pinned.copy_(result[b], non_blocking=True)
            ev_out[b].record(copy_out)
        if i > 0:
            ev_out[1 - b].synchronize()  # the previous step's result is on the host
        e2e_state["i"] = i + 1

    def drain_e2e():  # before the closing timestamp: every copy of the timed steps has finished
        cur = torch.cuda.current_stream()
        cur.wait_stream(copy_out)
        cur.wait_stream(copy_in)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = time_steps(torch, dist, world, step, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e = time_steps(torch, dist, world, step_e2e, args.steps, 1, drain=drain_e2e)
    finite = bool(torch.isfinite(r).all().item())

    # decode batch of 64 through the same stack
    dec = None
    if d_n > 0 and args.only is None:
        rd0 = r0_dev[:d_n].clone() if t_n >= d_n else torch.randn(d_n, D, device=dev)
        rd = torch.empty_like(rd0)

        def step_dec():
            rd.copy_(rd0)
            stack.forward(rd, d_n)

        dec_graph = capture(torch, step_dec)
        ms_dec = time_steps(torch, dist, world, dec_graph.replay, max(args.steps, 3), args.warmup)
        dec = {"tokens": DECODE_TOKENS, "ms_per_step": round(ms_dec, 3), "tokens_per_s": round(DECODE_TOKENS / ms_dec * 1e3, 1)}
        if world == 1:
            # HBM floor of one decode layer: the weights of the experts 64 tokens touch (about 126 of 128) + the router
            floor_us = (126 * 2654208 + 524288) / (peaks["hbm_gbs"] * 1e3)
            dec["us_per_layer"] = round(ms_dec * 1e3 / max(args.layers, 1), 2)
            dec["hbm_floor_us_per_layer"] = round(floor_us, 2)
            dec["frac_of_hbm_floor"] = round(floor_us / (ms_dec * 1e3 / max(args.layers, 1)), 4)

    # per-piece device times of one layer (every rank takes part: the exchange pieces meet at barriers)
    pieces = piece_times(torch, dist, world, stack, r, t_n) if args.layers > 0 else None

    # the dominant kernel of the prefill stack: the experts' gate+up GEMM, timed alone over the layers at N = 1
    roof = None
    if world == 1 and args.layers > 0:
        xn = stack.xn

        def gateup_all():
            for l in stack.layers:
                l.layer.encode(xn, r, t_n, only="gateup")

        step_eager()
        ms_gu = time_steps(torch, dist, 1, gateup_all, max(2, args.steps // 2), 1) / len(stack.layers)
        flops = 2.0 * t_n * TOPK * (2 * I) * D
        tf = flops / (ms_gu * 1e-3) / 1e12
        traffic, traffic_src = profiled_traffic("qmm_tc_grouped_gateup_down_prefill4096.md") if t_n == PREFILL_TOKENS else (None, None)
        roof = {"kernel": "experts gate+up+SwiGLU (grouped)", "bound": "tensor", "achieved": round(tf, 2),
                "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s", "frac": round(tf / peaks["bf16_tflops_sustained"], 4),
                "traffic": traffic, "traffic_source": traffic_src,
                "algorithmic_bytes": int(E * 2 * I * (D // 2 + D // 64 * 4) + t_n * D * 2 + t_n * TOPK * I * 2),
                "ms_per_launch": round(ms_gu, 4), "flops_per_launch": flops,
                "peak_source": peaks["source"] + " (sustained: the kernel runs inside a long step)"}

    colsplit = None
    if world > 1 and args.only is None:
        colsplit = bench_colsplit(torch, dist, dev, rank, world, peaks)

    line = None
    if rank == 0:
        qmv = bench_qmv(torch, dev, peaks) if args.only is None else None
        qmm = bench_qmm(torch, dev, peaks) if args.only is None else None
        from ingot_b200 import capi
        status = capi.context(local).device_status()
        if all_launches is not None:
            n_own = own_launches if own_launches is not None else all_launches
            launches = {"gpu_launches": n_own * args.steps,
                        "gpu_launches_source": (f"{n_own} kernel nodes of this library" if own_launches is not None else
                                                f"{all_launches} kernel nodes (their names could not be read; torch's "
                                                "residual copy is a memcpy node, so all of them are this library's)") +
                                               f" of {all_launches} kernel nodes counted in the step's CUDA graph, times the timed steps"}
        else:
            per_layer = 10 if world == 1 else 15
            launches = {"gpu_launches": per_layer * args.layers * args.steps,
                        "gpu_launches_source": "graph not inspectable: kernels per layer by the launch list x layers x steps"}
        line = {
            "metric": "moe_ffn_tokens_per_s", "value": round(T / ms * 1e3, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16 operands, f32 accumulate (4-bit codes)",
            "data": "synthetic",
            "config": {"workload": f"{args.layers}-layer MoE FFN stack, prefill {T} tokens: 128 experts top-8 d_model 2048 "
                                   "d_ff 768 4-bit g64, r += MoE(RMSNorm(r))",
                       "parallelism": f"ep{world}" if world > 1 else "single", "tokens": T, "layers": args.layers,
                       "l2": "per-step working set (weights of all layers) is far larger than L2",
                       "launch": "one CUDA graph per step", "exchange": "peer stores (every token row once per destination rank) + flag barrier (own kernels)" if world > 1 else "none"},
            "e2e": {"value": round(T / ms_e2e * 1e3, 1), "unit": "tokens/s", "ms_per_step": round(ms_e2e, 3),
                    "h2d_bytes_per_step": int(t_n * D * 4), "d2h_bytes_per_step": int(t_n * D * 4),
                    "copies": "pinned host memory, every step, on streams of their own: step i + 1's input arrives and "
                              "step i's result leaves while a step computes; all of them inside the timed region"},
            **launches,
            "clocks": clocks, "finite": finite, "device_status": status, "parity": parity,
            "roofline": roof if roof is not None else {"bound": "tensor", "achieved": None, "peak": peaks["bf16_tflops_sustained"],
                                                        "unit": "TFLOP/s", "frac": None, "traffic": None,
                                                        "note": "the dominant kernel is timed alone at N=1; see pieces_us"},
            "pieces_us": pieces, "decode": dec, "qmv": qmv, "qmm": qmm, "colsplit": colsplit,
        }
        if world == 1 and args.only is None:
            line["cpu_baseline"] = cpu_baseline(sample_tokens=args.cpu_tokens, reps=1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if line is not None:
        emit(line)


# ---------------------------------------------------------------------------------------------------------------------
# CPU arm: the C restatement of the reference's fp32 semantics, all host threads


_CPU_CASE = {}


def cpu_layer_inputs(sample_tokens: int, seed: int = 0):
    """Weights and activations of one layer on the host (drawn once, outside any timed region)."""
    import numpy as np

    from ingot_b200 import synth

    key = (sample_tokens, seed)
    if key not in _CPU_CASE:
        rng = np.random.default_rng(seed)
        g, u, d = synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, I, D, 4, E), synth.affine_np(rng, D, I, 4, E)
        _CPU_CASE[key] = (g, u, d, synth.router_np(rng, E, D), synth.activations_np(rng, sample_tokens, D))
    return _CPU_CASE[key]


def cpu_layer_once(sample_tokens: int, seed: int = 0):
    """One layer of the stack on the CPU (router logits, top-k, gate/up/SwiGLU, down, combine; dequantisation inside the
    timed region) on every hardware thread of the host, whatever OMP_NUM_THREADS the launcher exported. Returns
    (seconds, threads)."""
    import numpy as np

    from oracle import cref, qref

    g, u, d, wr, x = cpu_layer_inputs(sample_tokens, seed)
    cref.set_threads(0)
    t0 = time.perf_counter()
    logits = qref.router_logits(x, wr)
    inds, wts = cref.route(logits, E, TOPK)
    y, threads = cref.moe_ffn(x, inds, wts, g, u, d, "affine")
    dt = time.perf_counter() - t0
    assert np.isfinite(y).all()
    return dt, threads


def cpu_baseline(sample_tokens: int, reps: int = 1):
    best, threads = None, 1
    for _ in range(reps):
        dt, threads = cpu_layer_once(sample_tokens)
        best = dt if best is None else min(best, dt)
    return {"value": round(sample_tokens / (best * LAYERS), 2), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"one whole layer of the 48 at {sample_tokens} tokens on the host ({best:.2f} s, {threads} threads), "
                      "scaled by 48 layers; C restatement under oracle/, OpenMP"}


def run_reference(args):
    """The reference's CPU implementation of the path. ingot itself is Metal-only (no CPU or CUDA path to install), so
    this is the oracle port. One timed step = ONE layer of the stack at the full token count (a bounded sample: the 48
    layers are the same work 48 times); `ms_per_step` is that step as measured, `value` the tokens/s of the 48-layer job
    it implies (tokens / (48 x step time))."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = args.cpu_tokens
    cpu_layer_inputs(n)
    for _ in range(min(args.warmup, 1)):
        cpu_layer_once(n)
    times, threads = [], 1
    for _ in range(args.steps):
        dt, threads = cpu_layer_once(n)
        times.append(dt)
    sec = sum(times) / len(times)
    value = round(n / (sec * LAYERS), 2)
    sample = (f"each step is one layer of the {LAYERS} at {n} tokens ({sec:.2f} s on {threads} threads); value = tokens / "
              f"({LAYERS} x step time)")
    line = {
        "impl": "reference", "metric": "moe_ffn_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": round(sec * 1e3, 1),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{LAYERS}-layer MoE FFN stack, prefill {args.tokens} tokens: 128 experts top-8 d_model 2048 "
                               "d_ff 768 4-bit g64, r += MoE(RMSNorm(r))", "tokens": args.tokens, "layers": LAYERS,
                   "layers_per_timed_step": 1, "step_scaling": f"value = tokens / ({LAYERS} x ms_per_step)",
                   "sample_tokens": n},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "ingot has no CPU or CUDA implementation to install (Swift + Metal only); this arm runs the C restatement "
                "of its fp32 semantics kept under oracle/",
    }
    emit(line)


_RESULT_FD = None


def claim_stdout():
    """The one line on stdout is the result: everything else a library prints there (NCCL's version banner, for one)
    goes to stderr. File descriptor 1 is pointed at stderr and the original kept for emit()."""
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)


def emit(line: dict):
    data = (json.dumps(line) + "\n").encode()
    sys.stdout.flush()
    if _RESULT_FD is None:
        os.write(1, data)
    else:
        os.write(_RESULT_FD, data)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=PREFILL_TOKENS)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--cpu-tokens", type=int, default=PREFILL_TOKENS, help="tokens of the CPU sample (one layer per step)")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle check before the timing (profiling runs)")
    ap.add_argument("--only", choices=["stack", "qmv", "qmm"], default=None,
                    help="run one part alone (small profiling runs): the MoE stack without its side results, or the "
                         "GEMV / GEMM micro-benchmarks")
    ap.add_argument("--qmv-shape", default=None, help="with --only qmv: N,K,bits of another GEMV (an lm_head) instead of C0")
    args = ap.parse_args()
    claim_stdout()
    if args.only in ("qmv", "qmm"):
        import torch

        torch.cuda.set_device(0)
        if args.only == "qmv" and args.qmv_shape:
            n, k, bits = (int(v) for v in args.qmv_shape.split(","))
            emit(bench_qmv_shape(torch, torch.device("cuda", 0), measured_peaks(), n, k, bits))
            return
        fn = bench_qmv if args.only == "qmv" else bench_qmm
        emit(fn(torch, torch.device("cuda", 0), measured_peaks()))
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
