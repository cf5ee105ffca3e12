"""Expert-parallel MoE over the GPUs of one box and the layer stack used by the benchmark.

One process per GPU, `torch.distributed` (NCCL over NVLink on GPUs, gloo in the CPU tests of the host logic) for the
exchange. Experts are sharded in contiguous ranges: rank r of G holds experts [r·E/G, (r+1)·E/G). Tokens are data
parallel: each rank routes its own T/G tokens with the full (replicated) router, so routing indices do not depend on
G. A layer is: route + group (local) → pack rows in expert order (one contiguous segment per destination rank) →
all-to-all of the rows → gate/up/activation/down on the owner → all-to-all back → ordered combine at the sender.

The reference has no multi-GPU path; its nearest notion is the expert→slot table `smap` (Layers/MoE.swift:104).
The column-split dense linear (output features split N/G per rank, all-gather of the slices) is `ColumnSplitLinear`.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from . import capi
from .linear import DenseQ, VQMV, _dtype_id, _stream_ptr
from .moe import MoELayer


# ---- host logic (pure functions; exercised on CPU with gloo) -----------------------------------------------------------
def expert_range(rank: int, world: int, experts: int) -> Tuple[int, int]:
    """Experts owned by `rank`: a contiguous range; experts must divide evenly."""
    if experts % world != 0:
        raise ValueError(f"{experts} experts do not divide over {world} ranks")
    per = experts // world
    return rank * per, per


def plan_exchange(counts_all: np.ndarray, rank: int) -> Tuple[List[int], List[int]]:
    """counts_all[s, e] = rows rank s routes to expert e. Returns (send_splits, recv_splits) of `rank` in rows:
    send_splits[d] = rows this rank sends to rank d, recv_splits[s] = rows it receives from rank s."""
    world, experts = counts_all.shape
    per = experts // world
    send = [int(counts_all[rank, d * per:(d + 1) * per].sum()) for d in range(world)]
    recv = [int(counts_all[s, rank * per:(rank + 1) * per].sum()) for s in range(world)]
    return send, recv


def token_slice(rank: int, world: int, tokens: int) -> Tuple[int, int]:
    """Tokens [lo, lo + n) handled by `rank` (data parallel; the remainder goes to the first ranks)."""
    base, rem = divmod(tokens, world)
    lo = rank * base + min(rank, rem)
    return lo, base + (1 if rank < rem else 0)


# ---- device side ----------------------------------------------------------------------------------------------------------
class ExpertParallelMoE:
    """One rank's share of an MoE layer. `layer` holds this rank's experts (expert_lo/expert_count set)."""

    def __init__(self, layer: MoELayer, group: Optional[dist.ProcessGroup], max_local_tokens: int, max_rows: int,
                 shared: Optional["ExpertParallelMoE"] = None, yd_dtype: torch.dtype = torch.float32):
        # yd_dtype: element type of the expert outputs on the return path. float32 keeps the layer within 1e-3 of the
        # fp32 oracle; float16 (what the reference stores for affine experts) halves the bytes but adds a rounding.
        self.layer = layer
        self.group = group
        self.world = dist.get_world_size(group) if (group is not None or dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.max_rows = max_rows
        layer.reserve(max_local_tokens)
        dev = layer.device
        E, k, D = layer.router.experts, layer.router.top_k, layer.D
        if shared is not None:  # layers of a stack run in series and share their exchange buffers
            self.buf = shared.buf
        else:
            P = max_local_tokens * k
            self.buf = {
                "send": torch.empty(P, D, dtype=torch.float16, device=dev),
                "recv": torch.empty(max_rows, D, dtype=torch.float16, device=dev),
                "yd": torch.empty(max_rows, D, dtype=yd_dtype, device=dev),
                "back": torch.empty(P, D, dtype=yd_dtype, device=dev),
                "counts_all": torch.zeros(self.world, E, dtype=torch.int32, device=dev),
                "ws": torch.empty(layer.experts_workspace_bytes(max_rows, self.world), dtype=torch.uint8, device=dev),
            }

    def use_device_exchange(self, dx: "DeviceExchange"):
        """Switches the layer to the device-side exchange (`dx` is shared by the layers of a stack). Every source rank
        owns a region of dx.region_rows rows in each receive buffer, so the expert scratch covers world * region_rows."""
        self.dx = dx
        if "yd_dx" not in self.buf:
            dev = self.layer.device
            self.buf["yd_dx"] = torch.empty(dx.max_rows, self.layer.D, dtype=dx.yd_dtype, device=dev)
            self.buf["rows_dx"] = torch.zeros(dx.max_rows, dtype=torch.int64, device=dev)
            self.buf["xc_dx"] = torch.zeros(dx.max_rows if dx.fused_return == "compact" else 1, self.layer.D, dtype=torch.float16,
                                            device=dev)
            self.buf["index_dx"] = torch.zeros(dx.max_rows, dtype=torch.int32, device=dev)
            self.buf["ws_dx"] = torch.empty(self.layer.experts_workspace_bytes(dx.max_rows, self.world), dtype=torch.uint8,
                                            device=dev)

    def _encode_device(self, x, out, rows, accumulate):
        L, b, dx = self.layer, self.buf, self.dx
        k = L.router.top_k
        L.encode(x, out, rows, only=("router", "route", "group"))
        v = L.views(rows)
        by_token = dx.fused_return is True
        # rows and counts go out; no peer input needed
        (dx.pack_push_tokens if by_token else dx.pack_push)(x, rows, k, v["inds"], v["pos"], v["offsets"])
        dx.barrier(then_plan=True)
        # the kernels are picked for the rows this rank expects to receive (about as many as it sends)
        if dx.fused_return == "compact":
            # rows gathered expert-major (one run of rows per expert, whatever their source); the expert outputs then
            # go through the table of return addresses straight into the sources' buffers
            merged = dx.compact(b["xc_dx"], b["rows_dx"])
            L.experts(b["xc_dx"], min(rows * k, dx.max_rows), merged, 1, b["yd_dx"], b["ws_dx"], yd_rows=b["rows_dx"])
        elif dx.fused_return:
            # the same order as an index into the receive buffer: the experts' kernels fetch the rows themselves
            merged = (dx.index_tokens if by_token else dx.index)(b["index_dx"], b["rows_dx"])
            L.experts_indexed(dx.recv, b["index_dx"], min(rows * k, dx.max_rows), merged, b["yd_dx"], b["ws_dx"],
                              yd_rows=b["rows_dx"])
        else:
            L.experts(dx.recv, min(rows * k, dx.max_rows), dx.counts, self.world, b["yd_dx"], b["ws_dx"],
                      region_rows=dx.region_rows)
            dx.return_push(b["yd_dx"])
        dx.barrier()
        L.combine_rows(dx.back, out, rows, accumulate=accumulate)

    def encode(self, x: torch.Tensor, out: torch.Tensor, rows: int, accumulate: bool = False):
        if self.world == 1:
            self.layer.encode(x, out, rows, accumulate=accumulate)
            return
        if getattr(self, "dx", None) is not None:
            self._encode_device(x, out, rows, accumulate)
            return
        L, b = self.layer, self.buf
        k = L.router.top_k
        P = rows * k
        L.encode(x, out, rows, only=("router", "route", "group"))
        off = L.views(rows)["offsets"]
        counts = (off[1:] - off[:-1]).contiguous()
        dist.all_gather_into_tensor(b["counts_all"].view(-1), counts, group=self.group)
        send, recv = plan_exchange(b["counts_all"].cpu().numpy(), self.rank)  # the one host synchronisation per layer
        R = sum(recv)
        if R > self.max_rows:
            raise RuntimeError(f"rank {self.rank} received {R} rows, more than the {self.max_rows} reserved")
        L.pack_rows(x, b["send"], rows)
        dist.all_to_all_single(b["recv"][:R], b["send"][:P], recv, send, group=self.group)
        L.experts(b["recv"], R, b["counts_all"], self.world, b["yd"], b["ws"])
        dist.all_to_all_single(b["back"][:P], b["yd"][:R], send, recv, group=self.group)
        L.combine_rows(b["back"], out, rows, accumulate=accumulate)


class DeviceExchange:
    """The expert-parallel exchange done by this library's own kernels over NVLink peer memory: rows are stored straight
    into the owners' buffers, sizes are exchanged and read on the device, ranks meet at a flag barrier in peer memory.
    No host synchronisation and no library collective inside a layer, so a whole multi-layer step can be captured in one
    CUDA graph. Peer-addressable buffers come from torch's symmetric memory (plain peer pointers; multicast is not used).
    """

    def __init__(self, experts: int, top_k: int, d_model: int, max_local_tokens: int, yd_dtype: torch.dtype,
                 device: torch.device, group=None, fused_return=True):
        """max_local_tokens: the largest token count any rank handles per call (the same value on every rank).
        fused_return: True (every token row is sent once per destination rank, the experts fetch the received rows
        through an index and store their outputs straight into the sources' return buffers), "pairs" (the same with a
        row per routed pair on the way out), "compact" (pair rows gathered expert-major first) or False (a copy kernel
        returns the outputs)."""
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        P = max_local_tokens * top_k
        # region s of a receive buffer takes whatever source s sends, at most all of its P rows
        self.fused_return = fused_return
        self.tok_rows = max_local_tokens  # rows per source in the token layout of the receive buffer
        self.region_rows, max_rows = P, self.world * P
        self.max_rows, self.yd_dtype, self.d_model = max_rows, yd_dtype, d_model
        esz = torch.empty((), dtype=yd_dtype).element_size()
        sizes = [max_rows * d_model * 2, P * d_model * esz, 256, self.world * experts * 4]
        self._bufs, self._hdls, ptrs = [], [], []
        for n in sizes:
            t = symm_mem.empty((n + 255) // 256 * 256, dtype=torch.uint8, device=device)
            t.zero_()
            h = symm_mem.rendezvous(t, group)
            self._bufs.append(t)
            self._hdls.append(h)
            ptrs.append([int(p) for p in h.buffer_ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(group)
        self.recv = self._bufs[0].view(torch.float16)[: max_rows * d_model].view(max_rows, d_model)
        self.back = self._bufs[1].view(yd_dtype)[: P * d_model].view(P, d_model)
        self.counts = self._bufs[3].view(torch.int32)[: self.world * experts].view(self.world, experts)
        self.ctx = capi.context(device.index or 0)
        arr = lambda v: (C.c_void_p * self.world)(*v)
        self._h = C.c_void_p()
        self.ctx.check(capi.lib().iq_ep_create(self.ctx.handle, self.rank, self.world, experts, self.region_rows,
                                               arr(ptrs[0]), arr(ptrs[1]), arr(ptrs[2]), arr(ptrs[3]), C.byref(self._h)))

    def share_counts(self, offsets: torch.Tensor, stream=None):
        self.ctx.check(capi.lib().iq_ep_share_counts(self._h, _stream_ptr(stream), offsets.data_ptr()))

    def barrier(self, then_plan: bool = False, stream=None):
        self.ctx.check(capi.lib().iq_ep_barrier(self._h, _stream_ptr(stream), 1 if then_plan else 0))

    def plan(self, stream=None):
        self.ctx.check(capi.lib().iq_ep_plan(self._h, _stream_ptr(stream)))

    def pack_push(self, x: torch.Tensor, tokens: int, top_k: int, inds: torch.Tensor, pos: torch.Tensor,
                  offsets: torch.Tensor, stream=None):
        dt = {torch.float32: capi.IQ_F32, torch.float16: capi.IQ_F16, torch.bfloat16: capi.IQ_BF16}[x.dtype]
        self.ctx.check(capi.lib().iq_ep_pack_push(self._h, _stream_ptr(stream), x.data_ptr(), dt, x.stride(0), tokens, top_k,
                                                  self.d_model, inds.data_ptr(), pos.data_ptr(), offsets.data_ptr()))

    def pack_push_tokens(self, x: torch.Tensor, tokens: int, top_k: int, inds: torch.Tensor, pos: torch.Tensor,
                         offsets: torch.Tensor, stream=None):
        """The dispatch with each token row sent once per destination rank (and the token of every pair beside it)."""
        dt = {torch.float32: capi.IQ_F32, torch.float16: capi.IQ_F16, torch.bfloat16: capi.IQ_BF16}[x.dtype]
        self.ctx.check(capi.lib().iq_ep_pack_push_tokens(self._h, _stream_ptr(stream), x.data_ptr(), dt, x.stride(0), tokens,
                                                         top_k, self.d_model, inds.data_ptr(), pos.data_ptr(),
                                                         offsets.data_ptr(), self.tok_rows))

    def index_tokens(self, row_index: torch.Tensor, table: torch.Tensor, stream=None) -> int:
        """`index` for rows that arrived by `pack_push_tokens`."""
        dt = capi.IQ_F32 if self.yd_dtype == torch.float32 else capi.IQ_F16
        merged = C.c_void_p()
        self.ctx.check(capi.lib().iq_ep_index_tokens(self._h, _stream_ptr(stream), self.d_model, dt, self.tok_rows,
                                                     row_index.data_ptr(), table.data_ptr(), C.byref(merged)))
        return merged.value

    def return_push(self, yd: torch.Tensor, stream=None):
        dt = capi.IQ_F32 if yd.dtype == torch.float32 else capi.IQ_F16
        self.ctx.check(capi.lib().iq_ep_return_push(self._h, _stream_ptr(stream), yd.data_ptr(), dt, self.d_model))

    def compact(self, rows_out: torch.Tensor, table: torch.Tensor, stream=None) -> int:
        """Gathers the received rows expert-major into rows_out and fills `table` with their return addresses; returns
        the device address of this rank's per-expert row totals ([experts] uint32)."""
        dt = capi.IQ_F32 if self.yd_dtype == torch.float32 else capi.IQ_F16
        merged = C.c_void_p()
        self.ctx.check(capi.lib().iq_ep_compact(self._h, _stream_ptr(stream), self.recv.data_ptr(), self.d_model, dt,
                                                rows_out.data_ptr(), table.data_ptr(), C.byref(merged)))
        return merged.value

    def index(self, row_index: torch.Tensor, table: torch.Tensor, stream=None) -> int:
        """The expert-major order as an index into the receive buffer (row_index int32 [max_rows]) with the table of return
        addresses; returns the device address of this rank's per-expert row totals."""
        dt = capi.IQ_F32 if self.yd_dtype == torch.float32 else capi.IQ_F16
        merged = C.c_void_p()
        self.ctx.check(capi.lib().iq_ep_index(self._h, _stream_ptr(stream), self.d_model, dt, row_index.data_ptr(),
                                              table.data_ptr(), C.byref(merged)))
        return merged.value

    def return_rows(self, table: torch.Tensor, stream=None):
        dt = capi.IQ_F32 if self.yd_dtype == torch.float32 else capi.IQ_F16
        self.ctx.check(capi.lib().iq_ep_return_rows(self._h, _stream_ptr(stream), dt, self.d_model, table.data_ptr()))

    def close(self):
        if self._h:
            capi.lib().iq_ep_destroy(self._h)
            self._h = C.c_void_p()


def rmsnorm(x: torch.Tensor, out: torch.Tensor, rows: int, eps: float = 1e-6, stream=None):
    """out = x / sqrt(mean(x²) + eps), fp32 in, bf16/fp16/fp32 out (unit weight)."""
    ctx = capi.context(x.device.index or 0)
    dt = {torch.float32: capi.IQ_F32, torch.float16: capi.IQ_F16, torch.bfloat16: capi.IQ_BF16}[out.dtype]
    ctx.check(capi.lib().iq_rmsnorm(ctx.handle, _stream_ptr(stream), x.data_ptr(), x.stride(0), out.data_ptr(), dt,
                                    out.stride(0), rows, x.shape[1], eps))


class MoEStack:
    """L MoE FFN layers on an fp32 residual: per layer xn = RMSNorm(r) (unit weight, eps 1e-6), r += MoE(xn) — the
    reference's layer skeleton around its FFN (ModelRound.swift:194-221, accumulate: true)."""

    def __init__(self, layers: Sequence[ExpertParallelMoE], max_local_tokens: int, x_dtype=torch.bfloat16):
        self.layers = list(layers)
        D = layers[0].layer.D
        self.xn = torch.empty(max_local_tokens, D, dtype=x_dtype, device=layers[0].layer.device)

    def forward(self, r: torch.Tensor, rows: int):
        """r: fp32 [rows, D] residual of this rank's tokens, updated in place."""
        for l in self.layers:
            rmsnorm(r, self.xn, rows)
            l.encode(self.xn, r, rows, accumulate=True)
        return r


def column_shard(rank: int, world: int, n: int) -> Tuple[int, int]:
    """Output features [lo, lo + count) held by `rank` of a linear with n output features split by columns; every shard is
    a whole number of 16-row blocks (the GEMV's unit), so n must be a multiple of 16 * world."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} of {world}")
    if n % (16 * world) != 0:
        raise ValueError(f"{n} output features do not split into {world} shards of whole 16-row blocks")
    per = n // world
    return rank * per, per


def shard_rows(full: DenseQ, rank: int, world: int) -> DenseQ:
    """The shard of `rank`: rows [lo, lo + count) of w / scales / biases — one contiguous byte range of each tensor, the
    layout being row-major by output feature (the reference addresses such a range with nPrefix and its row
    concatenation, Layers/Linear.swift:107-183, 350-366)."""
    if full.experts != 1:
        raise ValueError("a column-split linear is one matrix, not a stack of experts")
    w, sc, b = shard_tensors(full.w, full.s, full.b, rank, world, full.N)
    return DenseQ(w, sc, b, full.N // world, full.K, full.bits, full.gs, full.mode)


def shard_tensors(w, scales, biases, rank: int, world: int, n: int):
    """Rows [lo, lo + count) of the three tensors of a matrix with n output features (torch tensors or numpy arrays,
    on any device; biases may be None): what `shard_rows` cuts, usable on the host before anything is uploaded."""
    lo, per = column_shard(rank, world, n)
    cut = lambda t: None if t is None else t.reshape(n, -1)[lo:lo + per]
    return cut(w), cut(scales), cut(biases)


def assemble_columns(y_all: torch.Tensor, rows: int) -> torch.Tensor:
    """y [rows, n] from the all-gathered slices y_all [world, max_rows, n / world] (slice r = output features of rank r)."""
    world, _, per = y_all.shape
    return y_all[:, :rows].permute(1, 0, 2).reshape(rows, world * per)


class ColumnSplitLinear:
    """A dense quantized linear split by output features over the GPUs of one box: rank r holds rows [r*N/G, (r+1)*N/G) of
    w / scales / biases, x is replicated, and every rank ends up with the whole y [rows, N]. Decode (rows <= 16) runs the
    GEMV kernel, larger row counts the tcgen05 GEMM.

    exchange="device" (default on GPUs): iq_linear_colsplit — the slice is computed straight into this rank's y, stored
    into every peer's y by the library's own kernel over peer memory and fenced by its flag barrier; no host
    synchronisation, graph-capturable. y and the flags live in torch symmetric memory (plain peer pointers, multicast off).
    exchange="nccl": the kernels write a local slice and `all_gather_into_tensor` assembles them (the baseline)."""

    def __init__(self, shard: DenseQ, n_total: int, group: Optional[dist.ProcessGroup], max_rows: int,
                 y_dtype: torch.dtype = torch.float32, exchange: str = "device", x_dtype: torch.dtype = torch.bfloat16):
        if exchange not in ("device", "nccl"):
            raise ValueError("exchange is 'device' or 'nccl'")
        self.shard, self.group, self.exchange = shard, group, exchange
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        lo, per = column_shard(self.rank, self.world, n_total)
        if shard.N != per:
            raise ValueError(f"the shard has {shard.N} output features, {n_total} / {self.world} = {per} expected")
        self.n_total, self.max_rows, self.y_dtype = n_total, max_rows, y_dtype
        dev = shard.w.device
        self.ctx = capi.context(dev.index or 0)
        self.ws = torch.empty(max(shard.qmm_workspace_bytes(max(max_rows, 64), x_dtype), 256), dtype=torch.uint8, device=dev)
        self._h = C.c_void_p()
        if exchange == "nccl":
            self.y_local = torch.empty(max_rows, per, dtype=y_dtype, device=dev)
            self.y_all = torch.empty(self.world, max_rows, per, dtype=y_dtype, device=dev)
            return
        esz = torch.empty((), dtype=y_dtype).element_size()
        if self.world > 1:
            import os

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            g = group if group is not None else dist.group.WORLD
            self._bufs, ptrs = [], []
            for nbytes in (max_rows * n_total * esz, 256):
                t = symm_mem.empty((nbytes + 255) // 256 * 256, dtype=torch.uint8, device=dev)
                t.zero_()
                h = symm_mem.rendezvous(t, g)
                self._bufs.append((t, h))
                ptrs.append([int(p) for p in h.buffer_ptrs])
            torch.cuda.synchronize(dev)
            dist.barrier(g)
            ybuf = self._bufs[0][0]
        else:
            ybuf = torch.zeros(max_rows * n_total * esz, dtype=torch.uint8, device=dev)
            self._flags = torch.zeros(64, dtype=torch.int32, device=dev)
            ptrs = [[ybuf.data_ptr()], [self._flags.data_ptr()]]
        self.y = ybuf[: max_rows * n_total * esz].view(y_dtype).view(max_rows, n_total)
        arr = lambda v: (C.c_void_p * self.world)(*v)
        self.ctx.check(capi.lib().iq_colsplit_create(self.ctx.handle, self.rank, self.world, n_total, max_rows,
                                                     _dtype_id(self.y), arr(ptrs[0]), arr(ptrs[1]), C.byref(self._h)))

    def encode(self, x: torch.Tensor, rows: int, stream=None) -> torch.Tensor:
        """Enqueues y[:rows] = x[:rows] W^T on every rank and returns y [max_rows, N] (valid in stream order)."""
        if rows > self.max_rows:
            raise ValueError(f"rows = {rows} exceeds the {self.max_rows} reserved")
        if self.exchange == "device":
            q = self.shard.qlinear()
            self.ctx.check(capi.lib().iq_linear_colsplit(self._h, _stream_ptr(stream), x.data_ptr(), _dtype_id(x), x.stride(0),
                                                         C.byref(q), rows, 0, self.ws.data_ptr(), self.ws.numel()))
            return self.y
        if rows <= VQMV.MAX_ROWS:
            VQMV.encode(x, self.shard, self.y_local, rows)
        else:
            self.shard.encode_qmm_f32(x, self.y_local, rows, workspace=self.ws)
        if self.world == 1:
            self.y_all[0].copy_(self.y_local)
        else:
            dist.all_gather_into_tensor(self.y_all.view(-1, self.y_all.shape[2]), self.y_local, group=self.group)
        return assemble_columns(self.y_all, self.max_rows)

    def close(self):
        if self._h:
            capi.lib().iq_colsplit_destroy(self._h)
            self._h = C.c_void_p()
