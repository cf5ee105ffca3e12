"""Host-side mirror of the reference's MoE operators (Sources/Ingot/Layers/MoE.swift, MoEPrefill.swift).

`MoELayer` holds the load-time state (router, stacked expert tensors, optional gpt-oss expert biases) and its scratch,
allocated once at construction like the reference (MoE.swift:220-241). `encode` runs router → top-k → group →
gate+up+activation → down → combine on a CUDA stream; `only=` selects pieces by the reference's names
(MoELayer.Piece MoE.swift:328, PrefillMoE.Piece MoEPrefill.swift:55). No CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Iterable, Optional

import torch

from . import capi
from .linear import DenseQ, _dtype_id, _need_cuda, _stream_ptr

PIECES = {
    "router": capi.IQ_PIECE_ROUTER, "route": capi.IQ_PIECE_ROUTE, "group": capi.IQ_PIECE_GROUP,
    "gateup": capi.IQ_PIECE_GATEUP, "down": capi.IQ_PIECE_DOWN, "combine": capi.IQ_PIECE_COMBINE,
}


class RouterSpec:
    """What the router does (the reference's RouterSpec, Loader/ModelSpecParts.swift:64): softmax over the chosen logits
    (score="softmax") or a sigmoid per expert (score="sigmoid") with an optional selection bias and eps."""

    def __init__(self, experts: int, top_k: int, scale: float = 1.0, logit_bias: Optional[torch.Tensor] = None,
                 per_expert_scale: Optional[torch.Tensor] = None, score: str = "softmax",
                 select_bias: Optional[torch.Tensor] = None, eps: float = 0.0):
        if score not in ("softmax", "sigmoid"):
            raise ValueError("score is 'softmax' or 'sigmoid'")
        self.experts, self.top_k, self.scale = experts, top_k, scale
        self.logit_bias, self.per_expert_scale = logit_bias, per_expert_scale
        self.score, self.select_bias, self.eps = score, select_bias, eps


class MoELayer:
    """One MoE FFN layer on one GPU, or one rank's share of it (experts [expert_lo, expert_lo + expert_count))."""

    def __init__(self, router: RouterSpec, router_w: torch.Tensor, gate: DenseQ, up: DenseQ, down: DenseQ,
                 act: str = "silu", limit: float = 7.0, router_scales: Optional[torch.Tensor] = None,
                 router_biases: Optional[torch.Tensor] = None, gate_bias: Optional[torch.Tensor] = None,
                 up_bias: Optional[torch.Tensor] = None, down_bias: Optional[torch.Tensor] = None, expert_lo: int = 0,
                 max_tokens: int = 16, shared: Optional[tuple] = None, shared_gate: Optional[DenseQ] = None):
        """shared: (gate, up, down) DenseQ of the shared expert (MoE.swift:140-154), with shared_gate the 8-bit [1, D]
        tensor of its sigmoid gate, or None for weight 1."""
        _need_cuda(router_w, gate_bias, up_bias, down_bias, router.logit_bias, router.per_expert_scale, router.select_bias)
        self.router, self.gate, self.up, self.down = router, gate, up, down
        self.D, self.I = gate.K, gate.N
        self.device = gate.w.device
        self._keep = [router_w, router_scales, router_biases, gate_bias, up_bias, down_bias, router.logit_bias,
                      router.per_expert_scale, router.select_bias]
        for t in (gate_bias, up_bias, down_bias, router.logit_bias, router.per_expert_scale, router.select_bias):
            if t is not None and (t.dtype != torch.float32 or not t.is_contiguous()):
                raise TypeError("expert biases, router bias and per-expert scale are contiguous float32 tensors")
        if router_w.dtype == torch.bfloat16:
            kind = capi.IQ_ROUTER_BF16
        elif router_w.dtype in (torch.int32, torch.uint32):
            kind = capi.IQ_ROUTER_Q8
        else:
            raise TypeError("router weights are bf16 [E, D] or 8-bit codes packed in 32-bit words")
        ptr = lambda t: 0 if t is None else t.data_ptr()
        d = capi.MoeDesc()
        d.experts, d.top_k, d.d_model, d.d_ff = router.experts, router.top_k, self.D, self.I
        d.act = {"silu": capi.IQ_ACT_SILU, "gelu": capi.IQ_ACT_GELU, "swiglu_oai": capi.IQ_ACT_SWIGLU_OAI,
                 "relu2": capi.IQ_ACT_RELU2}[act]
        d.act_limit = limit
        d.router_kind = kind
        d.routed_scale = router.scale
        d.router_w, d.router_scales, d.router_biases = ptr(router_w.contiguous()), ptr(router_scales), ptr(router_biases)
        d.router_logit_bias, d.per_expert_scale = ptr(router.logit_bias), ptr(router.per_expert_scale)
        d.gate, d.up, d.down = gate.qlinear(), up.qlinear(), down.qlinear()
        d.gate_bias, d.up_bias, d.down_bias = ptr(gate_bias), ptr(up_bias), ptr(down_bias)
        d.expert_lo, d.expert_count = expert_lo, gate.experts
        d.router_score = capi.IQ_SCORE_SIGMOID if router.score == "sigmoid" else capi.IQ_SCORE_SOFTMAX
        d.route_eps = router.eps
        d.router_select_bias = ptr(router.select_bias)
        self._shared = (shared, shared_gate)
        d.shared = capi.IQ_SHARED_NONE
        if shared is not None:
            d.shared = capi.IQ_SHARED_UNGATED if shared_gate is None else capi.IQ_SHARED_GATED
            d.shared_gate_proj, d.shared_up, d.shared_down = shared[0].qlinear(), shared[1].qlinear(), shared[2].qlinear()
            if shared_gate is not None:
                d.shared_gate = shared_gate.qlinear()
        self.ctx = capi.context(self.device.index or 0)
        self._h = C.c_void_p()
        self.ctx.check(capi.lib().iq_moe_create(self.ctx.handle, C.byref(d), C.byref(self._h)))
        self.max_tokens = 0
        self.workspace = None
        self.reserve(max_tokens)

    def reserve(self, max_tokens: int):
        """Sizes the scratch for up to max_tokens rows per call (the reference does this at construction)."""
        if max_tokens <= self.max_tokens:
            return
        n = C.c_size_t()
        self.ctx.check(capi.lib().iq_moe_workspace_bytes(self._h, max_tokens, C.byref(n)))
        self.workspace = torch.empty(n.value, dtype=torch.uint8, device=self.device)
        self.max_tokens = max_tokens

    def share_scratch(self, other: "MoELayer"):
        """Layers of one model run in series and share their scratch (the reference binds per-layer weights into one
        shared PrefillMoE, ModelPrefill.swift:367-374). Both layers must have the same shape."""
        if (other.router.experts, other.router.top_k, other.D, other.I) != (self.router.experts, self.router.top_k,
                                                                             self.D, self.I):
            raise ValueError("layers that share scratch must have the same shape")
        self.workspace, self.max_tokens = other.workspace, other.max_tokens

    def encode(self, x: torch.Tensor, out: torch.Tensor, rows: int, accumulate: bool = False,
               only: Optional[Iterable[str]] = None, stream: Optional[torch.cuda.Stream] = None):
        """out[rows, D] (+)= MoE(x[rows, D]) (MoELayer.encode MoE.swift:346-428; PrefillMoE.encodeAll
        MoEPrefill.swift:274). `only`: piece names to run, in the reference's vocabulary."""
        _need_cuda(x, out)
        if rows > self.max_tokens:
            raise ValueError(f"rows = {rows} exceeds the scratch reserved at construction ({self.max_tokens})")
        mask = capi.IQ_PIECE_ALL
        if only is not None:
            mask = 0
            for p in ([only] if isinstance(only, str) else only):
                mask |= PIECES[p]
        self.ctx.check(capi.lib().iq_moe_forward(
            self._h, _stream_ptr(stream), x.data_ptr(), _dtype_id(x), x.stride(0), out.data_ptr(), _dtype_id(out),
            out.stride(0), rows, capi.IQ_FLAG_ACCUMULATE if accumulate else 0, mask, self.workspace.data_ptr(),
            self.workspace.numel()))

    def route(self, logits: torch.Tensor, rows: int, stream: Optional[torch.cuda.Stream] = None):
        """Top-k on given fp32 logits [rows, ld]: returns (inds int32 [rows, k], wts float32 [rows, k])."""
        _need_cuda(logits)
        k = self.router.top_k
        inds = torch.empty(rows, k, dtype=torch.int32, device=logits.device)
        wts = torch.empty(rows, k, dtype=torch.float32, device=logits.device)
        self.ctx.check(capi.lib().iq_moe_route(self._h, _stream_ptr(stream), logits.data_ptr(), logits.stride(0), rows,
                                               inds.data_ptr(), wts.data_ptr()))
        return inds, wts

    def set_external_routing(self, inds: Optional[torch.Tensor], wts: Optional[torch.Tensor]):
        """Routing chosen by the caller (PrefillMoE.externalRouting, MoEPrefill.swift:80-86); None restores the router."""
        self._ext = (inds, wts)
        self.ctx.check(capi.lib().iq_moe_set_external_routing(
            self._h, 0 if inds is None else inds.data_ptr(), 0 if wts is None else wts.data_ptr()))

    def views(self, rows: int) -> dict:
        """Tensors aliasing the scratch after a call: logits, inds, wts, offsets, row_map, pos, h, yd."""
        v = capi.MoeViews()
        self.ctx.check(capi.lib().iq_moe_get_views(self._h, self.workspace.data_ptr(), rows, C.byref(v)))
        base = self.workspace.data_ptr()
        k, E = self.router.top_k, self.router.experts

        def view(ptr, dtype, shape):
            if ptr is None or ptr < base or ptr >= base + self.workspace.numel():
                return None
            n = 1
            for s in shape:
                n *= s
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            return self.workspace[ptr - base: ptr - base + nbytes].view(dtype).view(*shape)

        return {
            "logits": view(v.logits, torch.float32, (rows, v.ld)),
            "inds": view(v.inds, torch.int32, (rows, k)),
            "wts": view(v.wts, torch.float32, (rows, k)),
            "offsets": view(v.offsets, torch.int32, (E + 1,)),
            "row_map": view(v.row_map, torch.int32, (rows * k,)),
            "pos": view(v.pos, torch.int32, (rows * k,)),
            "h": view(v.h, torch.float16, (rows * k, self.I)),
            "yd": view(v.yd, torch.float16 if v.yd_dtype == capi.IQ_F16 else torch.float32, (rows * k, self.D)),
        }

    # ---- expert-parallel pieces (no counterpart in the single-GPU reference) ---------------------------------------
    def pack_rows(self, x: torch.Tensor, rows_f16: torch.Tensor, tokens: int, stream=None):
        """rows_f16[pos[pair]] = fp16(x[pair // top_k]) for the routing the `group` piece left in the scratch."""
        self.ctx.check(capi.lib().iq_moe_pack_rows(self._h, _stream_ptr(stream), x.data_ptr(), _dtype_id(x), x.stride(0),
                                                   tokens, self.workspace.data_ptr(), self.workspace.numel(),
                                                   rows_f16.data_ptr()))

    def experts_workspace_bytes(self, max_rows: int, sources: int) -> int:
        n = C.c_size_t()
        self.ctx.check(capi.lib().iq_moe_experts_workspace_bytes(self._h, max_rows, sources, C.byref(n)))
        return n.value

    def experts(self, rows_f16: torch.Tensor, total_rows: int, counts: torch.Tensor, sources: int, yd: torch.Tensor,
                workspace: torch.Tensor, region_rows: int = 0, yd_rows: Optional[torch.Tensor] = None, stream=None):
        """Gate/up/activation/down of this layer's own experts on received rows (source-major, expert order). yd_rows:
        int64 device tensor of one address per row; the outputs go there instead of into yd. counts: an int32 device
        tensor [sources, experts] or the device address of one."""
        self.ctx.check(capi.lib().iq_moe_experts(self._h, _stream_ptr(stream), rows_f16.data_ptr(), total_rows,
                                                 rows_f16.shape[0], counts.data_ptr() if hasattr(counts, "data_ptr") else int(counts),
                                                 sources, region_rows, yd.data_ptr(),
                                                 _dtype_id(yd), 0 if yd_rows is None else yd_rows.data_ptr(),
                                                 workspace.data_ptr(), workspace.numel()))

    def experts_indexed(self, rows_f16: torch.Tensor, row_index: torch.Tensor, total_rows: int, counts, yd: torch.Tensor,
                        workspace: torch.Tensor, yd_rows: Optional[torch.Tensor] = None, stream=None):
        """The same on rows left where they arrived: position i of the expert-major order is row row_index[i] of rows_f16
        (int32 device tensor); counts: per-expert totals, a device tensor [experts] or the device address of one."""
        self.ctx.check(capi.lib().iq_moe_experts_indexed(
            self._h, _stream_ptr(stream), rows_f16.data_ptr(), row_index.data_ptr(), total_rows, rows_f16.shape[0],
            counts.data_ptr() if hasattr(counts, "data_ptr") else int(counts), yd.data_ptr(), _dtype_id(yd),
            0 if yd_rows is None else yd_rows.data_ptr(), workspace.data_ptr(), workspace.numel()))

    def combine_rows(self, yd_rows: torch.Tensor, out: torch.Tensor, tokens: int, accumulate: bool = False, stream=None):
        self.ctx.check(capi.lib().iq_moe_combine_rows(self._h, _stream_ptr(stream), yd_rows.data_ptr(), _dtype_id(yd_rows),
                                                      tokens, out.data_ptr(), _dtype_id(out), out.stride(0),
                                                      capi.IQ_FLAG_ACCUMULATE if accumulate else 0,
                                                      self.workspace.data_ptr(), self.workspace.numel()))

    def close(self):
        if self._h:
            capi.lib().iq_moe_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# The reference keeps a separate prefill object that shares the layer's weights (PrefillMoE, MoEPrefill.swift:29);
# here the same layer serves any number of rows, so the name is an alias.
PrefillMoE = MoELayer
