"""ctypes binding of libingot_qmm.so (include/ingot_qmm.h). There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libingot_qmm.so")

IQ_F32, IQ_F16, IQ_BF16 = 0, 1, 2
IQ_MODE_AFFINE, IQ_MODE_MXFP4 = 0, 1
IQ_ACT_SILU, IQ_ACT_GELU, IQ_ACT_SWIGLU_OAI, IQ_ACT_RELU2 = 0, 1, 2, 3
IQ_ROUTER_BF16, IQ_ROUTER_Q8 = 0, 1
IQ_SCORE_SOFTMAX, IQ_SCORE_SIGMOID = 0, 1
IQ_SHARED_NONE, IQ_SHARED_GATED, IQ_SHARED_UNGATED = 0, 1, 2
IQ_FLAG_ACCUMULATE = 1
IQ_FLAG_NO_BARRIER = 2
IQ_PIECE_ROUTER, IQ_PIECE_ROUTE, IQ_PIECE_GROUP, IQ_PIECE_GATEUP, IQ_PIECE_DOWN, IQ_PIECE_COMBINE = 1, 2, 4, 8, 16, 32
IQ_PIECE_ALL = 63

# every symbol include/ingot_qmm.h declares (checked by the CPU test-suite against the built library)
SYMBOLS = [
    "iq_ctx_create", "iq_ctx_destroy", "iq_strerror", "iq_last_error", "iq_ctx_status", "iq_abi_version", "iq_qmv",
    "iq_qmm_workspace_bytes", "iq_qmm", "iq_dense_ffn_workspace_bytes", "iq_dense_ffn", "iq_moe_create",
    "iq_moe_destroy", "iq_moe_workspace_bytes", "iq_moe_forward", "iq_moe_route", "iq_moe_set_external_routing",
    "iq_moe_get_views", "iq_moe_pack_rows", "iq_moe_experts_workspace_bytes", "iq_moe_experts", "iq_moe_combine_rows",
    "iq_rmsnorm", "iq_qmm_noalloc", "iq_ep_create", "iq_ep_destroy", "iq_ep_share_counts", "iq_ep_barrier", "iq_ep_plan",
    "iq_ep_pack_push", "iq_ep_return_push", "iq_ep_return_rows", "iq_ep_compact",
    "iq_st_open", "iq_st_close", "iq_st_count", "iq_st_entry", "iq_st_find", "iq_st_last_error", "iq_widen4to8_words",
    "iq_scales_div16_bf16", "iq_argmax_rows", "iq_topk64_scratch_bytes", "iq_topk64", "iq_embed_rows",
    "iq_ctx_set_wait_cycles", "iq_colsplit_create", "iq_colsplit_destroy", "iq_linear_colsplit_workspace_bytes",
    "iq_linear_colsplit", "iq_had_rows", "iq_embed_rows_ternary", "iq_qmm_w8a8_workspace_bytes", "iq_qmm_w8a8",
    "iq_ep_index", "iq_moe_experts_indexed", "iq_ep_pack_push_tokens", "iq_ep_index_tokens",
]


class QLinear(C.Structure):
    _fields_ = [("w", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("n", C.c_int32), ("k", C.c_int32),
                ("bits", C.c_int32), ("group", C.c_int32), ("mode", C.c_int32), ("experts", C.c_int32)]


class MoeDesc(C.Structure):
    _fields_ = [("experts", C.c_int32), ("top_k", C.c_int32), ("d_model", C.c_int32), ("d_ff", C.c_int32),
                ("act", C.c_int32), ("act_limit", C.c_float), ("router_kind", C.c_int32), ("routed_scale", C.c_float),
                ("router_w", C.c_void_p), ("router_scales", C.c_void_p), ("router_biases", C.c_void_p),
                ("router_logit_bias", C.c_void_p), ("per_expert_scale", C.c_void_p),
                ("gate", QLinear), ("up", QLinear), ("down", QLinear),
                ("gate_bias", C.c_void_p), ("up_bias", C.c_void_p), ("down_bias", C.c_void_p),
                ("expert_lo", C.c_int32), ("expert_count", C.c_int32),
                ("router_score", C.c_int32), ("route_eps", C.c_float), ("router_select_bias", C.c_void_p),
                ("shared", C.c_int32), ("shared_gate_proj", QLinear), ("shared_up", QLinear), ("shared_down", QLinear),
                ("shared_gate", QLinear)]


class StTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_int32), ("rank", C.c_int32), ("shape", C.c_int64 * 8),
                ("file_offset", C.c_uint64), ("bytes", C.c_uint64), ("data", C.c_void_p)]


class MoeViews(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("ld", C.c_int32), ("inds", C.c_void_p), ("wts", C.c_void_p),
                ("offsets", C.c_void_p), ("row_map", C.c_void_p), ("pos", C.c_void_p), ("h", C.c_void_p),
                ("yd", C.c_void_p), ("yd_dtype", C.c_int32)]


class IngotError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"ingot_qmm status {status}: {message}")
        self.status = status


_lib = None


def lib() -> C.CDLL:
    """The loaded library. Raises if it has not been built (python -m ingot_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build the CUDA library with `python -m ingot_b200.build`; "
                               "there is no CPU path")
        l = C.CDLL(LIB_PATH)
        vp, i32, i64, u32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_size_t
        l.iq_ctx_create.argtypes = [i32, C.POINTER(vp)]
        l.iq_ctx_destroy.argtypes = [vp]
        l.iq_ctx_destroy.restype = None
        l.iq_strerror.argtypes = [i32]
        l.iq_strerror.restype = C.c_char_p
        l.iq_last_error.argtypes = [vp]
        l.iq_last_error.restype = C.c_char_p
        l.iq_abi_version.restype = i32
        l.iq_ctx_status.argtypes = [vp, C.POINTER(i32)]
        l.iq_ctx_status.restype = i32
        l.iq_qmv.argtypes = [vp, vp, vp, i32, i64, C.POINTER(QLinear), vp, i32, i64, i32, u32, i32]
        l.iq_qmm_workspace_bytes.argtypes = [vp, C.POINTER(QLinear), i32, i32, C.POINTER(sz)]
        l.iq_qmm.argtypes = [vp, vp, vp, i32, i64, C.POINTER(QLinear), vp, i32, i64, i32, u32, vp, sz]
        l.iq_dense_ffn_workspace_bytes.argtypes = [vp, C.POINTER(QLinear), C.POINTER(QLinear), i32, i32, C.POINTER(sz)]
        l.iq_dense_ffn.argtypes = [vp, vp, vp, i32, i64, C.POINTER(QLinear), C.POINTER(QLinear), i32, C.c_float, vp,
                                   i32, i64, i32, u32, vp, sz]
        l.iq_moe_create.argtypes = [vp, C.POINTER(MoeDesc), C.POINTER(vp)]
        l.iq_moe_destroy.argtypes = [vp]
        l.iq_moe_destroy.restype = None
        l.iq_moe_workspace_bytes.argtypes = [vp, i32, C.POINTER(sz)]
        l.iq_moe_forward.argtypes = [vp, vp, vp, i32, i64, vp, i32, i64, i32, u32, u32, vp, sz]
        l.iq_moe_route.argtypes = [vp, vp, vp, i32, i32, vp, vp]
        l.iq_moe_set_external_routing.argtypes = [vp, vp, vp]
        l.iq_moe_get_views.argtypes = [vp, vp, i32, C.POINTER(MoeViews)]
        l.iq_qmm_noalloc.argtypes = [vp, vp, vp, i32, i64, C.POINTER(QLinear), vp, i32, i64, i32, u32]
        l.iq_qmm_noalloc.restype = i32
        l.iq_argmax_rows.argtypes = [vp, vp, vp, i64, i32, i32, vp]
        l.iq_topk64_scratch_bytes.argtypes = [i32, i32, C.POINTER(sz)]
        l.iq_topk64.argtypes = [vp, vp, vp, i64, i32, i32, C.POINTER(C.c_float), i32, vp, vp, vp, vp, sz]
        l.iq_embed_rows.argtypes = [vp, vp, C.POINTER(QLinear), vp, i32, vp, vp, i64]
        for name in ("iq_argmax_rows", "iq_topk64_scratch_bytes", "iq_topk64", "iq_embed_rows"):
            getattr(l, name).restype = i32
        l.iq_st_open.argtypes = [C.c_char_p, C.POINTER(vp)]
        l.iq_st_close.argtypes = [vp]
        l.iq_st_close.restype = None
        l.iq_st_count.argtypes = [vp]
        l.iq_st_entry.argtypes = [vp, i32, C.POINTER(StTensor)]
        l.iq_st_find.argtypes = [vp, C.c_char_p, C.POINTER(StTensor)]
        l.iq_st_last_error.argtypes = []
        l.iq_st_last_error.restype = C.c_char_p
        l.iq_widen4to8_words.argtypes = [vp, vp, sz]
        l.iq_widen4to8_words.restype = None
        l.iq_scales_div16_bf16.argtypes = [vp, vp, sz]
        l.iq_scales_div16_bf16.restype = None
        for name in ("iq_st_open", "iq_st_count", "iq_st_entry", "iq_st_find"):
            getattr(l, name).restype = i32
        l.iq_ep_create.argtypes = [vp, i32, i32, i32, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]
        l.iq_ep_destroy.argtypes = [vp]
        l.iq_ep_destroy.restype = None
        l.iq_ep_share_counts.argtypes = [vp, vp, vp]
        l.iq_ep_barrier.argtypes = [vp, vp, i32]
        l.iq_ep_plan.argtypes = [vp, vp]
        l.iq_ep_pack_push.argtypes = [vp, vp, vp, i32, i64, i32, i32, i32, vp, vp, vp]
        l.iq_ep_return_push.argtypes = [vp, vp, vp, i32, i32]
        l.iq_ep_return_rows.argtypes = [vp, vp, i32, i32, vp]
        l.iq_ep_compact.argtypes = [vp, vp, vp, i32, i32, vp, vp, C.POINTER(vp)]
        for name in ("iq_ep_create", "iq_ep_share_counts", "iq_ep_barrier", "iq_ep_plan", "iq_ep_pack_push",
                     "iq_ep_return_push", "iq_ep_return_rows", "iq_ep_compact"):
            getattr(l, name).restype = i32
        l.iq_ctx_set_wait_cycles.argtypes = [vp, C.c_uint64]
        l.iq_colsplit_create.argtypes = [vp, i32, i32, i32, i32, i32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]
        l.iq_colsplit_destroy.argtypes = [vp]
        l.iq_colsplit_destroy.restype = None
        l.iq_linear_colsplit_workspace_bytes.argtypes = [vp, C.POINTER(QLinear), i32, i32, C.POINTER(sz)]
        l.iq_linear_colsplit.argtypes = [vp, vp, vp, i32, i64, C.POINTER(QLinear), i32, u32, vp, sz]
        for name in ("iq_ctx_set_wait_cycles", "iq_colsplit_create", "iq_linear_colsplit_workspace_bytes",
                     "iq_linear_colsplit"):
            getattr(l, name).restype = i32
        l.iq_had_rows.argtypes = [vp, vp, vp, i32, i64, vp, vp, i64, i32, i32]
        l.iq_embed_rows_ternary.argtypes = [vp, vp, C.POINTER(QLinear), vp, vp, i32, vp, vp, i64]
        l.iq_qmm_w8a8_workspace_bytes.argtypes = [vp, C.POINTER(QLinear), i32, C.POINTER(sz)]
        l.iq_qmm_w8a8.argtypes = [vp, vp, vp, i32, i64, C.POINTER(QLinear), vp, i32, i64, i32, u32, vp, sz]
        l.iq_qmm_w8a8_workspace_bytes.restype = i32
        l.iq_qmm_w8a8.restype = i32
        l.iq_ep_index.argtypes = [vp, vp, i32, i32, vp, vp, C.POINTER(vp)]
        l.iq_moe_experts_indexed.argtypes = [vp, vp, vp, vp, i32, i32, vp, vp, i32, vp, vp, sz]
        l.iq_ep_index.restype = i32
        l.iq_ep_pack_push_tokens.argtypes = [vp, vp, vp, i32, i64, i32, i32, i32, vp, vp, vp, i32]
        l.iq_ep_index_tokens.argtypes = [vp, vp, i32, i32, i32, vp, vp, C.POINTER(vp)]
        l.iq_ep_pack_push_tokens.restype = i32
        l.iq_ep_index_tokens.restype = i32
        l.iq_moe_experts_indexed.restype = i32
        l.iq_had_rows.restype = i32
        l.iq_embed_rows_ternary.restype = i32
        l.iq_moe_pack_rows.argtypes = [vp, vp, vp, i32, i64, i32, vp, sz, vp]
        l.iq_moe_experts_workspace_bytes.argtypes = [vp, i32, i32, C.POINTER(sz)]
        l.iq_moe_experts.argtypes = [vp, vp, vp, i32, i32, vp, i32, i32, vp, i32, vp, vp, sz]
        l.iq_moe_combine_rows.argtypes = [vp, vp, vp, i32, i32, vp, i32, i64, u32, vp, sz]
        l.iq_rmsnorm.argtypes = [vp, vp, vp, i64, vp, i32, i64, i32, i32, C.c_float]
        for name in ("iq_moe_pack_rows", "iq_moe_experts_workspace_bytes", "iq_moe_experts", "iq_moe_combine_rows",
                     "iq_rmsnorm"):
            getattr(l, name).restype = i32
        for name in ("iq_ctx_create", "iq_qmv", "iq_qmm_workspace_bytes", "iq_qmm", "iq_dense_ffn_workspace_bytes",
                     "iq_dense_ffn", "iq_moe_create", "iq_moe_workspace_bytes", "iq_moe_forward", "iq_moe_route",
                     "iq_moe_set_external_routing", "iq_moe_get_views"):
            getattr(l, name).restype = i32
        _lib = l
    return _lib


class Context:
    """One device context (iq_ctx). Mirrors the reference's MetalContext role: device + kernel configuration."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        st = lib().iq_ctx_create(device, C.byref(self._h))
        if st != 0:
            raise IngotError(st, lib().iq_strerror(st).decode() + f" (iq_ctx_create on device {device})")
        self.device = device

    @property
    def handle(self):
        return self._h

    def check(self, status: int):
        if status != 0:
            raise IngotError(status, lib().iq_last_error(self._h).decode())

    def device_status(self) -> int:
        """Synchronises the device and returns (and clears) the kernels' status word: 0 unless a bounded wait gave up."""
        v = C.c_int32(0)
        self.check(lib().iq_ctx_status(self._h, C.byref(v)))
        return v.value

    def set_wait_cycles(self, cycles: int):
        """Bound of the waits on another GPU, in SM clock cycles (iq_ctx_set_wait_cycles)."""
        self.check(lib().iq_ctx_set_wait_cycles(self._h, cycles))

    def close(self):
        if self._h:
            lib().iq_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_contexts = {}


def context(device: int = 0) -> Context:
    if device not in _contexts:
        _contexts[device] = Context(device)
    return _contexts[device]
