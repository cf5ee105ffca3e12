"""Host-side mirror of the reference's quantized-linear operators (Sources/Ingot/Layers/Linear.swift, Dense.swift).

`DenseQ` is the device container (three buffers + N, K, bits, group size, Linear.swift:17-33); `VQMV.encode` is the
decode GEMV launcher (Linear.swift:287-444); `DenseQ.encode_qmm_f32` the prefill GEMM launcher (Linear.swift:688-713);
`DenseMLP` the gated FFN (Dense.swift:9-96). Where the reference encodes a Metal dispatch onto a command encoder,
these enqueue CUDA kernels of libingot_qmm.so on a CUDA stream through the C ABI. torch is used for device memory and
streams only. There is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import capi

_DT = {torch.float32: capi.IQ_F32, torch.float16: capi.IQ_F16, torch.bfloat16: capi.IQ_BF16}


def _dtype_id(t: torch.Tensor) -> int:
    if t.dtype not in _DT:
        raise TypeError(f"unsupported element type {t.dtype} (float32, float16, bfloat16)")
    return _DT[t.dtype]


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def _need_cuda(*ts: torch.Tensor):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("tensors must live on a CUDA device: the operators have no CPU path")


class DenseQ:
    """A quantized matrix on the device in MLX layout (Linear.swift:17-33; Loader/Quant.swift:4-12).

    w: int32/uint32 tensor [experts?, N, K*bits/32] holding the packed codes; scales/biases bf16 [.., N, K/group]
    (affine) or scales uint8 [.., N, K/32] (mxfp4, biases None)."""

    def __init__(self, w: torch.Tensor, scales: torch.Tensor, biases: Optional[torch.Tensor], N: int, K: int, bits: int,
                 gs: int = 64, mode: str = "affine", experts: int = 1):
        self.had, self._rot = None, None
        if bits == 16:
            # a plain bf16 table (an unquantized embedding, Linear.swift:58-63): only encode_embed takes it
            _need_cuda(w)
            if w.dtype != torch.bfloat16 or w.numel() != N * K or scales is not None or biases is not None:
                raise ValueError("a 16-bit table is bf16 [N, K] without scales or biases")
            self.w, self.s, self.b = w.contiguous(), None, None
            self.N, self.K, self.bits, self.gs, self.mode, self.experts = N, K, 16, 64, "affine", 1
            return
        if bits == 2:
            # the rotated ternary format (xc_tern.metal): 2-bit codes, groups of 128, fp16 scales, w = (q - 1) * s
            _need_cuda(w, scales)
            if gs != 128 or mode != "affine" or scales.dtype != torch.float16 or experts != 1:
                raise ValueError("a 2-bit layer is ternary: groups of 128, fp16 scales, one matrix")
            if w.dtype not in (torch.int32, torch.uint32) or w.numel() != N * K // 16 or scales.numel() != N * (K // 128):
                raise ValueError(f"bits do not add up (packed {tuple(w.shape)}, N {N}, K {K}, 2 bits)")
            self.w, self.s, self.b = w.contiguous(), scales.contiguous(), None
            self.N, self.K, self.bits, self.gs, self.mode, self.experts = N, K, 2, 128, "affine", 1
            return
        _need_cuda(w, scales, biases)
        if mode not in ("affine", "mxfp4"):
            raise ValueError(f"quantization mode «{mode}» not supported (affine and mxfp4)")
        if w.dtype not in (torch.int32, torch.uint32):
            raise TypeError("packed codes must be 32-bit words")
        words = K * bits // 32
        if w.numel() != experts * N * words:
            raise ValueError(f"bits do not add up (packed {tuple(w.shape)}, N {N}, K {K}, bits {bits})")
        if mode == "mxfp4":
            if bits != 4 or gs != 32 or scales.dtype != torch.uint8 or biases is not None:
                raise ValueError("not an MLX mxfp4 layer (4 bits g32, uint8 scales, no biases)")
        else:
            if scales.dtype != torch.bfloat16 or biases is None or biases.dtype != torch.bfloat16:
                raise ValueError("affine scales/biases must be bf16")
            if biases.numel() != scales.numel():
                raise ValueError("scales and biases differ in shape")
        if scales.numel() != experts * N * (K // gs):
            raise ValueError(f"scales shape {tuple(scales.shape)} does not match N {N}, K {K}, group {gs}")
        self.w, self.s, self.b = w.contiguous(), scales.contiguous(), None if biases is None else biases.contiguous()
        self.N, self.K, self.bits, self.gs, self.mode, self.experts = N, K, bits, gs, mode, experts

    def qlinear(self) -> capi.QLinear:
        return capi.QLinear(self.w.data_ptr(), 0 if self.s is None else self.s.data_ptr(),
                            0 if self.b is None else self.b.data_ptr(), self.N,
                            self.K, self.bits, self.gs, capi.IQ_MODE_MXFP4 if self.mode == "mxfp4" else capi.IQ_MODE_AFFINE,
                            self.experts)

    @property
    def device_index(self) -> int:
        return self.w.device.index or 0

    def weight_bytes(self) -> int:
        """Bytes of codes + scales + biases (what one pass over the matrix reads)."""
        n = self.w.numel() * self.w.element_size() + (0 if self.s is None else self.s.numel() * self.s.element_size())
        return n + (0 if self.b is None else self.b.numel() * 2)

    # ---- input rotation of the ternary format (Linear.swift encodeRotate; had_rows_h, xc_tern.metal:29-40) ------
    def set_hadamard(self, signs: torch.Tensor):
        """Signs (float32 [K], +1 / -1) of the rotation x <- H_1024(x * signs) / 32 that precedes this matrix."""
        _need_cuda(signs)
        if signs.dtype != torch.float32 or signs.numel() != self.K or self.K % 1024 != 0:
            raise ValueError("the rotation's signs are float32 [K], K a multiple of 1024")
        self.had = signs.contiguous()

    def encode_rotate(self, x: torch.Tensor, rows: int, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
        """x[rows, K] rotated into a float16 scratch (grown on demand, like the reference's rotation buffer)."""
        if self._rot is None or self._rot.shape[0] < rows:
            self._rot = torch.empty(max(rows, 16), self.K, dtype=torch.float16, device=self.w.device)
        ctx = capi.context(self.device_index)
        ctx.check(capi.lib().iq_had_rows(ctx.handle, _stream_ptr(stream), x.data_ptr(), _dtype_id(x), x.stride(0),
                                         self.had.data_ptr(), self._rot.data_ptr(), self.K, rows, self.K))
        return self._rot

    # ---- embedding (Linear.swift:65-93) -------------------------------------------------------------------------
    def encode_embed(self, tok: torch.Tensor, rows: int, out_f: Optional[torch.Tensor] = None,
                     out_h: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None):
        """Rows tok[r] of the table, dequantised, into out_f (float32 [rows, >=K]) and / or out_h (float16): affine
        4-bit (groups of 64 or 32), 8-bit, or a bf16 table. tok is an int32/uint32 device tensor."""
        _need_cuda(tok, out_f, out_h)
        if tok.dtype not in (torch.int32, torch.uint32) or tok.numel() < rows:
            raise TypeError("tokens are 32-bit integers, one per row")
        if out_f is None and out_h is None:
            raise ValueError("one of out_f, out_h is needed")
        if (out_f is not None and out_f.dtype != torch.float32) or (out_h is not None and out_h.dtype != torch.float16):
            raise TypeError("out_f is float32, out_h float16")
        if out_f is not None and out_h is not None and out_f.stride(0) != out_h.stride(0):
            raise ValueError("out_f and out_h share one row stride")
        o = out_f if out_f is not None else out_h
        ctx = capi.context(self.device_index)
        q = self.qlinear()
        if self.bits == 2:  # ternary table: dequantise, then the inverse rotation (embed_rows_t, xc_tern.metal:44-65)
            if self.had is None:
                raise ValueError("a ternary table needs the rotation's signs (set_hadamard)")
            ctx.check(capi.lib().iq_embed_rows_ternary(ctx.handle, _stream_ptr(stream), C.byref(q), self.had.data_ptr(),
                                                       tok.data_ptr(), rows, 0 if out_f is None else out_f.data_ptr(),
                                                       0 if out_h is None else out_h.data_ptr(), o.stride(0)))
            return
        ctx.check(capi.lib().iq_embed_rows(ctx.handle, _stream_ptr(stream), C.byref(q), tok.data_ptr(), rows,
                                           0 if out_f is None else out_f.data_ptr(),
                                           0 if out_h is None else out_h.data_ptr(), o.stride(0)))

    # ---- prefill GEMM (Linear.swift:688-713) --------------------------------------------------------------------
    def qmm_workspace_bytes(self, rows: int, x_dtype: torch.dtype) -> int:
        ctx = capi.context(self.device_index)
        n = C.c_size_t()
        ql = self.qlinear()
        ctx.check(capi.lib().iq_qmm_workspace_bytes(ctx.handle, C.byref(ql), rows, _DT[x_dtype], C.byref(n)))
        return n.value

    def encode_qmm_f32(self, x: torch.Tensor, y: torch.Tensor, rows: int, accumulate: bool = False,
                       workspace: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None):
        """Y[rows, N] (+)= X[rows, K] · Wᵀ on the tensor cores. y may be float32 (the reference's default), float16
        (`halfOut`) or bfloat16. rows must be a multiple of 64 (Linear.swift:695)."""
        _need_cuda(x, y)
        ctx = capi.context(self.device_index)
        ql = self.qlinear()
        if self.had is not None:  # rotated basis: the rotation runs first, as in the reference's launcher
            x = self.encode_rotate(x, rows, stream)
        ws_ptr, ws_bytes = (0, 0) if workspace is None else (workspace.data_ptr(), workspace.numel() * workspace.element_size())
        ctx.check(capi.lib().iq_qmm(ctx.handle, _stream_ptr(stream), x.data_ptr(), _dtype_id(x), x.stride(0), C.byref(ql),
                                    y.data_ptr(), _dtype_id(y), y.stride(0), rows,
                                    capi.IQ_FLAG_ACCUMULATE if accumulate else 0, ws_ptr, ws_bytes))

    def encode_qmm_i8(self, x: torch.Tensor, y: torch.Tensor, rows: int, accumulate: bool = False,
                      scratch: Optional[torch.Tensor] = None, stream: Optional[torch.cuda.Stream] = None):
        """Y[rows, N] (+)= X · Wᵀ in rotated W8A8 (lossy; DenseQ.encodeQmmI8, Dense.swift:131-172): 4-bit weights and
        activations rotated along K, int8 per row, the product on the int8 tensor cores. `scratch` plays the reference's
        DenseI8Scratch (sized by `qmm_i8_scratch_bytes`; allocated here when absent). A ternary matrix takes the
        reference's encodeQmmI8T (Dense.swift:174-212): the format's own input rotation first, then int8 rows and the
        weights as int8 with one scale per row."""
        _need_cuda(x, y)
        ctx = capi.context(self.device_index)
        ql = self.qlinear()
        if self.bits == 2 and self.had is not None:
            x = self.encode_rotate(x, rows, stream)
        if scratch is None:
            scratch = torch.empty(self.qmm_i8_scratch_bytes(rows), dtype=torch.uint8, device=self.w.device)
        ctx.check(capi.lib().iq_qmm_w8a8(ctx.handle, _stream_ptr(stream), x.data_ptr(), _dtype_id(x), x.stride(0), C.byref(ql),
                                         y.data_ptr(), _dtype_id(y), y.stride(0), rows,
                                         capi.IQ_FLAG_ACCUMULATE if accumulate else 0, scratch.data_ptr(), scratch.numel()))

    def qmm_i8_scratch_bytes(self, rows: int) -> int:
        ctx = capi.context(self.device_index)
        n = C.c_size_t()
        ql = self.qlinear()
        ctx.check(capi.lib().iq_qmm_w8a8_workspace_bytes(ctx.handle, C.byref(ql), rows, C.byref(n)))
        return n.value

    def encode_qmm_noalloc(self, x: torch.Tensor, y: torch.Tensor, rows: int, accumulate: bool = False,
                           stream: Optional[torch.cuda.Stream] = None):
        """The prefill GEMM for callers that may not allocate device memory (a plugin inside an engine that owns the
        memory pool, a sealed pool, a no-allocation rule): same results as `encode_qmm_f32`, with the fp16 copy of
        bf16/fp32 activations kept in an 8 MiB array built into the library. rows * K must not exceed 4,194,304; calls
        that may overlap on the GPU share that array and must be ordered on one stream; make the first call on a device
        outside any stream capture."""
        _need_cuda(x, y)
        ctx = capi.context(self.device_index)
        ql = self.qlinear()
        ctx.check(capi.lib().iq_qmm_noalloc(ctx.handle, _stream_ptr(stream), x.data_ptr(), _dtype_id(x), x.stride(0),
                                            C.byref(ql), y.data_ptr(), _dtype_id(y), y.stride(0), rows,
                                            capi.IQ_FLAG_ACCUMULATE if accumulate else 0))


class VQMV:
    """Decode GEMV launcher (Linear.swift:287-444)."""

    MAX_ROWS = 16

    @staticmethod
    def encode(x: torch.Tensor, m: DenseQ, y: torch.Tensor, rows: int, ldx: Optional[int] = None,
               ldy: Optional[int] = None, accumulate: bool = False, n_prefix: Optional[int] = None,
               stream: Optional[torch.cuda.Stream] = None):
        """Y[rows, N] (+)= X[rows, K] · Wᵀ, rows ≤ 16. `ldx`/`ldy` are row strides in elements (default: the tensors'),
        `n_prefix` computes only the first rows of W (Linear.swift:350-366)."""
        _need_cuda(x, y)
        ctx = capi.context(m.device_index)
        ql = m.qlinear()
        if m.had is not None:  # Linear.swift:292-297: the input rotation first, then the kernel on the rotated rows
            x, ldx = m.encode_rotate(x, rows, stream), m.K
        ctx.check(capi.lib().iq_qmv(ctx.handle, _stream_ptr(stream), x.data_ptr(), _dtype_id(x),
                                    ldx if ldx is not None else (x.stride(0) if x.dim() > 1 else m.K), C.byref(ql),
                                    y.data_ptr(), _dtype_id(y),
                                    ldy if ldy is not None else (y.stride(0) if y.dim() > 1 else m.N), rows,
                                    capi.IQ_FLAG_ACCUMULATE if accumulate else 0, n_prefix or 0))


class DenseMLP:
    """Dense gated FFN with gate|up concatenated by rows ([2·I, D], gate rows first; Dense.swift:4-6,21-49)."""

    def __init__(self, gate_up: DenseQ, down: DenseQ, act: str = "silu", limit: float = 7.0):
        if gate_up.N % 2 or gate_up.N // 2 != down.K or gate_up.K != down.N:
            raise ValueError("gate|up and down do not chain")
        self.gate_up, self.down = gate_up, down
        self.act = {"silu": capi.IQ_ACT_SILU, "gelu": capi.IQ_ACT_GELU, "swiglu_oai": capi.IQ_ACT_SWIGLU_OAI,
                    "relu2": capi.IQ_ACT_RELU2}[act]
        self.limit = limit
        self._ws = None

    def _workspace(self, rows: int, x_dtype: torch.dtype) -> torch.Tensor:
        ctx = capi.context(self.gate_up.device_index)
        n = C.c_size_t()
        a, b = self.gate_up.qlinear(), self.down.qlinear()
        ctx.check(capi.lib().iq_dense_ffn_workspace_bytes(ctx.handle, C.byref(a), C.byref(b), rows, _DT[x_dtype], C.byref(n)))
        if self._ws is None or self._ws.numel() < n.value:
            self._ws = torch.empty(max(n.value, 256), dtype=torch.uint8, device=self.gate_up.w.device)
        return self._ws

    def encode(self, x: torch.Tensor, out: torch.Tensor, rows: int, accumulate: bool = False,
               stream: Optional[torch.cuda.Stream] = None):
        """out[rows, D] (+)= down(act(gate x)·up x) (Dense.swift:56-96). rows ≤ 16 runs the GEMV kernels, larger
        multiples of 64 the GEMM kernels. Scratch is sized on first use and reused."""
        _need_cuda(x, out)
        ctx = capi.context(self.gate_up.device_index)
        ws = self._workspace(rows, x.dtype)
        a, b = self.gate_up.qlinear(), self.down.qlinear()
        ctx.check(capi.lib().iq_dense_ffn(ctx.handle, _stream_ptr(stream), x.data_ptr(), _dtype_id(x), x.stride(0),
                                          C.byref(a), C.byref(b), self.act, self.limit, out.data_ptr(), _dtype_id(out),
                                          out.stride(0), rows, capi.IQ_FLAG_ACCUMULATE if accumulate else 0,
                                          ws.data_ptr(), ws.numel()))
