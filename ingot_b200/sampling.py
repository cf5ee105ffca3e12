"""What follows the lm_head GEMV on the decode path: arg-max per row and the sampler's 64 candidates per row
(argmax_rows, Shaders/verify.metal:525-547; TopK64, Shaders/zz_sample.metal and Tests/IngotTests/TopK64Tests.swift)."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import capi
from .linear import _need_cuda, _stream_ptr

CANDIDATES = 64


def argmax_rows(x: torch.Tensor, rows: int, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Index of the largest logit of each of the first `rows` rows of x (fp32 [*, n]); ties go to the lower index."""
    _need_cuda(x)
    if x.dtype != torch.float32:
        raise TypeError("logits are float32")
    ctx = capi.context(x.device.index or 0)
    out = torch.empty(rows, dtype=torch.int32, device=x.device)
    ctx.check(capi.lib().iq_argmax_rows(ctx.handle, _stream_ptr(stream), x.data_ptr(), x.stride(0), rows, x.shape[1],
                                        out.data_ptr()))
    return out


class TopK64:
    """Scratch sized once for (rows, vocabulary); `encode` enqueues the two kernels."""

    def __init__(self, max_rows: int, vocab: int, device: torch.device):
        n = C.c_size_t()
        if capi.lib().iq_topk64_scratch_bytes(max_rows, vocab, C.byref(n)) != 0:
            raise ValueError("TopK64 takes 1..16 rows and up to 262,144 logits per row")
        self.max_rows, self.vocab = max_rows, vocab
        self.scratch = torch.empty(n.value, dtype=torch.uint8, device=device)
        self.ctx = capi.context(device.index or 0)

    def encode(self, x: torch.Tensor, rows: int, temperatures: Sequence[float], stream: Optional[torch.cuda.Stream] = None):
        """Returns (idx int32 [rows, 64], val float32 [rows, 64], z float32 [rows, 2] = (max, sum exp((x - max) / T)))."""
        _need_cuda(x)
        if x.dtype != torch.float32 or rows > self.max_rows or x.shape[1] != self.vocab:
            raise ValueError("TopK64: float32 logits [rows <= max_rows, vocab]")
        idx = torch.empty(rows, CANDIDATES, dtype=torch.int32, device=x.device)
        val = torch.empty(rows, CANDIDATES, dtype=torch.float32, device=x.device)
        z = torch.empty(rows, 2, dtype=torch.float32, device=x.device)
        t = (C.c_float * len(temperatures))(*temperatures)
        self.ctx.check(capi.lib().iq_topk64(self.ctx.handle, _stream_ptr(stream), x.data_ptr(), x.stride(0), rows, self.vocab, t,
                                            len(temperatures), idx.data_ptr(), val.data_ptr(), z.data_ptr(),
                                            self.scratch.data_ptr(), self.scratch.numel()))
        return idx, val, z
