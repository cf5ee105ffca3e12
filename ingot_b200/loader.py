"""MLX safetensors checkpoints -> the device layouts the kernels read, with no conversion step.

Host-side mirror of the reference's loader:
  SafetensorsStore   Loader/Safetensors.swift:86-148 (shards, index.json, tensor table), :213-247 (layerPrefix)
  ModelConfig        Loader/Config.swift:96-118 (quantization default + per-path overrides from config.json)
  QuantizedLinear    Loader/Quant.swift:13-88 (shapes -> bits / group size / experts, checked against the config)
  dense_q            Layers/Linear.swift:104-183 (row concatenation of matrices sharing K, lossless 4 -> 8-bit widening
                     of the 4-bit pieces of a mixed concatenation, zero rows up to a multiple of pad_to)
  stacked_experts    Layers/Linear.swift:17-33 + Loader/Quant.swift:205-231 (stacked expert tensors as they are)
The file mapping, the header parse and the byte transforms are native (csrc/loader.cu behind iq_st_* / iq_widen4to8_words);
everything here is shapes and rules. Host arrays are numpy views into the mappings; `to_device` uploads with torch.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import capi

DTYPES = {capi_id: name for capi_id, name in enumerate(["BF16", "F16", "F32", "U32", "I32", "U8"])}
DTYPE_SIZE = {"BF16": 2, "F16": 2, "F32": 4, "U32": 4, "I32": 4, "U8": 1}
NP_VIEW = {"BF16": np.uint16, "F16": np.float16, "F32": np.float32, "U32": np.uint32, "I32": np.int32, "U8": np.uint8}

# Parts of a pack the engine never loads (Safetensors.swift:213-219)
SKIPPED_PARTS = ["mtp", "visual", "vision_tower", "audio_tower", "embed_vision", "embed_audio", "vision_embedder",
                 "multi_modal_projector", "vision_adapter", "vision_projection"]


class SafetensorsError(RuntimeError):
    """kind: 'io', 'format' or 'missing' (SafetensorsError, Safetensors.swift:35-44)."""

    def __init__(self, kind: str, message: str):
        super().__init__(message)
        self.kind = kind


def _raise(status: int):
    msg = capi.lib().iq_st_last_error().decode()
    kind = {-8: "io", -9: "format", -10: "missing"}.get(status, "format")
    raise SafetensorsError(kind, msg)


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    shard: int
    file_offset: int
    byte_count: int
    address: int  # of the bytes inside the mapping

    @property
    def count(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


class SafetensorsStore:
    """One or several shards of a directory (model.safetensors.index.json names them; else model.safetensors)."""

    def __init__(self, directory: str):
        self.directory = directory
        index = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                obj = json.load(f)
            if not isinstance(obj, dict) or not isinstance(obj.get("weight_map"), dict):
                raise SafetensorsError("format", "index.json without weight_map")
            names = sorted(set(obj["weight_map"].values()))
        else:
            names = ["model.safetensors"]
        self._files: List[C.c_void_p] = []
        self.tensors: Dict[str, TensorInfo] = {}
        lib = capi.lib()
        try:
            for shard, name in enumerate(names):
                h = C.c_void_p()
                st = lib.iq_st_open(os.path.join(directory, name).encode(), C.byref(h))
                if st != 0:
                    _raise(st)
                self._files.append(h)
                t = capi.StTensor()
                for i in range(lib.iq_st_count(h)):
                    lib.iq_st_entry(h, i, C.byref(t))
                    self.tensors[t.name.decode()] = TensorInfo(
                        t.name.decode(), DTYPES[t.dtype], tuple(t.shape[j] for j in range(t.rank)), shard, t.file_offset,
                        t.bytes, t.data or 0)
        except Exception:
            self.close()
            raise

    def close(self):
        for h in self._files:
            capi.lib().iq_st_close(h)
        self._files = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def info(self, name: str) -> TensorInfo:
        t = self.tensors.get(name)
        if t is None:
            raise SafetensorsError("missing", f"no such tensor {name}")
        return t

    def bytes(self, t: TensorInfo) -> np.ndarray:
        """The tensor's bytes inside the mapping (uint8, read-only view, possibly unaligned; valid while the store lives)."""
        if t.byte_count == 0:
            return np.zeros(0, dtype=np.uint8)
        buf = (C.c_ubyte * t.byte_count).from_address(t.address)
        a = np.frombuffer(buf, dtype=np.uint8)
        a.flags.writeable = False
        return a

    def array(self, t: TensorInfo) -> np.ndarray:
        """A copy of the tensor as a numpy array of its element type (bf16 as uint16 bit patterns)."""
        return self.bytes(t).copy().view(NP_VIEW[t.dtype]).reshape(t.shape)

    def alignment(self, t: TensorInfo) -> int:
        a = t.address
        return min(a & -a, 4096) if a else 4096

    @staticmethod
    def is_skipped(name: str) -> bool:
        return any(p in name for p in SKIPPED_PARTS)

    @staticmethod
    def preferred_prefix(cands) -> Optional[str]:
        """Under `language_model` first, then the shortest, then the first in lexicographic order."""
        cands = list(cands)
        if not cands:
            return None
        return min(cands, key=lambda s: (0 if "language_model" in s else 1, len(s), s))

    def layer_prefix(self, layer: int) -> str:
        key = f"layers.{layer}."
        cands = set()
        for name in self.tensors:
            i = name.find(key)
            if i >= 0 and not self.is_skipped(name):
                cands.add(name[: i + len(key)])
        p = self.preferred_prefix(cands)
        if p is None:
            raise SafetensorsError("missing", f"no such tensor layer {layer}")
        return p


@dataclass(frozen=True)
class QuantParams:
    bits: int
    group_size: int
    mode: str = "affine"


class ModelConfig:
    """The quantization part of config.json: a default and per-path overrides (Config.swift:96-118). An override
    without `mode` is affine: it does not inherit the default's mode."""

    def __init__(self, obj: dict):
        q = obj.get("quantization")
        if not isinstance(q, dict):
            q = obj.get("quantization_config") if isinstance(obj.get("quantization_config"), dict) else None
        self.quant_default: Optional[QuantParams] = None
        self.quant_overrides: Dict[str, QuantParams] = {}
        if q:
            if isinstance(q.get("bits"), int) and isinstance(q.get("group_size"), int):
                self.quant_default = QuantParams(q["bits"], q["group_size"], q.get("mode") or "affine")
            for k, v in q.items():
                if isinstance(v, dict) and isinstance(v.get("bits"), int) and isinstance(v.get("group_size"), int):
                    self.quant_overrides[k] = QuantParams(v["bits"], v["group_size"], v.get("mode") or "affine")

    @classmethod
    def from_file(cls, path: str) -> "ModelConfig":
        with open(path) as f:
            return cls(json.load(f))

    def quant(self, path: str) -> Optional[QuantParams]:
        return self.quant_overrides.get(path, self.quant_default)


class QuantizedLinear:
    """An MLX quantized layer of the store: the bits are deduced from the shapes and checked against the config."""

    def __init__(self, store: SafetensorsStore, path: str, config: Optional[ModelConfig], mxfp4: bool = False):
        self.path = path
        self.weight = store.info(path + ".weight")
        self.scales = store.info(path + ".scales")
        self.biases = store.tensors.get(path + ".biases")
        w, s = self.weight, self.scales
        if w.dtype != "U32" or len(w.shape) < 2 or len(s.shape) != len(w.shape):
            raise SafetensorsError("format", f"{path} does not look like an MLX quantized layer")
        packed, groups = w.shape[-1], s.shape[-1]
        self.out_features = w.shape[-2]
        self.experts = 1
        for d in w.shape[:-2]:
            self.experts *= d
        declared = config.quant(path) if config is not None else None
        if declared is not None and declared.mode != "affine" and not (declared.mode == "mxfp4" and mxfp4):
            extra = "; MXFP4 runs only in the MoE experts)" if declared.mode == "mxfp4" else ")"
            raise SafetensorsError("format", f"{path}: quantization mode «{declared.mode}» not supported (affine only{extra}")
        if declared is not None and declared.mode == "mxfp4":
            self.in_features = groups * 32
            if not (declared.bits == 4 and declared.group_size == 32 and packed * 8 == self.in_features and
                    s.dtype == "U8" and self.biases is None):
                raise SafetensorsError("format", f"{path}: not an MLX mxfp4 layer (4 bits g32, uint8 scales, no biases; "
                                                 f"packed {packed}, groups {groups}, scales {s.dtype})")
            self.params = QuantParams(4, 32, "mxfp4")
            return
        gs = declared.group_size if declared is not None else 64
        self.in_features = groups * gs
        bits = packed * 32 // self.in_features if self.in_features else 0
        if self.in_features == 0 or packed * 32 != bits * self.in_features or bits not in (2, 3, 4, 5, 6, 8):
            raise SafetensorsError("format", f"{path}: bits do not add up (packed {packed}, groups {groups})")
        if declared is not None and declared.bits != bits:
            raise SafetensorsError("format", f"{path}: config says {declared.bits} bits, the shapes say {bits}")
        self.params = QuantParams(bits, gs)

    @property
    def is_mxfp4(self) -> bool:
        return self.params.mode == "mxfp4"


@dataclass
class HostDenseQ:
    """Row-major host arrays of one dense quantized matrix, ready to upload: w uint32 [N, K*bits/32], s / b bf16 bit
    patterns (uint16) [N, K/gs]."""
    w: np.ndarray
    s: np.ndarray
    b: np.ndarray
    N: int
    K: int
    bits: int
    gs: int


def dense_q(store: SafetensorsStore, config: ModelConfig, paths: Sequence[str], pad_to: int = 1) -> HostDenseQ:
    """The matrices at `paths` (same K) stacked by rows into one (Linear.swift:104-183). Pieces at 4 and 8 bits are
    concatenated at 8 bits, the 4-bit ones widened losslessly (codes x 16, scales / 16); zero rows up to a multiple
    of pad_to."""
    ls = [QuantizedLinear(store, p, config) for p in paths]
    f = ls[0]
    mixed = {l.params.bits for l in ls} == {4, 8}
    ok = all(l.in_features == f.in_features and l.experts == 1 and
             ((l.params.group_size == 64 and l.params.mode == f.params.mode) if mixed else l.params == f.params) for l in ls)
    if not ok or f.params.bits not in (4, 6, 8):
        desc = [f"{l.params.bits} bits g{l.params.group_size}" for l in ls]
        raise SafetensorsError("format", f"cannot concatenate {list(paths)} ({desc}; mixed 4/8 bits only with groups of 64)")
    if not (f.params.group_size == 64 or (f.params.group_size == 32 and f.params.bits == 4)):
        raise SafetensorsError("format", f"{f.path}: {f.params.bits} bits with groups of {f.params.group_size} not supported "
                                         "(groups of 64, or 32 only with 4 bits)")
    for l in ls:
        bd = l.biases.dtype if l.biases is not None else "BF16"
        if l.scales.dtype != "BF16" or bd != "BF16":
            raise SafetensorsError("format", f"{l.path}: scales/biases are {l.scales.dtype}/{bd}, expected bf16")
        if l.biases is None:
            raise SafetensorsError("missing", f"no such tensor {l.path}.biases")
    K, gs = f.in_features, f.params.group_size
    bits = 8 if mixed else f.params.bits
    n0 = sum(l.out_features for l in ls)
    N = (n0 + pad_to - 1) // pad_to * pad_to
    wpr, spr = K * bits // 32, K // gs  # words / scale entries per row
    w = np.zeros((N, wpr), dtype=np.uint32)
    s = np.zeros((N, spr), dtype=np.uint16)
    b = np.zeros((N, spr), dtype=np.uint16)
    lib = capi.lib()
    r = 0
    for l in ls:
        n = l.out_features
        src_w, src_s, src_b = store.bytes(l.weight), store.bytes(l.scales), store.bytes(l.biases)
        if mixed and l.params.bits == 4:
            lib.iq_widen4to8_words(src_w.ctypes.data, w[r:r + n].ctypes.data, l.weight.byte_count // 4)
            lib.iq_scales_div16_bf16(src_s.ctypes.data, s[r:r + n].ctypes.data, l.scales.byte_count // 2)
        else:
            w[r:r + n] = src_w.view(np.uint8).copy().view(np.uint32).reshape(n, wpr)
            s[r:r + n] = src_s.copy().view(np.uint16).reshape(n, spr)
        b[r:r + n] = src_b.copy().view(np.uint16).reshape(n, spr)
        r += n
    return HostDenseQ(w, s, b, N, K, bits, gs)


def stacked_experts(store: SafetensorsStore, config: ModelConfig, path: str):
    """A stacked expert tensor [E, out, in] as it is in the checkpoint (affine 4-bit g64 or mxfp4): host arrays
    (w uint32 [E, N, words], s, b or None) and the QuantizedLinear that describes them."""
    l = QuantizedLinear(store, path, config, mxfp4=True)
    w = store.array(l.weight).reshape(l.experts, l.out_features, -1)
    s = store.array(l.scales).reshape(l.experts, l.out_features, -1)
    b = None if l.biases is None else store.array(l.biases).reshape(l.experts, l.out_features, -1)
    return w, s, b, l


def to_device(h: HostDenseQ, device):
    """Uploads a HostDenseQ as a linear.DenseQ (the three device buffers of DeviceQuantizedLinear, Quant.swift:205-231)."""
    import torch

    from .linear import DenseQ

    up = lambda a, dt: torch.from_numpy(a.view(dt)).to(device)
    return DenseQ(up(h.w, np.int32), up(h.s, np.int16).view(torch.bfloat16), up(h.b, np.int16).view(torch.bfloat16), h.N, h.K,
                  h.bits, h.gs, "affine", 1)
