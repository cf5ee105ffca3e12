"""From a safetensors file to the kernels: a mixed 4/8-bit concatenation read by the loader, uploaded, and multiplied by
the GEMV and the GEMM; parity with the oracle on the tensors as they were written."""
import json

import numpy as np
import pytest
import torch

from ingot_b200 import loader, synth
from ingot_b200.linear import VQMV
from oracle import qref
from gpu_util import TOL, x_tensor
from test_loader import affine_layer, write_safetensors

pytestmark = pytest.mark.gpu


def test_checkpoint_to_kernels(cuda_device, tmp_path):
    rng = np.random.default_rng(9)
    K = 2048
    t, raw = {}, {}
    for name, (N, bits) in {"m.qkv": (192, 8), "m.ab": (64, 4)}.items():
        d, r = affine_layer(rng, name, N, K, bits)
        t.update(d)
        raw[name] = r
    write_safetensors(tmp_path / "model.safetensors", t)
    cfg = loader.ModelConfig({"quantization": {"group_size": 64, "bits": 4, "m.qkv": {"group_size": 64, "bits": 8}}})
    st = loader.SafetensorsStore(str(tmp_path))
    h = loader.dense_q(st, cfg, ["m.qkv", "m.ab"], pad_to=64)
    m = loader.to_device(h, cuda_device)
    assert (m.N, m.K, m.bits) == (256, K, 8)
    wref = np.concatenate([qref.dequant_affine(*raw["m.qkv"], 8), qref.dequant_affine(*raw["m.ab"], 4)])
    x = synth.activations_np(rng, 64, K)
    xt = x_tensor(x, cuda_device)
    y = torch.zeros(3, m.N, dtype=torch.float32, device=cuda_device)
    VQMV.encode(xt[:3].contiguous(), m, y, 3)
    torch.cuda.synchronize()
    assert qref.max_rel(y.cpu().numpy(), qref.matmul_t(x[:3], wref)) <= TOL
    y2 = torch.zeros(64, m.N, dtype=torch.float32, device=cuda_device)
    ws = torch.empty(max(m.qmm_workspace_bytes(64, xt.dtype), 256), dtype=torch.uint8, device=cuda_device)
    m.encode_qmm_f32(xt, y2, 64, workspace=ws)
    torch.cuda.synchronize()
    assert qref.max_rel(y2.cpu().numpy(), qref.matmul_t(x, wref)) <= TOL
