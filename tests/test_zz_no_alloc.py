"""The allocation-free prefill GEMM (iq_qmm_noalloc) against the ordinary entry point.

Some hosts cannot hand this library a scratch buffer because they may not allocate device memory where they call it:
a plugin running inside an engine whose pool owns every byte, code that runs after the pool was sealed, a service under
a no-allocation rule. For them the library carries its own fixed scratch. This test calls the variant twice in a row
through the C ABI (the second call reuses whatever the first left in the scratch) and expects exactly the bits that
iq_qmm produces with a caller-provided workspace; it also checks that an oversized call is refused with a clear error.
The file name keeps it last in collection order, so a run that stops at the first failure has already run the rest.
"""
import numpy as np
import pytest
import torch

from ingot_b200 import capi, synth
from oracle import qref
from gpu_util import TOL, affine_case, deq, x_tensor

pytestmark = pytest.mark.gpu


def test_noalloc_matches_the_workspace_entry_point_twice(cuda_device):
    rng = np.random.default_rng(77)
    N, K = 256, 1024
    m, host = affine_case(rng, N, K, 4, cuda_device)
    wf = deq(host, 4)
    for call, M in enumerate((128, 64)):  # two calls in a row, different shapes: the scratch is reused, not cleared
        xh = synth.activations_np(rng, M, K)
        x = x_tensor(xh, cuda_device)  # bf16: the conversion pass writes the scratch
        ws = torch.empty(max(m.qmm_workspace_bytes(M, x.dtype), 256), dtype=torch.uint8, device=cuda_device)
        want = torch.zeros(M, N, dtype=torch.float32, device=cuda_device)
        m.encode_qmm_f32(x, want, M, workspace=ws)
        got = torch.full((M, N), float("nan"), dtype=torch.float32, device=cuda_device)
        m.encode_qmm_noalloc(x, got, M)
        assert capi.context(0).device_status() == 0
        assert torch.equal(got, want), f"call {call}: the allocation-free variant differs from iq_qmm"
        assert qref.max_rel(got.cpu().numpy(), qref.matmul_t(xh, wf)) <= TOL


def test_noalloc_refuses_sizes_beyond_its_scratch(cuda_device):
    rng = np.random.default_rng(78)
    m, _ = affine_case(rng, 64, 4096, 4, cuda_device)
    M = 2048  # 2048 * 4096 activations > 4,194,304
    x = torch.zeros(M, 4096, dtype=torch.bfloat16, device=cuda_device)
    y = torch.zeros(M, 64, dtype=torch.float32, device=cuda_device)
    with pytest.raises(capi.IngotError) as e:
        m.encode_qmm_noalloc(x, y, M)
    assert e.value.status == -4 and "scratch" in str(e.value)
