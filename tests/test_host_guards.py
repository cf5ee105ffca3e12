"""Host-side checks of the operator mirrors that need no GPU: shape/format guards raise before anything is launched."""
import pytest
import torch

from ingot_b200.linear import DenseQ, VQMV


def test_dense_q_rejects_cpu_tensors():
    w = torch.zeros(16, 8, dtype=torch.int32)
    s = torch.zeros(16, 1, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        DenseQ(w, s, s.clone(), 16, 64, 4)


def test_vqmv_has_the_reference_row_limit():
    assert VQMV.MAX_ROWS == 16


def test_bf16_table_and_embedding_have_no_cpu_path():
    t = torch.zeros(8, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        DenseQ(t, None, None, 8, 64, 16)
