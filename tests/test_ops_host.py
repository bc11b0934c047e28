"""Host-side argument checks of vectorsparse_b200.ops that need no GPU: operands that are not CUDA tensors, or that
are spread over two devices, are refused before anything is launched (the kernels, tensor maps, status word and
plan scratch of a call all belong to one device)."""
import types

import pytest
import torch

from vectorsparse_b200 import ops


def fake(device):
    """Stands in for a CUDA tensor where none can exist: _one_device only looks at is_cuda and device."""
    return types.SimpleNamespace(is_cuda=True, device=torch.device(device))


def test_one_device_accepts_a_single_device_and_skips_none():
    assert ops._one_device(a=fake("cuda:1"), b=fake("cuda:1"), c=None) == torch.device("cuda:1")


def test_operands_on_two_devices_are_refused():
    with pytest.raises(TypeError, match="share one device"):
        ops._one_device(values=fake("cuda:0"), rhs_matrix=fake("cuda:1"))


def test_cpu_tensors_are_refused_before_any_launch():
    i32 = torch.zeros(8, dtype=torch.int32)
    h = torch.zeros(64 * 64, dtype=torch.float16)
    with pytest.raises(TypeError, match="CUDA tensor"):
        ops.spmm.wmmaSpmm(1, 8, 64, 64, i32, i32, i32, h, h, h)
    with pytest.raises(TypeError, match="CUDA tensor"):
        ops.spmm.cudaSpmm(1, 8, 64, 64, i32, i32, i32, h, h, h)
    with pytest.raises(TypeError, match="CUDA tensor"):
        ops.sddmm.wmmaSddmm(1, 64, 64, 4, i32, i32, i32, h, h, h, 8)
    with pytest.raises(TypeError, match="CUDA tensor"):
        ops.softmax_cvse(1, 8, i32, i32, h, h)
    with pytest.raises(TypeError, match="CUDA tensor"):
        ops.spmm_t(1, 8, 64, 7, i32, i32, i32, h, h, h)


def test_short_index_and_value_arrays_are_refused_when_the_count_is_given():
    """The reference signature of SpMM carries no nonzero count; when the caller passes one, column_indices and values
    are checked against it on the host (here before the device check even looks at the tensors)."""
    i32 = torch.zeros(8, dtype=torch.int32)
    h = torch.zeros(64 * 64, dtype=torch.float16)
    cols = torch.zeros(3, dtype=torch.int32)
    with pytest.raises((ValueError, TypeError)) as e:
        ops.spmm.wmmaSpmm(1, 8, 64, 64, i32, i32, cols, h, h, h, nonzeros_vec=4)
    assert "column_indices" in str(e.value) or "CUDA" in str(e.value)
