"""Host-side argument checks of the Python mirror (no GPU needed): what the kernels would misread on
the device - a page table of the wrong dtype, on the wrong device or strided - is refused before any
launch, because a bad index on the GPU is an out-of-bounds read rather than an exception."""
import pytest
import torch

from amd_optimization_challenge_b200 import submission as sub

CPU = torch.device("cpu")


def test_index_tensor_checks():
    ok = torch.arange(9, dtype=torch.int32)
    sub._check_index_tensor("kv_indptr", ok, CPU, 2)
    sub._check_index_tensor("kv_indices", None, CPU)                       # optional arguments may be absent
    with pytest.raises(TypeError, match="int32"):
        sub._check_index_tensor("kv_indices", torch.arange(9), CPU)       # torch.arange defaults to int64
    with pytest.raises(TypeError, match="torch.Tensor"):
        sub._check_index_tensor("kv_indices", [0, 1, 2], CPU)
    with pytest.raises(ValueError, match="contiguous"):
        sub._check_index_tensor("kv_indices", torch.arange(18, dtype=torch.int32)[::2], CPU)
    with pytest.raises(ValueError, match="is on"):
        sub._check_index_tensor("kv_indices", torch.empty(9, dtype=torch.int32, device="meta"), CPU)
    with pytest.raises(ValueError, match="at least 10"):
        sub._check_index_tensor("kv_indices", ok, CPU, 10)


def test_plane_checks():
    sub._check_plane("kv[0]", torch.zeros(4, 1, 576, dtype=torch.uint8), CPU)
    sub._check_plane("scale", torch.zeros(1), CPU, torch.float32)
    with pytest.raises(TypeError, match="float32"):
        sub._check_plane("scale", torch.zeros(1, dtype=torch.float64), CPU, torch.float32)
    with pytest.raises(ValueError, match="unit stride"):
        sub._check_plane("kv[0]", torch.zeros(4, 576, dtype=torch.uint8).t(), CPU)
    with pytest.raises(ValueError, match="is on"):
        sub._check_plane("kv[0]", torch.empty(4, 576, dtype=torch.uint8, device="meta"), CPU)


def test_decode_refuses_cpu_tensors():
    q = torch.zeros(1, 16, 576, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        sub.mla_decode(q, None, "fp8", (torch.zeros(4, 576, dtype=torch.uint8), torch.ones(1)),
                       torch.tensor([0, 4], dtype=torch.int32), sm_scale=1.0)


def test_generator_device_default_is_cpu_and_seeded():
    import amd_optimization_challenge_b200 as pkg
    a = pkg.generate_input(2, 1, 8, seed=3, formats=("fp8",), device="cpu")
    b = pkg.generate_input(2, 1, 8, seed=3, formats=("fp8",), device="cpu", generator_device="cpu")
    assert torch.equal(a[0], b[0]) and torch.equal(a[1]["fp8"][0].view(torch.uint8), b[1]["fp8"][0].view(torch.uint8))
