"""The torch.library registration of the entry points, without a GPU: every operator exists with a
schema that names what it writes, shape functions work on meta tensors, and calling one on CPU
tensors fails loudly (the operators are CUDA-only: there is no CPU fallback)."""
import pytest
import torch


@pytest.fixture(scope="module")
def ops(pkg):
    from distributed_hipkittens_b200 import torch_ops
    return torch_ops


def test_every_operator_is_registered_with_its_schema(ops):
    for name in ops.OPS:
        assert hasattr(torch.ops.dk_b200, name), name
    s = str(torch.ops.dk_b200.gemm_rs.default._schema)
    assert "Tensor(a" in s and "out" in s          # `out` is declared as written
    s = str(torch.ops.dk_b200.moe_layer.default._schema)
    assert s.count("Tensor(") >= 2                 # out and workspace


def test_shape_functions_on_meta_tensors(ops):
    A = torch.empty(256, 128, dtype=torch.bfloat16, device="meta")
    Bt = torch.empty(512, 128, dtype=torch.bfloat16, device="meta")
    C = torch.ops.dk_b200.gemm(A, Bt)
    assert C.shape == (256, 512) and C.dtype == torch.bfloat16 and C.device.type == "meta"
    q, s, atoms = torch.ops.dk_b200.mx_quant(torch.empty(200, 256, device="meta"))
    assert q.shape == (200, 256) and s.shape == (200, 8) and atoms.shape == (2, 2, 512)
    assert torch.ops.dk_b200.gemm_mxfp8(q, atoms, q, atoms, True).dtype == torch.float32
    idx, w = torch.ops.dk_b200.moe_route(torch.empty(64, 8, device="meta"), 2)
    assert idx.shape == (64, 2) and idx.dtype == torch.int32 and w.dtype == torch.float32


def test_no_cpu_implementation(ops):
    a = torch.zeros(128, 64, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.dk_b200.gemm(a, a)
