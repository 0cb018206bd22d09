"""torch.ops.dk_b200.*: the operators run the same kernels as the tk_kernel calls (bit-identical
results), pass torch.library.opcheck, and can be traced by torch.compile's front end as opaque
calls (backend "eager": the graph is captured and replayed, nothing is code-generated)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(pkg):
    from distributed_hipkittens_b200 import torch_ops
    return torch_ops


def test_gemm_operator_matches_entry_point_and_oracle(ops, orc):
    import tk_kernel
    A, Bt = orc.make_gemm_inputs(384, 512, 256, seed=0)
    dA, dB = A.cuda(), Bt.cuda()
    C = torch.ops.dk_b200.gemm(dA, dB)
    C2 = torch.empty_like(C)
    tk_kernel.dispatch_micro(dA, dB, C2)
    torch.cuda.synchronize()
    assert torch.equal(C, C2)
    assert orc.rel_fro(C.float().cpu(), orc.gemm_ref(A, Bt)) <= 1e-2
    torch.library.opcheck(torch.ops.dk_b200.gemm.default, (dA, dB), test_utils=("test_schema", "test_faketensor"))


def test_mutating_and_tuple_operators(ops, orc):
    A, Bt = orc.make_gemm_inputs(256, 256, 128, seed=1)
    out = torch.full((256, 256), float("nan"), dtype=torch.bfloat16, device="cuda")
    torch.ops.dk_b200.gemm_rs(A.cuda(), Bt.cuda(), out, 0)          # view 0: one GPU
    out2 = torch.full_like(out, float("nan"))
    torch.ops.dk_b200.ag_gemm(A.cuda(), Bt.cuda(), out2, 0)
    torch.cuda.synchronize()
    ref = orc.gemm_ref(A, Bt)
    assert orc.rel_fro(out.float().cpu(), ref) <= 1e-2 and orc.rel_fro(out2.float().cpu(), ref) <= 1e-2
    x = torch.randn(256, 256, generator=torch.Generator().manual_seed(2))
    q, s, atoms = torch.ops.dk_b200.mx_quant(x.cuda())
    qr, sr = orc.mx_quant(x)
    assert torch.equal(q.cpu(), qr) and torch.equal(s.cpu(), sr)
    c = torch.ops.dk_b200.gemm_mxfp8(q, atoms, q, atoms, True)
    assert orc.rel_fro(c.cpu(), orc.mx_gemm_ref(qr, sr, qr, sr)) <= 1e-3
    idx, w = torch.ops.dk_b200.moe_route(torch.randn(100, 8, generator=torch.Generator().manual_seed(3)).cuda(), 2)
    assert idx.shape == (100, 2) and torch.allclose(w.sum(1).cpu(), torch.ones(100), atol=1e-5)


def test_operator_inside_a_captured_graph(ops, orc):
    A, Bt = orc.make_gemm_inputs(256, 512, 128, seed=4)

    def f(a, b):
        return torch.ops.dk_b200.gemm(a, b).float() * 2.0

    g = torch.compile(f, backend="eager", fullgraph=True)
    got = g(A.cuda(), Bt.cuda())
    torch.cuda.synchronize()
    assert orc.rel_fro(got.cpu(), 2.0 * orc.gemm_ref(A, Bt)) <= 1e-2
