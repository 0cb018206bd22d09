"""Parity of the tcgen05 GEMM with the oracle, through the C ABI and through the reference's
Python call (tk_kernel.dispatch_micro). Tolerance: relative Frobenius error <= 1e-2 against the
fp32 product of the bf16-rounded inputs; the reference example's own check (max-abs < 0.1 on its
seeds) is asserted as well."""
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
TOL = 1e-2


def _bf16(a):
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


@pytest.mark.parametrize("epilogue", [0, 1])
@pytest.mark.parametrize("shape", [
    (128, 256, 64), (128, 256, 512), (256, 512, 128), (384, 768, 320),
    (2048, 4096, 4096),          # the world_size = 1 case of the row-parallel GEMM
    (200, 264, 72), (1, 8, 8), (129, 8, 16), (1000, 1000, 992), (64, 4096, 64),   # ragged
])
def test_gemm_matches_oracle(capi, orc, shape, epilogue):
    M, N, K = shape
    A, Bt = orc.make_gemm_inputs(M, N, K, seed=0)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.gemm_bf16(A.cuda(), Bt.cuda(), C, epilogue=epilogue)
    torch.cuda.synchronize()
    assert capi.device_status()[0] == 0
    assert not torch.isnan(C.float()).any()
    assert orc.rel_fro(C.float().cpu(), orc.gemm_ref(A, Bt)) <= TOL


def test_gemm_golden_example_vectors(capi, orc):
    """The reference example's inputs and its acceptance test, on the committed vectors."""
    fx = np.load(GOLD / "gemm_example.npz")
    B = _bf16(fx["B"])
    for rank in (0, 1):
        A, C_ref = _bf16(fx[f"A{rank}"]), _bf16(fx[f"C{rank}"])
        C = capi.gemm_bf16(A.cuda(), B.cuda()).cpu()
        assert (C.float() - C_ref.float()).abs().max().item() < 0.1
        ok, _ = orc.example_check(C, A, B)
        assert ok
        assert orc.rel_fro(C.float(), orc.gemm_ref(A, B)) <= TOL


def test_gemm_linearity_at_full_size(capi):
    """Size-independent property at the benchmark's size (M=N=8192, K=28672), where the CPU oracle
    would take minutes: (A1 + A2) B == A1 B + A2 B up to bf16 rounding, and a sampled set of
    output entries against fp64 dot products."""
    M = N = 8192
    K = 28672
    g = torch.Generator(device="cuda").manual_seed(0)
    A1 = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    A2 = (torch.randn(M, K, device="cuda", generator=g) / 64).to(torch.bfloat16)
    # make A1 + A2 exactly representable: A2 is a copy of A1 scaled by a power of two
    A2 = (A1.float() * 0.5).to(torch.bfloat16)
    A3 = (A1.float() * 1.5).to(torch.bfloat16)            # == A1 + A2 exactly (3 significant bits more at most)
    Bt = (torch.randn(N, K, device="cuda", generator=g) / K ** 0.5).to(torch.bfloat16)
    C1 = capi.gemm_bf16(A1, Bt).float()
    C2 = capi.gemm_bf16(A2, Bt).float()
    C3 = capi.gemm_bf16(A3, Bt).float()
    torch.cuda.synchronize()
    lhs, rhs = C3, C1 + C2
    assert ((lhs - rhs).norm() / rhs.norm()).item() <= TOL
    idx_m = torch.randint(0, M, (64,), generator=torch.Generator().manual_seed(1))
    idx_n = torch.randint(0, N, (64,), generator=torch.Generator().manual_seed(2))
    ref = (A1[idx_m.cuda()].double() * Bt[idx_n.cuda()].double()).sum(1)
    got = C1[idx_m.cuda(), idx_n.cuda()].double()
    assert ((got - ref).norm() / ref.norm()).item() <= TOL
    assert capi.device_status()[0] == 0


def test_gemm_argument_errors(capi):
    a = torch.zeros(128, 60, dtype=torch.bfloat16, device="cuda")   # K % 8 != 0
    with pytest.raises(capi.DkError) as e:
        capi.gemm_bf16(a, a)
    assert e.value.code == capi.ERR_ARG
    b = torch.zeros(12, 64, dtype=torch.bfloat16, device="cuda")    # N % 8 != 0
    with pytest.raises(capi.DkError):
        capi.gemm_bf16(torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda"), b)
    with pytest.raises(RuntimeError):
        capi.gemm_bf16(torch.zeros(16, 64, device="cuda"), torch.zeros(16, 64, device="cuda"))


# (m, n, k) of the reference's single-GPU script kernels/cdna4/gemm/bf16fp32/test.py:6-14
REFERENCE_TEST_SHAPES = [(8192, 8192, 8192), (4096, 8192, 2048), (8192, 4096, 2048), (8192, 2048, 4096),
                         (512, 1024, 1024), (512, 1024, 2048), (2048, 1024, 512)]


@pytest.mark.parametrize("m,n,k", REFERENCE_TEST_SHAPES)
def test_dispatch_micro_three_argument_form(orc, m, n, k):
    """tk_kernel.dispatch_micro(A, Bt, C) as the reference's test.py:22-31 calls it: unscaled randn
    operands (seed 0), Bt = B.t().contiguous(), checked with its criterion
    (allclose(rtol=1e-2): elements whose value nearly cancels cannot meet a purely relative bound
    in bf16, so the share of elements inside it is asserted) and with the oracle's norm."""
    import tk_kernel
    g = torch.Generator().manual_seed(0)
    A = torch.randn(m, k, generator=g).to(torch.bfloat16)
    B = torch.randn(k, n, generator=g).to(torch.bfloat16)
    Bt = B.t().contiguous()
    C = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    tk_kernel.dispatch_micro(A.cuda(), Bt.cuda(), C)
    torch.cuda.synchronize()
    assert tk_kernel.device_status()[0] == 0
    ref = orc.gemm_ref(A, Bt)
    got = C.float().cpu()
    assert orc.rel_fro(got, ref) <= TOL
    # The reference compares with allclose(rtol=1e-2) against a bf16 matmul (test.py:29-31). Outputs
    # are ~N(0, K); an element that nearly cancels cannot meet a purely relative bound in bf16 under
    # any summation order, so every element is held to rtol 1e-2 plus an absolute floor scaled to the
    # output, 1e-2 * sqrt(K), against the bf16-rounded reference.
    ref16 = ref.to(torch.bfloat16).float()
    bad = (got - ref16).abs() > 1e-2 * ref16.abs() + 1e-2 * k ** 0.5
    assert not bad.any(), f"{int(bad.sum())} elements outside rtol 1e-2 + atol 1e-2*sqrt(K)"
    # and no tile may hide a local fault in the global norm: worst error of every 128x256 tile
    err = ((got - ref).abs() / k ** 0.5)
    tiles = err.reshape(m // 128, 128, n // 256, 256).amax(dim=(1, 3))
    assert tiles.max().item() <= 0.04, tiles.max().item()


def test_dispatch_micro_reference_call(orc):
    """The reference's call, argument for argument (distributed-kernels/bf16_gemm/example.py:110-121)."""
    import iris_py
    import tk_kernel
    iris = iris_py.Iris(heap_size_mb=64, verbose=False)
    assert iris.rank() == 0 and iris.world_size() == 1
    M_local, N, K = 384, 512, 256
    A, B = orc.example_inputs(M_local, N, K, rank=0)
    tA, tB, tC = (iris.empty([M_local, K]), iris.empty([N, K]), iris.empty([M_local, N]))
    dA = torch.as_tensor(tA, device="cuda").view(torch.bfloat16)
    dB = torch.as_tensor(tB, device="cuda").view(torch.bfloat16)
    dC = torch.as_tensor(tC, device="cuda").view(torch.bfloat16)
    assert dA.data_ptr() == tA.data_ptr() and dC.shape == (M_local, N)
    dA.copy_(A)
    dB.copy_(B)
    dC.zero_()
    iris.barrier()
    view = iris.get_device_view()
    assert view.cur_rank() == 0 and view.world_size() == 1
    tk_kernel.dispatch_micro(dA, dB, dC, view, M_local, N, K, 0)
    torch.cuda.synchronize()
    iris.barrier()
    ok, err = orc.example_check(dC.cpu(), A, B)
    assert ok, err
    assert orc.rel_fro(dC.float().cpu(), orc.gemm_ref(A, B)) <= TOL
    assert tk_kernel.device_status()[0] == 0


@pytest.mark.parametrize("mode", [1, 0])
def test_pair_and_single_cta_kernels_match_oracle(capi, orc, mode):
    """The cta_group::2 kernel (clusters of two CTAs per 256x256 tile, the default where M allows)
    and the one-CTA kernel give the same results; shapes with M % 256 != 0 fall back by themselves."""
    L = capi.lib()
    capi.check(L.dk_gemm_pair_mode(mode))
    try:
        outs = []
        for (M, N, K) in [(256, 256, 64), (512, 768, 320), (2048, 4096, 4096), (768, 264, 128),
                          (384, 512, 192)]:
            A, Bt = orc.make_gemm_inputs(M, N, K, seed=5)
            C = capi.gemm_bf16(A.cuda(), Bt.cuda())
            torch.cuda.synchronize()
            assert capi.device_status()[0] == 0
            assert orc.rel_fro(C.float().cpu(), orc.gemm_ref(A, Bt)) <= TOL
            outs.append(C)
        # bit-identical between the two kernels: same K order, same fp32 accumulation
        capi.check(L.dk_gemm_pair_mode(1 - mode))
        A, Bt = orc.make_gemm_inputs(512, 768, 320, seed=5)
        C2 = capi.gemm_bf16(A.cuda(), Bt.cuda())
        torch.cuda.synchronize()
        assert torch.equal(C2, outs[1])
    finally:
        capi.check(L.dk_gemm_pair_mode(1))
