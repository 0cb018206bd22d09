"""All-gather + GEMM (column-parallel projection). All ranks of a job run on ONE GPU here: every
rank's heap is a region of one device buffer; every rank's push runs first (its shard lands in the
other ranks' staging copies and counters), then every rank's GEMM. No launch waits for a later one.
Real peers: tests/test_multigpu_gpu.py. Oracle: gemm_ref on the gathered A; bf16 tolerance 1e-2."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _fake_job(capi, world, M, K):
    ws_bytes = capi.ag_gemm_workspace_bytes(M, K, world)
    region = capi.CTRL_BYTES + (ws_bytes + 4095) // 4096 * 4096
    buf = torch.zeros(world * region + 4096, dtype=torch.uint8, device="cuda")
    base0 = (buf.data_ptr() + 1023) // 1024 * 1024
    bases = [base0 + r * region for r in range(world)]
    views = [capi.make_view(r, world, bases, region) for r in range(world)]
    return buf, views, [b + capi.CTRL_BYTES for b in bases], ws_bytes


@pytest.fixture
def pair_mode(capi, request):
    capi.check(capi.lib().dk_gemm_pair_mode(request.param))
    yield request.param
    capi.check(capi.lib().dk_gemm_pair_mode(1))


@pytest.mark.parametrize("pair_mode", [1, 0], indirect=True)
@pytest.mark.parametrize("world,M,N,K", [(2, 512, 512, 256), (4, 1024, 264, 512), (8, 2048, 768, 128),
                                         (2, 256, 256, 1024), (4, 2048, 512, 320)])
def test_ag_gemm_all_ranks_on_one_gpu(capi, orc, world, M, N, K, pair_mode):
    buf, views, ws, ws_bytes = _fake_job(capi, world, M, K)
    shard = M // world
    stage_bytes = M * K * 2
    for seq in (1, 2, 3):          # staging parity 1, 0, 1; counters keep growing
        A, _ = orc.make_gemm_inputs(M, 8, K, seed=30 + seq)
        outs = []
        Bts = []
        for r in range(world):
            # poison the staging copy of this parity: what is read must have been pushed by this call
            capi.tensor_from_ptr(ws[r] + (seq & 1) * stage_bytes, (stage_bytes,), torch.uint8).fill_(0xFF)
            Bts.append(orc.make_gemm_inputs(8, N, K, seed=100 * seq + r)[1].cuda())
            outs.append(torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda"))
        dA = [A[r * shard:(r + 1) * shard].contiguous().cuda() for r in range(world)]
        torch.cuda.synchronize()
        for r in range(world):
            capi.ag_gemm_phase(dA[r], Bts[r], outs[r], ws[r], views[r], seq, 1)
        torch.cuda.synchronize()
        for r in range(world):
            capi.ag_gemm_phase(dA[r], Bts[r], outs[r], ws[r], views[r], seq, 2)
        torch.cuda.synchronize()
        assert capi.device_status()[0] == 0
        for r in range(world):
            got = outs[r].float().cpu()
            assert not torch.isnan(got).any()
            want = orc.gemm_ref(A, Bts[r].cpu())
            assert orc.rel_fro(got, want) <= TOL
            for s in range(world):       # every source shard by itself
                rows = slice(s * shard, (s + 1) * shard)
                assert orc.rel_fro(got[rows], want[rows]) <= TOL


def test_ag_gemm_world1_is_a_plain_gemm(orc):
    import iris_py
    import tk_kernel
    iris = iris_py.Iris(heap_size_mb=64)
    A, Bt = orc.make_gemm_inputs(256, 256, 128, seed=2)
    out = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    tk_kernel.ag_gemm(A.cuda(), Bt.cuda(), out, iris.get_device_view())
    torch.cuda.synchronize()
    assert orc.rel_fro(out.float().cpu(), orc.gemm_ref(A, Bt)) <= TOL
