"""GEMM + reduce-scatter. All ranks of a job are run on ONE GPU here: every rank's heap is a
region of one device buffer, the produce phase of every rank runs first (tiles and flags land in
the owners' staging areas), then every rank's reduce phase. No launch ever waits for a later one.
The multi-process path over real peer memory is exercised by bench.py --gpus N."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _fake_job(capi, world, M, N):
    ws_bytes = capi.gemm_rs_workspace_bytes(M, N, world)
    region = capi.CTRL_BYTES + (ws_bytes + 4095) // 4096 * 4096
    buf = torch.zeros(world * region + 4096, dtype=torch.uint8, device="cuda")
    base0 = (buf.data_ptr() + 1023) // 1024 * 1024
    bases = [base0 + r * region for r in range(world)]
    views = [capi.make_view(r, world, bases, region) for r in range(world)]
    ws = [b + capi.CTRL_BYTES for b in bases]
    return buf, views, ws


@pytest.fixture
def pair_mode(capi, request):
    """Two-CTA (1, the default) or one-CTA (0) kernel for the test; the default is restored."""
    capi.check(capi.lib().dk_gemm_pair_mode(request.param))
    yield request.param
    capi.check(capi.lib().dk_gemm_pair_mode(1))


@pytest.mark.parametrize("pair_mode", [1, 0], indirect=True)
@pytest.mark.parametrize("world,M,N,K", [(2, 512, 512, 256), (4, 1024, 768, 512), (8, 2048, 264, 1024),
                                         (2, 256, 512, 128), (4, 2048, 1024, 256),
                                         # more quarter-tile reduction items than CTAs (512 per rank), as at full size
                                         (8, 8192, 4096, 128)])
def test_gemm_rs_all_ranks_on_one_gpu(capi, orc, world, M, N, K, pair_mode):
    epilogue = -1
    buf, views, ws = _fake_job(capi, world, M, N)
    # staging area of one parity, in every rank's workspace: [world slots][tiles of the shard][64 KiB]
    stage_bytes = world * (M // world) * ((N + 255) // 256 * 256) * 2
    for seq in (1, 2, 3):     # parity 1, 0, 1: both staging buffers and flag reuse
        # other inputs on every call: a partial left over from an earlier call on the same parity
        # (a flag-epoch or parity bug) changes the answer instead of reproducing it
        A, Bt = orc.make_gemm_inputs(M, N, K, seed=10 + seq)
        As, Bs = orc.shard_k(A, Bt, world)
        want = orc.gemm_rs_ref(As, Bs)
        dA = [a.cuda() for a in As]
        dB = [b.cuda() for b in Bs]
        # poison outputs AND the staging buffers of the parity about to be used (bf16 0xffff = NaN):
        # whatever is read must have been written by this call
        outs = [torch.full((M // world, N), float("nan"), dtype=torch.bfloat16, device="cuda")
                for _ in range(world)]
        for r in range(world):
            stage = capi.tensor_from_ptr(ws[r] + (seq & 1) * stage_bytes, (stage_bytes,), torch.uint8)
            stage.fill_(0xFF)
        torch.cuda.synchronize()
        for r in range(world):
            capi.gemm_rs_phase(dA[r], dB[r], outs[r], ws[r], views[r], seq, 1, epilogue=epilogue)
        torch.cuda.synchronize()
        for r in range(world):
            capi.gemm_rs_phase(dA[r], dB[r], outs[r], ws[r], views[r], seq, 2, epilogue=epilogue)
        torch.cuda.synchronize()
        assert capi.device_status()[0] == 0
        for r in range(world):
            got = outs[r].float().cpu()
            assert not torch.isnan(got).any()
            assert orc.rel_fro(got, want[r]) <= TOL
        # all ranks together hold the full product
        full = torch.cat([o.float().cpu() for o in outs], 0)
        assert orc.rel_fro(full, orc.gemm_ref(A, Bt)) <= TOL


def test_gemm_rs_world1_is_a_plain_gemm(capi, orc):
    A, Bt = orc.make_gemm_inputs(256, 512, 128, seed=1)
    out = torch.empty(256, 512, dtype=torch.bfloat16, device="cuda")
    v = capi.make_view(0, 1, [0], 0)
    capi.gemm_rs(A.cuda(), Bt.cuda(), out, 0, v)
    torch.cuda.synchronize()
    assert orc.rel_fro(out.float().cpu(), orc.gemm_ref(A, Bt)) <= TOL


def test_gemm_rs_python_entry_point_world1(orc):
    import iris_py
    import tk_kernel
    iris = iris_py.Iris(heap_size_mb=64)
    A, Bt = orc.make_gemm_inputs(256, 256, 128, seed=2)
    out = torch.as_tensor(iris.empty([256, 256]), device="cuda").view(torch.bfloat16)
    tk_kernel.gemm_rs(A.cuda(), Bt.cuda(), out, iris.get_device_view())
    torch.cuda.synchronize()
    assert orc.rel_fro(out.float().cpu(), orc.gemm_ref(A, Bt)) <= TOL


def test_gemm_rs_rejects_bad_shapes(capi):
    buf, views, ws = _fake_job(capi, 2, 512, 256)
    a = torch.zeros(384, 64, dtype=torch.bfloat16, device="cuda")   # 384 % (2*128) != 0
    b = torch.zeros(256, 64, dtype=torch.bfloat16, device="cuda")
    o = torch.zeros(192, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(capi.DkError) as e:
        capi.gemm_rs_phase(a, b, o, ws[0], views[0], 1, 3)
    assert e.value.code == capi.ERR_ARG
