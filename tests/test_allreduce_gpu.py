"""TP all-reduce: all ranks of a job run inside one cooperative launch on one GPU (each rank's
heap is a region of one buffer). Result within 1e-2 relative Frobenius error of the fp32 sum, and
bit-identical on every rank."""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2


def _job(capi, world, nbytes):
    region = capi.CTRL_BYTES + 2 * ((nbytes + 4095) // 4096 * 4096)
    buf = torch.zeros(world * region + 4096, dtype=torch.uint8, device="cuda")
    base0 = (buf.data_ptr() + 1023) // 1024 * 1024
    bases = [base0 + r * region for r in range(world)]
    views = [capi.make_view(r, world, bases, region) for r in range(world)]
    off_x = capi.CTRL_BYTES
    off_o = capi.CTRL_BYTES + (nbytes + 4095) // 4096 * 4096
    return buf, views, bases, off_x, off_o


@pytest.mark.parametrize("algo", [0, 1, -1])
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("shape", [(64, 8192), (8, 64), (1024, 1024), (3, 8)])
def test_allreduce_all_ranks_on_one_gpu(capi, orc, world, shape, algo):
    n = shape[0] * shape[1]
    if algo == 1 and n % (8 * world) != 0:
        pytest.skip("two-shot needs n % (8*world) == 0")
    xs_cpu = orc.make_allreduce_inputs(shape, world)
    want = orc.allreduce_ref(xs_cpu)
    buf, views, bases, off_x, off_o = _job(capi, world, n * 2)
    xs = [capi.tensor_from_ptr(b + off_x, shape, torch.bfloat16) for b in bases]
    outs = [capi.tensor_from_ptr(b + off_o, shape, torch.bfloat16) for b in bases]
    for epoch in (1, 2):     # flags are reused: a second call must not see stale state
        for x, xc in zip(xs, xs_cpu):
            x.copy_(xc)
        for o in outs:
            o.fill_(float("nan"))
        capi.allreduce_all_ranks(views, xs, outs, algo, epoch)
        torch.cuda.synchronize()
        assert capi.device_status()[0] == 0
        got = [o.cpu() for o in outs]
        for gq in got:
            assert orc.rel_fro(gq.float(), want) <= TOL
            assert torch.equal(gq.view(torch.int16), got[0].view(torch.int16))   # identical bits


def test_allreduce_argument_errors(capi):
    buf, views, bases, off_x, off_o = _job(capi, 2, 4096)
    x = capi.tensor_from_ptr(bases[0] + off_x, (12,), torch.bfloat16)     # n % 8 != 0
    with pytest.raises(capi.DkError) as e:
        capi.allreduce_all_ranks(views, [x, x], [x, x], 0, 1)
    assert e.value.code == capi.ERR_ARG
    y = capi.tensor_from_ptr(bases[0] + off_x, (24,), torch.bfloat16)     # 24 % 16 != 0
    with pytest.raises(capi.DkError):
        capi.allreduce_all_ranks(views, [y, y], [y, y], 1, 1)
    with pytest.raises(capi.DkError) as e:
        capi.allreduce_all_ranks(views, [y, y], [y, y], 2, 1)             # NVLS not built
    assert e.value.code == capi.ERR_UNSUPPORTED


def test_allreduce_world1_is_a_copy(capi):
    h = capi.Heap(4 << 20)
    p = h.alloc(4096)
    x = capi.tensor_from_ptr(p, (2048,), torch.bfloat16)
    x.copy_(torch.arange(2048, dtype=torch.float32).to(torch.bfloat16))
    out = torch.zeros(2048, dtype=torch.bfloat16, device="cuda")
    capi.allreduce(x, out, h.view())
    torch.cuda.synchronize()
    assert torch.equal(out, x)
    del x
    h.free(p)
    h.close()
