"""dk_moe_permute_static: the permutation for callers that cannot allocate device memory.

Some users of this library run where cudaMalloc is not available to them: a host runtime that was
handed its buffers up front, or code inside a region where allocation is forbidden. For them the
library carries the permutation's scratch (per-chunk histograms) as a fixed 256 KiB device array.
This test calls that entry point through the C ABI twice in a row, with different routings, the
second smaller than the first so that it runs over leftovers of the first, and requires exactly
the results of dk_moe_permute (integer work: bit-exact). The outputs are preallocated here, by
the test, as any caller would; the entry point itself allocates nothing.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_static(capi, idx, E, pad, seg):
    L = capi.lib()
    T, k = idx.shape
    nseg = E // seg
    cap = L.dk_moe_rows_capacity(T, k, seg, pad)
    dev = idx.device
    rop = torch.empty((T, k), dtype=torch.int32, device=dev)
    por = torch.empty((nseg, cap), dtype=torch.int32, device=dev)
    offs = torch.empty((nseg, seg + 1), dtype=torch.int32, device=dev)
    counts = torch.empty((E,), dtype=torch.int32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.dk_moe_permute_static(C.c_void_p(idx.data_ptr()), T, k, E, pad, seg, C.c_void_p(rop.data_ptr()),
                                 C.c_void_p(por.data_ptr()), cap, C.c_void_p(offs.data_ptr()),
                                 C.c_void_p(counts.data_ptr()), stream)
    capi.check(rc)
    return rop, por, offs, counts


def _device_bytes_free():
    """Free device memory as the driver reports it (cudaMemGetInfo): it moves when anything on the
    device is allocated or released behind torch's caching allocator."""
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_static_permute_matches_allocating_entry_point_twice(capi, orc):
    assert capi.lib().dk_moe_permute_static_max_bytes() == 256 * 1024
    g = torch.Generator().manual_seed(123)
    cases = [(8192, 256, 8, 32), (1000, 8, 2, 8)]       # (T, E, k, experts per segment)
    for T, E, k, seg in cases:
        idx, _ = orc.moe_route(torch.randn(T, E, generator=g), k)
        d_idx = idx.cuda()
        want = capi.moe_permute(d_idx, E, 128, experts_per_segment=seg)
        got = _run_static(capi, d_idx, E, 128, seg)
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a.reshape(-1), b.reshape(-1))


def test_static_permute_leaves_device_memory_as_it_found_it(capi, orc):
    """The property the entry point exists for: with the outputs already there, a call (after the
    first one on the device, which looks the scratch array up) changes the amount of device memory
    in use by nothing, as the driver counts it."""
    L = capi.lib()
    T, E, k, seg, pad = 4096, 64, 4, 64, 128
    idx, _ = orc.moe_route(torch.randn(T, E, generator=torch.Generator().manual_seed(7)), k)
    d_idx = idx.cuda()
    cap = L.dk_moe_rows_capacity(T, k, seg, pad)
    rop = torch.empty((T, k), dtype=torch.int32, device="cuda")
    por = torch.empty((1, cap), dtype=torch.int32, device="cuda")
    offs = torch.empty((1, seg + 1), dtype=torch.int32, device="cuda")
    counts = torch.empty((E,), dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    P = lambda t: C.c_void_p(t.data_ptr())

    def call():
        capi.check(L.dk_moe_permute_static(P(d_idx), T, k, E, pad, seg, P(rop), P(por), cap, P(offs), P(counts),
                                           stream))
    call()                                  # first call on this device: set-up happens here
    before = _device_bytes_free()
    for _ in range(3):
        call()
    after = _device_bytes_free()
    assert after == before, (before, after)
    want = capi.moe_permute(d_idx, E, pad, experts_per_segment=seg)
    for a, b in zip((rop, por, offs, counts), want):
        assert torch.equal(a.reshape(-1), b.reshape(-1))


def test_static_permute_rejects_oversized_routing(capi):
    T, E, k = 70000, 256, 8          # 547 chunks x 256 experts x 4 bytes > 256 KiB
    assert capi.lib().dk_moe_permute_scratch_bytes(T, k, E) > 256 * 1024
    idx = torch.zeros((T, k), dtype=torch.int32, device="cuda")
    with pytest.raises(capi.DkError) as e:
        _run_static(capi, idx, E, 128, E)
    assert e.value.code == capi.ERR_ARG and "262144" in str(e.value)
