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


def test_static_permute_rejects_oversized_routing(capi):
    T, E, k = 70000, 256, 8          # 547 chunks x 256 experts x 4 bytes > 256 KiB
    assert capi.lib().dk_moe_permute_scratch_bytes(T, k, E) > 256 * 1024
    idx = torch.zeros((T, k), dtype=torch.int32, device="cuda")
    with pytest.raises(capi.DkError) as e:
        _run_static(capi, idx, E, 128, E)
    assert e.value.code == capi.ERR_ARG and "262144" in str(e.value)
