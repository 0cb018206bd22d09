"""iris_py on one GPU: the heap, its allocator, zero-copy views, object lifetimes."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_empty_dtypes_sizes_and_errors():
    import iris_py
    iris = iris_py.Iris(heap_size_mb=32)
    t = iris.empty([4, 8], "float32")
    assert t.shape == [4, 8] and t.dtype == "float32" and t.numel() == 32 and t.nbytes() == 128
    assert iris.empty([3], "half").nbytes() == 6
    assert iris.empty([2, 2]).dtype == "bfloat16"
    assert iris.empty([16], "float8_e4m3fn").nbytes() == 16
    with pytest.raises(RuntimeError, match="Unsupported dtype: int7"):
        iris.empty([1], "int7")
    with pytest.raises(RuntimeError, match="Failed to allocate iris memory"):
        iris.empty([64 * 1024 * 1024], "float32")      # 256 MiB from a 32 MiB heap


def test_allocations_live_inside_the_heap_and_are_zero_copy(capi):
    import iris_py
    iris = iris_py.Iris(heap_size_mb=32)
    view = iris.get_device_view()
    v = capi.DkView.from_address(view._addr())
    base, size = v.base[0], v.heap_bytes
    a = iris.empty([1024], "float32")
    b = iris.empty([1024], "float32")
    for t in (a, b):
        assert base + capi.CTRL_BYTES <= t.data_ptr() < base + size
        assert t.data_ptr() % 256 == 0
    assert abs(a.data_ptr() - b.data_ptr()) >= 4096
    ta = torch.as_tensor(a, device="cuda")
    assert ta.data_ptr() == a.data_ptr() and ta.dtype == torch.float32
    ta.fill_(3.0)
    tb = capi.tensor_from_ptr(a.data_ptr(), (1024,), torch.float32)
    assert float(tb.sum()) == 3072.0
    # freed blocks are reused: same sequence, same offsets
    pa = a.data_ptr()
    del ta, tb, a
    c = iris.empty([1024], "float32")
    assert c.data_ptr() == pa


def test_tensor_outlives_iris():
    """The reference's Tensor holds a raw context pointer (iris_py.cpp:17,24); here it keeps the
    heap alive, so this order of destruction is safe."""
    import gc
    import iris_py
    iris = iris_py.Iris(heap_size_mb=16)
    t = iris.empty([256], "float32")
    view = iris.get_device_view()
    del iris
    gc.collect()
    x = torch.as_tensor(t, device="cuda")
    x.fill_(1.0)
    torch.cuda.synchronize()
    assert float(x.sum()) == 256.0
    del x, t, view
    gc.collect()


def test_heap_allocator_first_fit_and_coalescing(capi):
    h = capi.Heap(8 << 20)
    free0 = h.bytes_free()
    p1, p2, p3 = h.alloc(1 << 20), h.alloc(1 << 20), h.alloc(1 << 20)
    assert p2 - p1 == 1 << 20 and p3 - p2 == 1 << 20
    h.free(p2)
    assert h.alloc(512 << 10) == p2               # first fit reuses the hole
    h.free(p1)
    with pytest.raises(capi.DkError):
        h.free(p1)                                # double free is an argument error
    h.free(p3)
    h.free(p2)
    assert h.bytes_free() == free0                # everything coalesced back
    h.close()
