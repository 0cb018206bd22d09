"""ctypes binding of libdk_b200.so (the C ABI declared in include/dk_b200.h).

This is the thin layer the parity tests and the benchmark call through. It never computes
anything itself: if the CUDA library is missing or a call fails, it raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libdk_b200.so"
DK_MAX_RANKS = 8

ERR_ARG, ERR_CUDA, ERR_DEVICE, ERR_BOOTSTRAP, ERR_NOMEM, ERR_UNSUPPORTED = 1, 2, 3, 4, 5, 6


class DkView(C.Structure):
    """Mirror of `dk_view`."""
    _fields_ = [
        ("rank", C.c_int),
        ("world", C.c_int),
        ("base", C.c_void_p * DK_MAX_RANKS),
        ("heap_bytes", C.c_uint64),
        ("mc_base", C.c_void_p),
        ("heap", C.c_void_p),
    ]


class DkMoeEpArgs(C.Structure):
    """Mirror of `dk_moe_ep_args`."""
    _fields_ = [
        ("T_loc", C.c_int), ("k", C.c_int), ("E", C.c_int), ("H", C.c_int), ("F", C.c_int),
        ("scale_mode", C.c_int),
        ("x", C.c_void_p), ("logits", C.c_void_p),
        ("w13q", C.c_void_p), ("w13s", C.c_void_p), ("w2q", C.c_void_p), ("w2s", C.c_void_p),
        ("out", C.c_void_p), ("workspace", C.c_void_p), ("counts_out", C.c_void_p),
        ("ev_gemm_begin", C.c_void_p), ("ev_gemm_end", C.c_void_p),
    ]


class DkError(RuntimeError):
    def __init__(self, code: int, what: str, detail: str):
        super().__init__(f"{what}: {detail}" if detail else what)
        self.code = code


_lib = None


def lib() -> C.CDLL:
    """Load the library once. Fails loudly when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: run `python distributed-hipkittens_b200/build.py` "
                "(there is no CPU fallback)")
        _lib = C.CDLL(str(LIB_PATH))
        _declare(_lib)
    return _lib


def _declare(L: C.CDLL) -> None:
    vp, i, sz = C.c_void_p, C.c_int, C.c_size_t
    L.dk_strerror.restype = C.c_char_p
    L.dk_strerror.argtypes = [i]
    L.dk_last_error_string.restype = C.c_char_p
    L.dk_last_error_string.argtypes = []
    L.dk_version.restype = i
    L.dk_last_device_status.argtypes = [C.POINTER(C.c_uint * 4)]
    L.dk_bootstrap_env.argtypes = [C.POINTER(i), C.POINTER(i), C.POINTER(i)]
    L.dk_gemm_bf16.argtypes = [vp, vp, vp, i, i, i, C.POINTER(DkView), i, vp]
    L.dk_heap_create.argtypes = [sz, i, i, C.c_char_p, C.POINTER(vp)]
    L.dk_heap_destroy.argtypes = [vp]
    L.dk_heap_alloc.restype = vp
    L.dk_heap_alloc.argtypes = [vp, sz, sz]
    L.dk_heap_free.argtypes = [vp, vp]
    L.dk_heap_barrier.argtypes = [vp]
    L.dk_heap_view.argtypes = [vp, C.POINTER(DkView)]
    L.dk_heap_enable_multicast.argtypes = [vp]
    L.dk_heap_bytes_free.restype = sz
    L.dk_heap_bytes_free.argtypes = [vp]
    L.dk_comm_create.argtypes = [i, i, C.c_char_p, i, C.POINTER(vp)]
    L.dk_comm_destroy.argtypes = [vp]
    L.dk_comm_barrier.argtypes = [vp]
    L.dk_comm_allgather_fd.argtypes = [vp, i, C.POINTER(i)]
    L.dk_comm_allgather.argtypes = [vp, vp, sz, vp]
    L.dk_gemm_rs_workspace_bytes.restype = sz
    L.dk_gemm_rs_workspace_bytes.argtypes = [i, i, i]
    L.dk_gemm_rs_workspace_init.argtypes = [vp, sz, C.POINTER(DkView), vp]
    L.dk_gemm_rs_workspace_get.argtypes = [C.POINTER(DkView), i, i, vp, C.POINTER(vp)]
    L.dk_gemm_rs.argtypes = [vp, vp, vp, i, i, i, vp, C.POINTER(DkView), vp]
    L.dk_gemm_rs_phase.argtypes = [vp, vp, vp, i, i, i, vp, C.POINTER(DkView), C.c_uint, i, i, vp]
    L.dk_ag_gemm_workspace_bytes.restype = sz
    L.dk_ag_gemm_workspace_bytes.argtypes = [i, i, i]
    L.dk_ag_gemm_workspace_init.argtypes = [vp, sz, C.POINTER(DkView), vp]
    L.dk_ag_gemm_workspace_get.argtypes = [C.POINTER(DkView), i, i, vp, C.POINTER(vp)]
    L.dk_ag_gemm.argtypes = [vp, vp, vp, i, i, i, vp, C.POINTER(DkView), vp]
    L.dk_ag_gemm_phase.argtypes = [vp, vp, vp, i, i, i, vp, C.POINTER(DkView), C.c_uint, i, vp]
    L.dk_allreduce.argtypes = [vp, vp, sz, i, C.POINTER(DkView), vp]
    L.dk_gemm_debug_counters.argtypes = [vp]
    L.dk_gemm_pair_mode.argtypes = [i]
    L.dk_moe_route.argtypes = [vp, i, i, i, vp, vp, vp]
    L.dk_moe_permute_scratch_bytes.restype = sz
    L.dk_moe_permute_scratch_bytes.argtypes = [i, i, i]
    L.dk_moe_rows_capacity.restype = sz
    L.dk_moe_rows_capacity.argtypes = [i, i, i, i]
    L.dk_moe_permute.argtypes = [vp, i, i, i, i, i, vp, vp, i, vp, vp, vp, sz, vp]
    L.dk_quant_block128.argtypes = [vp, i, i, vp, i, i, vp, vp, vp]
    L.dk_moe_permute_static_max_bytes.restype = sz
    L.dk_moe_permute_static_max_bytes.argtypes = []
    L.dk_moe_permute_static.argtypes = [vp, i, i, i, i, i, vp, vp, i, vp, vp, vp]
    L.dk_moe_combine.argtypes = [vp, vp, vp, i, i, i, vp, vp]
    L.dk_moe_grouped_gemm_fp8.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, vp, vp, vp]
    L.dk_mx_pair_mode.argtypes = [i]
    L.dk_mx_sf_bytes.restype = sz
    L.dk_mx_sf_bytes.argtypes = [i, i]
    L.dk_mx_quant.argtypes = [vp, i, i, i, vp, vp, vp, vp]
    L.dk_gemm_mxfp8.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, vp]
    L.dk_quant_block128_pow2.argtypes = [vp, i, i, vp, i, i, vp, vp, vp, vp, vp]
    L.dk_moe_grouped_gemm_mxfp8.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, vp, vp, vp, vp]
    L.dk_moe_ep_workspace_bytes.restype = sz
    L.dk_moe_ep_workspace_bytes.argtypes = [i, i, i, i, i, i]
    L.dk_moe_ep_layer.argtypes = [C.POINTER(DkMoeEpArgs), C.POINTER(DkView), C.c_uint, i, vp]
    L.dk_peer_barrier.argtypes = [C.POINTER(DkView), vp]
    L.dk_peer_barrier_epoch.argtypes = [C.POINTER(DkView), C.c_uint, vp]
    L.dk_set_peer_wait_ms.argtypes = [i]
    L.dk_set_log_level.argtypes = [i]
    L.dk_set_walk_band_bytes.argtypes = [sz]
    L.dk_allgather.argtypes = [vp, sz, vp, C.POINTER(DkView), vp]
    L.dk_moe_dispatch.argtypes = [vp, vp, vp, i, i, i, i, vp, C.POINTER(DkView), i, vp]
    L.dk_moe_combine_ep.argtypes = [vp, vp, vp, vp, i, i, i, i, vp, C.POINTER(DkView), i, vp]
    L.dk_allreduce_all_ranks.argtypes = [i, C.POINTER(DkView), C.POINTER(vp), C.POINTER(vp), sz, i,
                                         C.c_uint, vp]


def declare(name: str, argtypes, restype=C.c_int):
    f = getattr(lib(), name)
    f.argtypes = argtypes
    f.restype = restype
    return f


def check(rc: int) -> None:
    if rc != 0:
        L = lib()
        raise DkError(rc, L.dk_strerror(rc).decode(), L.dk_last_error_string().decode())


def device_status():
    """(code, block, site, detail) of the first device-side wait that gave up; clears it."""
    out = (C.c_uint * 4)()
    check(lib().dk_last_device_status(C.byref(out)))
    return tuple(int(x) for x in out)


def bootstrap_env():
    r, w, l = C.c_int(), C.c_int(), C.c_int()
    check(lib().dk_bootstrap_env(C.byref(r), C.byref(w), C.byref(l)))
    return r.value, w.value, l.value


def _stream_ptr(stream) -> C.c_void_p:
    if stream is None:
        import torch
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)
    return C.c_void_p(int(stream))


def _ptr(t) -> C.c_void_p:
    return C.c_void_p(t.data_ptr())


def _need_cuda(*tensors):
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("Tensor must be on CUDA device")
        if not t.is_contiguous():
            raise RuntimeError("Tensor must be contiguous")


def gemm_bf16(A, Bt, C_out=None, *, epilogue: int = -1, stream=None):
    """C[M,N] = A[M,K] @ Bt[N,K]^T on the GPU (bf16 in/out, fp32 accumulate)."""
    import torch
    _need_cuda(A, Bt)
    if A.dtype != torch.bfloat16 or Bt.dtype != torch.bfloat16:
        raise RuntimeError("gemm_bf16 expects bfloat16 operands")
    M, K = A.shape
    N, K2 = Bt.shape
    if K != K2:
        raise RuntimeError(f"inner dimensions differ: {K} vs {K2}")
    if C_out is None:
        C_out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    _need_cuda(C_out)
    check(lib().dk_gemm_bf16(_ptr(A), _ptr(Bt), _ptr(C_out), M, N, K, None, epilogue,
                             _stream_ptr(stream)))
    return C_out


CTRL_BYTES = 1 << 20  # control block at the start of every rank's heap (signal counters)


def make_view(rank: int, world: int, bases, heap_bytes: int, heap=None) -> DkView:
    v = DkView()
    v.rank, v.world = rank, world
    for r in range(world):
        v.base[r] = bases[r]
    v.heap_bytes = heap_bytes
    v.mc_base = None
    v.heap = heap
    return v


class Heap:
    """ctypes handle on a symmetric heap (dk_heap_*)."""

    def __init__(self, nbytes: int, rank: int = 0, world: int = 1, rendezvous: str | None = None):
        self._h = C.c_void_p()
        rv = rendezvous.encode() if rendezvous else None
        check(lib().dk_heap_create(nbytes, rank, world, rv, C.byref(self._h)))
        self.rank, self.world = rank, world

    def alloc(self, nbytes: int, align: int = 256) -> int:
        p = lib().dk_heap_alloc(self._h, nbytes, align)
        if not p:
            raise DkError(ERR_NOMEM, "Failed to allocate iris memory", "")
        return p

    def free(self, ptr: int) -> None:
        check(lib().dk_heap_free(self._h, C.c_void_p(ptr)))

    def barrier(self) -> None:
        check(lib().dk_heap_barrier(self._h))

    def enable_multicast(self) -> bool:
        """Collective: map the NVLink multicast object over all ranks' heaps; False if unavailable."""
        rc = lib().dk_heap_enable_multicast(self._h)
        if rc == ERR_UNSUPPORTED:
            return False
        check(rc)
        return True

    def view(self) -> DkView:
        v = DkView()
        check(lib().dk_heap_view(self._h, C.byref(v)))
        return v

    def bytes_free(self) -> int:
        return lib().dk_heap_bytes_free(self._h)

    def close(self) -> None:
        if self._h:
            check(lib().dk_heap_destroy(self._h))
            self._h = C.c_void_p()


def tensor_from_ptr(ptr: int, shape, dtype):
    """Zero-copy torch view of device memory at `ptr` (the caller keeps the owner alive)."""
    import torch
    n = 1
    for d in shape:
        n *= d
    esz = torch.empty((), dtype=dtype).element_size()

    class _W:
        pass
    w = _W()
    w.__cuda_array_interface__ = {"shape": (n * esz,), "typestr": "|u1", "data": (ptr, False),
                                  "version": 3, "strides": None}
    return torch.as_tensor(w, device="cuda").view(dtype).reshape(shape)


def gemm_rs_workspace_bytes(M: int, N: int, world: int) -> int:
    return lib().dk_gemm_rs_workspace_bytes(M, N, world)


def gemm_rs_workspace_init(ws_ptr: int, nbytes: int, view: DkView, stream=None) -> None:
    check(lib().dk_gemm_rs_workspace_init(C.c_void_p(ws_ptr), nbytes, C.byref(view), _stream_ptr(stream)))


def gemm_rs(A, Bt, out, ws_ptr, view: DkView, stream=None):
    """out[M/P,N] = reduce-scatter of A[M,K/P] @ Bt[N,K/P]^T over the ranks of `view`."""
    _need_cuda(A, Bt, out)
    M, Kloc = A.shape
    N = Bt.shape[0]
    check(lib().dk_gemm_rs(_ptr(A), _ptr(Bt), _ptr(out), M, N, Kloc,
                           C.c_void_p(ws_ptr) if ws_ptr else None, C.byref(view), _stream_ptr(stream)))
    return out


def gemm_rs_phase(A, Bt, out, ws_ptr, view: DkView, seq: int, phases: int, *, epilogue: int = -1,
                  stream=None):
    _need_cuda(A, Bt, out)
    M, Kloc = A.shape
    N = Bt.shape[0]
    check(lib().dk_gemm_rs_phase(_ptr(A), _ptr(Bt), _ptr(out), M, N, Kloc, C.c_void_p(ws_ptr),
                                 C.byref(view), seq, phases, epilogue, _stream_ptr(stream)))
    return out


def ag_gemm_workspace_bytes(M: int, K: int, world: int) -> int:
    return lib().dk_ag_gemm_workspace_bytes(M, K, world)


def ag_gemm_phase(A_shard, Bt, C_out, ws_ptr, view: DkView, seq: int, phases: int, stream=None):
    """C[M, N] = all-gather over ranks of A_shard[M/P, K] @ Bt[N, K]^T; phases 1 = push, 2 = GEMM."""
    _need_cuda(A_shard, Bt, C_out)
    M, N = C_out.shape
    K = A_shard.shape[1]
    check(lib().dk_ag_gemm_phase(_ptr(A_shard), _ptr(Bt), _ptr(C_out), M, N, K, C.c_void_p(ws_ptr), C.byref(view),
                                 seq, phases, _stream_ptr(stream)))
    return C_out


def allreduce(x, out, view: DkView, algo: int = -1, stream=None):
    """out = sum over ranks of x (bf16, fp32 accumulate). x (and out for two-shot) in the heap."""
    _need_cuda(x, out)
    check(lib().dk_allreduce(_ptr(x), _ptr(out), x.numel(), algo, C.byref(view), _stream_ptr(stream)))
    return out


def allreduce_all_ranks(views, xs, outs, algo: int, epoch: int, stream=None):
    """Every rank of a job in one cooperative launch on this GPU (see dk_allreduce_all_ranks)."""
    world = len(views)
    _need_cuda(*xs, *outs)
    va = (DkView * world)(*views)
    xa = (C.c_void_p * world)(*[t.data_ptr() for t in xs])
    oa = (C.c_void_p * world)(*[t.data_ptr() for t in outs])
    check(lib().dk_allreduce_all_ranks(world, va, xa, oa, xs[0].numel(), algo, epoch, _stream_ptr(stream)))
    return outs


# ---------------------------------------------------------------------------- MoE
def moe_route(logits, k: int, stream=None):
    """(topk_idx int32 [T,k], topk_w fp32 [T,k]) from fp32 logits [T,E]."""
    import torch
    _need_cuda(logits)
    if logits.dtype != torch.float32:
        raise RuntimeError("moe_route expects float32 logits")
    T, E = logits.shape
    idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    check(lib().dk_moe_route(_ptr(logits), T, E, k, _ptr(idx), _ptr(w), _stream_ptr(stream)))
    return idx, w


def moe_permute(topk_idx, E: int, pad: int = 128, experts_per_segment: int | None = None, stream=None):
    """Returns (row_of_pair [T,k], pair_of_row [nseg, cap], offsets [nseg, seg+1], counts [E]),
    all int32 on the device. With one segment the first two dimensions are squeezed."""
    import torch
    _need_cuda(topk_idx)
    T, k = topk_idx.shape
    seg = E if experts_per_segment is None else experts_per_segment
    nseg = E // seg
    cap = lib().dk_moe_rows_capacity(T, k, seg, pad)
    dev = topk_idx.device
    rop = torch.empty((T, k), dtype=torch.int32, device=dev)
    por = torch.empty((nseg, cap), dtype=torch.int32, device=dev)
    offs = torch.empty((nseg, seg + 1), dtype=torch.int32, device=dev)
    counts = torch.empty((E,), dtype=torch.int32, device=dev)
    sb = lib().dk_moe_permute_scratch_bytes(T, k, E)
    scratch = torch.empty((sb,), dtype=torch.uint8, device=dev)
    check(lib().dk_moe_permute(_ptr(topk_idx), T, k, E, pad, seg, _ptr(rop), _ptr(por), cap, _ptr(offs),
                               _ptr(counts), _ptr(scratch), sb, _stream_ptr(stream)))
    if nseg == 1:
        return rop, por[0], offs[0], counts
    return rop, por, offs, counts


def quant_block128(x, rows: int | None = None, row_map=None, map_mode: int = 0, k: int = 1, stream=None):
    """(q uint8 [R,C], s fp32 [R/128,C/128]) from bf16 x; see dk_quant_block128 for the row map."""
    import torch
    _need_cuda(x)
    if x.dtype != torch.bfloat16:
        raise RuntimeError("quant_block128 expects bfloat16")
    R = x.shape[0] if rows is None else rows
    Cc = x.shape[1]
    q = torch.empty((R, Cc), dtype=torch.uint8, device=x.device)
    s = torch.empty((R // 128, Cc // 128), dtype=torch.float32, device=x.device)
    check(lib().dk_quant_block128(_ptr(x), R, Cc, _ptr(row_map) if row_map is not None else None,
                                  map_mode, k, _ptr(q), _ptr(s), _stream_ptr(stream)))
    return q, s


def moe_combine(y, row_of_pair, topk_w, stream=None):
    import torch
    _need_cuda(y, row_of_pair, topk_w)
    T, k = row_of_pair.shape
    H = y.shape[1]
    out = torch.empty((T, H), dtype=torch.bfloat16, device=y.device)
    check(lib().dk_moe_combine(_ptr(y), _ptr(row_of_pair), _ptr(topk_w), T, k, H, _ptr(out),
                               _stream_ptr(stream)))
    return out


def moe_grouped_gemm_fp8(xq, xs, wq, ws, offsets, gated: bool, stream=None):
    """Grouped fp8 GEMM. gated: returns (hq uint8 [R,F], hs fp32 [R/128,F/128]); else Y bf16 [R,N].
    Output rows beyond offsets[E] are zero-initialised here for convenience."""
    import torch
    _need_cuda(xq, xs, wq, ws, offsets)
    R, K = xq.shape
    E = wq.shape[0]
    if gated:
        N = wq.shape[1] // 2
        out = torch.zeros((R, N), dtype=torch.uint8, device=xq.device)
        sc = torch.ones((R // 128, N // 128), dtype=torch.float32, device=xq.device)
    else:
        N = wq.shape[1]
        out = torch.zeros((R, N), dtype=torch.bfloat16, device=xq.device)
        sc = None
    check(lib().dk_moe_grouped_gemm_fp8(_ptr(xq), _ptr(xs), _ptr(wq), _ptr(ws), _ptr(offsets), E, R, N, K,
                                        1 if gated else 0, _ptr(out), _ptr(sc) if sc is not None else None,
                                        _stream_ptr(stream)))
    return (out, sc) if gated else out


def moe_ffn_fp8(xq, xs, w13q, w13s, w2q, w2s, offsets, stream=None):
    """gate/up grouped GEMM + SiLU*mul + requantise, then the down grouped GEMM. Returns Y bf16 [R,H]."""
    hq, hs = moe_grouped_gemm_fp8(xq, xs, w13q, w13s, offsets, True, stream)
    return moe_grouped_gemm_fp8(hq, hs, w2q, w2s, offsets, False, stream)


# ---------------------------------------------------------------------------- MXFP8
def mx_quant(x, stream=None):
    """x [R, K] bf16 or fp32 -> (q e4m3 bytes [R, K], s e8m0 bytes [R, K/32], scale atoms
    [ceil(R/128), K/128, 512] in the layout the tensor core reads)."""
    import torch
    _need_cuda(x)
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise RuntimeError("mx_quant expects bfloat16 or float32")
    R, K = x.shape
    q = torch.empty((R, K), dtype=torch.uint8, device=x.device)
    s = torch.empty((R, K // 32), dtype=torch.uint8, device=x.device)
    atoms = torch.empty(((R + 127) // 128, K // 128, 512), dtype=torch.uint8, device=x.device)
    check(lib().dk_mx_quant(_ptr(x), 1 if x.dtype == torch.float32 else 0, R, K, _ptr(q), _ptr(s), _ptr(atoms),
                            _stream_ptr(stream)))
    return q, s, atoms


def gemm_mxfp8(aq, sfa, bq, sfb, out_dtype=None, stream=None):
    """C[M, N] = dequant(A) @ dequant(B)^T from e4m3 bytes and scale atoms; bf16 (default) or fp32 out."""
    import torch
    _need_cuda(aq, sfa, bq, sfb)
    M, K = aq.shape
    N = bq.shape[0]
    f32 = out_dtype == torch.float32
    out = torch.empty((M, N), dtype=torch.float32 if f32 else torch.bfloat16, device=aq.device)
    check(lib().dk_gemm_mxfp8(_ptr(aq), _ptr(sfa), _ptr(bq), _ptr(sfb), _ptr(out), M, N, K, 1 if f32 else 0,
                              _stream_ptr(stream)))
    return out


def quant_block128_pow2(x, rows: int | None = None, row_map=None, map_mode: int = 0, k: int = 1, stream=None):
    """(q uint8 [R,C], s fp32 [R/128,C/128], e8 uint8 [R/128,C/128], block atoms uint8
    [R/128, ceil(C/512), 512]): 128x128 block quantisation with power-of-two scales."""
    import torch
    _need_cuda(x)
    if x.dtype != torch.bfloat16:
        raise RuntimeError("quant_block128_pow2 expects bfloat16")
    R = x.shape[0] if rows is None else rows
    Cc = x.shape[1]
    dev = x.device
    q = torch.empty((R, Cc), dtype=torch.uint8, device=dev)
    s = torch.empty((R // 128, Cc // 128), dtype=torch.float32, device=dev)
    e8 = torch.empty((R // 128, Cc // 128), dtype=torch.uint8, device=dev)
    atoms = torch.full((R // 128, (Cc // 128 + 3) // 4, 512), 127, dtype=torch.uint8, device=dev)
    check(lib().dk_quant_block128_pow2(_ptr(x), R, Cc, _ptr(row_map) if row_map is not None else None,
                                       map_mode, k, _ptr(q), _ptr(s), _ptr(e8), _ptr(atoms), _stream_ptr(stream)))
    return q, s, e8, atoms


def moe_grouped_gemm_mxfp8(xq, x_atoms, wq, w_atoms, offsets, gated: bool, stream=None):
    """Grouped GEMM on the block-scaled tensor-core path. gated: returns (hq uint8 [R,F], e8 uint8
    [R/128,F/128], block atoms [R/128,ceil(F/512),512]); else Y bf16 [R,N]. Rows beyond offsets[E]
    stay zero."""
    import torch
    _need_cuda(xq, x_atoms, wq, w_atoms, offsets)
    R, K = xq.shape
    E = wq.shape[0]
    dev = xq.device
    if gated:
        N = wq.shape[1] // 2
        out = torch.zeros((R, N), dtype=torch.uint8, device=dev)
        e8 = torch.full((R // 128, N // 128), 127, dtype=torch.uint8, device=dev)
        atoms = torch.full((R // 128, (N // 128 + 3) // 4, 512), 127, dtype=torch.uint8, device=dev)
        check(lib().dk_moe_grouped_gemm_mxfp8(_ptr(xq), _ptr(x_atoms), _ptr(wq), _ptr(w_atoms), _ptr(offsets), E,
                                              R, N, K, 1, _ptr(out), _ptr(e8), _ptr(atoms), _stream_ptr(stream)))
        return out, e8, atoms
    N = wq.shape[1]
    out = torch.zeros((R, N), dtype=torch.bfloat16, device=dev)
    check(lib().dk_moe_grouped_gemm_mxfp8(_ptr(xq), _ptr(x_atoms), _ptr(wq), _ptr(w_atoms), _ptr(offsets), E, R,
                                          N, K, 0, _ptr(out), None, None, _stream_ptr(stream)))
    return out


def moe_ffn_mxfp8(xq, x_atoms, w13q, w13_atoms, w2q, w2_atoms, offsets, stream=None):
    """gate/up + SiLU*mul + requantise, then down, with power-of-two block scales. Y bf16 [R,H]."""
    hq, _, h_atoms = moe_grouped_gemm_mxfp8(xq, x_atoms, w13q, w13_atoms, offsets, True, stream)
    return moe_grouped_gemm_mxfp8(hq, h_atoms, w2q, w2_atoms, offsets, False, stream)


# ---------------------------------------------------------------------------- expert parallel
def moe_ep_workspace_bytes(T_loc: int, k: int, E: int, H: int, F: int, world: int) -> int:
    return lib().dk_moe_ep_workspace_bytes(T_loc, k, E, H, F, world)


def moe_ep_layer(x, logits, w13q, w13s, w2q, w2s, out, workspace_ptr: int, view, k: int, scale_mode: int = 0,
                 epoch: int = 0, phases: int = 15, counts_out=None, gemm_events=None, stream=None):
    """One expert-parallel MoE layer (dk_moe_ep_layer). `workspace_ptr` addresses
    moe_ep_workspace_bytes(...) bytes (inside the heap when the view has more than one rank)."""
    _need_cuda(x, logits, w13q, w13s, w2q, w2s, out)
    a = DkMoeEpArgs()
    a.T_loc, a.H = x.shape
    a.E = logits.shape[1]
    a.k = k
    a.F = w2q.shape[2]
    a.scale_mode = scale_mode
    a.x, a.logits = x.data_ptr(), logits.data_ptr()
    a.w13q, a.w13s, a.w2q, a.w2s = w13q.data_ptr(), w13s.data_ptr(), w2q.data_ptr(), w2s.data_ptr()
    a.out = out.data_ptr()
    a.workspace = workspace_ptr
    a.counts_out = counts_out.data_ptr() if counts_out is not None else None
    if gemm_events is not None:      # two torch.cuda.Event(enable_timing=True) that have been recorded once
        a.ev_gemm_begin, a.ev_gemm_end = gemm_events[0].cuda_event, gemm_events[1].cuda_event
    check(lib().dk_moe_ep_layer(C.byref(a), C.byref(view) if view is not None else None, epoch, phases,
                                _stream_ptr(stream)))
    return out


def peer_barrier(view: DkView, stream=None):
    check(lib().dk_peer_barrier(C.byref(view), _stream_ptr(stream)))


def allgather(mine, all_out, view: DkView, stream=None):
    """all_out (in the heap) = concatenation over ranks of `mine`."""
    _need_cuda(mine, all_out)
    check(lib().dk_allgather(_ptr(mine), mine.numel() * mine.element_size(), _ptr(all_out), C.byref(view),
                             _stream_ptr(stream)))
    return all_out


def moe_dispatch(x, topk_idx, row_of_pair, experts_per_rank: int, xrecv, view: DkView, sync: bool = True,
                 stream=None):
    _need_cuda(x, topk_idx, row_of_pair, xrecv)
    T_loc, k = topk_idx.shape
    check(lib().dk_moe_dispatch(_ptr(x), _ptr(topk_idx), _ptr(row_of_pair), T_loc, k, x.shape[1],
                                experts_per_rank, _ptr(xrecv), C.byref(view), 1 if sync else 0,
                                _stream_ptr(stream)))
    return xrecv


def moe_combine_ep(y, topk_idx, row_of_pair, topk_w, experts_per_rank: int, view: DkView, sync: bool = True,
                   stream=None):
    import torch
    _need_cuda(y, topk_idx, row_of_pair, topk_w)
    T_loc, k = topk_idx.shape
    H = y.shape[1]
    out = torch.empty((T_loc, H), dtype=torch.bfloat16, device=y.device)
    check(lib().dk_moe_combine_ep(_ptr(y), _ptr(topk_idx), _ptr(row_of_pair), _ptr(topk_w), T_loc, k, H,
                                  experts_per_rank, _ptr(out), C.byref(view), 1 if sync else 0,
                                  _stream_ptr(stream)))
    return out
