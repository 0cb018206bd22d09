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
    for name in dir(L):
        pass
    # optional symbols are declared by the modules that use them (see declare_optional)


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
