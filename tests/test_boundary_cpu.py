"""The drop-in boundary without a GPU: the library loads and exports every declared symbol, the
pybind11 modules import with the reference's names and error strings, the host bootstrap works
between processes."""
import ctypes as C
import multiprocessing as mp
import os
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols():
    names = set()
    for h in (ROOT / "include").glob("*.h"):
        names |= set(re.findall(r"\b(dk_[a-z0-9_]+)\s*\(", h.read_text()))
    return sorted(names)


def test_library_exports_every_declared_symbol(capi):
    L = capi.lib()
    syms = declared_symbols()
    assert len(syms) >= 20
    for s in syms:
        assert hasattr(L, s), f"{s} is declared in include/ but not exported"
    assert L.dk_version() >= 1000
    assert L.dk_strerror(0) == b"ok" and L.dk_strerror(3).startswith(b"device-side error record pending")


def test_bootstrap_env(capi, monkeypatch):
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE",
              "OMPI_COMM_WORLD_LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    assert capi.bootstrap_env() == (0, 1, 0)
    monkeypatch.setenv("OMPI_COMM_WORLD_RANK", "3")
    monkeypatch.setenv("OMPI_COMM_WORLD_SIZE", "4")
    assert capi.bootstrap_env() == (3, 4, 3)
    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("WORLD_SIZE", "2")
    monkeypatch.setenv("LOCAL_RANK", "0")
    assert capi.bootstrap_env() == (1, 2, 0)
    monkeypatch.setenv("RANK", "5")
    with pytest.raises(capi.DkError):
        capi.bootstrap_env()


def test_pybind_surface_matches_reference():
    import iris_py
    import tk_kernel
    for name in ("Iris", "Tensor", "IrisDeviceView", "mpi_init", "mpi_finalize"):
        assert hasattr(iris_py, name)
    for m in ("rank", "world_size", "empty", "barrier", "get_device_view"):
        assert hasattr(iris_py.Iris, m)
    for m in ("data_ptr", "shape", "dtype", "numel", "nbytes"):
        assert hasattr(iris_py.Tensor, m)
    for m in ("cur_rank", "world_size"):
        assert hasattr(iris_py.IrisDeviceView, m)
    assert iris_py.mpi_init() == (int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)))
    assert iris_py.mpi_finalize() is None
    assert hasattr(tk_kernel, "dispatch_micro") and hasattr(tk_kernel, "gemm_rs")


def test_dispatch_micro_argument_errors():
    """Same checks and messages as the reference's from_object (include/pyutils/pyutils.cuh:14-47)."""
    import torch
    import tk_kernel
    with pytest.raises(RuntimeError, match="Expected a torch.Tensor"):
        tk_kernel.dispatch_micro(1, 2, 3, None, 1, 1, 1, 0)
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        tk_kernel.dispatch_micro(torch.zeros(2, 2), torch.zeros(2, 2), torch.zeros(2, 2), None, 2, 2, 2, 0)
    with pytest.raises(RuntimeError, match="Tensor must be contiguous"):
        tk_kernel.dispatch_micro(torch.zeros(4, 4).t()[:, :2], 0, 0, None, 2, 2, 2, 0)
    with pytest.raises(TypeError):
        tk_kernel.dispatch_micro(torch.zeros(2, 2))  # positional arity is part of the contract
    # the single-GPU three-argument form (kernels/cdna4/gemm/bf16fp32/256_256_64_32_with16x32.cpp:335-339)
    with pytest.raises(RuntimeError, match="Expected a torch.Tensor"):
        tk_kernel.dispatch_micro(1, 2, 3)
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        tk_kernel.dispatch_micro(torch.zeros(2, 2), torch.zeros(2, 2), torch.zeros(2, 2))


def test_product_path_has_no_cpu_fallback(capi):
    """Without a GPU the operators must fail loudly, not compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    a = torch.zeros(128, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        capi.gemm_bf16(a, a)
    import iris_py
    with pytest.raises(RuntimeError):
        iris_py.Iris(16)


def test_argument_errors_need_no_gpu(capi):
    """Argument checks come before any CUDA call, so they answer the same with or without a GPU."""
    L = capi.lib()
    assert L.dk_heap_enable_multicast(None) == capi.ERR_ARG
    assert b"heap is null" in L.dk_last_error_string()
    assert L.dk_gemm_pair_mode(7) == capi.ERR_ARG
    assert L.dk_gemm_pair_mode(1) == 0
    L.dk_gemm_rs_workspace_bytes.restype = C.c_size_t
    assert L.dk_gemm_rs_workspace_bytes(8192, 8192, 1) == 0
    # 2 parities x 8 slots x 1024 rows x 8192 columns x 2 bytes of staging + 2 x 256 tiles x 8 flags
    assert L.dk_gemm_rs_workspace_bytes(8192, 8192, 8) == 2 * 8 * 1024 * 8192 * 2 + 2 * 256 * 8 * 4
    assert L.dk_gemm_rs_workspace_bytes(8192, 8192, 9) == 0          # more ranks than supported
    assert L.dk_allreduce(None, None, 8, -1, None, None) == capi.ERR_ARG
    assert L.dk_set_peer_wait_ms(0) == capi.ERR_ARG
    assert L.dk_set_peer_wait_ms(20000) == 0
    assert L.dk_set_walk_band_bytes(0) == capi.ERR_ARG
    assert L.dk_set_walk_band_bytes(32 << 20) == 0
    assert L.dk_mx_pair_mode(2) == capi.ERR_ARG and L.dk_mx_pair_mode(-1) == 0
    # the one-call MoE layer: shapes and scale modes are checked before anything is launched
    assert capi.moe_ep_workspace_bytes(256, 2, 8, 256, 128, 1) > 0
    assert capi.moe_ep_workspace_bytes(256, 2, 8, 200, 128, 1) == 0       # H not a multiple of 128
    assert capi.moe_ep_workspace_bytes(256, 2, 9, 256, 128, 2) == 0       # E not a multiple of world
    a = capi.DkMoeEpArgs()
    a.T_loc, a.k, a.E, a.H, a.F, a.scale_mode = 256, 2, 8, 256, 128, 3
    for f in ("x", "logits", "w13q", "w13s", "w2q", "w2s", "out", "workspace"):
        setattr(a, f, 4096)
    assert L.dk_moe_ep_layer(C.byref(a), None, 0, 15, None) == capi.ERR_ARG
    assert b"scale_mode" in L.dk_last_error_string()
    a.scale_mode = 2
    assert L.dk_moe_ep_layer(C.byref(a), None, 0, 16, None) == capi.ERR_ARG      # phases outside 1..15


# ---- host bootstrap between two processes (no GPU involved) -----------------------------------
def _comm_worker(rank, world, name, q):
    import sys
    sys.path.insert(0, str(ROOT))
    from __graft_entry__ import load_package
    capi = load_package().capi
    L = capi.lib()
    c = C.c_void_p()
    rc = L.dk_comm_create(rank, world, name.encode(), 20000, C.byref(c))
    if rc != 0:
        q.put((rank, "create failed", L.dk_last_error_string().decode()))
        return
    # blob all-gather
    mine = (C.c_int * 2)(rank, 100 + rank)
    allb = (C.c_int * (2 * world))()
    rc1 = L.dk_comm_allgather(c, mine, C.sizeof(mine), allb)
    # fd all-gather: every rank shares a memfd holding its rank
    fd = os.memfd_create(f"dk{rank}")
    os.write(fd, bytes([65 + rank]) * 8)
    fds = (C.c_int * world)()
    rc2 = L.dk_comm_allgather_fd(c, fd, fds)
    seen = []
    for r in range(world):
        seen.append(os.pread(fds[r], 8, 0))   # the descriptors share one file offset: no seek
        os.close(fds[r])
    rc3 = L.dk_comm_barrier(c)
    L.dk_comm_destroy(c)
    q.put((rank, (rc1, rc2, rc3), list(allb), seen))


@pytest.mark.parametrize("world", [2, 4])
def test_comm_rendezvous_fd_exchange_barrier(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    name = f"pytest.{os.getpid()}.{world}"
    ps = [ctx.Process(target=_comm_worker, args=(r, world, name, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = [q.get(timeout=60) for _ in ps]
    for p in ps:
        p.join(30)
    for rank, rcs, blob, seen in res:
        assert rcs == (0, 0, 0), (rank, rcs, blob)
        assert blob == [v for r in range(world) for v in (r, 100 + r)]
        assert seen == [bytes([65 + r]) * 8 for r in range(world)]


def _lonely_worker(name, q):
    import sys
    sys.path.insert(0, str(ROOT))
    from __graft_entry__ import load_package
    L = load_package().capi.lib()
    c = C.c_void_p()
    rc = L.dk_comm_create(0, 2, name.encode(), 500, C.byref(c))
    q.put((rc, L.dk_last_error_string().decode()))


def test_comm_missing_rank_times_out_with_an_error():
    """Failure detection on the host: a rank that never joins ends the rendezvous with an error
    code after the timeout instead of hanging."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_worker, args=(f"pytest.lonely.{os.getpid()}", q))
    p.start()
    rc, msg = q.get(timeout=30)
    p.join(10)
    assert rc == 4 and "timed out" in msg


def test_comm_drops_a_connection_with_the_wrong_token_and_still_forms(capi, monkeypatch):
    """Whoever joins the rendezvous receives the descriptors of every rank's heap, so rank 0 accepts
    only its own user's processes whose hello carries the job's token (DK_JOB_TOKEN). An intruder with
    the wrong token (and one that says nothing) is dropped; the job still forms."""
    import socket
    import struct
    import threading
    monkeypatch.setenv("DK_JOB_TOKEN", "secret-of-this-job")
    L = capi.lib()
    name = f"tok{os.getpid()}"
    res = {}

    def rank(r):
        h = C.c_void_p()
        res[r] = L.dk_comm_create(r, 2, name.encode(), 15000, C.byref(h))
        if res[r] == 0:
            res[f"b{r}"] = L.dk_comm_barrier(h)
            L.dk_comm_destroy(h)

    t0 = threading.Thread(target=rank, args=(0,))
    t0.start()
    addr = "\0dk_b200." + name
    silent = None
    for _ in range(400):                    # wait for rank 0 to listen
        try:
            silent = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            silent.connect(addr)
            break
        except OSError:
            silent.close()
            silent = None
            import time
            time.sleep(0.01)
    assert silent is not None               # connected, and never says a word
    bad = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    bad.connect(addr)
    bad.sendall(struct.pack("<iIQ", 1, 0x646b3230, 12345))      # rank 1, right magic, wrong token
    t1 = threading.Thread(target=rank, args=(1,))
    t1.start()
    t0.join(30)
    t1.join(30)
    assert res.get(0) == 0 and res.get(1) == 0 and res.get("b0") == 0 and res.get("b1") == 0
    bad.settimeout(2)
    assert bad.recv(1) == b""               # rank 0 closed the intruder's connection
    bad.close()
    silent.close()


def test_comm_needs_a_job_name(capi, monkeypatch):
    for k in ("DK_JOB_ID", "MASTER_PORT"):
        monkeypatch.delenv(k, raising=False)
    h = C.c_void_p()
    assert capi.lib().dk_comm_create(0, 2, None, 500, C.byref(h)) == capi.ERR_BOOTSTRAP
    assert b"DK_JOB_ID" in capi.lib().dk_last_error_string()


def test_host_log_levels(capi, capfd):
    """DK_LOG / dk_set_log_level: silent by default, level 2 reports each rank that joins a
    rendezvous on stderr, one "[dk_b200] ..." line each."""
    import threading
    L = capi.lib()
    assert L.dk_set_log_level(3) == capi.ERR_ARG and L.dk_set_log_level(-1) == capi.ERR_ARG

    def job(name):
        def rank(r):
            h = C.c_void_p()
            if L.dk_comm_create(r, 2, name.encode(), 15000, C.byref(h)) == 0:
                L.dk_comm_destroy(h)
        ts = [threading.Thread(target=rank, args=(r,)) for r in range(2)]
        [t.start() for t in ts]
        [t.join(30) for t in ts]

    assert L.dk_set_log_level(0) == 0
    job(f"log0{os.getpid()}")
    assert "[dk_b200]" not in capfd.readouterr().err
    assert L.dk_set_log_level(2) == 0
    try:
        job(f"log2{os.getpid()}")
    finally:
        L.dk_set_log_level(0)
    err = capfd.readouterr().err
    assert "[dk_b200] rendezvous" in err and "rank 1 joined" in err
