"""torch.library custom operators over the `tk_kernel` entry points.

The reference binds its kernels as plain pybind11 callables that read raw pointers out of the
tensors (include/pyutils/pyutils.cuh:54-71: bind_kernel / bind_function). That is kept (the
`tk_kernel` module); this file adds what the PyTorch dispatcher needs to see the same operations:
a schema, which arguments are written, and a shape function, so that they can appear in traced or
compiled graphs, run under FakeTensorMode, and be checked with torch.library.opcheck. The
implementations are the CUDA kernels and nothing else: every operator is registered for the CUDA
device only and raises on any other (there is no CPU fallback).

A device view crosses the dispatcher as its address (`iris.get_device_view()._addr()`, an int;
0 = single GPU), because operator arguments must be tensors or plain scalars.

    import distributed_hipkittens_b200.torch_ops   # registers torch.ops.dk_b200.*
    C = torch.ops.dk_b200.gemm(A, Bt)
    torch.ops.dk_b200.gemm_rs(A, Bt, out, view._addr())
"""
from __future__ import annotations

import sys
from pathlib import Path
from typing import Tuple

import torch

_PKG = Path(__file__).resolve().parent
if str(_PKG) not in sys.path:
    sys.path.insert(0, str(_PKG))

NS = "dk_b200"


def _tk():
    import tk_kernel          # the CUDA extension; importing it fails loudly when it has not been built
    return tk_kernel


class _View:
    """What tk_kernel expects of a view argument: an object whose _addr() is the dk_view's address."""

    def __init__(self, addr: int):
        self._a = int(addr)

    def _addr(self) -> int:
        return self._a


def _view(addr: int):
    return _View(addr) if addr else None


# ---------------------------------------------------------------------------------------- GEMMs
@torch.library.custom_op(f"{NS}::gemm", mutates_args=(), device_types="cuda")
def gemm(A: torch.Tensor, Bt: torch.Tensor) -> torch.Tensor:
    """C[M,N] = A[M,K] @ Bt[N,K]^T, bf16 in/out, fp32 accumulate (tk_kernel.dispatch_micro)."""
    C = torch.empty((A.shape[0], Bt.shape[0]), dtype=torch.bfloat16, device=A.device)
    _tk().dispatch_micro(A, Bt, C)
    return C


@gemm.register_fake
def _(A, Bt):
    torch._check(A.dim() == 2 and Bt.dim() == 2 and A.shape[1] == Bt.shape[1], lambda: "A [M,K] and Bt [N,K] expected")
    return A.new_empty((A.shape[0], Bt.shape[0]), dtype=torch.bfloat16)


@torch.library.custom_op(f"{NS}::gemm_rs", mutates_args=("out",), device_types="cuda")
def gemm_rs(A: torch.Tensor, Bt: torch.Tensor, out: torch.Tensor, view: int) -> None:
    """out[M/P,N] = reduce-scatter over ranks of A[M,K/P] @ Bt[N,K/P]^T (tk_kernel.gemm_rs)."""
    _tk().gemm_rs(A, Bt, out, _view(view))


@gemm_rs.register_fake
def _(A, Bt, out, view):
    torch._check(A.shape[1] == Bt.shape[1] and out.shape[1] == Bt.shape[0], lambda: "shapes disagree")


@torch.library.custom_op(f"{NS}::ag_gemm", mutates_args=("out",), device_types="cuda")
def ag_gemm(A_shard: torch.Tensor, Bt: torch.Tensor, out: torch.Tensor, view: int) -> None:
    """out[M,N] = (all-gather over ranks of A_shard[M/P,K]) @ Bt[N,K]^T (tk_kernel.ag_gemm)."""
    _tk().ag_gemm(A_shard, Bt, out, _view(view))


@ag_gemm.register_fake
def _(A_shard, Bt, out, view):
    torch._check(A_shard.shape[1] == Bt.shape[1] and out.shape[1] == Bt.shape[0], lambda: "shapes disagree")


@torch.library.custom_op(f"{NS}::allreduce", mutates_args=("out",), device_types="cuda")
def allreduce(x: torch.Tensor, out: torch.Tensor, view: int, algo: int = -1) -> None:
    """out = sum over ranks of x (bf16); x inside the symmetric heap (tk_kernel.allreduce)."""
    _tk().allreduce(x, out, _view(view), algo)


@allreduce.register_fake
def _(x, out, view, algo=-1):
    torch._check(x.numel() == out.numel(), lambda: "x and out must hold the same number of elements")


# ---------------------------------------------------------------------------------------- MXFP8
@torch.library.custom_op(f"{NS}::mx_quant", mutates_args=(), device_types="cuda")
def mx_quant(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(e4m3 bytes [R,K], e8m0 scales [R,K/32], scale atoms [ceil(R/128),K/128,512])."""
    return tuple(_tk().mx_quant(x))


@mx_quant.register_fake
def _(x):
    R, K = x.shape
    torch._check(K % 128 == 0, lambda: "K must be a multiple of 128")
    u8 = dict(dtype=torch.uint8)
    return x.new_empty((R, K), **u8), x.new_empty((R, K // 32), **u8), x.new_empty(((R + 127) // 128, K // 128, 512), **u8)


@torch.library.custom_op(f"{NS}::gemm_mxfp8", mutates_args=(), device_types="cuda")
def gemm_mxfp8(Aq: torch.Tensor, Asf: torch.Tensor, Bq: torch.Tensor, Bsf: torch.Tensor,
               out_f32: bool = False) -> torch.Tensor:
    """C[M,N] = dequant(A) @ dequant(B)^T from e4m3 bytes and 1x32 e8m0 scale atoms."""
    return _tk().gemm_mxfp8(Aq, Asf, Bq, Bsf, out_f32)


@gemm_mxfp8.register_fake
def _(Aq, Asf, Bq, Bsf, out_f32=False):
    torch._check(Aq.shape[1] == Bq.shape[1], lambda: "A and B disagree on K")
    return Aq.new_empty((Aq.shape[0], Bq.shape[0]), dtype=torch.float32 if out_f32 else torch.bfloat16)


# ---------------------------------------------------------------------------------------- MoE
@torch.library.custom_op(f"{NS}::moe_route", mutates_args=(), device_types="cuda")
def moe_route(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(topk_idx int32 [T,k], topk_w fp32 [T,k])."""
    return tuple(_tk().moe_route(logits, k))


@moe_route.register_fake
def _(logits, k):
    T = logits.shape[0]
    return logits.new_empty((T, k), dtype=torch.int32), logits.new_empty((T, k), dtype=torch.float32)


@torch.library.custom_op(f"{NS}::moe_layer", mutates_args=("out", "workspace"), device_types="cuda")
def moe_layer(x: torch.Tensor, logits: torch.Tensor, k: int, w13q: torch.Tensor, w13s: torch.Tensor,
              w2q: torch.Tensor, w2s: torch.Tensor, out: torch.Tensor, workspace: torch.Tensor, view: int,
              scale_mode: int = 0, device_epoch: bool = False) -> None:
    """One expert-parallel fp8 MoE layer in one call (tk_kernel.moe_layer_ep). device_epoch: keep the
    call number on the device, which makes the call replayable from a CUDA graph."""
    _tk().moe_layer_ep(x, logits, k, w13q, w13s, w2q, w2s, out, workspace, _view(view), scale_mode, None,
                       device_epoch)


@moe_layer.register_fake
def _(x, logits, k, w13q, w13s, w2q, w2s, out, workspace, view, scale_mode=0, device_epoch=False):
    torch._check(x.shape == out.shape and x.shape[0] == logits.shape[0], lambda: "shapes disagree")


OPS = ("gemm", "gemm_rs", "ag_gemm", "allreduce", "mx_quant", "gemm_mxfp8", "moe_route", "moe_layer")
