"""Generates the golden fixtures in this directory. Run from the repository root:

    python tests/golden/make_golden.py

gemm_example.npz restates the only check the reference holds on this path, the example of
distributed-kernels/bf16_gemm/example.py: inputs drawn with its seeds and initialisation
(lines 93-96: torch.manual_seed(1234+rank) for A, 0 for B, bf16 randn / 10), reference output
torch.matmul(A, B.t()) in bf16 (line 105), acceptance max|C - C_ref| < 0.1 (lines 119-121).
The example itself cannot run here (it imports the HIP-built iris_py / tk_kernel), so the vectors
come from its formula evaluated by torch on the CPU of the build container.

moe_small.npz holds outputs of the oracle's routing / permutation / block quantisation on a small
seeded case. The reference has no such code, so these pin the oracle against drift, not against
the reference.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import dk_oracle as orc  # noqa: E402

OUT = Path(__file__).resolve().parent


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main():
    M_local, N, K = 128, 256, 128
    fx = {}
    for rank in (0, 1):
        A, B = orc.example_inputs(M_local, N, K, rank=rank)
        C_ref = torch.matmul(A, B.t())
        fx[f"A{rank}"] = bits(A)
        fx[f"C{rank}"] = bits(C_ref)
        fx["B"] = bits(B)
    np.savez_compressed(OUT / "gemm_example.npz", **fx)

    T, H, E, k = 64, 256, 8, 2
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(T, E, generator=g)
    logits[3, 1] = logits[3, 5]          # a tie: the lower index must win
    idx, w = orc.moe_route(logits, k)
    rop, por, offs, counts = orc.moe_permute(idx, E, 128)
    x = torch.randn(256, H, generator=g).to(torch.bfloat16)
    x[:128, :128] = 0                      # an all-zero block: scale must be 1
    q, s = orc.quant_block128(x)
    np.savez_compressed(OUT / "moe_small.npz", logits=logits.numpy(), topk_idx=idx.numpy(),
                        topk_w=w.numpy(), row_of_pair=rop.numpy(), pair_of_row=por.numpy(),
                        offsets=offs.numpy(), counts=counts.numpy(), x=bits(x), q=q.numpy(),
                        s=s.numpy())
    print("wrote", [p.name for p in OUT.glob("*.npz")])


if __name__ == "__main__":
    main()
