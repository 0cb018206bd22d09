"""The fp8 MoE FFN at the full layer sizes of the two MoE configurations, on a sample of experts.

Hidden and expert sizes are the configurations' own (Mixtral-shaped: hidden 4096, ffn 14336;
DeepSeek-V3-shaped: hidden 7168, expert inter 2048), so every tile walks the full K extent (32 / 112
and 56 / 16 K blocks) and the full row of column tiles. The CPU oracle cannot do all experts at this
size in seconds, so three experts are sampled: a hot one (two full 128-row tiles), an EMPTY one, and
a ragged one (200 rows, padded to 256). Gate/up + SiLU*mul + requantise, down, and combine are
compared with the block-dequantised fp32 oracle, <= 2e-2 relative Frobenius error, for both scale
formats (fp32 scales promoted in software; power-of-two scales applied by the tensor core).
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 2e-2

SHAPES = {"mixtral": (4096, 14336), "dsv3": (7168, 2048)}
ROWS = [256, 0, 200]          # pairs routed to the three sampled experts


def _inputs(capi, H, F, pow2):
    """Weights and activations drawn on the GPU and quantised with the library's quantisers (themselves
    bit-exact against the oracle, see test_moe_index_gpu / test_mx_gpu)."""
    g = torch.Generator(device="cuda").manual_seed(4)
    E = len(ROWS)
    offs = [0]
    for r in ROWS:
        offs.append(offs[-1] + (r + 127) // 128 * 128)
    R = offs[-1]
    x = torch.zeros(R, H, dtype=torch.bfloat16, device="cuda")
    valid = torch.zeros(R, dtype=torch.bool)
    for e, r in enumerate(ROWS):
        x[offs[e]:offs[e] + r] = torch.randn(r, H, device="cuda", generator=g).to(torch.bfloat16)
        valid[offs[e]:offs[e] + r] = True
    quant = capi.quant_block128_pow2 if pow2 else capi.quant_block128
    w13, w2 = [], []
    for _ in range(E):
        w13.append(quant((torch.randn(2 * F, H, device="cuda", generator=g) / math.sqrt(H)).to(torch.bfloat16)))
        w2.append(quant((torch.randn(H, F, device="cuda", generator=g) / math.sqrt(F)).to(torch.bfloat16)))
    xq = quant(x)
    st = lambda parts, i: torch.stack([p[i] for p in parts])
    return dict(offs=torch.tensor(offs, dtype=torch.int32), valid=valid, xq=xq, w13=[st(w13, i) for i in range(len(w13[0]))],
                w2=[st(w2, i) for i in range(len(w2[0]))])


@pytest.mark.parametrize("pow2", [False, True], ids=["fp32_scales", "pow2_scales"])
@pytest.mark.parametrize("shape", ["mixtral", "dsv3"])
def test_ffn_and_combine_at_full_layer_size(capi, orc, shape, pow2):
    H, F = SHAPES[shape]
    c = _inputs(capi, H, F, pow2)
    offs = c["offs"].cuda()
    if pow2:
        xq, xs, _, xa = c["xq"]
        w13q, w13s, _, w13a = c["w13"]
        w2q, w2s, _, w2a = c["w2"]
        y = capi.moe_ffn_mxfp8(xq, xa, w13q, w13a.reshape(-1, w13a.shape[-2], 512), w2q,
                               w2a.reshape(-1, w2a.shape[-2], 512), offs)
        ref = orc.moe_ffn_pow2_ref
    else:
        xq, xs = c["xq"]
        w13q, w13s = c["w13"]
        w2q, w2s = c["w2"]
        y = capi.moe_ffn_fp8(xq, xs, w13q, w13s, w2q, w2s, offs)
        ref = orc.moe_ffn_ref
    torch.cuda.synchronize()
    assert capi.device_status()[0] == 0
    want = ref(xq.cpu(), xs.cpu(), w13q.cpu(), w13s.cpu(), w2q.cpu(), w2s.cpu(), c["offs"])[0]
    got = y.float().cpu()
    valid = c["valid"]
    assert orc.rel_fro(got[valid], want[valid]) <= TOL
    # every 128-row tile by itself (an error confined to one tile would hide in the global norm)
    for r0 in range(0, got.shape[0], 128):
        v = valid[r0:r0 + 128]
        if v.any():
            assert orc.rel_fro(got[r0:r0 + 128][v], want[r0:r0 + 128][v]) <= TOL
    # combine over the sampled rows: token t owns rows t and T + t of the valid rows (k = 2)
    rows = valid.nonzero().flatten().to(torch.int32)
    T = rows.numel() // 2
    rop = torch.stack([rows[:T], rows[T:2 * T]], 1).contiguous()
    w = torch.rand(T, 2, generator=torch.Generator().manual_seed(3))
    w = w / w.sum(1, keepdim=True)
    out = capi.moe_combine(y, rop.cuda(), w.cuda())
    torch.cuda.synchronize()
    assert orc.rel_fro(out.float().cpu(), orc.moe_combine_ref(want, rop, w)) <= TOL
