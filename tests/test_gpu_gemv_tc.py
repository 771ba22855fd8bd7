"""The tensor-memory decode GEMV for matrices carved in 128 x 128 blocks (codes expanded straight
into tensor memory as the A operand) against the streaming kernel and a float64 product."""
import numpy as np
import pytest
import torch

import mortar_b200 as mb

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _dense(m):
    return torch.from_numpy(m.to_dense_codes()).double() * float(np.float32(m.scale))


@pytest.mark.parametrize("rows,planes", [(1, 3), (2, 3), (5, 3), (8, 2), (16, 1)])
@pytest.mark.parametrize("swiglu", [False, True])
def test_gemv_blocks_matches_float64(rows, planes, swiglu):
    out_f, in_f = (1024, 768) if swiglu else (640, 768)
    m = mb.synth.make_block_matrix(out_f, in_f, 0.4, seed=rows + 10 * planes)
    w = m.to_gemv_blocks(swiglu, DEV)
    x = mb.synth.make_activations(rows, in_f, seed=3, dtype=torch.float32).to(DEV)
    xp = mb.ops.act_prep(x, planes)
    xb = mb.ops.gemv_xprep(xp)
    y = mb.ops.gemv_blocks(w, xb, rows, planes)
    assert mb.ops.gemv_blocks_error() == 0
    xs = xp.double().sum(0).cpu()                       # what the planes represent
    full = xs @ _dense(m).T
    if swiglu:
        g, u = full[:, :out_f // 2], full[:, out_f // 2:]
        ref = g / (1 + torch.exp(-g)) * u
    else:
        ref = full
    tol = 1e-5 if planes == 3 else 2e-5
    assert float((y.cpu().double() - ref).abs().max()) <= tol * float(ref.abs().max())
    # and the streaming kernel on the same planes
    ys = mb.ops.linear_planes(m.to_stream(DEV), xp, swiglu=swiglu)
    assert float((y - ys).abs().max()) <= 1e-5 * float(ys.abs().max())
    # exact bf16 planes out: their sum is the fp32 result
    yp = mb.ops.gemv_blocks(w, xb, rows, planes, out_planes=3)
    assert float((yp.float().sum(0) - y).abs().max()) <= 1e-6 * float(y.abs().max())


def test_gemv_blocks_unfused_swiglu_for_unaligned_d_ff():
    """d_ff = 64 mod 128 (the published 30B shape has it): gate/up as a plain product, SwiGLU in the
    operand preparation of the down product."""
    d, f = 1024, 1984                                  # 1984 = 15.5 x 128
    gu_m = mb.synth.make_block_matrix(2 * f, d, 0.3, seed=4)
    dn_m = mb.synth.make_block_matrix(d, f + 64, 0.3, seed=5)      # in_features padded to a multiple of 128
    x = mb.synth.make_activations(2, d, seed=6, dtype=torch.float32).to(DEV)
    xp = mb.ops.act_prep(x, 3)
    gu32 = mb.ops.gemv_blocks(gu_m.to_gemv_blocks(False, DEV), mb.ops.gemv_xprep(xp), 2, 3)
    hb = mb.ops.gemv_xprep_swiglu(gu32, 3)
    hs = mb.ops.linear_planes(gu_m.to_stream(DEV), xp, swiglu=True, out_planes=3)
    ref_b = mb.ops.gemv_xprep(hs)
    hb_f = hb.view(torch.bfloat16).float().reshape(-1, 2, 2, 8, 8)      # [tile][col group][k half][col][k]
    rb_f = ref_b.view(torch.bfloat16).float().reshape(-1, 2, 2, 8, 8)
    # sums over the three planes (columns 2p + r) agree
    def total(t):
        cols = t.permute(0, 1, 3, 2, 4).reshape(-1, 16, 16)              # [tile][column][k]
        return cols[:, 0:6].reshape(-1, 3, 2, 16).sum(1)
    assert float((total(hb_f) - total(rb_f)).abs().max()) <= 1e-5 * float(total(rb_f).abs().max())
    with pytest.raises(ValueError):
        gu_m.to_gemv_blocks(True, DEV)                 # gate and up block rows do not pair up


def test_gemv_blocks_chain_large_shape():
    """gate/up with SwiGLU then down at an eighth of the published 30B shape, chained through planes."""
    d, f = 2048, 5632 - 5632 % 128 + 128 if 5632 % 128 else 5632
    gu_m = mb.synth.make_block_matrix(2 * f, d, 0.25, seed=1)
    dn_m = mb.synth.make_block_matrix(d, f, 0.25, seed=2)
    gu, dn = gu_m.to_gemv_blocks(True, DEV), dn_m.to_gemv_blocks(False, DEV)
    x = mb.synth.make_activations(1, d, seed=3, dtype=torch.float32).to(DEV)
    xp = mb.ops.act_prep(x, 3)
    hp = mb.ops.gemv_blocks(gu, mb.ops.gemv_xprep(xp), 1, 3, out_planes=3)
    y = mb.ops.gemv_blocks(dn, mb.ops.gemv_xprep(hp), 1, 3)
    assert mb.ops.gemv_blocks_error() == 0
    hs = mb.ops.linear_planes(gu_m.to_stream(DEV), xp, swiglu=True, out_planes=3)
    ys = mb.ops.linear_planes(dn_m.to_stream(DEV), hs, out_dtype=torch.float32)
    assert float((y - ys).abs().max()) <= 1e-5 * float(ys.abs().max())
