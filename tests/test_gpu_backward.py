"""Training backward of the carved linear: the weight gradient on the topology (sdd_at_b) and the
input gradient (dds on the transposed matrix), through the C ABI and through autograd of the
registered ``morph_stk::dds`` operator, against dense fp64 / autograd references."""
import numpy as np
import pytest
import torch

import mortar_b200 as mb
from test_gpu_parity import _assert_bf16_close

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("rows", [1, 50, 300])
def test_weight_gradient_tiles(rows):
    rng = np.random.default_rng(rows)
    R, C = 12, 9
    mask = rng.random((R, C)) < 0.4
    mask[3] = False                       # a tile row without tiles
    mask[4] = True                        # a full row (more than one work item)
    m = mb.MortarMatrix.from_codes(rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8), mask, 0.02)
    topo = mb.format.TopologyDev(m, DEV)
    dy = torch.randn(rows, R * 16, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    x = torch.randn(rows, C * 16, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16)
    tiles = mb.ops.sdd_tiles(dy.to(DEV), x.to(DEV), topo)
    full = dy.double().T @ x.double()                                   # [out, in]
    tr = np.repeat(np.arange(R), np.diff(m.row_ptr))
    ref = torch.stack([full[r * 16:(r + 1) * 16, c * 16:(c + 1) * 16] for r, c in zip(tr, m.col_idx.astype(int))])
    assert tiles.shape == (m.nnz, 16, 16)
    assert float((tiles.cpu().double() - ref).abs().max()) <= 1e-5 * max(float(ref.abs().max()), 1.0)
    tb = mb.ops.sdd_tiles(dy.to(DEV), x.to(DEV), topo, out_dtype=torch.bfloat16)
    assert torch.equal(tb, tiles.to(torch.bfloat16))


@pytest.mark.parametrize("rows", [64, 300, 1000, 4096])
@pytest.mark.parametrize("shape", ["ragged", "local"])
def test_weight_gradient_blocks(rows, shape):
    """The tensor-memory block kernel (whole 128 x 128 blocks of dW, kept tiles stored, token
    dimension split over CTAs) against the per-tile kernel and a float64 product: a ragged
    topology whose edges are not multiples of 128 features, and the local gate/up shape."""
    rng = np.random.default_rng(rows)
    if shape == "ragged":
        R, C = 21, 13                      # 336 x 208 features: partial blocks on both edges
        mask = rng.random((R, C)) < 0.4
        mask[3] = False
        mask[8:16, 8:13] = False           # a whole block without kept tiles
        m = mb.MortarMatrix.from_codes(rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8), mask, 0.02)
    else:
        m = mb.synth.make_layer(768, 2048, 0.25, seed=7).gate_up
        R, C = m.tile_rows, m.tile_cols
    topo = mb.format.TopologyDev(m, DEV)
    dy = torch.randn(rows, R * 16, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    x = torch.randn(rows, C * 16, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    blocks = mb.ops.sdd_tiles(dy, x, topo, path="blocks")
    assert mb.ops.sdd_error() == 0
    tiles = mb.ops.sdd_tiles(dy, x, topo, path="tiles")
    scale = max(float(tiles.abs().max()), 1.0)
    assert float((blocks - tiles).abs().max()) <= 2e-5 * scale
    if shape == "ragged":
        full = dy.double().T @ x.double()
        tr = np.repeat(np.arange(R), np.diff(m.row_ptr))
        ref = torch.stack([full[r * 16:(r + 1) * 16, c * 16:(c + 1) * 16] for r, c in zip(tr, m.col_idx.astype(int))])
        assert float((blocks.double() - ref).abs().max()) <= 1e-5 * scale
    # deterministic, and the bf16 output is the rounded fp32 one
    assert torch.equal(blocks, mb.ops.sdd_tiles(dy, x, topo, path="blocks"))
    assert torch.equal(mb.ops.sdd_tiles(dy, x, topo, out_dtype=torch.bfloat16, path="blocks"), blocks.to(torch.bfloat16))


@pytest.mark.parametrize("rows", [8, 256])
@pytest.mark.parametrize("blk", [16, 128])
def test_autograd_through_the_reference_operator(rows, blk):
    """loss = sum(w * dds(x, data, ...)): gradients wrt x and wrt the kept blocks, against autograd
    of the dense product on the same bf16 operands (the reference's dx = dds(dy, W) and
    dW = sdd_at_b(dy, x), custom_ops.py:91-133)."""
    out_f, in_f = 256, 384
    rng = np.random.default_rng(blk + rows)
    Rb, Cb = out_f // blk, in_f // blk
    bmask = rng.random((Rb, Cb)) < 0.5
    bmask[:, 0] = True
    idx = np.argwhere(bmask)
    off = np.concatenate([[0], np.cumsum(bmask.sum(1))]).astype(np.int32)
    ci = idx[:, 1].astype(np.int16)
    scale = torch.tensor(0.0173).to(torch.bfloat16).float()
    codes = torch.from_numpy(rng.integers(-1, 2, size=(len(idx), blk, blk)).astype(np.float32))
    data = (codes * scale).to(torch.bfloat16).to(DEV).requires_grad_(True)
    x = torch.randn(rows, in_f, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(DEV).requires_grad_(True)
    z = torch.zeros(1, dtype=torch.int16, device=DEV)
    offd, cid = torch.from_numpy(off).to(DEV), torch.from_numpy(ci).to(DEV)
    y = torch.ops.morph_stk.dds(x, data, offd, z, cid, z, z, z, in_f, out_f, True)
    wgt = torch.randn(rows, out_f, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).to(DEV)
    (y * wgt).sum().backward()
    # dense twin
    W = torch.zeros(out_f, in_f)
    for k, (r, c) in enumerate(idx):
        W[r * blk:(r + 1) * blk, c * blk:(c + 1) * blk] = codes[k] * scale
    Wd = W.to(torch.bfloat16).to(DEV).requires_grad_(True)
    xd = x.detach().clone().requires_grad_(True)
    yd = torch.nn.functional.linear(xd, Wd)
    _assert_bf16_close(y.detach(), yd.detach())
    (yd * wgt).sum().backward()
    _assert_bf16_close(x.grad, xd.grad, near_zero=1e-2)
    ref_blocks = torch.stack([Wd.grad[r * blk:(r + 1) * blk, c * blk:(c + 1) * blk] for r, c in idx])
    assert data.grad.shape == data.shape and data.grad.dtype == torch.bfloat16
    _assert_bf16_close(data.grad, ref_blocks, near_zero=1e-2)


def test_input_gradient_both_kernel_paths():
    """dx = dy @ W through the transposed matrix on the streaming and on the tensor-memory kernel."""
    L = mb.synth.make_layer(768, 2048, 0.25, seed=100)
    m = L.down                                      # [768, 2048]
    mt = m.transpose()
    W = torch.from_numpy(m.to_dense_codes()).float() * torch.tensor(m.scale).to(torch.bfloat16).float()
    for rows in (5, 300):
        dy = torch.randn(rows, 768, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16)
        ref = (dy.float() @ W.to(torch.bfloat16).float()).to(torch.bfloat16)
        got = mb.ops.linear(dy.to(DEV), mt.to_stream(DEV)) if rows < 128 else mb.ops.linear_tc(dy.to(DEV), mt.to_sched(False, DEV))
        _assert_bf16_close(got, ref, near_zero=1e-2)
