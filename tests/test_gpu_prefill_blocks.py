"""The block path of the prefill kernels (topologies carved at 128 x 128: expanded blocks as plain
tensor-core operands, pairs of block rows, two accumulator sets) against the CPU oracle, the tile
path and the golden fixture made by the reference at blocking 128."""
import numpy as np
import pytest
import torch

import mortar_b200 as mb
from conftest import bf16_from_bits, load_golden
from oracle import mortar_oracle as orc
from test_gpu_parity import _assert_bf16_close, _dense

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _clean():
    assert mb.ops.prefill_error() == 0, "a bounded wait in the prefill kernel expired"


@pytest.fixture(params=["single", "pairs"])
def kernel_mode(request):
    """Both kernels of the block path at every size (by default the row count chooses)."""
    prev = mb.ops.linear_blocks_mode(request.param)
    yield request.param
    mb.ops.linear_blocks_mode(prev)


@pytest.mark.parametrize("rows", [1, 100, 128, 300, 1000])
def test_linear_blocks_ragged(rows, kernel_mode):
    """edges that are not multiples of 128, an empty block row, an odd number of block rows, blocks
    with dropped tiles inside."""
    rng = np.random.default_rng(7)
    R, C = 43, 21                                      # 688 x 336 features: 6 x 3 blocks with ragged edges
    mask = np.zeros((R, C), dtype=bool)
    for rb, cb in [(0, 0), (0, 2), (1, 1), (3, 0), (3, 1), (3, 2), (4, 2), (5, 0), (5, 2)]:   # block row 2 is empty
        mask[rb * 8:(rb + 1) * 8, cb * 8:(cb + 1) * 8] = True
    mask[1, 2] = False                                 # a dropped tile inside a kept block
    mask[30:32, 20] = False
    codes = rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8)
    m = mb.MortarMatrix.from_codes(codes, mask, 0.0173)
    x = torch.randn(rows, C * 16, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16)
    y = mb.ops.linear_blocks(x.to(DEV), m.to_blocks(False, DEV))
    _clean()
    W = torch.from_numpy(m.to_dense_codes()).float() * torch.tensor(0.0173).to(torch.bfloat16).float()
    ref = torch.nn.functional.linear(x, W.to(torch.bfloat16))
    _assert_bf16_close(y, ref)
    assert float(y[:, 256:384].float().abs().max()) == 0.0           # the empty block row


@pytest.mark.parametrize("rows", [128, 391, 2048])
def test_mlp_blocks_cloud_shape_vs_oracle_and_tile_path(rows, kernel_mode):
    d, f = 2048, 5632
    gu_m = mb.synth.make_block_matrix(2 * f, d, 0.25, seed=11)
    dn_m = mb.synth.make_block_matrix(d, f, 0.25, seed=12)
    assert mb.format.block_fill(gu_m) == 1.0
    x = mb.synth.make_activations(rows, d, seed=rows).to(DEV)
    bg, bd = gu_m.to_blocks(True, DEV), dn_m.to_blocks(False, DEV)
    y = mb.ops.mlp_prefill_blocks(x, bg, bd)
    _clean()
    ref = orc.swiglu_mlp(x.cpu().float(), _dense(gu_m), _dense(dn_m), dtype=torch.bfloat16)
    _assert_bf16_close(y, ref, near_zero=1e-2)
    # exact integer activations: both paths must agree bit for bit (every sum is exact)
    xi = torch.randint(-3, 4, (rows, d), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    hb = mb.ops.linear_blocks(xi, gu_m.to_blocks(False, DEV))
    ht = mb.ops.linear_tc(xi, gu_m.to_sched(False, DEV))
    assert torch.equal(hb, ht)
    ncls = f // 16
    L = type("L", (), {"gate_up": gu_m, "down": dn_m, "d_ff": f, "d_model": d})
    gates = mb.synth.make_gates(rows, L, ncls, ncls // 4, seed=3).to(DEV)
    yg = mb.ops.mlp_prefill_blocks(x, bg, bd, gates=gates, n_clusters=ncls)
    refg = orc.swiglu_mlp(x.cpu().float(), _dense(gu_m), _dense(dn_m), gates.cpu(), ncls, dtype=torch.bfloat16)
    _assert_bf16_close(yg, refg, near_zero=1e-2)
    _clean()
    # token blocks are independent: a 128-row slice gives the same bits, from either kernel
    if rows >= 256:
        assert torch.equal(mb.ops.mlp_prefill_blocks(x[128:256], bg, bd), y[128:256])
        mb.ops.linear_blocks_mode("pairs" if kernel_mode == "single" else "single")
        assert torch.equal(mb.ops.mlp_prefill_blocks(x[128:256], bg, bd), y[128:256])
        assert torch.equal(mb.ops.mlp_prefill_blocks(x, bg, bd), y)
        mb.ops.linear_blocks_mode(kernel_mode)


@pytest.mark.parametrize("rows", [130, 300])
def test_mlp_blocks_hidden_width_not_a_multiple_of_128(rows, kernel_mode):
    """d_ff = 448: the gate and the up half are cut into blocks from their own first rows, the last
    block row of each half is half empty, and so is the last block column of the down matrix."""
    d, f = 256, 448
    L = mb.synth.make_layer(d, f, 0.3, seed=13)
    x = mb.synth.make_activations(rows, d, seed=rows).to(DEV)
    bg, bd = L.gate_up.to_blocks(True, DEV), L.down.to_blocks(False, DEV)
    assert bg.n_pairs == 4 and bg.n_out == f
    y = mb.ops.mlp_prefill_blocks(x, bg, bd)
    _clean()
    ref = orc.swiglu_mlp(x.cpu().float(), _dense(L.gate_up), _dense(L.down), dtype=torch.bfloat16)
    _assert_bf16_close(y, ref, near_zero=1e-2)
    ncls = f // 16
    gates = mb.synth.make_gates(rows, L, ncls, ncls // 4, seed=3).to(DEV)
    yg = mb.ops.mlp_prefill_blocks(x, bg, bd, gates=gates, n_clusters=ncls)
    refg = orc.swiglu_mlp(x.cpu().float(), _dense(L.gate_up), _dense(L.down), gates.cpu(), ncls, dtype=torch.bfloat16)
    _assert_bf16_close(yg, refg, near_zero=1e-2)
    # the hidden block itself, against the per-tile path bit for bit on exact integer activations
    xi = torch.randint(-3, 4, (rows, d), generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).to(DEV)
    assert torch.equal(mb.ops.linear_blocks(xi, L.gate_up.to_blocks(False, DEV)),
                       mb.ops.linear_tc(xi, L.gate_up.to_sched(False, DEV)))
    _clean()


def test_blocks_at_the_large_model_shape_match_the_tile_path():
    """The shape of the reference's large-model decode bench (d_model 8192, d_ff 21824 -- not a
    multiple of 128 --, 25% ragged 128-blocks): step lists beyond the shared-memory cache, padded last
    block rows, 5456 blocks.  On exact integer activations every sum is exact, so the block path and
    the per-tile path (itself checked against the oracle at small sizes) must agree bit for bit."""
    d, f, rows = 8192, 21824, 256
    gu_m = mb.synth.make_block_matrix(2 * f, d, 0.25, seed=1)
    dn_m = mb.synth.make_block_matrix(d, f, 0.25, seed=2)
    xi = torch.randint(-2, 3, (rows, d), generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).to(DEV)
    bg = gu_m.to_blocks(False, DEV)
    assert bg.n_steps > 1024
    g_blocks = mb.ops.linear_blocks(xi, bg)
    g_tiles = mb.ops.linear_tc(xi, gu_m.to_sched(False, DEV))
    _clean()
    assert torch.equal(g_blocks, g_tiles)
    del bg, g_blocks, g_tiles
    hi = torch.randint(-2, 3, (rows, f), generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).to(DEV)
    assert torch.equal(mb.ops.linear_blocks(hi, dn_m.to_blocks(False, DEV)), mb.ops.linear_tc(hi, dn_m.to_sched(False, DEV)))
    _clean()
    # the fused MLP: SwiGLU pairing with the padded last block row of each half
    x = mb.synth.make_activations(rows, d, seed=6).to(DEV)
    yb = mb.ops.mlp_prefill_blocks(x, gu_m.to_blocks(True, DEV), dn_m.to_blocks(False, DEV))
    yt = mb.ops.mlp_prefill_tc(x, gu_m.to_sched(True, DEV), dn_m.to_sched(False, DEV))
    _clean()
    _assert_bf16_close(yb, yt.cpu(), near_zero=1e-2)


def test_step_list_larger_than_the_shared_memory_cache(kernel_mode):
    """More than 1024 steps: the roles read the step list from global memory instead of the copy in
    shared memory."""
    m = mb.synth.make_block_matrix(16384, 2176, 1.0, seed=21)
    b = m.to_blocks(False, DEV)
    assert b.n_steps > 1024
    x = mb.synth.make_activations(256, 2176, seed=9).to(DEV)
    y = mb.ops.linear_blocks(x, b)
    _clean()
    W = torch.from_numpy(m.to_dense_codes()).float() * torch.tensor(m.scale).to(torch.bfloat16).float()
    ref = torch.nn.functional.linear(x.cpu(), W.to(torch.bfloat16))
    _assert_bf16_close(y, ref)


def test_blocks_golden_fixture_and_module_dispatch():
    """The reference's own 128-blocking carve (fixture made by running it) through the block path, and
    the module forward choosing that path by itself."""
    g = load_golden("mlp_blk128_d256")
    if g is not None:
        d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
        assert blk == 128
        mats = {}
        for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
            mats[tag] = mb.MortarMatrix.from_reference_bcsr(
                g[f"{tag}_offsets"], g[f"{tag}_column_indices"], g[f"{tag}_packed"],
                float(g[f"{tag}_scale"]), blk, O, I)
        if d_ff % 128 == 0:
            x = bf16_from_bits(g["x_bf16"])
            y = mb.ops.mlp_prefill_blocks(x.to(DEV), mats["gu"].to_blocks(True, DEV), mats["dn"].to_blocks(False, DEV))
            _clean()
            _assert_bf16_close(y, bf16_from_bits(g["y_bf16"]))
    gu_m = mb.synth.make_block_matrix(2 * 512, 256, 0.5, seed=1)
    dn_m = mb.synth.make_block_matrix(256, 512, 0.5, seed=2)
    mlp = mb.SwiGLUMortar.from_matrices(gu_m, dn_m, device=DEV)
    x = mb.synth.make_activations(256, 256, seed=4).to(DEV)
    n0 = mb.ops.kernel_counts().get("prefill_blocks", 0)
    y = mlp(x)
    assert mb.ops.kernel_counts()["prefill_blocks"] - n0 == 2
    ref = orc.swiglu_mlp(x.cpu().float(), _dense(gu_m), _dense(dn_m), dtype=torch.bfloat16)
    _assert_bf16_close(y, ref, near_zero=1e-2)
    # the registered operators on raw tensors, eager and through a fake-tensor trace
    bg, bd = gu_m.to_blocks(True, DEV), dn_m.to_blocks(False, DEV)
    a, b = mb.torch_ops.blocks_args(bg), mb.torch_ops.blocks_args(bd)
    y_op = torch.ops.mortar_b200.mlp_prefill_blocks(x, *a[:5], a[6], *b[:5], b[6], None, 0)
    assert torch.equal(y_op, y)
    h_op = torch.ops.mortar_b200.linear_blocks(x, *a, None, 0)
    assert torch.equal(h_op, mb.ops.linear_blocks(x, bg))
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode(allow_non_fake_inputs=True):
        fy = torch.ops.mortar_b200.mlp_prefill_blocks(torch.empty(300, 256, dtype=torch.bfloat16, device=DEV),
                                                      *a[:5], a[6], *b[:5], b[6], None, 0)
    assert tuple(fy.shape) == (300, 256) and fy.dtype == torch.bfloat16
    # a sparse tile-16 topology keeps the per-tile path
    L = mb.synth.make_layer(1024, 512, 0.02, seed=3)
    assert max(mb.format.block_fill(L.gate_up), mb.format.block_fill(L.down)) < mb.format.BLOCK_PATH_MIN_FILL
    mlp2 = mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=DEV)
    n1 = mb.ops.kernel_counts().get("prefill_panel", 0)
    mlp2(mb.synth.make_activations(256, 1024, seed=6).to(DEV))
    assert mb.ops.kernel_counts()["prefill_panel"] - n1 == 2
    # the reference operator on a 128-carved layer takes the block path too
    z = torch.zeros(1, dtype=torch.int16, device=DEV)
    Rb, Cb = 256 // 128, 512 // 128
    rows = np.repeat(np.arange(dn_m.tile_rows), np.diff(dn_m.row_ptr))
    kept = np.zeros((Rb, Cb), dtype=bool)
    kept[rows // 8, dn_m.col_idx.astype(int) // 8] = True
    idx = np.argwhere(kept)
    dense = torch.from_numpy(dn_m.to_dense_codes()).float() * torch.tensor(dn_m.scale).to(torch.bfloat16).float()
    data = torch.stack([dense[r * 128:(r + 1) * 128, c * 128:(c + 1) * 128] for r, c in idx]).to(torch.bfloat16).to(DEV)
    off = torch.from_numpy(np.concatenate([[0], np.cumsum(kept.sum(1))]).astype(np.int32)).to(DEV)
    ci = torch.from_numpy(idx[:, 1].astype(np.int16)).to(DEV)
    hx = mb.synth.make_activations(256, 512, seed=5).to(DEV)
    n2 = mb.ops.kernel_counts().get("prefill_blocks", 0)
    yd = torch.ops.morph_stk.dds(hx, data, off, z, ci, z, z, z, 512, 256, True)
    assert mb.ops.kernel_counts()["prefill_blocks"] - n2 == 1
    assert torch.equal(yd, mb.ops.linear_blocks(hx, dn_m.to_blocks(False, DEV)))
