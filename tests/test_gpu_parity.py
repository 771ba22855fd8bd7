"""Parity of the CUDA path (through the C ABI) against the CPU oracle and the golden
fixtures.  Needs a B200."""
import numpy as np
import pytest
import torch

import mortar_b200 as mb
from conftest import GOLDEN_CASES, bf16_from_bits, load_golden
from oracle import mortar_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"

# fp32 (decode) semantics: reassociation noise only
F32_TOL = 1e-5
# bf16 (prefill) semantics: the official tolerance of the path ...
BF16_RTOL, BF16_ATOL = 1e-2, 1e-3


def _assert_bf16_close(y: torch.Tensor, ref: torch.Tensor, near_zero: float = 4e-3):
    """... and the internal gate: an output may differ from the oracle only where an fp32 sum
    landed on a bf16 rounding boundary -- by at most two bf16 steps of its own magnitude, or
    (for outputs that cancel to nearly zero) by 4e-3 of the output RMS, the size of one-step
    flips of a few hidden activations -- and only a small fraction of outputs may differ.
    `near_zero` is that allowance in units of the output RMS.  The flips add up like a random walk
    over the terms of an output, so tests over 10^7 outputs (further out on the tail) and
    row-clustered topologies (outputs with several times the average number of terms) pass 1e-2."""
    y, ref = y.cpu().reshape(-1).float(), ref.cpu().reshape(-1).float()
    torch.testing.assert_close(y, ref, rtol=BF16_RTOL, atol=BF16_ATOL)
    rms = float(ref.pow(2).mean().sqrt())
    bound = torch.maximum(ref.abs() * 2.0 ** -7, torch.full_like(ref, near_zero * rms))
    excess = ((y - ref).abs() - bound).max()
    assert float(excess) <= 0, f"error exceeds two bf16 steps by {float(excess):.3e} (rms {rms:.3e})"
    frac = float((y != ref).float().mean())
    assert frac < 0.02, f"{frac:.4f} of outputs differ"


def _oracle_meta(m):
    rows = np.repeat(np.arange(m.tile_rows), np.diff(m.row_ptr))
    codes = torch.from_numpy(
        np.ascontiguousarray(orc.unpack_ternary(m.codes.reshape(-1), m.nnz * 256).reshape(m.nnz, 16, 16)))
    meta = (torch.from_numpy(rows), torch.from_numpy(m.col_idx.astype(np.int64)),
            m.out_features, m.in_features)
    return codes, meta


def _decode_oracle(x, layer, gates=None, ncls=0, rms_w=None):
    cg, mg = _oracle_meta(layer.gate_up)
    cd, md = _oracle_meta(layer.down)
    return orc.swiglu_mlp_decode(x.float(), cg, torch.tensor(layer.gate_up.scale), mg, cd,
                                 torch.tensor(layer.down.scale), md, gates, ncls, rms_w)


def _dense(m, bf16_scale=True):
    c, meta = _oracle_meta(m)
    return orc.mortar_dense(c, torch.tensor(m.scale), meta[0], meta[1], meta[2], meta[3], bf16_scale)


@pytest.fixture(scope="module")
def local_layer():
    L = mb.synth.make_layer(768, 2048, 0.25, seed=100)
    return L, L.gate_up.to_stream(DEV), L.down.to_stream(DEV)


@pytest.mark.parametrize("B", [1, 3, 8, 13, 64])
@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float32])
def test_mlp_decode_fp32_semantics(local_layer, B, in_dtype):
    L, gu, dn = local_layer
    x = mb.synth.make_activations(B, 768, seed=B).to(in_dtype)
    y = mb.ops.mlp_decode(x.to(DEV), gu, dn, n_planes=3, out_dtype=torch.float32)
    ref = _decode_oracle(x, L)
    assert float((y.cpu() - ref).abs().max()) <= F32_TOL * float(ref.abs().max())


@pytest.mark.parametrize("B", [1, 8, 64])
def test_mlp_decode_rmsnorm_and_gates(local_layer, B):
    L, gu, dn = local_layer
    gen = torch.Generator().manual_seed(77 + B)
    x = torch.randn(B, 768, generator=gen) * 3.0
    rms_w = 1.0 + 0.1 * torch.randn(768, generator=gen)
    ncls, k = 16, 8
    gates = mb.synth.make_gates(B, L, ncls, k, seed=5 + B)
    y = mb.ops.mlp_decode(x.to(DEV), gu, dn, rms_weight=rms_w.to(DEV), eps=1e-6, gates=gates.to(DEV),
                          n_clusters=ncls, n_planes=3)
    ref = _decode_oracle(x, L, gates, ncls, rms_w)
    assert float((y.cpu() - ref).abs().max()) <= F32_TOL * float(ref.abs().max())
    # fine-grained groups (one 16-neuron group per tile, k-1 = 31 of 128 active)
    gates = mb.synth.make_gates(B, L, 128, 32, seed=9 + B)
    y = mb.ops.mlp_decode(x.to(DEV), gu, dn, rms_weight=rms_w.to(DEV), gates=gates.to(DEV),
                          n_clusters=128, n_planes=3)
    ref = _decode_oracle(x, L, gates, 128, rms_w)
    assert float((y.cpu() - ref).abs().max()) <= F32_TOL * float(ref.abs().max())


@pytest.mark.parametrize("rows", [5, 64, 200])
def test_mlp_prefill_bf16_rounding_points(local_layer, rows):
    L, gu, dn = local_layer
    x = mb.synth.make_activations(rows, 768, seed=3 * rows)
    y = mb.ops.mlp_prefill(x.to(DEV), gu, dn)
    assert y.dtype == torch.bfloat16
    ref = orc.swiglu_mlp(x.float(), _dense(L.gate_up), _dense(L.down), dtype=torch.bfloat16)
    _assert_bf16_close(y, ref)
    gates = mb.synth.make_gates(rows, L, 16, 8, seed=rows)
    y = mb.ops.mlp_prefill(x.to(DEV), gu, dn, gates=gates.to(DEV), n_clusters=16)
    ref = orc.swiglu_mlp(x.float(), _dense(L.gate_up), _dense(L.down), gates, 16, dtype=torch.bfloat16)
    _assert_bf16_close(y, ref)


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_golden_fixtures_through_reference_storage(case):
    """Reference storage (offsets / column_indices / mortar_packed / scale at blocking 16 and
    128) -> converter -> kernels, against outputs the reference itself produced."""
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    mats = {}
    for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
        mats[tag] = mb.MortarMatrix.from_reference_bcsr(
            g[f"{tag}_offsets"], g[f"{tag}_column_indices"], g[f"{tag}_packed"],
            float(g[f"{tag}_scale"]), blk, O, I).to_stream(DEV)
    x = bf16_from_bits(g["x_bf16"])
    lead = x.shape[:-1]
    # bf16 (prefill) semantics vs the reference's autocast outputs
    y = mb.ops.mlp_prefill(x.to(DEV), mats["gu"], mats["dn"])
    _assert_bf16_close(y, bf16_from_bits(g["y_bf16"]))
    gates = torch.from_numpy(g["gates_autocast"])
    y = mb.ops.mlp_prefill(x.to(DEV), mats["gu"], mats["dn"], gates=gates.to(DEV), n_clusters=ncls)
    _assert_bf16_close(y, bf16_from_bits(g["y_routed_bf16"]))
    # fp32 semantics vs the reference's fp32 outputs: the reference folds bf16(scale) into the
    # weights, the decode algebra multiplies by the fp32 scale after the sum, so the two agree
    # to bf16-scale precision (2^-9 relative per matrix).
    y32 = mb.ops.mlp_decode(x.float().to(DEV), mats["gu"], mats["dn"], n_planes=3).cpu()
    ref = torch.from_numpy(g["y_fp32"])
    assert float((y32 - ref).abs().max()) <= 1.5e-2 * float(ref.abs().max())
    gates = torch.from_numpy(g["gates_fp32"])
    y32 = mb.ops.mlp_decode(x.float().to(DEV), mats["gu"], mats["dn"], gates=gates.to(DEV),
                            n_clusters=ncls, n_planes=3).cpu()
    ref = torch.from_numpy(g["y_routed_fp32"])
    assert float((y32 - ref).abs().max()) <= 1.5e-2 * float(ref.abs().max())
    # rmsnorm prologue vs the reference RMSNorm module
    xn = mb.ops.rmsnorm_rows(torch.from_numpy(g["x_raw"]).to(DEV), torch.from_numpy(g["rms_weight"]).to(DEV), 1e-6)
    np.testing.assert_allclose(xn.cpu().numpy(), g["x_normed"], rtol=3e-6, atol=1e-7)


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_mortar_gemv_shim_matches_reference_algebra(case):
    """The reference-signature shim against the restatement of the reference's two decode
    kernels on ITS strip layout and work list, flags at the reference's block granularity."""
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])

    class FakeCms:      # the attributes mortar_pack_strips reads from a packed CMSBlockLinear
        pass
    packs, sps = {}, {}
    for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
        c = FakeCms()
        c._mortar, c._mortar_blocking = True, blk
        c.mortar_packed = torch.from_numpy(g[f"{tag}_packed"])
        c.mortar_scale = torch.tensor(float(g[f"{tag}_scale"]))
        c.mortar_offsets = torch.from_numpy(g[f"{tag}_offsets"])
        c.mortar_column_indices = torch.from_numpy(g[f"{tag}_column_indices"])
        c.out_features, c.in_features = O, I
        packs[tag] = mb.ops.mortar_pack_strips(c, DEV)
        sps[tag] = orc.pack_strips(g[f"{tag}_codes"], g[f"{tag}_column_indices"], g[f"{tag}_offsets"],
                                   g[f"{tag}_scale"])
    x = torch.from_numpy(g["x_normed"]).reshape(-1, d_model)[:4].contiguous()
    gates = g["gates_fp32"].reshape(-1, ncls)[:4]
    cs = d_ff // ncls
    rlo, rhi, clo, chi = orc.cluster_spans(d_ff, ncls, blk)
    ract_o, cact_o = orc.route_flags(gates, rlo, rhi, clo, chi)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    ract = torch.zeros(4, 512, dtype=torch.int32, device=DEV)[:, :len(rlo)]
    cact = torch.zeros(4, 512, dtype=torch.int32, device=DEV)[:, :len(clo)]
    mb.ops.route_flags(t(gates), t(rlo), t(rhi), t(clo), t(chi), ract, cact)
    np.testing.assert_array_equal(ract.cpu().numpy(), ract_o)
    np.testing.assert_array_equal(cact.cpu().numpy(), cact_o)
    # unrouted
    h = mb.ops.mortar_gemv(x.to(DEV), packs["gu"], swiglu_out=True)
    y = mb.ops.mortar_gemv(h, packs["dn"])
    ho = orc.mortar_gemv(x.numpy(), sps["gu"], swiglu_out=True)
    yo = orc.mortar_gemv(ho, sps["dn"])
    assert np.abs(h.cpu().numpy() - ho).max() <= F32_TOL * np.abs(ho).max()
    assert np.abs(y.cpu().numpy() - yo).max() <= F32_TOL * np.abs(yo).max()
    # routed, with gather flags
    h = mb.ops.mortar_gemv(x.to(DEV), packs["gu"], swiglu_out=True, row_act=ract, gates=t(gates),
                           cluster_size=cs)
    y = mb.ops.mortar_gemv(h, packs["dn"], col_act=cact)
    ho = orc.mortar_gemv(x.numpy(), sps["gu"], swiglu_out=True, row_act=ract_o, gates=gates, cluster_size=cs)
    yo = orc.mortar_gemv(ho, sps["dn"], col_act=cact_o)
    assert np.abs(h.cpu().numpy() - ho).max() <= F32_TOL * np.abs(ho).max()
    assert np.abs(y.cpu().numpy() - yo).max() <= F32_TOL * np.abs(yo).max()
    # legacy swiglu-on-load form
    gu_full = mb.ops.mortar_gemv(x.to(DEV), packs["gu"])
    y2 = mb.ops.mortar_gemv(gu_full, packs["dn"], swiglu_x=True)
    yo2 = orc.mortar_gemv(orc.mortar_gemv(x.numpy(), sps["gu"], swiglu_out=True), sps["dn"])
    assert np.abs(y2.cpu().numpy() - yo2).max() <= 2 * F32_TOL * np.abs(yo2).max()


def test_linear_edge_topologies():
    """empty rows, a single tile, a full row, ragged tails; every batch remainder."""
    rng = np.random.default_rng(11)
    R, C = 19, 21
    mask = rng.random((R, C)) < 0.3
    mask[0] = False
    mask[1] = True
    mask[2] = False; mask[2, 20] = True
    codes = rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8)
    m = mb.MortarMatrix.from_codes(codes, mask, 0.37)
    s = m.to_stream(DEV)
    W = torch.from_numpy(m.to_dense_codes()).float()
    for rows in (1, 2, 7, 8, 9, 16, 31, 33, 64, 65, 130):
        x = torch.randn(rows, C * 16, generator=torch.Generator().manual_seed(rows))
        y = mb.ops.linear(x.to(DEV), s)
        ref = (x.double() @ W.double().T * np.float32(0.37)).float()
        assert float((y.cpu() - ref).abs().max()) <= F32_TOL * float(ref.abs().max())
        assert float(y[:, :16].abs().max()) == 0.0      # the empty tile row yields exact zeros
    assert mb.ops.linear(torch.zeros(0, C * 16, device=DEV), s).shape == (0, R * 16)
    with pytest.raises(ValueError):
        mb.ops.linear(torch.zeros(2, C * 16 + 16, device=DEV), s)


@pytest.mark.parametrize("path", ["plain", "staged", "persistent"])
@pytest.mark.parametrize("B", [1, 2, 5, 8, 24, 64])
@pytest.mark.parametrize("in_dtype", [torch.bfloat16, torch.float32])
def test_mlp_decode_every_kernel_path(local_layer, path, B, in_dtype):
    """The three paths of the linear kernel (per-lane loads, bulk-copy staging, persistent with
    producer warps) pinned one by one; a path that cannot serve a call (the persistent one past
    8 MMA columns) falls back, so every combination must still match the oracle."""
    L, gu, dn = local_layer
    x = mb.synth.make_activations(B, 768, seed=40 + B).to(in_dtype)
    y = mb.ops.mlp_decode(x.to(DEV), gu, dn, n_planes=3, out_dtype=torch.float32, path=path)
    ref = _decode_oracle(x, L)
    assert float((y.cpu() - ref).abs().max()) <= F32_TOL * float(ref.abs().max())
    assert mb.ops.linear_error() == 0


@pytest.mark.parametrize("path", ["staged", "persistent"])
def test_routed_decode_on_pinned_paths(local_layer, path):
    """Routing inputs: the staged path honours gates and gather flags, the persistent one has none
    and must hand such calls to a path that does."""
    L, gu, dn = local_layer
    B, ncls, k = 4, 16, 8
    gen = torch.Generator().manual_seed(123)
    x = torch.randn(B, 768, generator=gen) * 2.0
    rms_w = 1.0 + 0.1 * torch.randn(768, generator=gen)
    gates = mb.synth.make_gates(B, L, ncls, k, seed=31)
    y = mb.ops.mlp_decode(x.to(DEV), gu, dn, rms_weight=rms_w.to(DEV), gates=gates.to(DEV),
                          n_clusters=ncls, n_planes=3, path=path)
    ref = _decode_oracle(x, L, gates, ncls, rms_w)
    assert float((y.cpu() - ref).abs().max()) <= F32_TOL * float(ref.abs().max())
    assert mb.ops.linear_error() == 0


@pytest.mark.parametrize("path", ["plain", "staged", "persistent"])
def test_linear_edge_topologies_on_pinned_paths(path):
    """empty rows, one tile, a full row, rows longer than one stage (more than 16 groups), ragged
    tails; exact integer arithmetic, so every path must agree bit for bit."""
    rng = np.random.default_rng(13)
    R, C = 23, 300
    mask = rng.random((R, C)) < 0.25
    mask[0] = False
    mask[1] = True                                  # 300 tiles = 38 groups: three stages and a tail
    mask[2] = False; mask[2, C - 1] = True
    mask[3] = False; mask[3, :8] = True             # exactly one full group
    mask[4] = False; mask[4, :129] = True           # 16 groups and one padded group
    codes = rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8)
    m = mb.MortarMatrix.from_codes(codes, mask, 0.5)
    s = m.to_stream(DEV)
    W = torch.from_numpy(m.to_dense_codes()).float().to(DEV)
    for rows in (1, 2, 3, 8, 9, 40):
        xi = torch.randint(-4, 5, (rows, C * 16), generator=torch.Generator().manual_seed(rows)).float()
        for planes in ((xi.to(torch.bfloat16).unsqueeze(0)),
                       torch.stack([xi.to(torch.bfloat16), torch.zeros_like(xi, dtype=torch.bfloat16),
                                    torch.zeros_like(xi, dtype=torch.bfloat16)])):
            y = mb.ops.linear_planes(s, planes.contiguous().to(DEV), out_dtype=torch.float32, path=path)
            assert torch.equal(y, (xi.to(DEV) @ W.T) * np.float32(0.5))
    assert mb.ops.linear_error() == 0


def test_linear_is_linear_and_exact_on_integers():
    """size-independent properties: integer-valued activations make every partial sum exact,
    so the kernel must agree with integer arithmetic bit for bit."""
    L = mb.synth.make_layer(2048, 5632, 0.25, seed=200)
    s = L.gate_up.to_stream(DEV)
    gen = torch.Generator().manual_seed(4)
    xi = torch.randint(-8, 9, (40, 2048), generator=gen).float()
    y = mb.ops.linear_planes(s, xi.to(torch.bfloat16).unsqueeze(0).to(DEV), out_dtype=torch.float32)
    Wc = torch.from_numpy(L.gate_up.to_dense_codes()).to(DEV).float()
    exact = (xi.to(DEV) @ Wc.T)                     # integer sums below 2^24: exact in fp32
    assert torch.equal(y, exact * np.float32(L.gate_up.scale))


@pytest.mark.parametrize("mask", ["uniform", "zipf_rows"])
@pytest.mark.parametrize("density", [0.125, 0.5, 1.0])
def test_topology_sweep_cloud_shape(mask, density):
    """density / topology sweep on the cloud-shape MLP against a dense evaluation of the same
    codes on the GPU (row-clustered Zipf masks have empty and very long rows)."""
    L = mb.synth.make_layer(2048, 5632, density, seed=300, mask=mask)
    gu, dn = L.gate_up.to_stream(DEV), L.down.to_stream(DEV)
    x = mb.synth.make_activations(96, 2048, seed=1).to(DEV)
    y = mb.ops.mlp_decode(x, gu, dn, n_planes=3, out_dtype=torch.float32)
    Wg = torch.from_numpy(L.gate_up.to_dense_codes()).to(DEV).double()
    Wd = torch.from_numpy(L.down.to_dense_codes()).to(DEV).double()
    gu_ = (x.double() @ Wg.T) * float(np.float32(L.gate_up.scale))
    g_, u_ = gu_.chunk(2, dim=-1)
    ref = ((g_ * torch.sigmoid(g_) * u_) @ Wd.T) * float(np.float32(L.down.scale))
    assert float((y.double() - ref).abs().max()) <= 2e-5 * float(ref.abs().max())


def test_module_mirror_matches_ops(local_layer):
    L, gu, dn = local_layer
    mlp = mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=DEV)
    x = mb.synth.make_activations(4 * 9, 768, seed=8).reshape(4, 9, 768).to(DEV)
    y = mlp(x)
    assert y.shape == (4, 9, 768) and y.dtype == torch.bfloat16
    assert torch.equal(y.reshape(-1, 768), mb.ops.mlp_prefill(x.reshape(-1, 768), gu, dn))
    y32 = mlp(x.float(), iter_idx=3)
    assert y32.dtype == torch.float32
    lin = mlp.down
    assert lin.is_compact and lin.bias is None and abs(lin.get_density() - 0.25) < 1e-6
    with pytest.raises(AssertionError):
        lin.carve()


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_registered_ops_and_dds_shim_against_reference_outputs(case):
    """The MLP assembled from the reference operator's own call (stk_dds twice, the elementwise
    steps in torch as transformer.py:402-431 has them) and through the registered
    mortar_b200:: ops, against the bf16 outputs the reference produced."""
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    x = bf16_from_bits(g["x_bf16"]).to(DEV)
    x2 = x.reshape(-1, d_model)
    z = torch.zeros(1, dtype=torch.int16, device=DEV)
    datas, mats = {}, {}
    for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
        sc = torch.tensor(float(g[f"{tag}_scale"])).to(torch.bfloat16)
        datas[tag] = ((torch.from_numpy(g[f"{tag}_codes"]).float() * sc.float()).to(torch.bfloat16).to(DEV),
                      torch.from_numpy(g[f"{tag}_offsets"]).to(DEV),
                      torch.from_numpy(g[f"{tag}_column_indices"]).to(DEV), I, O)
        mats[tag] = mb.MortarMatrix.from_reference_bcsr(
            g[f"{tag}_offsets"], g[f"{tag}_column_indices"], g[f"{tag}_packed"],
            float(g[f"{tag}_scale"]), blk, O, I).to_stream(DEV)

    def dds(inp, tag):
        data, off, ci, I, O = datas[tag]
        return mb.torch_ops.stk_dds(inp, data, off, z, ci, z, z, z, I, O, True)

    gu = dds(x2, "gu")
    assert gu.dtype == torch.bfloat16 and gu.shape == (x2.shape[0], 2 * d_ff)
    gate, up = gu.chunk(2, dim=-1)
    h = torch.nn.functional.silu(gate) * up
    y = dds(h.contiguous(), "dn").reshape(*x.shape[:-1], d_model)
    _assert_bf16_close(y, bf16_from_bits(g["y_bf16"]))
    # the registered ops, unrouted and routed
    args = (*mb.torch_ops.stream_args(mats["gu"]), *mb.torch_ops.stream_args(mats["dn"]))
    y = torch.ops.mortar_b200.mlp_prefill(x, *args, None, 0)
    _assert_bf16_close(y, bf16_from_bits(g["y_bf16"]))
    gates = torch.from_numpy(g["gates_autocast"]).to(DEV)
    y = torch.ops.mortar_b200.mlp_prefill(x, *args, gates, ncls)
    _assert_bf16_close(y, bf16_from_bits(g["y_routed_bf16"]))
    y32 = torch.ops.mortar_b200.mlp_decode(x.float(), None, 1e-6, *args, None, 0).cpu()
    ref = torch.from_numpy(g["y_fp32"])
    assert float((y32 - ref).abs().max()) <= 1.5e-2 * float(ref.abs().max())
    y1 = torch.ops.mortar_b200.linear(x, *mb.torch_ops.stream_args(mats["gu"]))
    assert torch.equal(y1.reshape(-1, 2 * d_ff), gu)


def test_remoe_cloud_configuration():
    """The routed configuration at its own sizes: d_model 2048, d_ff 5632, 352 groups of 16 hidden
    neurons, k = 88 (87 active per token).  A 64-token decode batch against the oracle; the
    4096-token prefill through properties that do not need a CPU pass of that size: a token
    whose gates are all zero yields exact zeros, and the routed output of a token equals the
    one it gets inside a smaller batch (tokens are independent)."""
    L = mb.synth.make_layer(2048, 5632, 0.25, seed=200)
    gu, dn = L.gate_up.to_stream(DEV), L.down.to_stream(DEV)
    ncls, k = 352, 88
    x = mb.synth.make_activations(64, 2048, seed=5, dtype=torch.float32)
    gates = mb.synth.make_gates(64, L, ncls, k, seed=6)
    assert int((gates > 0).sum(dim=1).max()) == k - 1
    y = mb.ops.mlp_decode(x.to(DEV), gu, dn, gates=gates.to(DEV), n_clusters=ncls, n_planes=3)
    ref = _decode_oracle(x, L, gates, ncls)
    assert float((y.cpu() - ref).abs().max()) <= F32_TOL * float(ref.abs().max())
    # prefill at 4096 tokens on the tensor-core path
    gs, ds = L.gate_up.to_sched(True, DEV), L.down.to_sched(False, DEV)
    xb = mb.synth.make_activations(4096, 2048, seed=7).to(DEV)
    g4 = mb.synth.make_gates(4096, L, ncls, k, seed=8).to(DEV)
    g4[17] = 0.0
    y4 = mb.ops.mlp_prefill_tc(xb, gs, ds, gates=g4, n_clusters=ncls)
    assert mb.ops.prefill_error() == 0
    assert float(y4[17].float().abs().max()) == 0.0
    sub = slice(1000, 1128)
    ysub = mb.ops.mlp_prefill_tc(xb[sub].contiguous(), gs, ds, gates=g4[sub].contiguous(), n_clusters=ncls)
    assert torch.equal(ysub, y4[sub])
    ref = orc.swiglu_mlp(xb[sub].cpu().float(), _dense(L.gate_up), _dense(L.down), g4[sub].cpu(), ncls,
                         dtype=torch.bfloat16)
    _assert_bf16_close(ysub, ref)


@pytest.mark.parametrize("ncls,k", [(352, 88), (16, 8), (704, 176)])
@pytest.mark.parametrize("rows", [9, 64, 300])
def test_per_token_tile_gather(ncls, k, rows):
    """Routed batches of more than 8 rows: the gather schedule lists exactly the (row, hidden tile
    row) pairs with a positive gate; the gathered gate/up stage runs only those and the MLP still
    equals the multiply semantics of the oracle, in both arithmetic modes.  704 clusters = two
    clusters inside one tile row (a listed row may still have gated-off neurons)."""
    L = mb.synth.make_layer(2048, 5632, 0.25, seed=200)
    gu, dn = L.gate_up.to_stream(DEV), L.down.to_stream(DEV)
    gates = mb.synth.make_gates(rows, L, ncls, k, seed=rows + ncls)
    cs = 5632 // ncls
    cnt, lst = mb.ops.route_gather(gates.to(DEV), cs, 352)
    act = gates.reshape(rows, ncls).numpy() > 0
    for u in (0, 1, 17, 200, 351):
        lo, hi = (u * 16) // cs, (u * 16 + 15) // cs
        want = np.nonzero(act[:, lo:hi + 1].any(axis=1))[0]
        assert int(cnt[u]) == len(want)
        np.testing.assert_array_equal(lst[u, :len(want)].cpu().numpy(), want)
    listed = int(cnt.sum())
    assert listed < 0.6 * rows * 352                        # most (row, tile row) pairs are skipped
    x = mb.synth.make_activations(rows, 2048, seed=rows, dtype=torch.float32)
    before = mb.ops.kernel_counts()
    y = mb.ops.mlp_decode(x.to(DEV), gu, dn, gates=gates.to(DEV), n_clusters=ncls, n_planes=3)
    after = mb.ops.kernel_counts()
    assert after.get("bcsr_gather", 0) == before.get("bcsr_gather", 0) + 1
    ref = _decode_oracle(x, L, gates, ncls)
    assert float((y.cpu() - ref).abs().max()) <= F32_TOL * float(ref.abs().max())
    xb = x.to(torch.bfloat16)
    yb = mb.ops.mlp_prefill(xb.to(DEV), gu, dn, gates=gates.to(DEV), n_clusters=ncls)
    refb = orc.swiglu_mlp(xb.float(), _dense(L.gate_up), _dense(L.down), gates, ncls, dtype=torch.bfloat16)
    _assert_bf16_close(yb, refb)
    # a row whose gates are all zero yields exact zeros
    g0 = gates.clone()
    g0[rows // 2] = 0.0
    y0 = mb.ops.mlp_decode(x.to(DEV), gu, dn, gates=g0.to(DEV), n_clusters=ncls, n_planes=3)
    assert float(y0[rows // 2].abs().max()) == 0.0


def test_decode_side_steps_fused():
    """The steps either side of the MLP in the decode engine: the hyper-connection POST write as
    the down projection's epilogue, and the row-scaled dense ternary GEMV -- against the outputs
    the reference's eager code produced and against the oracle."""
    g = load_golden("decode_sides")
    t = lambda k: torch.from_numpy(g[k]).to(DEV)
    # row-scaled stack: three ternary layers with their own scales as one product
    pack = mb.ops.ternary_pack_rs(torch.from_numpy(g["rs_codes"]), torch.from_numpy(g["rs_row_scale"]), DEV)
    y = mb.ops.ternary_gemv_rs(t("rs_x"), pack)
    assert y.shape == (5, 144)
    np.testing.assert_allclose(y.cpu().numpy(), g["rs_out"], rtol=2e-5, atol=1e-6)
    # O not a multiple of 16 (the reference's ctx_w = 2730 stacks)
    rng = np.random.default_rng(5)
    O, I = 2730, 256
    dense = rng.integers(-1, 2, size=(O, I)).astype(np.int8)
    st = (dense + 1).astype(np.uint8).reshape(O, 4, I // 4)
    packed = st[:, 0] | (st[:, 1] << 2) | (st[:, 2] << 4) | (st[:, 3] << 6)
    rs = rng.random(O).astype(np.float32) * 0.05
    x = rng.standard_normal((3, I)).astype(np.float32)
    y = mb.ops.ternary_gemv_rs(torch.from_numpy(x).to(DEV), mb.ops.ternary_pack_rs(torch.from_numpy(packed),
                                                                                  torch.from_numpy(rs), DEV))
    ref = orc.ternary_gemv_rs(x, packed, rs)
    assert y.shape == (3, O)
    assert float(np.abs(y.cpu().numpy() - ref).max()) <= F32_TOL * float(np.abs(ref).max())
    # POST write fused behind the MLP: golden mapping tensors, MLP output from the oracle
    L = mb.synth.make_layer(256, 512, 0.25, seed=1)
    gu, dn = L.gate_up.to_stream(DEV), L.down.to_stream(DEV)
    h = t("hc_h")                                            # [3, 1, 4, 256]
    xbar = h.mean(dim=2)                                     # a single-stream input [3, 1, 256]
    y_ref = _decode_oracle(xbar.reshape(-1, 256).cpu(), L)
    for term in (None, t("hc_term")):
        want = orc.hc_post(t("hc_hres").cpu(), t("hc_hpost_row").cpu(), h.cpu(), y_ref.reshape(3, 1, 256),
                           None if term is None else term.cpu())
        out = mb.ops.mlp_decode_hc(xbar, gu, dn, t("hc_hres"), t("hc_hpost_row"), h, term=term)
        assert out.shape == h.shape
        assert float((out.cpu() - want).abs().max()) <= F32_TOL * float(want.abs().max())
    # in place on the carrier, with the MLP replaced by a known y: the reference's own output
    carrier = h.clone()
    mb.ops.mlp_decode_hc(xbar, gu, dn, t("hc_hres"), t("hc_hpost_row"), carrier, out=carrier)
    want = orc.hc_post(t("hc_hres").cpu(), t("hc_hpost_row").cpu(), h.cpu(), y_ref.reshape(3, 1, 256))
    assert float((carrier.cpu() - want).abs().max()) <= F32_TOL * float(want.abs().max())
