"""Parity at the sizes the benchmark times (not only at sizes the oracle finishes quickly):
the single-layer configuration (4 x 4096 tokens at 768/2048), one cloud-shape application at
16384 tokens, the density / topology sweep at 8192 tokens on the tensor-memory path, and the
whole 42-application decode stack at batch 1, 8 and 64 -- each against the CPU oracle, full
size where the oracle is fast enough and on a row sample plus size-independent properties
(tokens are independent: a block computed inside a large launch equals the same block
computed alone) where it is not.  Also: which kernel the module forward and the registered
operators actually run."""
import numpy as np
import pytest
import torch

import mortar_b200 as mb
from oracle import mortar_oracle as orc
from test_gpu_parity import _assert_bf16_close, _decode_oracle, _dense, _oracle_meta

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _clean():
    assert mb.ops.prefill_error() == 0, "a bounded wait in the prefill kernel expired"


def _delta(before, name):
    return mb.ops.kernel_counts().get(name, 0) - before.get(name, 0)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_single_layer_configuration_full_size(seed, monkeypatch):
    """4 x 4096 tokens, d_model 768, d_ff 2048, top-25% tiles by L2, bf16 RMS-normed input:
    the tensor-memory operator and the module forward against the oracle's bf16 path on every
    one of the 16384 x 768 outputs."""
    L = mb.synth.make_layer(768, 2048, 0.25, seed=seed)
    x = mb.synth.make_activations(4 * 4096, 768, seed=seed).reshape(4, 4096, 768)
    ref = orc.swiglu_mlp(x.reshape(-1, 768).float(), _dense(L.gate_up), _dense(L.down), dtype=torch.bfloat16)
    y = mb.ops.mlp_prefill_tc(x.to(DEV), L.gate_up.to_sched(True, DEV), L.down.to_sched(False, DEV))
    _clean()
    assert y.shape == (4, 4096, 768)
    _assert_bf16_close(y, ref, near_zero=1e-2)         # 12.6 million outputs
    # the module forward: 25% random tiles fill the touched 128 x 128 blocks above the dispatch
    # threshold, so it takes the block path; pinned to the per-tile path it returns y's bits
    mlp = mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=DEV)
    before = mb.ops.kernel_counts()
    y2 = mlp(x.to(DEV))
    assert _delta(before, "prefill_blocks") == 2 and _delta(before, "bcsr_stream") == 0
    _clean()
    _assert_bf16_close(y2, ref, near_zero=1e-2)
    monkeypatch.setattr(mb.format, "BLOCK_PATH_MIN_FILL", 2.0)
    mlp = mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=DEV)
    before = mb.ops.kernel_counts()
    y3 = mlp(x.to(DEV))
    assert _delta(before, "prefill_panel") == 2 and _delta(before, "prefill_blocks") == 0
    assert torch.equal(y3, y)


def test_cloud_application_16384_tokens():
    """One cloud-shape MLP (2048/5632, 25%) on 16384 tokens, the size of the prefill benchmark:
    512 rows drawn from every residue of the 128-row blocks and from the first and last work item
    of a CTA against the oracle, and every row bit-equal to the same block computed alone (a
    launch of 128 rows holds one work item per CTA; the full launch makes every CTA walk ~19
    items through its rings and both accumulator phases)."""
    d, f, n = 2048, 5632, 16384
    L = mb.synth.make_layer(d, f, 0.25, seed=200)
    gu, dn = L.gate_up.to_sched(True, DEV), L.down.to_sched(False, DEV)
    x = mb.synth.make_activations(n, d, seed=7).to(DEV)
    y = mb.ops.mlp_prefill_tc(x, gu, dn)
    _clean()
    rng = np.random.default_rng(0)
    rows = np.concatenate([np.arange(0, 128), np.arange(n - 128, n),            # first / last item of CTA 0 / the last CTA
                           rng.integers(0, n // 128, 256) * 128 + np.arange(256) % 128])   # every residue twice
    rows = np.unique(rows)
    assert len(rows) >= 500
    ref = orc.swiglu_mlp(x[rows].cpu().float(), _dense(L.gate_up), _dense(L.down), dtype=torch.bfloat16)
    _assert_bf16_close(y[rows], ref)
    for b in range(0, n // 128, 1):
        sl = slice(b * 128, (b + 1) * 128)
        if b % 8 == 0:      # every 8th block alone (16 launches of one block), all other blocks via the sample above
            assert torch.equal(mb.ops.mlp_prefill_tc(x[sl], gu, dn), y[sl]), f"block {b}"
    _clean()


@pytest.mark.parametrize("mask", ["uniform", "zipf_rows"])
@pytest.mark.parametrize("density", [0.125, 0.25, 0.5, 1.0])
def test_topology_sweep_8192_tokens_vs_oracle(mask, density):
    """The density / topology sweep at its own size (8192 tokens, cloud shape) on the
    tensor-memory path, against the oracle on 256 sampled rows; the row-clustered masks give long
    vertical runs and very uneven panels."""
    d, f, n = 2048, 5632, 8192
    L = mb.synth.make_layer(d, f, density, seed=300, mask=mask)
    x = mb.synth.make_activations(n, d, seed=3).to(DEV)
    y = mb.ops.mlp_prefill_tc(x, L.gate_up.to_sched(True, DEV), L.down.to_sched(False, DEV))
    _clean()
    rows = np.unique(np.concatenate([np.arange(0, n, 61), np.arange(n - 64, n)]))[:256]
    ref = orc.swiglu_mlp(x[rows].cpu().float(), _dense(L.gate_up), _dense(L.down), dtype=torch.bfloat16)
    _assert_bf16_close(y[rows], ref, near_zero=1e-2 if mask == "zipf_rows" else 4e-3)


def _decode_stack_layers(cfg_seed0=100, n_layers=12, d=768, f=2048):
    gen = torch.Generator().manual_seed(cfg_seed0 + 999)
    layers, rms = [], []
    for i in range(n_layers):
        layers.append(mb.synth.make_layer(d, f, 0.25, seed=cfg_seed0 + i))
        rms.append(1.0 + 0.05 * torch.randn(d, generator=gen))
    return layers, rms


@pytest.fixture(scope="module")
def full_stack():
    layers, rms = _decode_stack_layers()
    order = list(range(3)) + [3 + i for _ in range(6) for i in range(6)] + [9, 10, 11]
    stack = mb.ops.DecodeStack([(L.gate_up, L.down, w) for L, w in zip(layers, rms)], order, DEV)
    dense = []
    for L in layers:
        ws = []
        for m in (L.gate_up, L.down):
            c, meta = _oracle_meta(m)
            ws.append(orc.mortar_dense(c, torch.tensor(m.scale), meta[0], meta[1], meta[2], meta[3], False))
        dense.append(ws)
    return layers, rms, order, stack, dense


@pytest.mark.parametrize("batch", [1, 8, 64])
def test_whole_decode_stack_vs_oracle(full_stack, batch):
    """The launch the headline times: 12 layers, 42 applications (3 + 6 x 6 + 3), fp32 residual
    carrier, against x <- x + mlp_i(rmsnorm_i(x)) chained on the CPU in fp32."""
    layers, rms, order, stack, dense = full_stack
    assert len(order) == 42
    x0 = mb.synth.make_activations(batch, 768, seed=batch, dtype=torch.float32)
    ref = x0.clone()
    for i in order:
        ref = ref + orc.swiglu_mlp(orc.rmsnorm_rows(ref, rms[i], 1e-6), dense[i][0], dense[i][1])
    for planes in (mb.ops.PLANES_HALF2, 3):        # the default (two scaled fp16 planes) and three bf16 planes
        x = x0.clone().to(DEV)
        mb.ops.stack_decode(x, stack, n_planes=planes)
        assert stack.error() == 0
        rel = float((x.cpu() - ref).abs().max()) / float(ref.abs().max())
        print(f"batch {batch} planes {planes}: max relative error {rel:.2e}")
        assert rel <= 1e-5, f"batch {batch} planes {planes}: relative error {rel:.2e}"
    # the per-application path on the same chain
    x2 = x0.clone().to(DEV)
    streams = [(L.gate_up.to_stream(DEV), L.down.to_stream(DEV)) for L in layers]
    for i in order:
        mb.ops.mlp_decode(x2, *streams[i], rms_weight=rms[i].to(DEV), n_planes=3, out=x2, accumulate=True)
    assert float((x2.cpu() - ref).abs().max()) / float(ref.abs().max()) <= 1e-5


def test_stack_decode_takes_norm_weights_as_an_argument(full_stack):
    """The C entry point as its header describes it: blobs WITHOUT an embedded norm weight
    (hdr[11] = 0) and the weights passed as `rms_weights` [n_layers, d_model]."""
    layers, rms, order, stack, dense = full_stack
    bare = mb.ops.DecodeStack([(L.gate_up, L.down, None) for L in layers[:3]], [0, 1, 2, 1], DEV, cluster_sizes=(8,))
    v = bare.variants[8]
    x0 = mb.synth.make_activations(13, 768, seed=5, dtype=torch.float32) * 1.7
    w = torch.stack(rms[:3]).to(DEV).contiguous()
    x = x0.clone().to(DEV)
    mb.ops.stack_decode_raw(x, v.blobs, v.table, bare.app_layer, w, bare.status, 3, 768, 2048, v.max_a, v.max_b, 8)
    assert bare.error() == 0
    ref = x0.clone()
    for i in [0, 1, 2, 1]:
        ref = ref + orc.swiglu_mlp(orc.rmsnorm_rows(ref, rms[i], 1e-6), dense[i][0], dense[i][1])
    assert float((x.cpu() - ref).abs().max()) / float(ref.abs().max()) <= 1e-5
    # without weights: no normalisation
    x = x0.clone().to(DEV)
    mb.ops.stack_decode_raw(x, v.blobs, v.table, bare.app_layer, None, bare.status, 3, 768, 2048, v.max_a, v.max_b, 8)
    ref = x0.clone()
    for i in [0, 1, 2, 1]:
        ref = ref + orc.swiglu_mlp(ref, dense[i][0], dense[i][1])
    assert float((x.cpu() - ref).abs().max()) / float(ref.abs().max()) <= 1e-5
    # the registered operator runs the same launch in place
    x = x0.clone().to(DEV)
    torch.ops.mortar_b200.stack_decode(x, v.blobs, v.table, bare.app_layer, None, bare.status, 3, 768, 2048,
                                       v.max_a, v.max_b, 8, 1e-6, 3)
    assert float((x.cpu() - ref).abs().max()) / float(ref.abs().max()) <= 1e-5


def test_module_forward_and_operators_pick_the_kernel_by_row_count(monkeypatch):
    """bf16 token blocks of 128 rows or more run the tcgen05 kernel through every public door
    (module forward, MortarLinear, mortar_b200::mlp_prefill / linear, morph_stk::dds); smaller
    blocks and fp32 rows run the streaming kernel; results agree with the explicit operators.
    (The per-tile path is pinned here; the choice between it and the block path has its own test.)"""
    monkeypatch.setattr(mb.format, "BLOCK_PATH_MIN_FILL", 2.0)
    L = mb.synth.make_layer(768, 2048, 0.25, seed=100)
    mlp = mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=DEV)
    gs, ds = L.gate_up.to_sched(True, DEV), L.down.to_sched(False, DEV)
    gu, dn = L.gate_up.to_stream(DEV), L.down.to_stream(DEV)
    big = mb.synth.make_activations(300, 768, seed=1).to(DEV)
    small = big[:40].contiguous()
    for x, tc in ((big, True), (small, False)):
        b = mb.ops.kernel_counts()
        y = mlp(x)
        assert (_delta(b, "prefill_panel"), _delta(b, "bcsr_stream")) == ((2, 0) if tc else (0, 2))
        assert torch.equal(y, mb.ops.mlp_prefill_tc(x, gs, ds) if tc else mb.ops.mlp_prefill(x, gu, dn))
        b = mb.ops.kernel_counts()
        y1 = mlp.gate_up(x)
        assert (_delta(b, "prefill_panel"), _delta(b, "bcsr_stream")) == ((1, 0) if tc else (0, 1))
        assert torch.equal(y1, mb.ops.linear_tc(x, L.gate_up.to_sched(False, DEV)) if tc else mb.ops.linear(x, gu))
        b = mb.ops.kernel_counts()
        args = (*mb.torch_ops.stream_args(gu), *mb.torch_ops.stream_args(dn))
        y2 = torch.ops.mortar_b200.mlp_prefill(x, *args, None, 0)
        assert (_delta(b, "prefill_panel") > 0) == tc and torch.equal(y2, y)
    b = mb.ops.kernel_counts()
    y32 = mlp(big.float())
    assert _delta(b, "prefill_panel") == 0 and y32.dtype == torch.float32
    with torch.autocast("cuda", dtype=torch.bfloat16):
        b = mb.ops.kernel_counts()
        ya = mlp(big.float())
        assert _delta(b, "prefill_panel") == 2 and ya.dtype == torch.bfloat16 and torch.equal(ya, mlp(big))
    # the reference operator's name and argument list
    z = torch.zeros(1, dtype=torch.int16, device=DEV)
    m = L.down
    data = (torch.from_numpy(mb.format.unpack_codes_2bit(m.codes).reshape(-1, 16, 16)).float()
            * torch.tensor(m.scale).to(torch.bfloat16).float()).to(torch.bfloat16).to(DEV)
    off = torch.from_numpy(m.row_ptr).to(DEV)
    ci = torch.from_numpy(m.col_idx.astype(np.int16)).to(DEV)
    h = mb.synth.make_activations(256, 2048, seed=2).to(DEV)
    b = mb.ops.kernel_counts()
    y = torch.ops.morph_stk.dds(h, data, off, z, ci, z, z, z, 2048, 768, True)
    assert _delta(b, "prefill_panel") == 1
    assert torch.equal(y, mb.ops.linear_tc(h, ds))
    y = torch.ops.morph_stk.dds(h[:8].contiguous(), data, off, z, ci, z, z, z, 2048, 768, True)
    assert torch.equal(y, mb.ops.linear(h[:8].contiguous(), dn))
    # a weight update behind the same index buffers is noticed (the reference passes a fresh
    # temporary every forward, so address and version cannot be trusted)
    data2 = -data
    y = torch.ops.morph_stk.dds(h, data2, off, z, ci, z, z, z, 2048, 768, True)
    assert torch.equal(y, -mb.ops.linear_tc(h, ds))
    _clean()


def test_module_decode_stack_hook():
    layers, rms = _decode_stack_layers(n_layers=2)
    mlps = [mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=DEV) for L in layers]
    stack = mb.modules.decode_stack(mlps, [w.to(DEV) for w in rms], order=[0, 1, 0])
    x0 = mb.synth.make_activations(8, 768, seed=9, dtype=torch.float32)
    x = x0.clone().to(DEV)
    mb.ops.stack_decode(x, stack)
    ref = x0.clone().to(DEV)
    for i in [0, 1, 0]:
        xn = mb.ops.rmsnorm_rows(ref, rms[i].to(DEV), 1e-6)
        ref = ref + mlps[i](xn)
    assert float((x - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
