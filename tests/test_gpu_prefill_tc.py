"""Parity of the tcgen05 / tensor-memory prefill kernels (through the C ABI) against the CPU
oracle's bf16 path, the golden fixtures, and the already-checked streaming kernels."""
import numpy as np
import pytest
import torch

import mortar_b200 as mb
from conftest import GOLDEN_CASES, bf16_from_bits, load_golden
from oracle import mortar_oracle as orc
from test_gpu_parity import _assert_bf16_close, _dense

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _check_clean():
    assert mb.ops.prefill_error() == 0, "a bounded wait in the prefill kernel expired"


@pytest.mark.parametrize("rows", [1, 100, 128, 300])
def test_linear_tc_small_matrix(rows):
    """ragged topology with an empty row, a full row and partial last panel / chunk."""
    rng = np.random.default_rng(21)
    R, C = 40, 23
    mask = rng.random((R, C)) < 0.3
    mask[0] = False
    mask[1] = True
    codes = rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8)
    m = mb.MortarMatrix.from_codes(codes, mask, 0.0173)
    x = torch.randn(rows, C * 16, generator=torch.Generator().manual_seed(rows)).to(torch.bfloat16)
    y = mb.ops.linear_tc(x.to(DEV), m.to_sched(False, DEV))
    _check_clean()
    W = torch.from_numpy(m.to_dense_codes()).float() * torch.tensor(0.0173).to(torch.bfloat16).float()
    ref = torch.nn.functional.linear(x, W.to(torch.bfloat16))
    _assert_bf16_close(y, ref)
    assert float(y[:, :16].float().abs().max()) == 0.0


@pytest.mark.parametrize("shape", ["local", "cloud"])
@pytest.mark.parametrize("rows", [128, 391])
def test_mlp_prefill_tc_matches_oracle(shape, rows):
    d, f = (768, 2048) if shape == "local" else (2048, 5632)
    L = mb.synth.make_layer(d, f, 0.25, seed=100 if shape == "local" else 200)
    gu, dn = L.gate_up.to_sched(True, DEV), L.down.to_sched(False, DEV)
    x = mb.synth.make_activations(rows, d, seed=rows)
    y = mb.ops.mlp_prefill_tc(x.to(DEV), gu, dn)
    _check_clean()
    ref = orc.swiglu_mlp(x.float(), _dense(L.gate_up), _dense(L.down), dtype=torch.bfloat16)
    _assert_bf16_close(y, ref)
    ncls = f // 16
    gates = mb.synth.make_gates(rows, L, ncls, ncls // 4, seed=3)
    y = mb.ops.mlp_prefill_tc(x.to(DEV), gu, dn, gates=gates.to(DEV), n_clusters=ncls)
    _check_clean()
    ref = orc.swiglu_mlp(x.float(), _dense(L.gate_up), _dense(L.down), gates, ncls, dtype=torch.bfloat16)
    _assert_bf16_close(y, ref)


@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_golden_fixtures_tc(case):
    g = load_golden(case)
    d_model, d_ff, blk, ncls = (int(v) for v in g["meta"])
    mats = {}
    for tag, (O, I) in (("gu", (2 * d_ff, d_model)), ("dn", (d_model, d_ff))):
        mats[tag] = mb.MortarMatrix.from_reference_bcsr(
            g[f"{tag}_offsets"], g[f"{tag}_column_indices"], g[f"{tag}_packed"],
            float(g[f"{tag}_scale"]), blk, O, I)
    gu, dn = mats["gu"].to_sched(True, DEV), mats["dn"].to_sched(False, DEV)
    x = bf16_from_bits(g["x_bf16"])
    y = mb.ops.mlp_prefill_tc(x.to(DEV), gu, dn)
    _check_clean()
    _assert_bf16_close(y, bf16_from_bits(g["y_bf16"]))
    gates = torch.from_numpy(g["gates_autocast"])
    y = mb.ops.mlp_prefill_tc(x.to(DEV), gu, dn, gates=gates.to(DEV), n_clusters=ncls)
    _check_clean()
    _assert_bf16_close(y, bf16_from_bits(g["y_routed_bf16"]))


@pytest.mark.parametrize("mask", ["uniform", "zipf_rows"])
@pytest.mark.parametrize("density", [0.125, 0.5, 1.0])
def test_topology_sweep_tc_vs_stream(mask, density):
    """density / topology sweep on the cloud shape: the tensor-memory path against the
    streaming path (itself checked against the oracle); dense and row-clustered masks fuse
    tiles into long runs (N up to 256)."""
    L = mb.synth.make_layer(2048, 5632, density, seed=300, mask=mask)
    x = mb.synth.make_activations(256, 2048, seed=1).to(DEV)
    y = mb.ops.mlp_prefill_tc(x, L.gate_up.to_sched(True, DEV), L.down.to_sched(False, DEV))
    _check_clean()
    ref = mb.ops.mlp_prefill(x, L.gate_up.to_stream(DEV), L.down.to_stream(DEV))
    _assert_bf16_close(y, ref)
