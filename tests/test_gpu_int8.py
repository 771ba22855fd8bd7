"""The opt-in 8-bit arm of the prefill kernel (tcgen05 kind::i8 on per-row quantised activations).

It is NOT the reference's arithmetic, so it is checked two ways: bit for bit against the bf16
kernel on activations the quantiser represents exactly, and against the CPU oracle on ordinary
activations with the error measured relative to the output's RMS (the quantisation error of a
sum does not shrink with the sum, so small outputs miss the element-wise bf16 tolerance)."""
import numpy as np
import pytest
import torch

import mortar_b200 as mb
from oracle import mortar_oracle as orc
from test_gpu_parity import _dense

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _integer_activations(rows, cols, seed):
    g = torch.Generator().manual_seed(seed)
    x = torch.randint(-127, 128, (rows, cols), generator=g).float()
    x[:, 0] = 127.0                                  # every row's scale is exactly 1
    return x.to(torch.bfloat16)                      # |v| <= 127 is exact in bf16


def test_quantize_rows_matches_definition():
    x = (torch.randn(300, 2048, generator=torch.Generator().manual_seed(1)) * 0.7).to(torch.bfloat16)
    x[7] = 0
    q, s = mb.ops.quantize_rows(x.to(DEV))
    m = x.float().abs().amax(dim=1)
    inv = torch.where(m > 0, torch.tensor(127.0) / m, torch.zeros(()))
    ref = torch.clamp(torch.round(x.float() * inv[:, None]), -127, 127).to(torch.int8)
    assert torch.equal(q.cpu(), ref)
    assert torch.equal(s.cpu(), m / 127.0)


@pytest.mark.parametrize("rows", [100, 128, 391])
@pytest.mark.parametrize("density", [0.3, 1.0])
def test_linear_i8_equals_bf16_kernel_on_exact_activations(rows, density):
    """ragged topology, odd tile-column count (the last pair of the int8 schedule is half empty)."""
    rng = np.random.default_rng(21)
    R, C = 40, 23
    mask = rng.random((R, C)) < density
    if density < 1:
        mask[0] = False
        mask[1] = True
    codes = rng.integers(-1, 2, size=(R * 16, C * 16)).astype(np.int8)
    m = mb.MortarMatrix.from_codes(codes, mask, 0.0173)
    x = _integer_activations(rows, C * 16, rows).to(DEV)
    y8 = mb.ops.linear_tc_i8(x, m.to_sched(False, DEV, arith="i8"))
    assert mb.ops.prefill_error() == 0
    y16 = mb.ops.linear_tc(x, m.to_sched(False, DEV))
    assert torch.equal(y8, y16)
    W = torch.from_numpy(m.to_dense_codes()).float() * torch.tensor(0.0173).to(torch.bfloat16).float()
    assert torch.equal(y8.cpu(), torch.nn.functional.linear(x.cpu().float(), W).to(torch.bfloat16))


@pytest.mark.parametrize("mask", ["uniform", "zipf_rows"])
def test_swiglu_i8_equals_bf16_kernel_on_exact_activations(mask):
    """gate/up with the SwiGLU epilogue and cluster gates on the cloud shape."""
    L = mb.synth.make_layer(2048, 5632, 0.25, seed=300, mask=mask)
    x = _integer_activations(256, 2048, 5).to(DEV)
    ncls = 5632 // 16
    gates = mb.synth.make_gates(256, L, ncls, ncls // 4, seed=3).to(DEV)
    s8, s16 = L.gate_up.to_sched(True, DEV, arith="i8"), L.gate_up.to_sched(True, DEV)
    assert torch.equal(mb.ops.linear_tc_i8(x, s8), mb.ops.linear_tc(x, s16))
    assert torch.equal(mb.ops.linear_tc_i8(x, s8, gates=gates, cluster_size=16),
                       mb.ops.linear_tc(x, s16, gates=gates, cluster_size=16))
    assert mb.ops.prefill_error() == 0


def test_mlp_i8_against_oracle_reports_margin(record_property):
    """Ordinary activations: error relative to the output RMS stays within a few percent; the
    fraction of elements outside the bf16 element-wise tolerance (1e-2 relative + 1e-3 absolute)
    is recorded -- it is why this arm is opt-in."""
    d, f, rows = 2048, 5632, 256
    L = mb.synth.make_layer(d, f, 0.25, seed=200)
    x = mb.synth.make_activations(rows, d, seed=9)
    y = mb.ops.mlp_prefill_tc_i8(x.to(DEV), L.gate_up.to_sched(True, DEV, arith="i8"),
                                 L.down.to_sched(False, DEV, arith="i8")).cpu().float()
    assert mb.ops.prefill_error() == 0
    ref = orc.swiglu_mlp(x.float(), _dense(L.gate_up), _dense(L.down), dtype=torch.bfloat16).float()
    rms = float(ref.pow(2).mean().sqrt())
    err = (y - ref).abs()
    rel_rms = float(err.pow(2).mean().sqrt()) / rms
    outside = float((err > 1e-2 * ref.abs() + 1e-3).float().mean())
    record_property("i8_rms_error_over_rms", rel_rms)
    record_property("i8_fraction_outside_bf16_tolerance", outside)
    print(f"int8 arm: rms error / rms output = {rel_rms:.4f}, max error / rms = {float(err.max()) / rms:.4f}, "
          f"fraction outside 1e-2/1e-3 = {outside:.4f}")
    assert rel_rms < 3e-2
    assert float(err.max()) / rms < 0.25
