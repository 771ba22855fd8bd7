"""The persistent stack-decode launch against the per-application entry point (itself checked
against the oracle) and against the oracle directly."""
import numpy as np
import pytest
import torch

import mortar_b200 as mb
from test_gpu_parity import _decode_oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _stack(d, f, n_layers, seed0, rms=True):
    layers, host = [], []
    gen = torch.Generator().manual_seed(seed0 + 77)
    for i in range(n_layers):
        L = mb.synth.make_layer(d, f, 0.25, seed=seed0 + i)
        w = (1.0 + 0.05 * torch.randn(d, generator=gen)) if rms else None
        layers.append((L.gate_up, L.down, w))
        host.append((L, w))
    return layers, host


PLANES = [3, mb.ops.PLANES_HALF2]


@pytest.mark.parametrize("planes", PLANES)
@pytest.mark.parametrize("cs", [8, 16])
@pytest.mark.parametrize("rows", [1, 8, 13, 64])
def test_stack_matches_per_application_calls(rows, cs, planes):
    layers, host = _stack(768, 2048, 3, 100)
    order = [0, 1, 2, 1, 2, 0]
    stack = mb.ops.DecodeStack(layers, order, DEV)
    x0 = mb.synth.make_activations(rows, 768, seed=rows, dtype=torch.float32) * 2.0
    x = x0.clone().to(DEV)
    mb.ops.stack_decode(x, stack, cluster_size=cs, n_planes=planes)
    assert stack.error() == 0
    ref = x0.clone().to(DEV)
    streams = [(gu.to_stream(DEV), dn.to_stream(DEV), w.to(DEV)) for gu, dn, w in layers]
    for i in order:
        gu, dn, w = streams[i]
        mb.ops.mlp_decode(ref, gu, dn, rms_weight=w, n_planes=3, out=ref, accumulate=True)
    assert float((x - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    # and against the oracle for the first application alone
    x1 = x0.clone().to(DEV)
    mb.ops.stack_decode(x1, mb.ops.DecodeStack(layers, [0], DEV), n_planes=planes)
    L, w = host[0]
    y = _decode_oracle(x0, L, rms_w=w)
    assert float((x1.cpu() - (x0 + y)).abs().max()) <= 1e-5 * float((x0 + y).abs().max())


@pytest.mark.parametrize("cs", [8, 16])
def test_half_planes_follow_the_magnitude_of_every_row(cs):
    """fp16 planes: rows whose magnitudes span twelve decades, with and without an RMSNorm, stay
    within 1e-5 of each row's own largest output (every row has its own power-of-two scales)."""
    mags = torch.tensor([1e-6, 1e-3, 0.05, 1.0, 7.0, 3e2, 1e4, 1e6, 1e-5, 2.0, 1e3])[:, None]
    x0 = mb.synth.make_activations(11, 768, seed=5, dtype=torch.float32) * mags
    for rms in (True, False):
        layers, host = _stack(768, 2048, 1, 500, rms=rms)
        x = x0.clone().to(DEV)
        stack = mb.ops.DecodeStack(layers, [0], DEV)
        mb.ops.stack_decode(x, stack, n_planes=mb.ops.PLANES_HALF2, cluster_size=cs)
        assert stack.error() == 0
        L, w = host[0]
        y = _decode_oracle(x0, L, rms_w=w)
        ref = x0 + y
        err = (x.cpu() - ref).abs().amax(dim=1)
        assert bool((err <= 1e-5 * ref.abs().amax(dim=1)).all()), (err / ref.abs().amax(dim=1)).tolist()
        # the update itself, not only the carrier it is added to
        dy = ((x.cpu() - x0) - y).abs().amax(dim=1)
        assert bool((dy <= 2e-5 * y.abs().amax(dim=1) + 1e-6 * x0.abs().amax(dim=1)).all())


@pytest.mark.parametrize("planes", PLANES)
def test_stack_without_norm_and_limits(planes):
    layers, host = _stack(256, 1024, 1, 300, rms=False)
    stack = mb.ops.DecodeStack(layers, [0, 0], DEV)
    x0 = mb.synth.make_activations(20, 256, seed=3, dtype=torch.float32)
    x = x0.clone().to(DEV)
    mb.ops.stack_decode(x, stack, n_planes=planes)
    assert stack.error() == 0
    ref = x0.clone().to(DEV)
    gu, dn = layers[0][0].to_stream(DEV), layers[0][1].to_stream(DEV)
    for _ in range(2):
        mb.ops.mlp_decode(ref, gu, dn, n_planes=3, out=ref, accumulate=True)
    assert float((x - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    # the cloud shape does not fit a rank's shared memory: refused, not silently slow
    big, _ = _stack(2048, 5632, 1, 200, rms=False)
    with pytest.raises(ValueError):
        mb.ops.stack_decode(torch.zeros(8, 2048, device=DEV), mb.ops.DecodeStack(big, [0], DEV))
