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


@pytest.mark.parametrize("cs", [8, 16])
@pytest.mark.parametrize("rows", [1, 8, 13, 64])
def test_stack_matches_per_application_calls(rows, cs):
    layers, host = _stack(768, 2048, 3, 100)
    order = [0, 1, 2, 1, 2, 0]
    stack = mb.ops.DecodeStack(layers, order, DEV)
    x0 = mb.synth.make_activations(rows, 768, seed=rows, dtype=torch.float32) * 2.0
    x = x0.clone().to(DEV)
    mb.ops.stack_decode(x, stack, cluster_size=cs)
    assert stack.error() == 0
    ref = x0.clone().to(DEV)
    streams = [(gu.to_stream(DEV), dn.to_stream(DEV), w.to(DEV)) for gu, dn, w in layers]
    for i in order:
        gu, dn, w = streams[i]
        mb.ops.mlp_decode(ref, gu, dn, rms_weight=w, n_planes=3, out=ref, accumulate=True)
    assert float((x - ref).abs().max()) <= 1e-5 * float(ref.abs().max())
    # and against the oracle for the first application alone
    x1 = x0.clone().to(DEV)
    mb.ops.stack_decode(x1, mb.ops.DecodeStack(layers, [0], DEV))
    L, w = host[0]
    y = _decode_oracle(x0, L, rms_w=w)
    assert float((x1.cpu() - (x0 + y)).abs().max()) <= 1e-5 * float((x0 + y).abs().max())


def test_stack_without_norm_and_limits():
    layers, host = _stack(256, 1024, 1, 300, rms=False)
    stack = mb.ops.DecodeStack(layers, [0, 0], DEV)
    x0 = mb.synth.make_activations(20, 256, seed=3, dtype=torch.float32)
    x = x0.clone().to(DEV)
    mb.ops.stack_decode(x, stack)
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
