"""The allocation-free MLP entry point (``mortar_mlp_decode_static``) against the regular one.

Some callers of this library cannot provide device memory: a foreign runtime that binds the
C ABI without a CUDA allocator of its own, or a latency-critical loop where ``cudaMalloc`` is
off limits because it synchronises the device.  For them the library keeps the MLP's
intermediate activation planes in an 8 MiB array compiled into it.  This file checks, through
the C ABI, that the variant returns what ``mortar_mlp_decode`` returns -- on two calls in a
row, because the second call finds the first call's data still in the shared array -- and
that a batch too large for the array is refused with a clear error.  It is named to be
collected last, so a run that stops at the first failure has already run everything else.
"""
import pytest
import torch

import mortar_b200 as mb

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL = 1e-5      # the decode-path tolerance of the other GPU tests (relative to max |y|)


def _layer():
    L = mb.synth.make_layer(768, 2048, 0.25, seed=100)
    return L, L.gate_up.to_stream(DEV), L.down.to_stream(DEV)


def test_static_scratch_matches_workspace_entry_point_twice():
    L, gu, dn = _layer()
    rms_w = (1.0 + 0.05 * torch.randn(768, generator=torch.Generator().manual_seed(5))).to(DEV)
    for call, (rows, seed, routed) in enumerate([(64, 1, False), (8, 2, True)]):
        x = (mb.synth.make_activations(rows, 768, seed=seed, dtype=torch.float32) * 2.5).to(DEV)
        gates = mb.synth.make_gates(rows, L, 16, 8, seed=seed).to(DEV).contiguous() if routed else None
        ref = mb.ops.mlp_decode(x, gu, dn, rms_weight=rms_w, gates=gates, n_clusters=16 if routed else 0,
                                n_planes=3)
        out = torch.full_like(x, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        mb.ops.mlp_decode_static(x, gu, dn, out, rms_weight=rms_w, gates=gates,
                                 n_clusters=16 if routed else 0, n_planes=3)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before, "the static entry point must not allocate"
        err = float((out - ref).abs().max()) / float(ref.abs().max())
        assert err <= TOL, f"call {call}: relative error {err}"


def test_static_scratch_against_the_oracle_bf16_input_and_accumulate():
    """The same entry point against the CPU oracle (not only against its sibling), on the path
    that skips the plane kernel (bf16 input, no norm: two launches) and with the residual add."""
    from test_gpu_parity import _decode_oracle
    L, gu, dn = _layer()
    xb = mb.synth.make_activations(24, 768, seed=11)                       # bf16
    ref = _decode_oracle(xb, L)
    out = torch.full((24, 768), float("nan"), device=DEV)
    before = mb.ops.kernel_counts()
    mb.ops.mlp_decode_static(xb.to(DEV), gu, dn, out, n_planes=3)
    after = mb.ops.kernel_counts()
    assert after.get("act_prep", 0) == before.get("act_prep", 0)           # bf16 rows are used as a plane directly
    assert float((out.cpu() - ref).abs().max()) <= TOL * float(ref.abs().max())
    carrier = torch.randn(24, 768, generator=torch.Generator().manual_seed(3))
    acc = carrier.clone().to(DEV)
    mb.ops.mlp_decode_static(xb.to(DEV), gu, dn, acc, n_planes=3, accumulate=True)
    want = carrier + ref
    assert float((acc.cpu() - want).abs().max()) <= TOL * float(want.abs().max())
    import ctypes as C
    gus, dns = gu.c_struct(), dn.c_struct()
    rc = mb._lib.lib().mortar_mlp_decode_static(C.byref(gus), C.byref(dns), None, 0, 768, -1, None, 1e-6, None, 0, 0,
                                               None, 0, 768, 3, 0, None)
    assert rc == -2                                                        # MORTAR_ERR_SHAPE for a negative row count


def test_static_scratch_rejects_oversized_batches():
    L, gu, dn = _layer()
    limit = mb._lib.lib().mortar_mlp_static_scratch_bytes()
    assert limit == 8 << 20
    rows = 1
    while mb._lib.lib().mortar_mlp_workspace_bytes(rows, 768, 2048, 3) <= limit:
        rows *= 2
    x = torch.zeros(rows, 768, device=DEV)
    with pytest.raises(ValueError, match="too small"):
        mb.ops.mlp_decode_static(x, gu, dn, torch.empty_like(x), n_planes=3)
