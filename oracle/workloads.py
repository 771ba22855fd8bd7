"""Seeded benchmark workloads for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

The CPU baseline and the reference arm of the benchmark must not load the CUDA library, so
the synthetic layers of the benchmark configurations are restated here with numpy / CPU
PyTorch alone: same generator seeds, same weights, same topology rule, same ternarisation as
the product's own generator, checked equal to it in the test-suite.  Nothing here reads a
dataset: weights are N(0, 0.02) cast to bf16, topology is one magnitude block-prune step at
blocking 16 (block_sparse.py:659-743, via ``prune_blocks_once``), kept values are ternarised
with the deploy rule (deploy_quant.py:81-95, 356-358), activations are N(0,1) RMS-normalised.
"""
from __future__ import annotations

import torch

from . import mortar_oracle as orc

Tensor = torch.Tensor
TILE = 16


def dense_matrix(w: Tensor, density: float, bf16_scale: bool = False):
    """bf16-valued weight [out, in] -> (effective dense weight = code * scale with zeros in
    pruned tiles, kept-tile count).  Top `density` of the 16x16 tiles by Frobenius norm, each
    tile row keeping its best tile."""
    O, I = w.shape
    R, C = O // TILE, I // TILE
    if density >= 1.0:
        mask = torch.ones(R, C, dtype=torch.bool)
    else:
        mask = orc.prune_blocks_once(orc.tile_l2_scores(w), 1.0 - density, density, blocking=TILE)
    tiles = w.reshape(R, TILE, C, TILE).permute(0, 2, 1, 3)
    kept = tiles[mask]                                              # [nnz, 16, 16], row-major tile order
    q, scale = orc.ternary_quantize(kept)
    s = scale.to(torch.bfloat16).float() if bf16_scale else scale.float()
    dense = torch.zeros(R, C, TILE, TILE)
    dense[mask] = q.float() * s
    return dense.permute(0, 2, 1, 3).reshape(O, I).contiguous(), int(mask.sum())


def dense_layer(d_model: int, d_ff: int, density: float, seed: int, bf16_scale: bool = False):
    """(W_gate_up [2*d_ff, d_model], W_down [d_model, d_ff], kept tiles of both) of the
    benchmark layer with this seed."""
    gen = torch.Generator().manual_seed(seed)
    out, nnz = [], 0
    for (O, I) in ((2 * d_ff, d_model), (d_model, d_ff)):
        w = (torch.randn(O, I, generator=gen) * 0.02).to(torch.bfloat16).float()
        d, n = dense_matrix(w, density, bf16_scale)
        out.append(d)
        nnz += n
    return out[0], out[1], nnz


def activations(rows: int, d_model: int, seed: int, dtype=torch.bfloat16) -> Tensor:
    """x ~ N(0,1), RMS-normalised (eps 1e-6, unit weight), cast to `dtype`."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, d_model, generator=gen)
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    return x.to(dtype)


def norm_weights(n_layers: int, d_model: int, seed: int):
    """Per-layer RMSNorm weights 1 + 0.05 N(0,1), drawn in layer order from one generator."""
    gen = torch.Generator().manual_seed(seed)
    return [1.0 + 0.05 * torch.randn(d_model, generator=gen) for _ in range(n_layers)]


def decode_stack_step(x: Tensor, dense, rms, order) -> Tensor:
    """x <- x + mlp_i(rmsnorm_i(x)) for the listed applications, fp32: the reference's CPU path
    for the carved MLP (dense reconstruction + F.linear, engine.py:74-84,
    transformer.py:402-431) chained with the residual add."""
    for i in order:
        x = x + orc.swiglu_mlp(orc.rmsnorm_rows(x, rms[i], 1e-6), dense[i][0], dense[i][1])
    return x
