"""Seeded synthetic MORTAR layers, topologies and routing inputs in the shapes the benchmark
configurations name.  Nothing here reads a dataset or a checkpoint: weights are
N(0, 0.02) cast to bf16, topologies come from the generators below, activations are
N(0,1) RMS-normalised, router logits are N(0,1).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .format import TILE, MortarMatrix, ternary_quantize

# shapes named by the benchmark configurations
LOCAL = dict(d_model=768, d_ff=2048)        # default 3+6xT+3 stack
CLOUD = dict(d_model=2048, d_ff=5632)       # 4+8xT+4 stack


def topk_l2_mask(w: torch.Tensor, density: float, min_one_per_row: bool = True) -> torch.Tensor:
    """Keep the globally top `density` fraction of 16x16 tiles by Frobenius norm, never
    dropping a tile row's best tile -- one magnitude-scored block-prune step of the reference
    at blocking 16 (morph/model/layers/block_sparse.py:659-743)."""
    O, I = w.shape
    R, C = O // TILE, I // TILE
    sal = w.float().reshape(R, TILE, C, TILE).pow(2).sum(dim=(1, 3)).sqrt()
    total = R * C
    keep = max(R, int(round(density * total)))
    if keep >= total:
        return torch.ones(R, C, dtype=torch.bool)
    new_alive = max(keep, min(int(math.floor(total * density)), total - 1))
    n_drop = total - new_alive
    droppable = sal.clone()
    if min_one_per_row:
        droppable[torch.arange(R), sal.argmax(dim=1)] = float("inf")
    n_drop = min(n_drop, int(torch.isfinite(droppable).sum()))
    alive = torch.ones(total, dtype=torch.bool)
    if n_drop > 0:
        alive[droppable.flatten().topk(n_drop, largest=False).indices] = False
    return alive.view(R, C)


def uniform_mask(R: int, C: int, density: float, gen: torch.Generator) -> torch.Tensor:
    """Uniform-random choice of round(density*R*C) tiles."""
    total = R * C
    keep = int(round(density * total))
    alive = torch.zeros(total, dtype=torch.bool)
    alive[torch.randperm(total, generator=gen)[:keep]] = True
    return alive.view(R, C)


def zipf_row_mask(R: int, C: int, density: float, gen: torch.Generator, a: float = 1.2) -> torch.Tensor:
    """Row-clustered topology: every tile row keeps ONE contiguous run of tile columns whose
    length follows a Zipf(a) row-popularity weight (normalised so the total is
    density*R*C, capped at C), at a uniform random start without wrap-around."""
    ranks = torch.randperm(R, generator=gen).float() + 1.0
    wgt = ranks.pow(-a)
    target = density * R * C
    lens = torch.zeros(R)
    # water-filling so that capping rows at C keeps the requested total
    free = torch.ones(R, dtype=torch.bool)
    remaining = target
    for _ in range(8):
        share = wgt * free
        if share.sum() <= 0:
            break
        prop = share / share.sum() * remaining
        over = (prop >= C) & free
        if not over.any():
            lens[free] = prop[free]
            break
        lens[over] = C
        free &= ~over
        remaining = target - lens[~free].sum()
    lens = lens.round().clamp(0, C).long()
    mask = torch.zeros(R, C, dtype=torch.bool)
    for r in range(R):
        n = int(lens[r])
        if n == 0:
            continue
        start = int(torch.randint(0, C - n + 1, (1,), generator=gen))
        mask[r, start:start + n] = True
    return mask


@dataclass
class SynthLayer:
    """One MLP: canonical matrices plus the dense code matrices for checking."""
    d_model: int
    d_ff: int
    gate_up: MortarMatrix
    down: MortarMatrix

    def dense_codes(self):
        return (torch.from_numpy(self.gate_up.to_dense_codes()),
                torch.from_numpy(self.down.to_dense_codes()))


def make_layer(d_model: int, d_ff: int, density: float = 0.25, seed: int = 0,
               mask: str = "topk_l2") -> SynthLayer:
    """W ~ N(0, 0.02) in bf16 per seed; topology by `mask` ("topk_l2", "uniform",
    "zipf_rows"); kept values ternarised with the deploy rule (scale = mean |kept|)."""
    gen = torch.Generator().manual_seed(seed)
    mats = []
    for (O, I) in ((2 * d_ff, d_model), (d_model, d_ff)):
        w = (torch.randn(O, I, generator=gen) * 0.02).to(torch.bfloat16).float()
        R, C = O // TILE, I // TILE
        if density >= 1.0:
            tm = torch.ones(R, C, dtype=torch.bool)
        elif mask == "topk_l2":
            tm = topk_l2_mask(w, density)
        elif mask == "uniform":
            tm = uniform_mask(R, C, density, gen)
        elif mask == "zipf_rows":
            tm = zipf_row_mask(R, C, density, gen)
        else:
            raise ValueError(f"unknown mask generator {mask!r}")
        mats.append(MortarMatrix.from_weight(w, tm))
    return SynthLayer(d_model, d_ff, mats[0], mats[1])


def make_block_matrix(out_features: int, in_features: int, density: float = 0.25, blocking: int = 128,
                      ragged: bool = True, seed: int = 0, scale: float = 0.02) -> MortarMatrix:
    """Block-aligned ragged topology in the shape of the reference's large-model decode bench
    (tile-prover/proofs/decode/gemv_bw_30b.py:124-165): every block row keeps
    round(density*C*(0.5+u)) random block columns, u ~ U(0,1); codes are uniform over {-1,0,+1}.
    Returned in the canonical tile-16 format (each kept block = (blocking/16)^2 tiles)."""
    rng = np.random.default_rng(seed)
    Rb, Cb = out_features // blocking, in_features // blocking
    tpb = blocking // TILE
    rows_cols = []
    for _ in range(Rb):
        k = int(round(density * Cb * (0.5 + rng.random()))) if ragged else int(round(density * Cb))
        k = max(1, min(Cb, k))
        rows_cols.append(np.sort(rng.permutation(Cb)[:k]))
    row_ptr = [0]
    col_idx = []
    for cols in rows_cols:
        tile_cols = (cols[:, None] * tpb + np.arange(tpb)[None, :]).reshape(-1)
        for _ in range(tpb):
            col_idx.append(tile_cols)
            row_ptr.append(row_ptr[-1] + tile_cols.size)
    col_idx = np.concatenate(col_idx).astype(np.uint16)
    nnz = int(row_ptr[-1])
    stored = rng.integers(0, 3, size=(nnz, 64, 4), dtype=np.uint8)
    codes = (stored[..., 0] | (stored[..., 1] << 2) | (stored[..., 2] << 4) | (stored[..., 3] << 6))
    return MortarMatrix(out_features, in_features, np.asarray(row_ptr, dtype=np.int32), col_idx,
                        np.ascontiguousarray(codes.astype(np.uint8)), float(scale))


def make_activations(rows: int, d_model: int, seed: int, dtype=torch.bfloat16) -> torch.Tensor:
    """x ~ N(0,1), RMS-normalised (eps 1e-6, unit weight), cast to `dtype`."""
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, d_model, generator=gen)
    x = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    return x.to(dtype)


def remoe_gates(logits: torch.Tensor, k: int) -> torch.Tensor:
    """relu(logits - kth largest) * k / clamp(sum, 1e-6): the k-th group lands on exactly 0, so
    k-1 groups are active (morph/model/routing.py:236-260)."""
    G = logits.shape[-1]
    if k < G:
        kth = logits.topk(k, dim=-1).values[..., -1:]
        g = torch.relu(logits - kth)
    else:
        g = torch.relu(logits)
    return g * (k / g.sum(dim=-1, keepdim=True).clamp(min=1e-6))


def make_gates(rows: int, layer: SynthLayer, n_clusters: int, k: int, seed: int) -> torch.Tensor:
    """Router logits ~ N(0,1) over `n_clusters` contiguous hidden groups; groups with no
    surviving tile in gate_up or down are masked to -inf first; gates by the ReMoE rule."""
    gen = torch.Generator().manual_seed(seed)
    logits = torch.randn(rows, n_clusters, generator=gen)
    cs = layer.d_ff // n_clusters
    F_ = layer.d_ff // TILE
    gu_rows = np.diff(layer.gate_up.row_ptr)                      # tiles per gate_up tile row
    hidden_alive = (gu_rows[:F_] > 0) | (gu_rows[F_:] > 0)
    dn_cols = np.zeros(F_, dtype=bool)
    dn_cols[layer.down.col_idx.astype(np.int64)] = True
    tile_alive = torch.from_numpy(hidden_alive & dn_cols)         # per hidden tile row
    neuron_alive = tile_alive.repeat_interleave(TILE)
    cluster_alive = neuron_alive.view(n_clusters, cs).any(dim=1)
    logits = logits.masked_fill(~cluster_alive.unsqueeze(0), float("-inf"))
    return remoe_gates(logits, k)
