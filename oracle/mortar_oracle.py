"""CPU oracle for the MORTAR sparse-MLP path.  TEST INFRASTRUCTURE ONLY.

This module is a plain restatement, in numpy / CPU PyTorch, of the arithmetic the
reference performs on the carved block-sparse ternary SwiGLU MLP.  It exists so the
CUDA kernels can be checked against something that does not share any code with
them.  Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it; the product package never does.

Parity status: PINNED.  Every function below is checked against fixtures under
``tests/golden/`` that were produced by importing and running the reference's own
Python code on CPU (``tests/golden/make_golden.py`` is the generating script).

Each function cites the reference file:line it follows (paths are relative to the
reference project root).
"""
from __future__ import annotations

import math
from typing import NamedTuple, Optional

import numpy as np
import torch
import torch.nn.functional as F

Tensor = torch.Tensor


# ---------------------------------------------------------------------------------
# 2-bit ternary packing            morph/inference/deploy_quant.py:56-95
# ---------------------------------------------------------------------------------

def ternary_quantize(w: Tensor, threshold: float = 0.5) -> tuple[Tensor, Tensor]:
    """(codes int8 in {-1,0,1}, scale fp32 0-dim).  deploy_quant.py:81-95.

    scale = mean(|w|) over ALL elements handed in (the caller passes kept tiles only,
    deploy_quant.py:356-358), clamped at 1e-8; code = sign(w/scale) where |w/scale| >
    threshold, evaluated in fp32.
    """
    wf = w.detach().float()
    scale = wf.abs().mean().clamp(min=1e-8)
    wn = wf / scale
    q = (torch.sign(wn) * (wn.abs() > threshold)).to(torch.int8)
    return q, scale


def pack_ternary_codes(q: np.ndarray) -> np.ndarray:
    """Flat 2-bit pack: byte k holds elements 4k..4k+3, element i in bits 2i..2i+1,
    stored value = code + 1; tail padded with stored 0.  deploy_quant.py:56-71."""
    flat = np.asarray(q).reshape(-1).astype(np.int16) + 1
    pad = (-flat.size) % 4
    if pad:
        flat = np.concatenate([flat, np.zeros(pad, dtype=np.int16)])
    u = flat.astype(np.uint8).reshape(-1, 4)
    return (u[:, 0] | (u[:, 1] << 2) | (u[:, 2] << 4) | (u[:, 3] << 6)).astype(np.uint8)


def unpack_ternary(packed: np.ndarray, numel: int) -> np.ndarray:
    """Inverse of :func:`pack_ternary_codes` -> int8 codes.  deploy_quant.py:74-78."""
    p = np.asarray(packed, dtype=np.uint8)
    u = (p[:, None] >> np.array([0, 2, 4, 6], dtype=np.uint8)) & 3
    return (u.reshape(-1)[:numel].astype(np.int8) - 1)


def magic_dequant(byte: int, stride: int) -> float:
    """Magic-number dequant of one 2-bit field.  fused_decode_step.py:1394-1411:
    bitcast_f32(((byte >> 2*stride) & 3) | 0x4B400000) - 12582913.0 == code."""
    bits = np.array([((byte >> (2 * stride)) & 3) | 0x4B400000], dtype=np.uint32)
    return float(bits.view(np.float32)[0] - np.float32(12582913.0))


# ---------------------------------------------------------------------------------
# Topology selection + carve       morph/model/layers/block_sparse.py:659-743, 810-907
# ---------------------------------------------------------------------------------

def tile_l2_scores(w: Tensor, tile: int = 16) -> Tensor:
    """Per-tile Frobenius norm [out/tile, in/tile] in fp32 -- the quantity the
    reference's ``score_mode="magnitude"`` accumulates (block_sparse.py:484-486)."""
    O, I = w.shape
    t = w.float().reshape(O // tile, tile, I // tile, tile)
    return t.pow(2).sum(dim=(1, 3)).sqrt()


def prune_blocks_once(tile_scores: Tensor, prune_rate: float, target_density: float,
                      blocking: int = 16, tile: int = 16) -> Tensor:
    """One ``prune_step_blocks`` call starting from an all-alive mask.

    block_sparse.py:659-743: pool tile scores to blocks, drop the lowest-score blocks
    GLOBALLY (not per row), never dropping each block-row's best block; the number
    kept is max(target_keep, min(floor(alive*(1-rate)), alive-1)) with
    target_keep = max(Rb, round(target_density*total)).  Returns the [R, C] bool tile
    mask (True = alive)."""
    R, C = tile_scores.shape
    tpb = blocking // tile
    Rb, Cb = R // tpb, C // tpb
    total = Rb * Cb
    cur_alive = total
    target_keep = max(Rb, int(round(target_density * total)))
    if cur_alive <= target_keep:
        return torch.ones(R, C, dtype=torch.bool)
    new_alive = int(math.floor(cur_alive * (1.0 - prune_rate)))
    new_alive = max(target_keep, min(new_alive, cur_alive - 1))
    n_drop = cur_alive - new_alive
    sal = tile_scores.float().view(Rb, tpb, Cb, tpb).sum(dim=(1, 3))
    row_best = sal.argmax(dim=1)
    droppable = sal.clone()
    droppable[torch.arange(Rb), row_best] = float("inf")
    n_drop = min(n_drop, int(torch.isfinite(droppable).sum()))
    alive = torch.ones(Rb * Cb, dtype=torch.bool)
    if n_drop > 0:
        _, drop_idx = droppable.flatten().topk(n_drop, largest=False)
        alive[drop_idx] = False
    return (alive.view(Rb, 1, Cb, 1).expand(Rb, tpb, Cb, tpb).reshape(R, C).contiguous())


class Carved(NamedTuple):
    """BCSR storage exactly as ``carve()`` leaves it (block_sparse.py:874-899)."""
    data: Tensor               # [nnz, blk, blk] (dtype of w)
    row_indices: Tensor        # int16 [nnz]
    column_indices: Tensor     # int16 [nnz], ascending inside a row
    offsets: Tensor            # int32 [Rb+1]
    column_indices_t: Tensor   # int16 [nnz]
    offsets_t: Tensor          # int32 [Cb+1]
    block_offsets_t: Tensor    # int32 [nnz]
    blocking: int
    out_features: int
    in_features: int


def carve(w: Tensor, tile_mask: Optional[Tensor], blocking: int, tile: int = 16) -> Carved:
    """Masked-dense weight -> BCSR blocks.  block_sparse.py:810-907 and the stk
    transpose metadata of morph/sparse/stk/matrix.py:107-125.  A block is kept if ANY
    of its tiles is alive; dead tiles inside a kept block ride along as zeros.  Raises
    if a block-row keeps nothing (block_sparse.py:871-872)."""
    O, I = w.shape
    if O % blocking or I % blocking:
        raise ValueError(f"carve: [{O},{I}] not divisible by blocking {blocking}")
    if blocking % tile:
        raise ValueError(f"carve: blocking ({blocking}) not divisible by tile_size ({tile})")
    tpb = blocking // tile
    Rb, Cb = O // blocking, I // blocking
    if tile_mask is None:
        tile_mask = torch.ones(O // tile, I // tile, dtype=torch.bool)
    elem = tile_mask.repeat_interleave(tile, 0).repeat_interleave(tile, 1)
    w = w * elem.to(w.dtype)
    block_mask = tile_mask.view(Rb, tpb, Cb, tpb).any(dim=3).any(dim=1)
    if not bool(block_mask.any(dim=1).all()):
        raise RuntimeError("carve: a block-row has zero kept blocks")
    idx = block_mask.nonzero()
    row_indices = idx[:, 0].to(torch.int16).contiguous()
    column_indices = idx[:, 1].to(torch.int16).contiguous()
    offsets = torch.cat([torch.zeros(1, dtype=torch.int32),
                         block_mask.sum(dim=1).to(torch.int32).cumsum(0, dtype=torch.int32)])
    blocks = w.reshape(Rb, blocking, Cb, blocking).permute(0, 2, 1, 3)
    data = blocks[idx[:, 0], idx[:, 1]].contiguous()
    gather = column_indices.argsort()
    column_indices_t = row_indices.gather(0, gather.long())
    block_offsets_t = gather.int()
    nnz_per_col = torch.bincount(column_indices.long(), minlength=Cb).to(torch.int32)
    offsets_t = torch.cat([torch.zeros(1, dtype=torch.int32),
                           nnz_per_col.cumsum(0, dtype=torch.int32)])
    return Carved(data, row_indices, column_indices, offsets, column_indices_t, offsets_t,
                  block_offsets_t, blocking, O, I)


def mortar_dense(codes: Tensor, scale: Tensor, row_indices: Tensor, column_indices: Tensor,
                 out_features: int, in_features: int, bf16_weights: bool = True) -> Tensor:
    """Dense fp32 reconstruction of the effective weight (pruned blocks exact zeros).

    morph/inference/engine.py:74-84 composed with the deploy dequant of
    deploy_quant.py:367-369: effective block = codes.to(bf16) * scale.to(bf16), widened
    to fp32.  With ``bf16_weights=False`` the fp32 scale is used instead (the decode
    kernels' algebra, fused_decode_step.py:1441-1459)."""
    nnz, blk, _ = codes.shape
    if bf16_weights:
        eff = (codes.to(torch.bfloat16) * scale.to(torch.bfloat16)).float()
    else:
        eff = codes.float() * scale.float()
    W = torch.zeros(out_features, in_features, dtype=torch.float32)
    W4 = W.view(out_features // blk, blk, in_features // blk, blk)
    W4[row_indices.long(), :, column_indices.long()] = eff
    return W


# ---------------------------------------------------------------------------------
# Decode strip pack + work list    morph/kernels/triton/fused_decode_step.py:1465-1499
# ---------------------------------------------------------------------------------

class StripPack(NamedTuple):
    strips: np.ndarray     # uint8 [nnz, blk, blk//4]
    col_idx: np.ndarray    # int32 [nnz]
    offsets: np.ndarray    # int32 [R+1]
    scale: np.float32
    out_features: int
    ent: np.ndarray        # int32 [3, E]  (row, first block, slot)
    nspl_max: int
    cnts: np.ndarray       # int32 [R]


MORTAR_CB = 4  # blocks per work-list entry, fused_decode_step.py:1462


def pack_strips(codes: np.ndarray, col_idx: np.ndarray, offsets: np.ndarray,
                scale: float) -> StripPack:
    """Strip layout: byte b of row lr holds the codes of columns
    {b, b+blk/4, b+2blk/4, b+3blk/4} (stored code+1, little-endian 2-bit fields), plus
    the balanced work list of <=CB consecutive blocks of one row per entry."""
    codes = np.asarray(codes)
    nnz, blk, _ = codes.shape
    u = (codes.astype(np.int16) + 1).astype(np.uint8).reshape(nnz, blk, 4, blk // 4)
    strips = (u[:, :, 0] | (u[:, :, 1] << 2) | (u[:, :, 2] << 4) | (u[:, :, 3] << 6))
    offsets = np.asarray(offsets, dtype=np.int32)
    R = offsets.size - 1
    rows, j0s, slots = [], [], []
    nspl_max = 0
    for r in range(R):
        lo, hi = int(offsets[r]), int(offsets[r + 1])
        nch = -(-(hi - lo) // MORTAR_CB)
        nspl_max = max(nspl_max, nch)
        for s in range(nch):
            rows.append(r); j0s.append(lo + s * MORTAR_CB); slots.append(s)
    ent = np.array([rows, j0s, slots], dtype=np.int32).reshape(3, -1)
    cnts = (-(-(offsets[1:] - offsets[:-1]) // MORTAR_CB)).astype(np.int32)
    return StripPack(np.ascontiguousarray(strips), np.asarray(col_idx, dtype=np.int32), offsets,
                     np.float32(scale), R * blk, ent, nspl_max, cnts)


def mortar_gemv(x: np.ndarray, pack: StripPack, swiglu_out: bool = False,
                row_act: Optional[np.ndarray] = None, col_act: Optional[np.ndarray] = None,
                gates: Optional[np.ndarray] = None, cluster_size: int = 0) -> np.ndarray:
    """The decode GEMV in the reference's own order of operations.

    fused_decode_step.py:1341-1413 (partials per work-list entry, fp32, exact +-x
    products, rows/columns skipped by the per-stream activity flags) followed by
    :1416-1459 (sum partial slots in slot order, multiply by the per-tensor scale AFTER
    the sum, optional silu(g)*u and cluster gate).  x [B, I] fp32 -> [B, O] or [B, O/2]."""
    x = np.asarray(x, dtype=np.float32)
    B = x.shape[0]
    nnz, blk, q = pack.strips.shape
    O = pack.out_features
    part = np.zeros((max(pack.nspl_max, 1), B, O), dtype=np.float32)
    E = pack.ent.shape[1]
    sh = np.array([0, 2, 4, 6], dtype=np.uint8)
    for e in range(E):
        r, j0, sl = (int(v) for v in pack.ent[:, e])
        hi = int(pack.offsets[r + 1])
        for b in range(B):
            if row_act is not None and row_act[b, r] == 0:
                part[sl, b, r * blk:(r + 1) * blk] = 0.0
                continue
            acc = np.zeros((blk, q), dtype=np.float32)
            for jj in range(MORTAR_CB):
                j = j0 + jj
                if j >= hi:
                    continue
                cb = int(pack.col_idx[j])
                if col_act is not None and col_act[b, cb] == 0:
                    continue
                p = pack.strips[j]                              # [blk, blk/4]
                for st in range(4):
                    w = ((p >> sh[st]) & 3).astype(np.float32) - np.float32(1.0)
                    xs = x[b, cb * blk + st * q: cb * blk + (st + 1) * q]
                    acc += w * xs[None, :]
            part[sl, b, r * blk:(r + 1) * blk] = acc.sum(axis=1, dtype=np.float32)
    cnt_row = np.repeat(pack.cnts, blk)                          # [O]
    tot = np.zeros((B, O), dtype=np.float32)
    for s in range(pack.nspl_max):
        tot += np.where((s < cnt_row)[None, :], part[s], np.float32(0.0))
    tot = tot * pack.scale
    if not swiglu_out:
        return tot
    FF = O // 2
    g, u = tot[:, :FF], tot[:, FF:]
    h = g * (np.float32(1.0) / (np.float32(1.0) + np.exp(-g, dtype=np.float32))) * u
    if gates is not None:
        h = h * np.repeat(np.asarray(gates, dtype=np.float32), cluster_size, axis=1)
    return h.astype(np.float32)


# ---------------------------------------------------------------------------------
# ReMoE routing inputs             morph/model/routing.py:236-260; engine.py:384-413
# ---------------------------------------------------------------------------------

def remoe_gates(logits: Tensor, k: int) -> Tensor:
    """gates = relu(logits - kth_largest) * k / clamp(sum, 1e-6).  The k-th largest
    logit maps to exactly 0, so k-1 groups are strictly active.  routing.py:236-260."""
    G = logits.shape[-1]
    if k < G:
        kth = logits.topk(k, dim=-1).values[..., -1:]
        g = F.relu(logits - kth)
    else:
        g = F.relu(logits)
    s = g.sum(dim=-1, keepdim=True).clamp(min=1e-6)
    return g * (k / s)


def router_logits(x: np.ndarray, wq: np.ndarray, iter_vec: np.ndarray, ln_w: np.ndarray, ln_b: np.ndarray,
                  ln_eps: float, ska: np.ndarray, skb: np.ndarray, gbias: np.ndarray) -> np.ndarray:
    """Group logits of the ReMoE router for rows x[N, d] (float64 accumulation, returned as
    float32).  routing.py:166-204: q = LayerNorm(x Wq^T + iter_embed); product-key scores of the
    two halves of q; the nsk^2 sums sa[a] + sb[b] (a-major) mapped onto G groups 1:1, as the G
    largest in descending order, or repeated cyclically; + group_bias."""
    x = np.asarray(x, dtype=np.float64)
    qv = x @ np.asarray(wq, dtype=np.float64).T + np.asarray(iter_vec, dtype=np.float64)
    mean = qv.mean(axis=1, keepdims=True)
    var = ((qv - mean) ** 2).mean(axis=1, keepdims=True)          # biased, as torch LayerNorm
    q = (qv - mean) / np.sqrt(var + ln_eps) * np.asarray(ln_w, dtype=np.float64) + np.asarray(ln_b, dtype=np.float64)
    d2 = x.shape[1] // 2
    sa = q[:, :d2] @ np.asarray(ska, dtype=np.float64).T
    sb = q[:, d2:] @ np.asarray(skb, dtype=np.float64).T
    nsk = sa.shape[1]
    prod = (sa[:, :, None] + sb[:, None, :]).reshape(x.shape[0], nsk * nsk)
    G = gbias.shape[0]
    if nsk * nsk == G:
        lg = prod
    elif nsk * nsk > G:
        lg = -np.sort(-prod, axis=1, kind="stable")[:, :G]
    else:
        lg = prod[:, np.arange(G) % (nsk * nsk)]
    return (lg + np.asarray(gbias, dtype=np.float64)).astype(np.float32)


def cluster_spans(d_ff: int, n_clusters: int, blk: int):
    """Cluster span (lo, hi) of every gate_up output block-row (gate half then up half,
    same neuron mapping) and every down input block-column.  engine.py:384-413."""
    cls = d_ff // n_clusters
    rh = np.arange(d_ff // blk)
    lo = (rh * blk) // cls
    hi = (rh * blk + blk - 1) // cls
    return (np.concatenate([lo, lo]).astype(np.int32), np.concatenate([hi, hi]).astype(np.int32),
            lo.astype(np.int32), hi.astype(np.int32))


def route_flags(gates: np.ndarray, rlo, rhi, clo, chi):
    """A block is active iff either spanned cluster has gate > 0.
    fused_decode_step.py:1883-1910.  Returns (ract [B,NR], cact [B,NC]) int32."""
    g = np.asarray(gates, dtype=np.float32)
    ract = ((g[:, rlo] > 0) | (g[:, rhi] > 0)).astype(np.int32)
    cact = ((g[:, clo] > 0) | (g[:, chi] > 0)).astype(np.int32)
    return ract, cact


def rmsnorm_rows(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """(x * rsqrt(mean(x^2) + eps)) * w in fp32.  fused_decode_step.py:293-302."""
    xf = x.float()
    r = 1.0 / torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * r) * weight.float()


# ---------------------------------------------------------------------------------
# The MLP itself                   morph/model/transformer.py:402-431
# ---------------------------------------------------------------------------------

def swiglu_mlp(x: Tensor, w_gu: Tensor, w_dn: Tensor, gates: Optional[Tensor] = None,
               n_clusters: int = 0, dtype: torch.dtype = torch.float32) -> Tensor:
    """gu = x W_gu^T; gate, up = gu.chunk(2); h = silu(gate)*up; h *= gates per
    contiguous cluster; y = h W_dn^T.  With ``dtype=torch.bfloat16`` every op rounds
    to bf16 exactly where the reference's autocast path does (gu, silu, product, gate
    multiply, y) because the same torch ops run on bf16 tensors."""
    xd = x.to(dtype)
    gu = F.linear(xd, w_gu.to(dtype))
    gate, up = gu.chunk(2, dim=-1)
    h = F.silu(gate) * up
    if gates is not None:
        d_ff = h.shape[-1]
        cs = d_ff // n_clusters
        g = gates.to(h.dtype)
        h = (h.unflatten(-1, (n_clusters, cs)) * g.unsqueeze(-1)).flatten(-2)
    return F.linear(h, w_dn.to(dtype))


def swiglu_mlp_decode(x: Tensor, codes_gu: Tensor, scale_gu: Tensor, meta_gu,
                      codes_dn: Tensor, scale_dn: Tensor, meta_dn,
                      gates: Optional[Tensor] = None, n_clusters: int = 0,
                      rms_weight: Optional[Tensor] = None, eps: float = 1e-6) -> Tensor:
    """Decode-engine semantics (engine.py:936-986): fp32 throughout, optional rmsnorm
    in front, exact ternary codes, the per-tensor scale applied once after each sum,
    silu as g*sigmoid(g), cluster gates multiplied in fp32.  ``meta_*`` is
    (row_indices, column_indices, out_features, in_features)."""
    xf = x.float()
    if rms_weight is not None:
        xf = rmsnorm_rows(xf, rms_weight, eps)
    one = torch.ones((), dtype=torch.float32)
    Cgu = mortar_dense(codes_gu, one, meta_gu[0], meta_gu[1], meta_gu[2], meta_gu[3], False)
    Cdn = mortar_dense(codes_dn, one, meta_dn[0], meta_dn[1], meta_dn[2], meta_dn[3], False)
    gu = F.linear(xf, Cgu) * scale_gu.float()
    g, u = gu.chunk(2, dim=-1)
    h = g * torch.sigmoid(g) * u
    if gates is not None:
        cs = h.shape[-1] // n_clusters
        h = h * gates.float().repeat_interleave(cs, dim=-1)
    return F.linear(h, Cdn) * scale_dn.float()


# ---------------------------------------------------------------------------------
# The steps beside the MLP in the decode engine
# ---------------------------------------------------------------------------------

def hc_post(hres: Tensor, hpost_row: Tensor, h: Tensor, y: Tensor, term: Optional[Tensor] = None) -> Tensor:
    """Hyper-connection POST write: out[..., i, c] = sum_j Hres[..., i, j] h[..., j, c]
    + Hpost_row[..., i] y[..., c] (+ term[..., c] on every stream).  Follows
    morph/kernels/triton/fused_hyper_connection.py:933-977 (_hc_post_fwd_kernel; eager twin
    hc_post_reference :1426-1433); called after the MLP at morph/inference/engine.py:1001-1060."""
    out = torch.einsum("...ij,...jc->...ic", hres.float(), h.float()) + hpost_row.float().unsqueeze(-1) * y.float().unsqueeze(-2)
    if term is not None:
        out = out + term.float().unsqueeze(-2)
    return out


def unpack_row_strips(codes: np.ndarray) -> np.ndarray:
    """Strip-packed dense ternary rows [O, I/4] uint8 -> int8 codes [O, I]: byte j of a row holds
    columns j, j+I/4, j+I/2, j+3I/4 in its four 2-bit fields, stored value = code + 1
    (ternary_pack, morph/kernels/triton/fused_decode_step.py:1181-1204)."""
    p = np.asarray(codes, dtype=np.uint8)
    O, I4 = p.shape
    out = np.zeros((O, 4, I4), dtype=np.int8)
    for st in range(4):
        out[:, st] = ((p >> (2 * st)) & 3).astype(np.int8) - 1
    return out.reshape(O, 4 * I4)


def ternary_gemv_rs(x: np.ndarray, codes: np.ndarray, row_scale: np.ndarray) -> np.ndarray:
    """out[b, o] = row_scale[o] * sum_i code[o, i] x[b, i]: the row-scaled dense ternary GEMV
    (_ternary_rs_kernel, morph/kernels/triton/fused_decode_step.py:1754-1791): exact +-x products,
    fp32 accumulate, the scale applied once after the sum."""
    w = unpack_row_strips(codes).astype(np.float32)
    return (np.asarray(x, dtype=np.float32) @ w.T) * np.asarray(row_scale, dtype=np.float32)[None, :]
