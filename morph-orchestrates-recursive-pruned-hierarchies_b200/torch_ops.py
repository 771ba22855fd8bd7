"""The operators as ``torch.library`` custom ops (namespace ``mortar_b200``), plus a shim with
the signature of the reference's block-sparse operator.

The reference registers ``morph_stk::dds`` as a CUDA-only custom op with a fake kernel so the
model can be traced (morph/sparse/stk/backend/custom_ops.py:35-66).  The ops here play that role
for the replacement: tensors only in the schema (the stream arrays of a matrix travel as three
tensors and four scalars), ``device_types="cuda"``, ``mutates_args=()``, and a fake kernel that
returns an empty tensor of the right shape and dtype.  There is no CPU implementation: calling
an op with CPU tensors raises ``NotImplementedError``, like the reference's.

    mortar_b200::linear(x, grp_ptr, grp_cols, grp_codes, scale, out_features, in_features, n_groups) -> y
    mortar_b200::mlp_decode(x, rms_weight?, eps, <gate_up stream>, <down stream>, gates?, n_clusters) -> y
    mortar_b200::mlp_prefill(x, <gate_up stream>, <down stream>, gates?, n_clusters) -> y

``stk_dds`` takes the reference operator's argument list (lhs, data, offsets, row_indices,
column_indices, offsets_t, column_indices_t, block_offsets_t, shape0, shape1, transpose_b) and
runs the same contraction through ``mortar_b200::linear``; ``data`` must hold ternary effective
weights (code * scale), which is what a ternarised MORTAR layer feeds the reference op
(block_sparse.py:909-919, 951-956).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

from . import ops
from .format import MortarMatrix, StreamMatrix

_LIB = "mortar_b200"


def _stream(grp_ptr, grp_cols, grp_codes, scale, out_features, in_features, n_groups) -> StreamMatrix:
    nnz = 0   # only used for accounting
    return StreamMatrix(out_features, in_features, scale, n_groups, nnz, grp_ptr, grp_cols, grp_codes, 0)


def stream_args(w: StreamMatrix):
    """The (tensors..., scalars...) of a stream matrix in the order the ops take them."""
    return (w.grp_ptr, w.grp_cols, w.grp_codes, float(w.scale), int(w.out_features),
            int(w.in_features), int(w.n_groups))


@torch.library.custom_op(f"{_LIB}::linear", mutates_args=(), device_types="cuda")
def linear(x: torch.Tensor, grp_ptr: torch.Tensor, grp_cols: torch.Tensor, grp_codes: torch.Tensor,
           scale: float, out_features: int, in_features: int, n_groups: int) -> torch.Tensor:
    w = _stream(grp_ptr, grp_cols, grp_codes, scale, out_features, in_features, n_groups)
    return ops.linear(x, w)


@linear.register_fake
def _(x, grp_ptr, grp_cols, grp_codes, scale, out_features, in_features, n_groups):
    return x.new_empty((*x.shape[:-1], out_features))


@torch.library.custom_op(f"{_LIB}::mlp_decode", mutates_args=(), device_types="cuda")
def mlp_decode(x: torch.Tensor, rms_weight: Optional[torch.Tensor], eps: float,
               gu_ptr: torch.Tensor, gu_cols: torch.Tensor, gu_codes: torch.Tensor, gu_scale: float,
               gu_out: int, gu_in: int, gu_groups: int,
               dn_ptr: torch.Tensor, dn_cols: torch.Tensor, dn_codes: torch.Tensor, dn_scale: float,
               dn_out: int, dn_in: int, dn_groups: int,
               gates: Optional[torch.Tensor], n_clusters: int) -> torch.Tensor:
    gu = _stream(gu_ptr, gu_cols, gu_codes, gu_scale, gu_out, gu_in, gu_groups)
    dn = _stream(dn_ptr, dn_cols, dn_codes, dn_scale, dn_out, dn_in, dn_groups)
    return ops.mlp_decode(x, gu, dn, rms_weight=rms_weight, eps=eps, gates=gates, n_clusters=n_clusters)


@mlp_decode.register_fake
def _(x, rms_weight, eps, gu_ptr, gu_cols, gu_codes, gu_scale, gu_out, gu_in, gu_groups,
      dn_ptr, dn_cols, dn_codes, dn_scale, dn_out, dn_in, dn_groups, gates, n_clusters):
    return x.new_empty((*x.shape[:-1], dn_out))


@torch.library.custom_op(f"{_LIB}::mlp_prefill", mutates_args=(), device_types="cuda")
def mlp_prefill(x: torch.Tensor,
                gu_ptr: torch.Tensor, gu_cols: torch.Tensor, gu_codes: torch.Tensor, gu_scale: float,
                gu_out: int, gu_in: int, gu_groups: int,
                dn_ptr: torch.Tensor, dn_cols: torch.Tensor, dn_codes: torch.Tensor, dn_scale: float,
                dn_out: int, dn_in: int, dn_groups: int,
                gates: Optional[torch.Tensor], n_clusters: int) -> torch.Tensor:
    gu = _stream(gu_ptr, gu_cols, gu_codes, gu_scale, gu_out, gu_in, gu_groups)
    dn = _stream(dn_ptr, dn_cols, dn_codes, dn_scale, dn_out, dn_in, dn_groups)
    return ops.mlp_prefill(x, gu, dn, gates=gates, n_clusters=n_clusters)


@mlp_prefill.register_fake
def _(x, gu_ptr, gu_cols, gu_codes, gu_scale, gu_out, gu_in, gu_groups,
      dn_ptr, dn_cols, dn_codes, dn_scale, dn_out, dn_in, dn_groups, gates, n_clusters):
    return x.new_empty((*x.shape[:-1], dn_out), dtype=torch.bfloat16)


# ---------------------------------------------------------------------------------------
# shim with the reference operator's signature
# ---------------------------------------------------------------------------------------

_DDS_CACHE: "OrderedDict" = OrderedDict()
_DDS_CACHE_MAX = 256            # layers whose converted weights are kept (least recently used goes first)


def _ternary_matrix_from_data(data: torch.Tensor, offsets: torch.Tensor, column_indices: torch.Tensor,
                              out_features: int, in_features: int) -> MortarMatrix:
    """[nnz, blk, blk] effective weights (code * scale) + BCSR row pointers / column ids of the
    reference (block_sparse.py:874-899) -> canonical tile-16 matrix."""
    d = data.detach().float().cpu().numpy()
    nnz, blk, _ = d.shape
    scale = float(np.abs(d).max()) if d.size else 1.0
    if scale == 0.0:
        scale = 1.0
    codes = np.rint(d / scale)
    if not np.array_equal(codes * np.float32(scale), d) or np.abs(codes).max(initial=0) > 1:
        raise ValueError("stk_dds shim: `data` is not ternary (code * one scale); only ternarised "
                         "MORTAR layers can run on the packed kernels")
    off = offsets.detach().cpu().numpy().astype(np.int64)
    ci = column_indices.detach().cpu().numpy().astype(np.int64)
    dense = np.zeros((out_features, in_features), dtype=np.int8)
    mask = np.zeros((out_features // 16, in_features // 16), dtype=bool)
    t = blk // 16
    for r in range(out_features // blk):
        for j in range(int(off[r]), int(off[r + 1])):
            c = int(ci[j])
            dense[r * blk:(r + 1) * blk, c * blk:(c + 1) * blk] = codes[j].astype(np.int8)
            mask[r * t:(r + 1) * t, c * t:(c + 1) * t] = True
    return MortarMatrix.from_codes(dense, mask, scale)


def stk_dds(lhs: torch.Tensor, data: torch.Tensor, offsets: torch.Tensor, row_indices: torch.Tensor,
            column_indices: torch.Tensor, offsets_t: torch.Tensor, column_indices_t: torch.Tensor,
            block_offsets_t: torch.Tensor, shape0: int, shape1: int, transpose_b: bool = True) -> torch.Tensor:
    """``torch.ops.morph_stk.dds`` (custom_ops.py:35-56) on the packed kernels:
    ``out[M, shape1] = lhs[M, shape0] @ W^T`` for the BCSR matrix W[shape1, shape0] whose kept
    blocks are ``data`` -- the call CMSBlockLinear._forward_mortar makes with
    ``(in_features, out_features, True)`` (block_sparse.py:956-966).  The transposed metadata is
    not needed.
    The conversion of ``data`` is cached per storage, so a layer converts once."""
    if not transpose_b:
        raise ValueError("stk_dds shim: only the transpose_b=True form of the MLP forward is served")
    if not lhs.is_cuda:
        raise NotImplementedError("morph_stk::dds is a CUDA-only operator (no CPU path)")
    key = (data.data_ptr(), data._version, tuple(data.shape), offsets.data_ptr(), int(shape0), int(shape1))
    w = _DDS_CACHE.get(key)
    if w is None:
        w = _ternary_matrix_from_data(data, offsets, column_indices, int(shape1), int(shape0)).to_stream(lhs.device)
        _DDS_CACHE[key] = w
        while len(_DDS_CACHE) > _DDS_CACHE_MAX:
            _DDS_CACHE.popitem(last=False)
    else:
        _DDS_CACHE.move_to_end(key)
    return linear(lhs, *stream_args(w))
