"""The operators as ``torch.library`` custom ops (namespace ``mortar_b200``), plus the reference's
own block-sparse operator ``morph_stk::dds`` served by the packed kernels.

The reference registers ``morph_stk::dds`` as a CUDA-only custom op with a fake kernel so the
model can be traced (morph/sparse/stk/backend/custom_ops.py:35-66).  The ops here play that role
for the replacement: tensors only in the schema (the arrays of a matrix travel as tensors plus
scalars), ``device_types="cuda"``, and a fake kernel that returns an empty tensor of the right
shape and dtype.  There is no CPU implementation: calling an op with CPU tensors raises
``NotImplementedError``, like the reference's.

    mortar_b200::linear(x, <stream>) -> y
    mortar_b200::mlp_decode(x, rms_weight?, eps, <gate_up stream>, <down stream>, gates?, n_clusters) -> y
    mortar_b200::mlp_prefill(x, <gate_up stream>, <down stream>, gates?, n_clusters) -> y
    mortar_b200::linear_tc(x, <sched>, gates?, cluster_size) -> y            (tcgen05 kernel)
    mortar_b200::mlp_prefill_tc(x, <gate_up sched>, <down sched>, gates?, n_clusters) -> y
    mortar_b200::stack_decode(x!, blobs, table, app_layer, status!, ...) -> ()   (in place)
    <stream> = grp_ptr, grp_cols, grp_codes, scale, out_features, in_features, n_groups
    <sched>  = step_data, step_off, step_meta, panel_step_ptr, panel_mask, n_tiles, n_runs, n_steps,
               data_units, n_panels, out_features, in_features, swiglu, scale

``mlp_prefill`` and ``linear`` send bf16 token blocks of ``TC_MIN_ROWS`` rows or more to the
tcgen05 kernel (the panel schedule is rebuilt from the stream arrays once per matrix and cached).

``install_morph_stk_dds()`` (run at import) makes ``torch.ops.morph_stk.dds`` -- the reference's
name and schema (lhs, data, offsets, row_indices, column_indices, offsets_t, column_indices_t,
block_offsets_t, shape0, shape1, transpose_b) -- resolve to the packed kernels, so an unmodified
``CMSBlockLinear._forward_mortar`` (block_sparse.py:921-970) runs on them.  ``data`` must hold
ternary effective weights (code * scale), which is what a ternarised MORTAR layer feeds the
reference op (block_sparse.py:909-919, 951-956).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

from . import ops
from .format import (BlockSched, MortarMatrix, SchedMatrix, StreamMatrix, TopologyDev, matrix_from_stream, pack_codes_2bit,
                     wants_block_path)

_LIB = "mortar_b200"
TC_MIN_ROWS = 128        # bf16 token blocks of at least this many rows run the tcgen05 kernel


def _stream(grp_ptr, grp_cols, grp_codes, scale, out_features, in_features, n_groups) -> StreamMatrix:
    nnz = 0   # only used for accounting
    return StreamMatrix(out_features, in_features, scale, n_groups, nnz, grp_ptr, grp_cols, grp_codes, 0)


def stream_args(w: StreamMatrix):
    """The (tensors..., scalars...) of a stream matrix in the order the ops take them."""
    return (w.grp_ptr, w.grp_cols, w.grp_codes, float(w.scale), int(w.out_features),
            int(w.in_features), int(w.n_groups))


def sched_args(w: SchedMatrix):
    """The (tensors..., scalars...) of a panel schedule in the order the ``*_tc`` ops take them."""
    return (w.step_data, w.step_off, w.step_meta, w.panel_step_ptr, w.panel_mask, int(w.n_tiles),
            int(w.n_runs), int(w.n_steps), int(w.data_units), int(w.n_panels), int(w.out_features),
            int(w.in_features), bool(w.swiglu), float(w.scale))


def _sched(step_data, step_off, step_meta, panel_step_ptr, panel_mask, n_tiles, n_runs, n_steps,
           data_units, n_panels, out_features, in_features, swiglu, scale) -> SchedMatrix:
    return SchedMatrix.from_tensors(step_data, step_off, step_meta, panel_step_ptr, panel_mask, n_tiles,
                                    n_runs, n_steps, data_units, n_panels, out_features, in_features,
                                    swiglu, scale)


# panel schedules rebuilt from stream arrays, keyed by the stream's code buffer
_SCHED_FROM_STREAM: "OrderedDict" = OrderedDict()
_CACHE_MAX = 256            # matrices whose derived layouts are kept (least recently used goes first)


def _sched_for_stream(w: StreamMatrix, swiglu: bool) -> SchedMatrix:
    key = (w.grp_codes.data_ptr(), w.grp_ptr.data_ptr(), w.out_features, w.in_features, bool(swiglu))
    hit = _SCHED_FROM_STREAM.get(key)
    if hit is None:
        hit = matrix_from_stream(w).to_sched(swiglu, w.grp_codes.device)
        _SCHED_FROM_STREAM[key] = hit
        while len(_SCHED_FROM_STREAM) > _CACHE_MAX:
            _SCHED_FROM_STREAM.popitem(last=False)
    else:
        _SCHED_FROM_STREAM.move_to_end(key)
    return hit


def _takes_tc(x: torch.Tensor, features: int) -> bool:
    return x.dtype == torch.bfloat16 and x.numel() // max(features, 1) >= TC_MIN_ROWS


@torch.library.custom_op(f"{_LIB}::linear", mutates_args=(), device_types="cuda")
def linear(x: torch.Tensor, grp_ptr: torch.Tensor, grp_cols: torch.Tensor, grp_codes: torch.Tensor,
           scale: float, out_features: int, in_features: int, n_groups: int) -> torch.Tensor:
    w = _stream(grp_ptr, grp_cols, grp_codes, scale, out_features, in_features, n_groups)
    if _takes_tc(x, in_features):
        return ops.linear_tc(x, _sched_for_stream(w, False))
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
    if x.numel() // max(gu_in, 1) >= TC_MIN_ROWS:
        return ops.mlp_prefill_tc(x, _sched_for_stream(gu, True), _sched_for_stream(dn, False), gates=gates,
                                  n_clusters=n_clusters)
    return ops.mlp_prefill(x, gu, dn, gates=gates, n_clusters=n_clusters)


@mlp_prefill.register_fake
def _(x, gu_ptr, gu_cols, gu_codes, gu_scale, gu_out, gu_in, gu_groups,
      dn_ptr, dn_cols, dn_codes, dn_scale, dn_out, dn_in, dn_groups, gates, n_clusters):
    return x.new_empty((*x.shape[:-1], dn_out), dtype=torch.bfloat16)


@torch.library.custom_op(f"{_LIB}::linear_tc", mutates_args=(), device_types="cuda")
def linear_tc(x: torch.Tensor, step_data: torch.Tensor, step_off: torch.Tensor, step_meta: torch.Tensor,
              panel_step_ptr: torch.Tensor, panel_mask: torch.Tensor, n_tiles: int, n_runs: int,
              n_steps: int, data_units: int, n_panels: int, out_features: int, in_features: int,
              swiglu: bool, scale: float, gates: Optional[torch.Tensor], cluster_size: int) -> torch.Tensor:
    w = _sched(step_data, step_off, step_meta, panel_step_ptr, panel_mask, n_tiles, n_runs, n_steps,
               data_units, n_panels, out_features, in_features, swiglu, scale)
    return ops.linear_tc(x, w, gates=gates, cluster_size=cluster_size)


@linear_tc.register_fake
def _(x, step_data, step_off, step_meta, panel_step_ptr, panel_mask, n_tiles, n_runs, n_steps, data_units,
      n_panels, out_features, in_features, swiglu, scale, gates, cluster_size):
    return x.new_empty((*x.shape[:-1], out_features // 2 if swiglu else out_features), dtype=torch.bfloat16)


@torch.library.custom_op(f"{_LIB}::mlp_prefill_tc", mutates_args=(), device_types="cuda")
def mlp_prefill_tc(x: torch.Tensor,
                   gu_data: torch.Tensor, gu_off: torch.Tensor, gu_meta: torch.Tensor, gu_psp: torch.Tensor,
                   gu_mask: torch.Tensor, gu_tiles: int, gu_runs: int, gu_steps: int, gu_units: int,
                   gu_panels: int, gu_out: int, gu_in: int, gu_scale: float,
                   dn_data: torch.Tensor, dn_off: torch.Tensor, dn_meta: torch.Tensor, dn_psp: torch.Tensor,
                   dn_mask: torch.Tensor, dn_tiles: int, dn_runs: int, dn_steps: int, dn_units: int,
                   dn_panels: int, dn_out: int, dn_in: int, dn_scale: float,
                   gates: Optional[torch.Tensor], n_clusters: int) -> torch.Tensor:
    gu = _sched(gu_data, gu_off, gu_meta, gu_psp, gu_mask, gu_tiles, gu_runs, gu_steps, gu_units, gu_panels,
                gu_out, gu_in, True, gu_scale)
    dn = _sched(dn_data, dn_off, dn_meta, dn_psp, dn_mask, dn_tiles, dn_runs, dn_steps, dn_units, dn_panels,
                dn_out, dn_in, False, dn_scale)
    return ops.mlp_prefill_tc(x, gu, dn, gates=gates, n_clusters=n_clusters)


@mlp_prefill_tc.register_fake
def _(x, gu_data, gu_off, gu_meta, gu_psp, gu_mask, gu_tiles, gu_runs, gu_steps, gu_units, gu_panels, gu_out,
      gu_in, gu_scale, dn_data, dn_off, dn_meta, dn_psp, dn_mask, dn_tiles, dn_runs, dn_steps, dn_units,
      dn_panels, dn_out, dn_in, dn_scale, gates, n_clusters):
    return x.new_empty((*x.shape[:-1], dn_out), dtype=torch.bfloat16)


def mlp_prefill_tc_args(gu: SchedMatrix, dn: SchedMatrix):
    """Arguments between ``x`` and ``gates`` of ``mortar_b200::mlp_prefill_tc`` for two schedules."""
    a, b = sched_args(gu), sched_args(dn)
    return (*a[:12], a[13], *b[:12], b[13])


def blocks_args(w: BlockSched):
    """The tensors and scalars that describe a block layout in the registered ops' argument order."""
    return (w.data, w.pair_ptr, w.steps, w.out_features, w.in_features, w.swiglu, w.scale)


@torch.library.custom_op(f"{_LIB}::linear_blocks", mutates_args=(), device_types="cuda")
def linear_blocks(x: torch.Tensor, data: torch.Tensor, pair_ptr: torch.Tensor, steps: torch.Tensor,
                  out_features: int, in_features: int, swiglu: bool, scale: float,
                  gates: Optional[torch.Tensor], cluster_size: int) -> torch.Tensor:
    """``ops.linear_blocks`` on raw tensors (``MortarMatrix.to_blocks`` builds them)."""
    w = BlockSched.from_tensors(data, pair_ptr, steps, out_features, in_features, swiglu, scale)
    return ops.linear_blocks(x, w, gates=gates, cluster_size=cluster_size)


@linear_blocks.register_fake
def _(x, data, pair_ptr, steps, out_features, in_features, swiglu, scale, gates, cluster_size):
    return x.new_empty((*x.shape[:-1], out_features // 2 if swiglu else out_features), dtype=torch.bfloat16)


@torch.library.custom_op(f"{_LIB}::mlp_prefill_blocks", mutates_args=(), device_types="cuda")
def mlp_prefill_blocks(x: torch.Tensor,
                       gu_data: torch.Tensor, gu_pairs: torch.Tensor, gu_steps: torch.Tensor, gu_out: int,
                       gu_in: int, gu_scale: float,
                       dn_data: torch.Tensor, dn_pairs: torch.Tensor, dn_steps: torch.Tensor, dn_out: int,
                       dn_in: int, dn_scale: float,
                       gates: Optional[torch.Tensor], n_clusters: int) -> torch.Tensor:
    """``_SwiGLUMortar.forward`` on a token block through the block path of the tcgen05 kernels."""
    gu = BlockSched.from_tensors(gu_data, gu_pairs, gu_steps, gu_out, gu_in, True, gu_scale)
    dn = BlockSched.from_tensors(dn_data, dn_pairs, dn_steps, dn_out, dn_in, False, dn_scale)
    return ops.mlp_prefill_blocks(x, gu, dn, gates=gates, n_clusters=n_clusters)


@mlp_prefill_blocks.register_fake
def _(x, gu_data, gu_pairs, gu_steps, gu_out, gu_in, gu_scale, dn_data, dn_pairs, dn_steps, dn_out, dn_in,
      dn_scale, gates, n_clusters):
    return x.new_empty((*x.shape[:-1], dn_out), dtype=torch.bfloat16)


@torch.library.custom_op(f"{_LIB}::stack_decode", mutates_args=("x", "status"), device_types="cuda")
def stack_decode(x: torch.Tensor, blobs: torch.Tensor, blob_table: torch.Tensor, app_layer: torch.Tensor,
                 rms_weights: Optional[torch.Tensor], status: torch.Tensor, n_layers: int, d_model: int,
                 d_ff: int, max_gate_up_bytes: int, max_down_bytes: int, cluster_size: int, eps: float,
                 n_planes: int) -> None:
    """x <- x + MLP_i(rmsnorm_i(x)) for every application listed in ``app_layer``, one launch
    (``ops.stack_decode`` on raw tensors; ``ops.DecodeStack`` builds them)."""
    ops.stack_decode_raw(x, blobs, blob_table, app_layer, rms_weights, status, n_layers, d_model, d_ff,
                         max_gate_up_bytes, max_down_bytes, cluster_size, eps, n_planes)


@stack_decode.register_fake
def _(x, blobs, blob_table, app_layer, rms_weights, status, n_layers, d_model, d_ff, max_gate_up_bytes,
      max_down_bytes, cluster_size, eps, n_planes):
    return None


# ---------------------------------------------------------------------------------------
# the reference operator: morph_stk::dds
# ---------------------------------------------------------------------------------------

_DDS_CACHE: "OrderedDict" = OrderedDict()
_HASH_WEIGHTS: dict = {}
_DDS_ASSUME_FROZEN = False


def clear_dds_cache() -> None:
    """Forget every matrix converted for ``morph_stk::dds``."""
    _DDS_CACHE.clear()


def dds_assume_frozen(flag: bool = True) -> None:
    """With frozen weights (inference) the content check of ``morph_stk::dds`` can be skipped: a
    cached conversion is then reused as long as the layer's index buffers are the same tensors.
    Off by default, because the reference hands the op a fresh temporary every forward
    (block_sparse.py:909-919, 951-956) whose address and version say nothing about its content."""
    global _DDS_ASSUME_FROZEN
    _DDS_ASSUME_FROZEN = bool(flag)


def _fingerprint(data: torch.Tensor) -> int:
    """Exact integer hash of the bit pattern of ``data`` (one pass on the device, one scalar read)."""
    v = data.detach().contiguous().view(torch.int16 if data.element_size() == 2 else torch.int32).reshape(-1)
    key = (v.numel(), v.device)
    wts = _HASH_WEIGHTS.get(key)
    if wts is None:
        wts = ((torch.arange(v.numel(), device=v.device, dtype=torch.int64) * 2654435761) % 1000003 + 1)
        _HASH_WEIGHTS.clear()           # one shape at a time is enough; keeps the memory bounded
        _HASH_WEIGHTS[key] = wts
    return int((v.to(torch.int64) * wts).sum().item())


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
        raise ValueError("morph_stk::dds: `data` is not ternary (code * one scale); only ternarised "
                         "MORTAR layers can run on the packed kernels")
    packed = pack_codes_2bit(codes.astype(np.int8).reshape(-1, 4)).reshape(-1)
    return MortarMatrix.from_reference_bcsr(offsets.detach().cpu().numpy(), column_indices.detach().cpu().numpy(),
                                            packed, scale, blk, out_features, in_features)


class _DdsEntry:
    def __init__(self, matrix: MortarMatrix, fingerprint: int, device):
        self.matrix, self.fingerprint, self.device = matrix, fingerprint, device
        self._stream = self._sched = self._stream_t = self._sched_t = None
        self._blocks = {}

    def stream(self, transposed: bool = False):
        if transposed:
            if self._stream_t is None:
                self._stream_t = self.matrix.transpose().to_stream(self.device)
            return self._stream_t
        if self._stream is None:
            self._stream = self.matrix.to_stream(self.device)
        return self._stream

    def sched(self, transposed: bool = False):
        if transposed:
            if self._sched_t is None:
                self._sched_t = self.matrix.transpose().to_sched(False, self.device)
            return self._sched_t
        if self._sched is None:
            self._sched = self.matrix.to_sched(False, self.device)
        return self._sched


    def blocks(self, transposed: bool = False):
        """Layout of the block path, or None when the topology is too sparse for it."""
        if transposed not in self._blocks:
            m = self.matrix.transpose() if transposed else self.matrix
            self._blocks[transposed] = m.to_blocks(False, self.device) if wants_block_path(m, False) else None
        return self._blocks[transposed]


def stk_dds(lhs: torch.Tensor, data: torch.Tensor, offsets: torch.Tensor, row_indices: torch.Tensor,
            column_indices: torch.Tensor, offsets_t: torch.Tensor, column_indices_t: torch.Tensor,
            block_offsets_t: torch.Tensor, shape0: int, shape1: int, transpose_b: bool = True) -> torch.Tensor:
    """``torch.ops.morph_stk.dds`` (custom_ops.py:35-56) on the packed kernels.
    transpose_b=True: the BCSR matrix W is [shape1, shape0] and the result is ``lhs @ W^T`` -- the
    call CMSBlockLinear._forward_mortar makes with ``(in_features, out_features, True)``
    (block_sparse.py:956-966).  transpose_b=False: W is [shape0, shape1] and the result is
    ``lhs @ W`` -- the input gradient of that forward (custom_ops.py:112-124), served by the same
    kernels on the transposed matrix.  The reference's transposed metadata is not needed.
    A layer is recognised by its persistent index buffers (``offsets`` / ``column_indices``); its
    converted weights are reused while an exact hash of ``data`` stays the same and converted
    again when it changes (a weight update, a reloaded checkpoint).  ``dds_assume_frozen()`` skips
    the hash for inference."""
    if not lhs.is_cuda:
        raise NotImplementedError("morph_stk::dds is a CUDA-only operator (no CPU path)")
    out_f, in_f = (int(shape1), int(shape0)) if transpose_b else (int(shape0), int(shape1))
    key = (offsets.data_ptr(), column_indices.data_ptr(), tuple(data.shape), out_f, in_f)
    ent = _DDS_CACHE.get(key)
    fp = None
    if ent is not None and not _DDS_ASSUME_FROZEN:
        fp = _fingerprint(data)
        if fp != ent.fingerprint:
            ent = None
    if ent is None:
        if fp is None:
            fp = _fingerprint(data)
        ent = _DdsEntry(_ternary_matrix_from_data(data, offsets, column_indices, out_f, in_f), fp, lhs.device)
        _DDS_CACHE[key] = ent
        while len(_DDS_CACHE) > _CACHE_MAX:
            _DDS_CACHE.popitem(last=False)
    else:
        _DDS_CACHE.move_to_end(key)
    k_features = in_f if transpose_b else out_f
    if _takes_tc(lhs, k_features):
        blk = ent.blocks(not transpose_b)
        if blk is not None:
            return ops.linear_blocks(lhs, blk)
        return ops.linear_tc(lhs, ent.sched(not transpose_b))
    return ops.linear(lhs, ent.stream(not transpose_b))


# topologies (no values) for the weight gradient, keyed by the layer's index buffers
_TOPO_CACHE: "OrderedDict" = OrderedDict()


def _topology(offsets: torch.Tensor, column_indices: torch.Tensor, blk: int, device):
    key = (offsets.data_ptr(), column_indices.data_ptr(), int(blk))
    hit = _TOPO_CACHE.get(key)
    if hit is not None:
        _TOPO_CACHE.move_to_end(key)
        return hit
    off = offsets.detach().cpu().numpy().astype(np.int64)
    ci = column_indices.detach().cpu().numpy().astype(np.int64)
    t = blk // 16
    Rb = len(off) - 1
    n_cols = int(ci.max(initial=-1)) + 1
    row_ptr, cols, gather = [0], [], np.zeros((len(ci), t, t), dtype=np.int64)
    for R in range(Rb):
        bc = ci[off[R]:off[R + 1]]
        n_r = len(bc)
        tile_cols = (bc[:, None] * t + np.arange(t)[None, :]).reshape(-1)
        for i in range(t):
            base = row_ptr[-1]
            cols.append(tile_cols)
            row_ptr.append(base + n_r * t)
            # tile (block c of this row, sub-row i, sub-column j) sits at base + c*t + j
            gather[off[R]:off[R + 1], i, :] = base + np.arange(n_r)[:, None] * t + np.arange(t)[None, :]
    col_idx = np.concatenate(cols).astype(np.uint16) if cols else np.zeros(0, dtype=np.uint16)
    m = MortarMatrix(Rb * blk, max(n_cols, 1) * blk, np.asarray(row_ptr, dtype=np.int32), col_idx,
                     np.zeros((len(col_idx), 64), dtype=np.uint8), 1.0)
    hit = (TopologyDev(m, device), torch.from_numpy(gather).to(device))
    _TOPO_CACHE[key] = hit
    while len(_TOPO_CACHE) > _CACHE_MAX:
        _TOPO_CACHE.popitem(last=False)
    return hit


def stk_sdd_at_b(a: torch.Tensor, b: torch.Tensor, data: torch.Tensor, offsets: torch.Tensor,
                 row_indices: torch.Tensor, column_indices: torch.Tensor) -> torch.Tensor:
    """``torch.ops.morph_stk.sdd_at_b`` (custom_ops.py:68-89): ``a^T @ b`` restricted to the BCSR
    topology of ``data`` -> [nnz, blk, blk] in the dtype of ``a``; with a = dy [M, out] and
    b = x [M, in] this is the weight gradient of the carved forward.  ``data`` supplies only the
    block shape."""
    if not a.is_cuda:
        raise NotImplementedError("morph_stk::sdd_at_b is a CUDA-only operator (no CPU path)")
    nnz, blk, _ = data.shape
    topo, gather = _topology(offsets, column_indices, blk, a.device)
    if b.shape[-1] != topo.tile_cols * 16:
        # the column count of the topology comes from the largest kept column; widen to the operand
        topo.tile_cols = b.shape[-1] // 16
    tiles = ops.sdd_tiles(a, b, topo, out_dtype=torch.float32)                    # [nnz16, 16, 16]
    t = blk // 16
    blocks = tiles[gather]                                                        # [nnz, t, t, 16, 16]
    return blocks.permute(0, 1, 3, 2, 4).reshape(nnz, blk, blk).to(a.dtype)


def _dds_setup_context(ctx, inputs, output):
    (lhs, data, offsets, row_indices, column_indices, offsets_t, column_indices_t, block_offsets_t,
     shape0, shape1, transpose_b) = inputs
    ctx.save_for_backward(lhs, data, offsets, row_indices, column_indices, offsets_t, column_indices_t,
                          block_offsets_t)
    ctx.shape0, ctx.shape1, ctx.transpose_b = shape0, shape1, transpose_b


def _dds_backward(ctx, grad):
    """dlhs = grad @ (W or W^T) -- another dds; ddata = the product of the two dense operands on
    the topology -- sdd_at_b (the reference's rule, custom_ops.py:91-133)."""
    (lhs, data, offsets, row_indices, column_indices, offsets_t, column_indices_t, block_offsets_t) = ctx.saved_tensors
    dy = grad if grad.is_contiguous() else grad.contiguous()
    dlhs = ddata = None
    if ctx.needs_input_grad[0]:
        dlhs = torch.ops.morph_stk.dds(dy, data, offsets, row_indices, column_indices, offsets_t, column_indices_t,
                                       block_offsets_t, ctx.shape1, ctx.shape0, not ctx.transpose_b)
    if ctx.needs_input_grad[1]:
        a, b = (dy, lhs) if ctx.transpose_b else (lhs, dy)
        ddata = torch.ops.morph_stk.sdd_at_b(a, b, data, offsets, row_indices, column_indices)
    return (dlhs, ddata, None, None, None, None, None, None, None, None, None)


def _dds_fake(lhs, data, offsets, row_indices, column_indices, offsets_t, column_indices_t, block_offsets_t,
              shape0, shape1, transpose_b):
    return lhs.new_empty((lhs.size(0), shape1))


_DDS_SCHEMA = ("(Tensor lhs, Tensor data, Tensor offsets, Tensor row_indices, Tensor column_indices, "
               "Tensor offsets_t, Tensor column_indices_t, Tensor block_offsets_t, SymInt shape0, "
               "SymInt shape1, bool transpose_b) -> Tensor")
_SDD_SCHEMA = ("(Tensor a, Tensor b, Tensor data, Tensor offsets, Tensor row_indices, Tensor column_indices) "
               "-> Tensor")
_morph_stk_libs = []        # keeps the torch.library.Library objects alive


def _sdd_fake(a, b, data, offsets, row_indices, column_indices):
    return a.new_empty(data.shape)


def install_morph_stk_dds() -> str:
    """Makes ``torch.ops.morph_stk.dds`` and ``torch.ops.morph_stk.sdd_at_b`` run the packed
    kernels.  When nothing has defined the ops yet they are defined here with the reference's
    schemas (custom_ops.py:35-133: CUDA-only, ``mutates_args=()``, fake kernels for tracing, the
    dds autograd rule) and "defined" is returned; when the reference package was imported first and
    owns the definitions (and the autograd rule, which calls the two ops), their CUDA kernels are
    replaced and "overridden" is returned.  Idempotent."""
    if _morph_stk_libs:
        return _morph_stk_libs[0][1]
    try:
        have = hasattr(torch.ops.morph_stk, "dds")
    except (AttributeError, RuntimeError):
        have = False
    if not have:
        lib = torch.library.Library("morph_stk", "FRAGMENT")
        lib.define("dds" + _DDS_SCHEMA)
        lib.define("sdd_at_b" + _SDD_SCHEMA)
        lib.impl("dds", stk_dds, "CUDA")
        lib.impl("sdd_at_b", stk_sdd_at_b, "CUDA")
        torch.library.register_fake("morph_stk::dds", _dds_fake, lib=lib)
        torch.library.register_fake("morph_stk::sdd_at_b", _sdd_fake, lib=lib)
        torch.library.register_autograd("morph_stk::dds", _dds_backward, setup_context=_dds_setup_context, lib=lib)
        _morph_stk_libs.append((lib, "defined"))
    else:
        lib = torch.library.Library("morph_stk", "IMPL")
        lib.impl("dds", stk_dds, "CUDA", allow_override=True)
        lib.impl("sdd_at_b", stk_sdd_at_b, "CUDA", allow_override=True)
        _morph_stk_libs.append((lib, "overridden"))
    return _morph_stk_libs[0][1]


install_morph_stk_dds()
