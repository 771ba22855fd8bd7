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
from .format import MortarMatrix, SchedMatrix, StreamMatrix, matrix_from_stream, pack_codes_2bit

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
        self._stream = None
        self._sched = None

    def stream(self):
        if self._stream is None:
            self._stream = self.matrix.to_stream(self.device)
        return self._stream

    def sched(self):
        if self._sched is None:
            self._sched = self.matrix.to_sched(False, self.device)
        return self._sched


def stk_dds(lhs: torch.Tensor, data: torch.Tensor, offsets: torch.Tensor, row_indices: torch.Tensor,
            column_indices: torch.Tensor, offsets_t: torch.Tensor, column_indices_t: torch.Tensor,
            block_offsets_t: torch.Tensor, shape0: int, shape1: int, transpose_b: bool = True) -> torch.Tensor:
    """``torch.ops.morph_stk.dds`` (custom_ops.py:35-56) on the packed kernels:
    ``out[M, shape1] = lhs[M, shape0] @ W^T`` for the BCSR matrix W[shape1, shape0] whose kept
    blocks are ``data`` -- the call CMSBlockLinear._forward_mortar makes with
    ``(in_features, out_features, True)`` (block_sparse.py:956-966).  The transposed metadata is
    not needed.
    A layer is recognised by its persistent index buffers (``offsets`` / ``column_indices``); its
    converted weights are reused while an exact hash of ``data`` stays the same and converted
    again when it changes (a weight update, a reloaded checkpoint).  ``dds_assume_frozen()`` skips
    the hash for inference."""
    if not transpose_b:
        raise ValueError("morph_stk::dds: only the transpose_b=True form of the MLP forward is served")
    if not lhs.is_cuda:
        raise NotImplementedError("morph_stk::dds is a CUDA-only operator (no CPU path)")
    key = (offsets.data_ptr(), column_indices.data_ptr(), tuple(data.shape), int(shape0), int(shape1))
    ent = _DDS_CACHE.get(key)
    fp = None
    if ent is not None and not _DDS_ASSUME_FROZEN:
        fp = _fingerprint(data)
        if fp != ent.fingerprint:
            ent = None
    if ent is None:
        if fp is None:
            fp = _fingerprint(data)
        ent = _DdsEntry(_ternary_matrix_from_data(data, offsets, column_indices, int(shape1), int(shape0)),
                        fp, lhs.device)
        _DDS_CACHE[key] = ent
        while len(_DDS_CACHE) > _CACHE_MAX:
            _DDS_CACHE.popitem(last=False)
    else:
        _DDS_CACHE.move_to_end(key)
    if _takes_tc(lhs, int(shape0)):
        return ops.linear_tc(lhs, ent.sched())
    return ops.linear(lhs, ent.stream())


def _dds_fake(lhs, data, offsets, row_indices, column_indices, offsets_t, column_indices_t, block_offsets_t,
              shape0, shape1, transpose_b):
    return lhs.new_empty((lhs.size(0), shape1))


_DDS_SCHEMA = ("(Tensor lhs, Tensor data, Tensor offsets, Tensor row_indices, Tensor column_indices, "
               "Tensor offsets_t, Tensor column_indices_t, Tensor block_offsets_t, SymInt shape0, "
               "SymInt shape1, bool transpose_b) -> Tensor")
_morph_stk_libs = []        # keeps the torch.library.Library objects alive


def install_morph_stk_dds() -> str:
    """Makes ``torch.ops.morph_stk.dds`` run the packed kernels.  When nothing has defined the op
    yet it is defined here with the reference's schema (custom_ops.py:35-66: CUDA-only,
    ``mutates_args=()``, a fake kernel for tracing) and "defined" is returned; when the reference
    package was imported first and owns the definition, its CUDA kernel is replaced and
    "overridden" is returned.  Idempotent."""
    if _morph_stk_libs:
        return _morph_stk_libs[0][1]
    try:
        have = hasattr(torch.ops.morph_stk, "dds")
    except (AttributeError, RuntimeError):
        have = False
    if not have:
        lib = torch.library.Library("morph_stk", "FRAGMENT")
        lib.define("dds" + _DDS_SCHEMA)
        lib.impl("dds", stk_dds, "CUDA")
        torch.library.register_fake("morph_stk::dds", _dds_fake, lib=lib)
        _morph_stk_libs.append((lib, "defined"))
    else:
        lib = torch.library.Library("morph_stk", "IMPL")
        lib.impl("dds", stk_dds, "CUDA", allow_override=True)
        _morph_stk_libs.append((lib, "overridden"))
    return _morph_stk_libs[0][1]


install_morph_stk_dds()
