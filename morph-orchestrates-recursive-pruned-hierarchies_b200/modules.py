"""Drop-in mirrors of the reference's module API for the carved MLP
(morph/model/sparsity.py:33-166 ``MortarLinear``; morph/model/layers/block_sparse.py:182-1044
``CMSBlockLinear`` in its carved state; morph/model/transformer.py:319-431 ``_SwiGLUMortar``).
Same constructor signatures, attribute names, ``state_dict`` keys, argument meaning and error
behaviour; the forward runs the sm_100a kernels of this package.

Only the carved (post-``carve()``) phase is served: the dense pre-carve phase, saliency
scoring and pruning belong to training.  A layer built with the reference constructor holds
no weights until a carved ``state_dict`` is loaded into it (the reference's own
``mortar_*`` keys, unpacked or 2-bit packed) or it is filled with ``from_matrix`` /
``from_reference``.

Kernel choice of the forward (``TC_MIN_ROWS``): bf16 token blocks of at least that many rows
run the tcgen05 / tensor-memory kernel (``ops.linear_tc`` / ``ops.mlp_prefill_tc``), smaller
blocks and fp32 activations the streaming kernel (``ops.linear`` / ``ops.mlp_decode``).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.nn as nn

from . import ops
from .format import TILE, BlockSched, MortarMatrix, SchedMatrix, StreamMatrix, wants_block_path

# bf16 token blocks with at least this many rows take the tensor-memory kernel.  Measured on
# B200 at the 768/2048 and 2048/5632 shapes: the streaming kernel wins below 128 rows, the
# tcgen05 kernel (whose work item is a block of 128 rows) from 128 rows on.
TC_MIN_ROWS = 128


class CarvedStorage(nn.Module):
    """The carved state of the reference's ``CMSBlockLinear`` (what ``MortarLinear._cms`` is
    after ``carve()``): BCSR index buffers ``mortar_offsets`` / ``mortar_row_indices`` /
    ``mortar_column_indices`` and their transposed twins, ``mortar_ternary`` = [flag, threshold],
    and the values either as ``mortar_data`` [nnz, blk, blk] (block_sparse.py:783-799) or 2-bit
    packed as ``mortar_packed`` + ``mortar_scale`` (deploy_quant.py:361-365).  The kernels'
    layouts are derived from these buffers on first use and cached."""

    _INDEX_KEYS = ("mortar_row_indices", "mortar_column_indices", "mortar_offsets",
                   "mortar_column_indices_t", "mortar_offsets_t", "mortar_block_offsets_t")

    def __init__(self, in_features: int, out_features: int, tile_size: int = TILE, bias: bool = True,
                 device=None, dtype=None):
        super().__init__()
        if in_features % tile_size or out_features % tile_size:
            raise ValueError(f"features [{out_features},{in_features}] must be divisible by tile_size "
                             f"({tile_size})")
        if tile_size != TILE:
            raise ValueError(f"tile_size must be {TILE}")
        self.in_features, self.out_features, self.tile_size = in_features, out_features, tile_size
        self.R, self.C = out_features // tile_size, in_features // tile_size
        self.density = 1.0
        self._dense_mode = True            # no carved weights yet
        self._mortar = False
        self._mortar_blocking = 0
        self._values_ternary_mode = True   # the packed kernels only run ternary values
        self._values_threshold = 0.5
        self._device = torch.device(device) if device is not None else torch.device("cpu")
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype))
        else:
            self.register_parameter("bias", None)
        self._matrix: Optional[MortarMatrix] = None
        self._stream: Optional[StreamMatrix] = None
        self._sched = {}

    # ---- filling ------------------------------------------------------------------------
    def _install(self, tensors: dict, blocking: int) -> None:
        for k in list(self._buffers):
            if k.startswith("mortar_"):
                del self._buffers[k]
        if "mortar_data" in self._parameters:
            del self._parameters["mortar_data"]
        for k, v in tensors.items():
            if k == "mortar_data":
                self.mortar_data = nn.Parameter(v, requires_grad=False)
            else:
                self.register_buffer(k, v)
        self._mortar, self._mortar_blocking, self._dense_mode = True, int(blocking), False
        Rb, Cb = self.out_features // blocking, self.in_features // blocking
        self.density = int(tensors["mortar_column_indices"].shape[0]) / float(Rb * Cb)
        self.invalidate()

    def set_matrix(self, m: MortarMatrix, device=None) -> None:
        """Install a canonical tile-16 matrix as carved storage at blocking 16 in the packed
        flavour (its codes ARE the reference's flat pack at that blocking)."""
        if (m.out_features, m.in_features) != (self.out_features, self.in_features):
            raise ValueError("matrix shape does not match the layer")
        dev = device if device is not None else self._device
        rows = np.repeat(np.arange(m.tile_rows), np.diff(m.row_ptr)).astype(np.int16)
        cols = m.col_idx.astype(np.int16)
        order = np.argsort(cols, kind="stable")
        off_t = np.zeros(m.tile_cols + 1, dtype=np.int32)
        np.cumsum(np.bincount(cols.astype(np.int64), minlength=m.tile_cols), out=off_t[1:])
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        self._install({
            "mortar_row_indices": t(rows), "mortar_column_indices": t(cols),
            "mortar_offsets": t(m.row_ptr.astype(np.int32)),
            "mortar_column_indices_t": t(rows[order]), "mortar_offsets_t": t(off_t),
            "mortar_block_offsets_t": t(order.astype(np.int32)),
            "mortar_ternary": torch.tensor([1.0, self._values_threshold], dtype=torch.float32, device=dev),
            "mortar_packed": t(m.codes.reshape(-1)),
            "mortar_scale": torch.tensor(m.scale, dtype=torch.float32, device=dev),
        }, TILE)
        self._matrix = m

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        """Takes the keys the reference persists for a carved layer
        (block_sparse.py:983-1036): storage is created with the checkpoint's shapes, then the
        default loader fills it.  Dense (never carved) checkpoints are refused."""
        off_key = prefix + "mortar_offsets"
        if off_key in state_dict:
            if prefix + "mortar_data" in state_dict:
                blocking = int(state_dict[prefix + "mortar_data"].shape[-1])
                values = ["mortar_data"]
            elif prefix + "mortar_packed" in state_dict:
                nnz = int(state_dict[prefix + "mortar_column_indices"].shape[0])
                numel = int(state_dict[prefix + "mortar_packed"].numel()) * 4
                blocking = int(round((numel / max(nnz, 1)) ** 0.5)) if nnz else TILE
                values = ["mortar_packed", "mortar_scale"]
            else:
                raise RuntimeError(f"{prefix}: carved index buffers without mortar_data / mortar_packed")
            mt = state_dict.get(prefix + "mortar_ternary")
            if mt is not None:
                self._values_ternary_mode = bool(float(mt[0]) > 0)
                self._values_threshold = float(mt[1])
            # row ids and the transposed index arrays only serve the reference's backward; a
            # checkpoint without them gets them rebuilt from offsets / column_indices
            off = state_dict[off_key].detach().cpu().numpy().astype(np.int64)
            cols = state_dict[prefix + "mortar_column_indices"].detach().cpu().numpy().astype(np.int64)
            rows = np.repeat(np.arange(len(off) - 1), np.diff(off))
            order = np.argsort(cols, kind="stable")
            n_cols = self.in_features // blocking
            off_t = np.zeros(n_cols + 1, dtype=np.int64)
            np.cumsum(np.bincount(cols, minlength=n_cols), out=off_t[1:])
            derived = {"mortar_row_indices": torch.from_numpy(rows.astype(np.int16)),
                       "mortar_column_indices_t": torch.from_numpy(rows[order].astype(np.int16)),
                       "mortar_offsets_t": torch.from_numpy(off_t.astype(np.int32)),
                       "mortar_block_offsets_t": torch.from_numpy(order.astype(np.int32))}
            for k, v in derived.items():
                state_dict.setdefault(prefix + k, v)
            dev = self._device
            tensors = {}
            for k in list(self._INDEX_KEYS) + values + (["mortar_ternary"] if mt is not None else []):
                tensors[k] = torch.empty_like(state_dict[prefix + k], device=dev)
            self._install(tensors, blocking)
        elif prefix + "weight" in state_dict and not self._mortar:
            raise RuntimeError(f"{prefix}weight: dense (pre-carve) checkpoint; this layer runs carved "
                               f"MORTAR storage only -- carve and pack the model first")
        for k in ("block_score_ema", "math_score_ema", "_prune_mask", "weight"):
            state_dict.pop(prefix + k, None)                   # training-side state of the reference
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self.invalidate()

    def _apply(self, fn, *a, **k):
        out = super()._apply(fn, *a, **k)
        for t in list(self._buffers.values()) + list(self._parameters.values()):
            if t is not None:
                self._device = t.device
                break
        self._stream, self._sched = None, {}
        return out

    def invalidate(self) -> None:
        """Drop the cached kernel layouts (call after changing the carved buffers in place)."""
        self._matrix, self._stream, self._sched = None, None, {}

    # ---- derived layouts --------------------------------------------------------------
    def matrix(self) -> MortarMatrix:
        if not self._mortar:
            raise RuntimeError("layer holds no carved weights: load a carved state_dict, or build it "
                               "with from_matrix / from_reference (the dense pre-carve phase is not "
                               "part of this package)")
        if self._matrix is None:
            self._matrix = MortarMatrix.from_reference_cms(self)
        return self._matrix

    def stream(self) -> StreamMatrix:
        if self._stream is None:
            self._stream = self.matrix().to_stream(self._device)
        return self._stream

    def sched(self, swiglu: bool) -> SchedMatrix:
        if swiglu not in self._sched:
            self._sched[swiglu] = self.matrix().to_sched(swiglu, self._device)
        return self._sched[swiglu]

    def blocks(self, swiglu: bool) -> Optional[BlockSched]:
        """Layout of the block path when the touched 128 x 128 blocks are full enough
        (format.BLOCK_PATH_MIN_FILL); None otherwise."""
        key = ("blocks", swiglu)
        if key not in self._sched:
            m = self.matrix()
            self._sched[key] = m.to_blocks(swiglu, self._device) if wants_block_path(m, swiglu) else None
        return self._sched[key]

    # ---- reference API ------------------------------------------------------------------
    def accumulate_scores(self) -> None:
        """No-op: saliency scoring stops at carve time (block_sparse.py:453-493 returns early
        for carved layers)."""

    def get_density(self) -> float:
        return self.density

    def carve(self, blocking: int = 128) -> int:
        assert not self._mortar, "carve() already applied"
        raise NotImplementedError("carving a dense layer is a training-side step; load carved weights")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        rows = x.numel() // max(self.in_features, 1)
        if torch.is_autocast_enabled() and x.is_cuda and x.dtype == torch.float32:
            x = x.to(torch.get_autocast_dtype("cuda"))           # as _forward_mortar does (block_sparse.py:947-955)
        if x.dtype == torch.bfloat16 and rows >= TC_MIN_ROWS and x.is_cuda:
            blk = self.blocks(False)
            y = ops.linear_blocks(x, blk) if blk is not None else ops.linear_tc(x, self.sched(False))
        else:
            y = ops.linear(x, self.stream())
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*lead, self.out_features)


class MortarLinear(nn.Module):
    """``MortarLinear`` (morph/model/sparsity.py:33-166) in its MORTAR mode: y = x @ W^T over
    the kept 16x16 ternary tiles.  Same constructor signature as the reference;
    ``initial_density`` and ``score_ema_alpha`` are accepted and unused (they steer the dense
    phase)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, tile_size: int = TILE,
                 initial_density: float = 1.0, score_ema_alpha: float = 0.95, device=None, dtype=None):
        super().__init__()
        self._cms = CarvedStorage(in_features, out_features, tile_size, bias, device, dtype)
        self.in_features, self.out_features, self.tile_size = in_features, out_features, tile_size

    @classmethod
    def from_matrix(cls, matrix: MortarMatrix, bias: Optional[torch.Tensor] = None,
                    device="cuda") -> "MortarLinear":
        new = cls(matrix.in_features, matrix.out_features, bias=bias is not None, device=device)
        new._cms.set_matrix(matrix, torch.device(device))
        if bias is not None:
            with torch.no_grad():
                new._cms.bias.copy_(bias.detach().to(new._cms.bias.dtype))
        return new

    @classmethod
    def from_reference(cls, layer, device="cuda") -> "MortarLinear":
        """`layer` is a reference ``MortarLinear`` or its ``CMSBlockLinear`` after carve()."""
        cms = getattr(layer, "_cms", layer)
        return cls.from_matrix(MortarMatrix.from_reference_cms(cms), bias=cms.bias, device=device)

    @property
    def is_compact(self) -> bool:
        return not self._cms._dense_mode

    @property
    def bias(self):
        return self._cms.bias

    @property
    def matrix(self) -> MortarMatrix:
        return self._cms.matrix()

    @property
    def stream(self) -> StreamMatrix:
        return self._cms.stream()

    def accumulate_scores(self) -> None:
        self._cms.accumulate_scores()

    def carve(self, blocking: int = 128) -> int:
        return self._cms.carve(blocking=blocking)

    def get_density(self) -> float:
        return self._cms.get_density()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self._cms(x)

    def extra_repr(self) -> str:
        mode = "mortar" if self.is_compact else "empty"
        return (f"in={self.in_features}, out={self.out_features}, tile={self.tile_size}, "
                f"density={self.get_density():.2f}, mode={mode}")


class SwiGLUMortar(nn.Module):
    """``_SwiGLUMortar`` (morph/model/transformer.py:319-431): gate_up -> chunk (gate first) ->
    silu(gate)*up -> [* cluster gates] -> down, evaluated by the fused kernels.  bf16 inputs
    (and fp32 inputs under autocast) follow the reference's autocast rounding points; plain
    fp32 inputs follow the decode engine's fp32 algebra (morph/inference/engine.py:936-986)."""

    def __init__(self, d_model: int, d_ff: int, device=None):
        super().__init__()
        self.gate_up = MortarLinear(d_model, d_ff * 2, bias=False, initial_density=1.0, device=device)
        self.down = MortarLinear(d_ff, d_model, bias=False, initial_density=1.0, device=device)
        self.d_model, self.d_ff = d_model, d_ff
        self.router: Optional[nn.Module] = None
        self.n_clusters = 0
        self._last_aux_loss = None
        self._aux_detach_input = True

    @classmethod
    def from_matrices(cls, gate_up: MortarMatrix, down: MortarMatrix, device="cuda") -> "SwiGLUMortar":
        if gate_up.out_features != 2 * down.in_features or gate_up.in_features != down.out_features:
            raise ValueError("gate_up must be [2*d_ff, d_model] and down [d_model, d_ff]")
        new = cls(gate_up.in_features, down.in_features, device=device)
        new.gate_up._cms.set_matrix(gate_up, torch.device(device))
        new.down._cms.set_matrix(down, torch.device(device))
        return new

    @classmethod
    def from_reference(cls, mlp, device="cuda") -> "SwiGLUMortar":
        """`mlp` is a carved reference ``_SwiGLUMortar`` (its router, if any, is reused)."""
        new = cls.from_matrices(MortarMatrix.from_reference_cms(mlp.gate_up._cms),
                                MortarMatrix.from_reference_cms(mlp.down._cms), device=device)
        if getattr(mlp, "router", None) is not None:
            new.attach_router(mlp.router.to(device), int(mlp.n_clusters))
        return new

    def _device(self):
        return self.gate_up._cms._device

    def attach_router(self, router: nn.Module, n_clusters: int) -> None:
        """`router(x, iter_idx=...) -> (gates[..., n_clusters], aux)` as ``TileRouter.forward``
        (morph/model/routing.py:159)."""
        self.router = router
        self.n_clusters = int(n_clusters)
        base, rem = divmod(self.d_ff, self.n_clusters)
        sizes = torch.tensor([base + (1 if c < rem else 0) for c in range(self.n_clusters)])
        h2c = torch.repeat_interleave(torch.arange(self.n_clusters), sizes)
        self.register_buffer("hidden_to_cluster", h2c.to(self._device()))

    def enable_routing(self, n_clusters: int = 16, activation_ratio: float = 0.5,
                       aux_loss_coeff: float = 1e-2, n_iters: int = 1, n_sub_keys: int = 0,
                       detach_input: bool = True) -> None:
        from .router import TileRouter
        self._aux_detach_input = bool(detach_input)
        self.attach_router(TileRouter(n_clusters, self.d_model, activation_ratio, n_sub_keys,
                                      aux_loss_coeff, n_iters).to(self._device()), n_clusters)

    def forward(self, x: torch.Tensor, iter_idx: int = 0) -> torch.Tensor:
        gates = None
        if self.router is not None:
            if self.d_ff % self.n_clusters:
                raise NotImplementedError("uneven clusters are not supported by the fused kernels")
            _rx = x.detach() if self._aux_detach_input else x
            gates, aux = self.router(_rx, iter_idx=iter_idx)
            self._last_aux_loss = aux
        if torch.is_autocast_enabled() and x.is_cuda and x.dtype == torch.float32:
            x = x.to(torch.get_autocast_dtype("cuda"))
        gu, dn = self.gate_up._cms, self.down._cms
        if x.dtype == torch.bfloat16:
            rows = x.numel() // self.d_model
            if rows >= TC_MIN_ROWS and x.is_cuda:
                bg, bd = gu.blocks(True), dn.blocks(False)
                if bg is not None and bd is not None:
                    return ops.mlp_prefill_blocks(x, bg, bd, gates=gates, n_clusters=self.n_clusters)
                return ops.mlp_prefill_tc(x, gu.sched(True), dn.sched(False), gates=gates,
                                          n_clusters=self.n_clusters)
            return ops.mlp_prefill(x, gu.stream(), dn.stream(), gates=gates, n_clusters=self.n_clusters)
        return ops.mlp_decode(x, gu.stream(), dn.stream(), gates=gates, n_clusters=self.n_clusters,
                              n_planes=3)


def decode_stack(mlps: Sequence[SwiGLUMortar], norm_weights: Sequence[Optional[torch.Tensor]],
                 order: Optional[Sequence[int]] = None, device=None) -> "ops.DecodeStack":
    """One persistent launch for the MLP sites of a decode step: a list of ``SwiGLUMortar``
    modules with the weights of their pre-norms (``block.norm_mlp.weight``; None = no norm) and the
    order the sites run in (indices into ``mlps``; default: once each, in list order) becomes an
    ``ops.DecodeStack``; ``ops.stack_decode(x, stack)`` then performs
    x <- x + mlp_i(rmsnorm_i(x)) for every site (the MLP sites of
    StaticDecodeEngine._block, morph/inference/engine.py:207-213, 936-994) in one launch on the
    fp32 residual carrier.  Routed modules are not supported on this path."""
    mlps = list(mlps)
    if len(norm_weights) != len(mlps):
        raise ValueError("one norm weight (or None) per module")
    for m in mlps:
        if m.router is not None:
            raise NotImplementedError("routed MLPs run per application (ops.mlp_decode with gates)")
    dev = device if device is not None else mlps[0]._device()
    layers = [(m.gate_up.matrix, m.down.matrix, w) for m, w in zip(mlps, norm_weights)]
    return ops.DecodeStack(layers, list(order) if order is not None else list(range(len(mlps))), dev)
