"""Matrix formats of the MORTAR path and the converters between them.

Canonical format (``MortarMatrix``): tile-16 BCSR with 2-bit ternary codes and one
absmean scale per matrix -- byte-identical to what the reference's
``carve(blocking=16)`` + ``pack_mortar_ternary`` produce
(morph/model/layers/block_sparse.py:874-899, morph/inference/deploy_quant.py:56-95,
344-374).  Execution layout (``StreamMatrix``): the 8-tile-group stream the kernels read,
built by the native packer; counterpart of ``mortar_pack_strips``
(morph/kernels/triton/fused_decode_step.py:1465-1499).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib

TILE = 16


def ternary_quantize(w: torch.Tensor, threshold: float = 0.5):
    """Per-tensor symmetric ternarisation in fp32: scale = mean|w| (clamped at 1e-8) over
    the values handed in, code = sign(w/scale) where |w/scale| > threshold.  Same rule as
    deploy_quant.py:81-95; callers pass kept tiles only (deploy_quant.py:356-358)."""
    wf = w.detach().float()
    scale = wf.abs().mean().clamp(min=1e-8)
    wn = wf / scale
    q = (torch.sign(wn) * (wn.abs() > threshold)).to(torch.int8)
    return q, float(scale)


def pack_codes_2bit(codes: np.ndarray) -> np.ndarray:
    """int8 codes (last dim a multiple of 4) -> bytes, 4 per byte, stored value = code+1,
    element i of a byte in bits 2i..2i+1 (deploy_quant.py:56-71)."""
    u = (np.asarray(codes).astype(np.int16) + 1).astype(np.uint8)
    u = u.reshape(*u.shape[:-1], u.shape[-1] // 4, 4)
    return (u[..., 0] | (u[..., 1] << 2) | (u[..., 2] << 4) | (u[..., 3] << 6)).astype(np.uint8)


def unpack_codes_2bit(packed: np.ndarray) -> np.ndarray:
    p = np.asarray(packed, dtype=np.uint8)
    u = (p[..., None] >> np.array([0, 2, 4, 6], dtype=np.uint8)) & 3
    return (u.reshape(*p.shape[:-1], p.shape[-1] * 4).astype(np.int8) - 1)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


@dataclass
class MortarMatrix:
    """Canonical tile-16 BCSR ternary matrix W[out, in] (host, numpy)."""
    out_features: int
    in_features: int
    row_ptr: np.ndarray      # int32 [R+1]
    col_idx: np.ndarray      # uint16 [nnz]
    codes: np.ndarray        # uint8 [nnz, 64]
    scale: float

    @property
    def tile_rows(self) -> int:
        return self.out_features // TILE

    @property
    def tile_cols(self) -> int:
        return self.in_features // TILE

    @property
    def nnz(self) -> int:
        return int(self.col_idx.shape[0])

    @property
    def density(self) -> float:
        return self.nnz / float(self.tile_rows * self.tile_cols)

    def validate(self) -> None:
        """Raises ValueError on malformed metadata (non-monotone row pointers, column index
        out of range or unsorted, unused code value)."""
        if self.out_features <= 0 or self.in_features <= 0 or self.out_features % TILE \
                or self.in_features % TILE:
            raise ValueError(f"features [{self.out_features},{self.in_features}] must be positive "
                             f"multiples of {TILE}")
        if self.row_ptr.dtype != np.int32 or self.col_idx.dtype != np.uint16 \
                or self.codes.dtype != np.uint8:
            raise ValueError("row_ptr must be int32, col_idx uint16, codes uint8")
        if self.row_ptr.shape != (self.tile_rows + 1,) or self.codes.shape != (self.nnz, 64):
            raise ValueError("row_ptr / codes have the wrong shape for these features")
        rp = np.ascontiguousarray(self.row_ptr)
        ci = np.ascontiguousarray(self.col_idx)
        cd = np.ascontiguousarray(self.codes)
        _lib.check(_lib.lib().mortar_validate_bcsr(_ptr(rp), _ptr(ci), _ptr(cd), self.tile_rows,
                                                   self.tile_cols, self.nnz), "mortar_validate_bcsr")

    # ---- constructors -------------------------------------------------------------
    @staticmethod
    def from_codes(codes: np.ndarray, tile_mask: Optional[np.ndarray], scale: float) -> "MortarMatrix":
        """Dense int8 code matrix [out, in] + bool tile mask [R, C] (None = keep every tile)."""
        codes = np.asarray(codes, dtype=np.int8)
        O, I = codes.shape
        R, Cc = O // TILE, I // TILE
        if tile_mask is None:
            tile_mask = np.ones((R, Cc), dtype=bool)
        tile_mask = np.asarray(tile_mask, dtype=bool)
        rows, cols = np.nonzero(tile_mask)                      # row-major: sorted by row, then col
        row_ptr = np.zeros(R + 1, dtype=np.int32)
        np.cumsum(tile_mask.sum(axis=1), out=row_ptr[1:])
        tiles = codes.reshape(R, TILE, Cc, TILE).transpose(0, 2, 1, 3)[rows, cols]   # [nnz,16,16]
        packed = pack_codes_2bit(tiles.reshape(-1, TILE * TILE))
        m = MortarMatrix(O, I, row_ptr, cols.astype(np.uint16), np.ascontiguousarray(packed),
                         float(scale))
        m.validate()
        return m

    @staticmethod
    def from_weight(w: torch.Tensor, tile_mask: Optional[torch.Tensor], threshold: float = 0.5):
        """Masked-dense weight -> canonical matrix, ternarising the KEPT values only with the
        deploy rule (the composition carve + pack_mortar_ternary of the reference)."""
        O, I = w.shape
        R, Cc = O // TILE, I // TILE
        if tile_mask is None:
            tile_mask = torch.ones(R, Cc, dtype=torch.bool)
        tm = tile_mask.cpu().bool()
        rows, cols = tm.nonzero(as_tuple=True)
        tiles = w.detach().cpu().reshape(R, TILE, Cc, TILE).permute(0, 2, 1, 3)[rows, cols]
        q, scale = ternary_quantize(tiles, threshold)
        dense = torch.zeros(R, Cc, TILE, TILE, dtype=torch.int8)
        dense[rows, cols] = q
        dense = dense.permute(0, 2, 1, 3).reshape(O, I)
        return MortarMatrix.from_codes(dense.numpy(), tm.numpy(), scale)

    @staticmethod
    def from_reference_bcsr(offsets, column_indices, packed, scale: float, blocking: int,
                            out_features: int, in_features: int,
                            drop_zero_tiles: bool = False) -> "MortarMatrix":
        """Reference carved+packed storage (``mortar_offsets`` int32, ``mortar_column_indices``
        int16, ``mortar_packed`` uint8 flat 2-bit over [nnz, blk, blk], ``mortar_scale``) at
        any blocking that is a multiple of 16 -> canonical tiles (each block becomes
        (blk/16)^2 tiles)."""
        off = np.ascontiguousarray(np.asarray(offsets, dtype=np.int32))
        ci = np.ascontiguousarray(np.asarray(column_indices, dtype=np.int16))
        pk = np.ascontiguousarray(np.asarray(packed, dtype=np.uint8))
        Rb, Cb = out_features // blocking, in_features // blocking
        if off.shape != (Rb + 1,):
            raise ValueError("offsets length does not match out_features / blocking")
        nnzb = int(off[-1])
        if ci.shape[0] != nnzb or pk.shape[0] < nnzb * blocking * blocking // 4:
            raise ValueError("column_indices / packed shorter than offsets[-1] blocks")
        L = _lib.lib()
        tpb = blocking // TILE
        row_ptr = np.zeros(Rb * tpb + 1, dtype=np.int32)
        nnz = C.c_int64(0)
        _lib.check(L.mortar_split_blocks(_ptr(off), _ptr(ci), _ptr(pk), Rb, Cb, blocking,
                                         int(drop_zero_tiles), _ptr(row_ptr), None, None,
                                         C.byref(nnz)), "mortar_split_blocks")
        col_idx = np.zeros(nnz.value, dtype=np.uint16)
        codes = np.zeros((nnz.value, 64), dtype=np.uint8)
        _lib.check(L.mortar_split_blocks(_ptr(off), _ptr(ci), _ptr(pk), Rb, Cb, blocking,
                                         int(drop_zero_tiles), _ptr(row_ptr), _ptr(col_idx),
                                         _ptr(codes), C.byref(nnz)), "mortar_split_blocks")
        m = MortarMatrix(out_features, in_features, row_ptr, col_idx, codes, float(scale))
        m.validate()
        return m

    @staticmethod
    def from_reference_cms(cms, drop_zero_tiles: bool = False,
                           threshold: Optional[float] = None) -> "MortarMatrix":
        """A carved reference ``CMSBlockLinear`` (``MortarLinear._cms``): packed
        (``mortar_packed``/``mortar_scale``, deploy_quant.py:361-365) or still holding
        ``mortar_data`` (block_sparse.py:783-799).  Unpacked values are ternarised the way the
        layer itself would: with its own ``_values_threshold`` when its values-ternary STE is on
        (block_sparse.py:909-919), else with the deploy packer's rule and default threshold 0.5
        (``pack_mortar_ternary``, deploy_quant.py:344-358) -- i.e. the conversion of a layer
        that is not in ternary mode is the deploy-time snap, not its training forward.
        ``threshold`` overrides both."""
        if not getattr(cms, "_mortar", False):
            raise ValueError("layer is not carved: call carve() first, or use from_weight with "
                             "its _prune_mask")
        blk = int(cms._mortar_blocking)
        if hasattr(cms, "mortar_packed"):
            packed = cms.mortar_packed.detach().cpu().numpy()
            scale = float(cms.mortar_scale)
        else:
            if threshold is None:
                threshold = float(cms._values_threshold) if getattr(cms, "_values_ternary_mode", False) else 0.5
            q, scale = ternary_quantize(cms.mortar_data.data, threshold)
            packed = pack_codes_2bit(q.cpu().numpy().reshape(-1, 4)).reshape(-1)
        return MortarMatrix.from_reference_bcsr(
            cms.mortar_offsets.detach().cpu().numpy(), cms.mortar_column_indices.detach().cpu().numpy(),
            packed, scale, blk, cms.out_features, cms.in_features, drop_zero_tiles)

    @staticmethod
    def from_state_dict(state: dict, prefix: str, out_features: int, in_features: int,
                        blocking: int = 128, drop_zero_tiles: bool = False) -> "MortarMatrix":
        """A carved layer straight from a checkpoint ``state_dict``: the keys the reference
        persists (``{prefix}mortar_offsets``, ``mortar_column_indices`` and either the packed pair
        ``mortar_packed`` / ``mortar_scale`` of deploy_quant.py:361-365 or the unpacked
        ``mortar_data`` of block_sparse.py:783-799, which is ternarised with the deploy rule)."""
        def get(name):
            v = state[prefix + name]
            return v.detach().cpu() if isinstance(v, torch.Tensor) else torch.as_tensor(v)
        for k in ("mortar_offsets", "mortar_column_indices"):
            if prefix + k not in state:
                raise KeyError(f"{prefix}{k} missing: the layer was not carved when it was saved")
        if prefix + "mortar_packed" in state:
            packed = get("mortar_packed").numpy()
            scale = float(get("mortar_scale"))
        elif prefix + "mortar_data" in state:
            data = get("mortar_data")
            blocking = int(data.shape[1])
            threshold = 0.5
            if prefix + "mortar_ternary" in state:             # [flag, threshold] (block_sparse.py:796)
                mt = get("mortar_ternary")
                if float(mt[0]) > 0:
                    threshold = float(mt[1])
            q, scale = ternary_quantize(data, threshold)
            packed = pack_codes_2bit(q.numpy().reshape(-1, 4)).reshape(-1)
        else:
            raise KeyError(f"neither {prefix}mortar_packed nor {prefix}mortar_data in the state dict")
        return MortarMatrix.from_reference_bcsr(get("mortar_offsets").numpy(),
                                                get("mortar_column_indices").numpy(), packed, scale,
                                                blocking, out_features, in_features, drop_zero_tiles)

    # ---- views ----------------------------------------------------------------------
    def to_dense_codes(self) -> np.ndarray:
        """int8 [out, in] with zeros in pruned tiles."""
        R, Cc = self.tile_rows, self.tile_cols
        tiles = unpack_codes_2bit(self.codes).reshape(self.nnz, TILE, TILE)
        rows = np.repeat(np.arange(R), np.diff(self.row_ptr))
        dense = np.zeros((R, Cc, TILE, TILE), dtype=np.int8)
        dense[rows, self.col_idx.astype(np.int64)] = tiles
        return dense.transpose(0, 2, 1, 3).reshape(self.out_features, self.in_features)

    def tile_mask(self) -> np.ndarray:
        R, Cc = self.tile_rows, self.tile_cols
        m = np.zeros((R, Cc), dtype=bool)
        rows = np.repeat(np.arange(R), np.diff(self.row_ptr))
        m[rows, self.col_idx.astype(np.int64)] = True
        return m

    def slice_tile_rows(self, tile_rows) -> "MortarMatrix":
        """Sub-matrix made of the listed tile rows, in the listed order (same columns, same scale)."""
        tile_rows = np.asarray(tile_rows, dtype=np.int64)
        counts = (self.row_ptr[tile_rows + 1] - self.row_ptr[tile_rows]).astype(np.int64)
        idx = np.concatenate([np.arange(self.row_ptr[r], self.row_ptr[r + 1]) for r in tile_rows]) \
            if len(tile_rows) else np.zeros(0, dtype=np.int64)
        row_ptr = np.zeros(len(tile_rows) + 1, dtype=np.int32)
        np.cumsum(counts, out=row_ptr[1:])
        return MortarMatrix(len(tile_rows) * TILE, self.in_features, row_ptr,
                            np.ascontiguousarray(self.col_idx[idx]), np.ascontiguousarray(self.codes[idx]),
                            self.scale)

    def slice_tile_cols(self, c0: int, c1: int) -> "MortarMatrix":
        """Sub-matrix of tile columns [c0, c1) (all rows; column indices become local)."""
        keep = (self.col_idx >= c0) & (self.col_idx < c1)
        rows = np.repeat(np.arange(self.tile_rows), np.diff(self.row_ptr))
        counts = np.bincount(rows[keep], minlength=self.tile_rows)
        row_ptr = np.zeros(self.tile_rows + 1, dtype=np.int32)
        np.cumsum(counts, out=row_ptr[1:])
        return MortarMatrix(self.out_features, (c1 - c0) * TILE, row_ptr,
                            np.ascontiguousarray((self.col_idx[keep] - c0).astype(np.uint16)),
                            np.ascontiguousarray(self.codes[keep]), self.scale)

    def transpose(self) -> "MortarMatrix":
        """W^T as a canonical matrix [in, out]: tiles transposed one by one and re-sorted by their
        new row (the matrix the input gradient dx = dy @ W runs the forward kernels on)."""
        rows = np.repeat(np.arange(self.tile_rows), np.diff(self.row_ptr))
        cols = self.col_idx.astype(np.int64)
        order = np.lexsort((rows, cols))                       # by new row (= old column), then new column
        tiles = unpack_codes_2bit(self.codes).reshape(self.nnz, TILE, TILE).transpose(0, 2, 1)[order]
        row_ptr = np.zeros(self.tile_cols + 1, dtype=np.int32)
        np.cumsum(np.bincount(cols, minlength=self.tile_cols), out=row_ptr[1:])
        return MortarMatrix(self.in_features, self.out_features, row_ptr, rows[order].astype(np.uint16),
                            np.ascontiguousarray(pack_codes_2bit(tiles.reshape(self.nnz, TILE * TILE))),
                            self.scale)

    def algorithmic_bytes(self) -> int:
        """Bytes a kernel must read to use this matrix once: 64 per tile of codes, 2 per tile of
        column index, 4 per row pointer, 4 of scale."""
        return 64 * self.nnz + 2 * self.nnz + 4 * (self.tile_rows + 1) + 4

    def build_stream_host(self):
        """(grp_ptr int32[R+1], grp_cols uint16[8G], grp_codes uint8[512G]) on the host."""
        L = _lib.lib()
        rp = np.ascontiguousarray(self.row_ptr)
        ci = np.ascontiguousarray(self.col_idx)
        cd = np.ascontiguousarray(self.codes)
        G = L.mortar_stream_groups(_ptr(rp), self.tile_rows)
        if G < 0:
            _lib.check(int(G), "mortar_stream_groups")
        grp_ptr = np.zeros(self.tile_rows + 1, dtype=np.int32)
        grp_cols = np.zeros(max(G, 1) * 8, dtype=np.uint16)
        grp_codes = np.zeros(max(G, 1) * 512, dtype=np.uint8)
        _lib.check(L.mortar_build_stream(_ptr(rp), _ptr(ci), _ptr(cd), self.tile_rows, self.tile_cols,
                                         self.nnz, _ptr(grp_ptr), _ptr(grp_cols), _ptr(grp_codes)),
                   "mortar_build_stream")
        return grp_ptr, grp_cols, grp_codes, int(G)

    def to_sched(self, swiglu: bool, device="cuda", arith: str = "bf16") -> "SchedMatrix":
        """Prefill (tcgen05) execution layout; `swiglu` pairs gate rows with up rows;
        ``arith="i8"`` builds the layout of the opt-in 8-bit arm."""
        return SchedMatrix(self, swiglu, device, arith)

    def to_gemv_blocks(self, swiglu: bool, device="cuda") -> "GemvBlocks":
        """Layout of the tensor-memory decode GEMV (matrices carved in 128 x 128 blocks)."""
        return GemvBlocks(self, swiglu, device)

    def to_blocks(self, swiglu: bool, device="cuda") -> "BlockSched":
        """Prefill execution layout of the block path (topologies carved at 128 x 128)."""
        return BlockSched(self, swiglu, device)

    def to_stream(self, device="cuda") -> "StreamMatrix":
        grp_ptr, grp_cols, grp_codes, G = self.build_stream_host()
        return StreamMatrix(self.out_features, self.in_features, self.scale, G, self.nnz,
                            torch.from_numpy(grp_ptr).to(device),
                            torch.from_numpy(grp_cols.view(np.int16)).to(device),
                            torch.from_numpy(grp_codes).to(device),
                            self.algorithmic_bytes())


class TopologyDev:
    """Canonical topology of a matrix on the device plus the work list of the weight-gradient
    kernel (items of up to 8 consecutive kept tiles of one tile row)."""

    def __init__(self, m: "MortarMatrix", device="cuda"):
        self.tile_rows, self.tile_cols, self.nnz = m.tile_rows, m.tile_cols, m.nnz
        item_row, item_first = [], []
        for r in range(m.tile_rows):
            for f in range(int(m.row_ptr[r]), int(m.row_ptr[r + 1]), 8):
                item_row.append(r)
                item_first.append(f)
        t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(np.asarray(a, dtype=dt))).to(device)
        self.row_ptr = t(m.row_ptr, np.int32)
        self.col_idx = t(m.col_idx.view(np.int16), np.int16)
        self.item_row, self.item_first = t(item_row, np.int32), t(item_first, np.int32)
        self.n_items = len(item_row)
        # work list of the block kernel: every 128 x 128 block with a kept tile, and where its 64
        # tile positions land in the [nnz] output (-1 = not kept)
        rows = np.repeat(np.arange(m.tile_rows), np.diff(m.row_ptr)).astype(np.int64)
        cols = m.col_idx.astype(np.int64)
        n_bc = (m.tile_cols + 7) // 8
        key = (rows // 8) * n_bc + cols // 8
        blocks, inv = np.unique(key, return_inverse=True)
        tiles = np.full((len(blocks), 64), -1, dtype=np.int32)
        tiles[inv, (rows % 8) * 8 + cols % 8] = np.arange(m.nnz, dtype=np.int32)
        self.blk_rc = t(np.stack([blocks // n_bc, blocks % n_bc], axis=1), np.int32)
        self.blk_tiles = t(tiles, np.int32)
        self.n_blocks = len(blocks)


PANEL_ROWS, CHUNK_COLS, STEP_TILES = 16, 4, 48


def build_sched_host(m: "MortarMatrix", swiglu: bool, arith: str = "bf16"):
    """Host arrays of the prefill panel schedule of `m` (see ``mortar_sched`` in the header);
    ``arith="i8"`` builds the paired-tile schedule of the int8 arm."""
    if arith not in ("bf16", "i8"):
        raise ValueError(f"unknown schedule arithmetic {arith!r}")
    L = _lib.lib()
    f_sizes = L.mortar_sched_sizes if arith == "bf16" else L.mortar_sched_sizes_i8
    f_build = L.mortar_build_sched if arith == "bf16" else L.mortar_build_sched_i8
    rp = np.ascontiguousarray(m.row_ptr)
    ci = np.ascontiguousarray(m.col_idx)
    cd = np.ascontiguousarray(m.codes)
    nt, nr, ns, du = C.c_int64(0), C.c_int64(0), C.c_int64(0), C.c_int64(0)
    npan = C.c_int32(0)
    _lib.check(f_sizes(_ptr(rp), _ptr(ci), m.tile_rows, m.tile_cols, int(swiglu),
                       C.byref(nt), C.byref(nr), C.byref(ns), C.byref(npan),
                       C.byref(du)), "mortar_sched_sizes")
    data = np.zeros(max(du.value, 1) * 16, dtype=np.uint8)
    off = np.zeros(ns.value + 1, dtype=np.uint32)
    meta = np.zeros(max(ns.value, 1), dtype=np.uint32)
    psp = np.zeros(npan.value + 1, dtype=np.int32)
    mask = np.zeros(npan.value, dtype=np.uint32)
    _lib.check(f_build(_ptr(rp), _ptr(ci), _ptr(cd), m.tile_rows, m.tile_cols, m.nnz,
                       int(swiglu), _ptr(data), _ptr(off), _ptr(meta), _ptr(psp),
                       _ptr(mask)), "mortar_build_sched")
    return dict(step_data=data, step_off=off, step_meta=meta, panel_step_ptr=psp, panel_mask=mask,
                n_tiles=nt.value, n_runs=nr.value, n_steps=ns.value, n_panels=npan.value,
                data_units=du.value)


class SchedMatrix:
    """Device-resident prefill schedule of one matrix (owns its tensors)."""

    def __init__(self, m: "MortarMatrix", swiglu: bool, device="cuda", arith: str = "bf16"):
        h = build_sched_host(m, swiglu, arith)
        self.arith = arith
        self.out_features, self.in_features = m.out_features, m.in_features
        self.swiglu, self.scale, self.nnz = bool(swiglu), float(m.scale), m.nnz
        self.n_tiles, self.n_runs, self.n_steps = h["n_tiles"], h["n_runs"], h["n_steps"]
        self.n_panels, self.data_units = h["n_panels"], h["data_units"]
        t = lambda a: torch.from_numpy(a).to(device)
        self.step_data = t(h["step_data"])
        self.step_off = t(h["step_off"].view(np.int32))
        self.step_meta = t(h["step_meta"].view(np.int32))
        self.panel_step_ptr = t(h["panel_step_ptr"])
        self.panel_mask = t(h["panel_mask"].view(np.int32))
        self._c = None

    @classmethod
    def from_tensors(cls, step_data, step_off, step_meta, panel_step_ptr, panel_mask, n_tiles, n_runs,
                     n_steps, data_units, n_panels, out_features, in_features, swiglu, scale) -> "SchedMatrix":
        """A schedule whose arrays already live on the device (the registered ops pass them as
        tensors); borrows the tensors."""
        self = cls.__new__(cls)
        self.arith = "bf16"
        self.out_features, self.in_features = int(out_features), int(in_features)
        self.swiglu, self.scale, self.nnz = bool(swiglu), float(scale), 0
        self.n_tiles, self.n_runs, self.n_steps = int(n_tiles), int(n_runs), int(n_steps)
        self.n_panels, self.data_units = int(n_panels), int(data_units)
        self.step_data, self.step_off, self.step_meta = step_data, step_off, step_meta
        self.panel_step_ptr, self.panel_mask = panel_step_ptr, panel_mask
        self._c = None
        return self

    @property
    def n_out(self) -> int:
        return self.out_features // 2 if self.swiglu else self.out_features

    def c_struct(self) -> _lib.Sched:
        if self._c is None:
            self._c = _lib.Sched(self.step_data.data_ptr(), self.step_off.data_ptr(),
                                 self.step_meta.data_ptr(), self.panel_step_ptr.data_ptr(),
                                 self.panel_mask.data_ptr(), self.n_tiles, self.n_runs, self.n_steps,
                                 self.data_units, self.n_panels, self.out_features // TILE,
                                 self.in_features // TILE, int(self.swiglu), self.scale,
                                 1 if self.arith == "i8" else 0)
        return self._c


BLOCK = 128

# Token blocks run the block path of the prefill kernels (every touched 128 x 128 block executed
# densely, dropped tiles as zeros) when the touched blocks are at least this full.  Measured on the
# cloud shape the dense blocks run at the tensor pipe's rate whatever their fill, while the per-tile
# path pays a narrow MMA per tile and a fixed cost per panel: the block path was faster down to 3%
# random tiles (0.38 ms against 0.41 ms per MLP at 8192 tokens; 187 against 147 TFLOP/s useful at
# 12.5%).  The price is memory: the expanded blocks take 2 bytes per element of every touched
# block, built on the first forward with 128 rows or more.  Below this fill that price buys
# little, and the per-tile path keeps the packed footprint.
BLOCK_PATH_MIN_FILL = 0.05


def wants_block_path(m: "MortarMatrix", swiglu: bool) -> bool:
    """Whether token blocks of `m` should take the block path (see BLOCK_PATH_MIN_FILL)."""
    return block_fill(m) >= BLOCK_PATH_MIN_FILL


def block_fill(m: "MortarMatrix") -> float:
    """Kept tiles / (64 x the number of 128 x 128 blocks that hold a kept tile): 1.0 for a topology
    carved at 128, about the tile density for a random tile-16 one."""
    if m.nnz == 0:
        return 0.0
    rows = np.repeat(np.arange(m.tile_rows), np.diff(m.row_ptr)).astype(np.int64)
    key = (rows // 8) * ((m.tile_cols + 7) // 8) + m.col_idx.astype(np.int64) // 8
    return float(m.nnz) / (64.0 * np.unique(key).size)


class BlockSched:
    """Device-resident layout of one matrix for the block path of the prefill kernels: every
    128 x 128 block that holds a kept tile, expanded to bf16 codes (dropped tiles inside it are
    zeros), and the step lists of the pairs of block rows (see ``mortar_blocks`` in the header)."""

    def __init__(self, m: "MortarMatrix", swiglu: bool, device="cuda"):
        self.out_features, self.in_features = m.out_features, m.in_features
        self.swiglu, self.scale, self.nnz = bool(swiglu), float(m.scale), m.nnz
        Cb = -(-m.in_features // BLOCK)
        rows = np.repeat(np.arange(m.tile_rows), np.diff(m.row_ptr)).astype(np.int64)
        codes = m.to_dense_codes()
        if swiglu:
            # gate rows and up rows each start on a block boundary, so that block row g of the gate
            # half and block row g of the up half cover the same hidden columns whatever d_ff is
            # (a d_ff that is not a multiple of 128 leaves the last block row of each half partly empty)
            d_ff = m.out_features // 2
            Hb = -(-d_ff // BLOCK)
            Rb = 2 * Hb
            dense = np.zeros((Rb * BLOCK, Cb * BLOCK), dtype=np.int8)
            dense[:d_ff, :m.in_features] = codes[:d_ff]
            dense[Hb * BLOCK:Hb * BLOCK + d_ff, :m.in_features] = codes[d_ff:]
            ht = d_ff // TILE
            brow_of_tile = np.where(rows < ht, rows // 8, (rows - ht) // 8 + Hb)
        else:
            Rb = -(-m.out_features // BLOCK)
            dense = np.zeros((Rb * BLOCK, Cb * BLOCK), dtype=np.int8)
            dense[:m.out_features, :m.in_features] = codes
            brow_of_tile = rows // 8
        key = np.unique(brow_of_tile * Cb + m.col_idx.astype(np.int64) // 8)          # ascending (row, column)
        brow, bcol = key // Cb, key % Cb
        blocks = dense.reshape(Rb, BLOCK, Cb, BLOCK).transpose(0, 2, 1, 3)[brow, bcol]   # [nb, 128, 128]
        self.n_blocks = int(key.size)
        index = {(int(r), int(c)): i for i, (r, c) in enumerate(zip(brow, bcol))}
        cols_of = [[] for _ in range(Rb)]
        for r, c in zip(brow, bcol):
            cols_of[int(r)].append(int(c))
        if swiglu:
            half = Rb // 2
            pairs = [(g, g + half) for g in range(half)]
        else:
            pairs = [(2 * q, 2 * q + 1 if 2 * q + 1 < Rb else -1) for q in range((Rb + 1) // 2)]
        pair_ptr, steps = [0], []
        for ra, rb in pairs:
            ca = set(cols_of[ra])
            cb = set(cols_of[rb]) if rb >= 0 else set()
            # block columns both rows keep first: from then on both accumulators are in the same
            # state and every such step is one N = 256 MMA
            for c in sorted(ca | cb, key=lambda c: (not (c in ca and c in cb), c)):
                steps.append((c, index[(ra, c)] if c in ca else -1, index[(rb, c)] if c in cb else -1, 0))
            pair_ptr.append(len(steps))
        self.n_pairs, self.n_steps = len(pairs), len(steps)
        self.data = torch.from_numpy(np.ascontiguousarray(blocks)).to(device=device, dtype=torch.bfloat16)
        self.pair_ptr = torch.tensor(pair_ptr, dtype=torch.int32, device=device)
        self.steps = torch.tensor(steps if steps else [(0, -1, -1, 0)], dtype=torch.int32, device=device).reshape(-1, 4)
        self._c = None

    @classmethod
    def from_tensors(cls, data, pair_ptr, steps, out_features, in_features, swiglu, scale) -> "BlockSched":
        """A block layout whose arrays already live on the device (the registered ops pass them as
        tensors); borrows the tensors."""
        self = cls.__new__(cls)
        self.out_features, self.in_features = int(out_features), int(in_features)
        self.swiglu, self.scale, self.nnz = bool(swiglu), float(scale), 0
        self.data, self.pair_ptr, self.steps = data, pair_ptr, steps
        self.n_blocks = int(data.shape[0]) if data.dim() == 3 else int(data.numel() // (BLOCK * BLOCK))
        self.n_pairs = int(pair_ptr.numel()) - 1
        # the step list of a matrix without blocks is one placeholder row that no pair points at
        self.n_steps = int(steps.shape[0]) if self.n_blocks > 0 else 0
        self._c = None
        return self

    @property
    def n_out(self) -> int:
        return self.out_features // 2 if self.swiglu else self.out_features

    def c_struct(self) -> _lib.Blocks:
        if self._c is None:
            self._c = _lib.Blocks(self.data.data_ptr(), self.pair_ptr.data_ptr(), self.steps.data_ptr(),
                                  self.n_blocks, self.n_pairs, self.n_steps, self.out_features, self.in_features,
                                  int(self.swiglu), self.scale)
        return self._c


class GemvBlocks:
    """Device-resident layout of a matrix carved in 128 x 128 blocks for the tensor-memory decode
    GEMV (see ``mortar_gemv_pack`` in the header): per kept block 128 rows of 8 permuted row words."""

    def __init__(self, m: "MortarMatrix", swiglu: bool, device="cuda"):
        if m.out_features % BLOCK or m.in_features % BLOCK or (swiglu and (m.out_features // 2) % BLOCK):
            raise ValueError("the block GEMV needs feature counts that are multiples of 128")
        self.out_features, self.in_features = m.out_features, m.in_features
        self.swiglu, self.scale, self.nnz = bool(swiglu), float(m.scale), m.nnz
        Rb, Cb = m.out_features // BLOCK, m.in_features // BLOCK
        rows = np.repeat(np.arange(m.tile_rows), np.diff(m.row_ptr)).astype(np.int64)
        cols = m.col_idx.astype(np.int64)
        key = np.unique((rows // 8) * Cb + cols // 8)
        brow, bcol = key // Cb, key % Cb
        nb = int(key.size)
        # canonical row words (code e of a tile row at bits 2e) -> even columns low half, odd columns high half
        canon = np.ascontiguousarray(m.codes).view(np.uint32).reshape(m.nnz, 16)
        perm = np.zeros_like(canon)
        for q in range(8):
            perm |= ((canon >> np.uint32(4 * q)) & np.uint32(3)) << np.uint32(2 * q)
            perm |= ((canon >> np.uint32(4 * q + 2)) & np.uint32(3)) << np.uint32(16 + 2 * q)
        words = np.full((nb, 8, 16, 8), 0x55555555, dtype=np.uint32)          # [block][tile row][row][tile col]
        blk_of = np.searchsorted(key, (rows // 8) * Cb + cols // 8)
        words[blk_of, rows % 8, :, cols % 8] = perm
        blk_ptr = np.concatenate([[0], np.cumsum(np.bincount(brow, minlength=Rb))]).astype(np.int32)
        per_row = np.diff(blk_ptr)
        if swiglu:
            half = Rb // 2
            size = per_row[:half] + per_row[half:]
            items = np.argsort(-size, kind="stable").astype(np.int32)
        else:
            items = np.argsort(-per_row, kind="stable").astype(np.int32)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        self.n_blocks, self.n_items = nb, int(items.size)
        self.row_words = t(words.reshape(nb, 128, 8).view(np.int32))
        self.blk_ptr, self.blk_col, self.items = t(blk_ptr), t(bcol.astype(np.int32)), t(items)
        self._c = None

    @property
    def n_out(self) -> int:
        return self.out_features // 2 if self.swiglu else self.out_features

    def c_struct(self) -> _lib.GemvPack:
        if self._c is None:
            self._c = _lib.GemvPack(self.row_words.data_ptr(), self.blk_ptr.data_ptr(), self.blk_col.data_ptr(),
                                    self.items.data_ptr(), self.n_blocks, self.n_items, self.out_features,
                                    self.in_features, int(self.swiglu), self.scale)
        return self._c


def unpack_stream_host(grp_ptr, grp_cols, grp_codes, row_ptr, tile_rows):
    """Inverse of build_stream_host -> (col_idx uint16[nnz], codes uint8[nnz,64])."""
    nnz = int(row_ptr[-1])
    col_idx = np.zeros(nnz, dtype=np.uint16)
    codes = np.zeros((nnz, 64), dtype=np.uint8)
    rp = np.ascontiguousarray(row_ptr, dtype=np.int32)
    _lib.check(_lib.lib().mortar_unpack_stream(_ptr(np.ascontiguousarray(grp_ptr)),
                                               _ptr(np.ascontiguousarray(grp_cols)),
                                               _ptr(np.ascontiguousarray(grp_codes)), _ptr(rp),
                                               tile_rows, _ptr(col_idx), _ptr(codes)),
               "mortar_unpack_stream")
    return col_idx, codes


def matrix_from_stream(w: "StreamMatrix") -> MortarMatrix:
    """Canonical matrix recovered from a device-resident stream layout (padding slots carry the
    column sentinel 0xFFFF and are dropped)."""
    grp_ptr = w.grp_ptr.detach().cpu().numpy().astype(np.int32)
    grp_cols = w.grp_cols.detach().cpu().numpy().view(np.uint16).reshape(-1)
    grp_codes = w.grp_codes.detach().cpu().numpy().reshape(-1)
    R = w.out_features // TILE
    G = int(grp_ptr[-1])
    live = (grp_cols[:G * 8] != 0xFFFF).reshape(G, 8).sum(axis=1)
    per_group = np.concatenate([[0], np.cumsum(live)]).astype(np.int64)
    row_ptr = per_group[grp_ptr.astype(np.int64)].astype(np.int32)
    col_idx, codes = unpack_stream_host(grp_ptr, grp_cols, grp_codes, row_ptr, R)
    m = MortarMatrix(w.out_features, w.in_features, row_ptr, col_idx, codes, w.scale)
    m.validate()
    return m


class StreamMatrix:
    """Device-resident execution layout of one matrix.  Owns its torch tensors; the C struct
    handed to the library borrows their pointers."""

    def __init__(self, out_features, in_features, scale, n_groups, nnz, grp_ptr, grp_cols,
                 grp_codes, algorithmic_bytes, row_scale=None):
        self.out_features, self.in_features = int(out_features), int(in_features)
        self.scale, self.n_groups, self.nnz = float(scale), int(n_groups), int(nnz)
        self.grp_ptr, self.grp_cols, self.grp_codes = grp_ptr, grp_cols, grp_codes
        self.algorithmic_bytes = int(algorithmic_bytes)
        self.row_scale = row_scale          # optional fp32 [out_features] on the device: per-row scales
        self._c = None

    @property
    def device(self):
        return self.grp_ptr.device

    def to(self, device) -> "StreamMatrix":
        return StreamMatrix(self.out_features, self.in_features, self.scale, self.n_groups, self.nnz,
                            self.grp_ptr.to(device), self.grp_cols.to(device),
                            self.grp_codes.to(device), self.algorithmic_bytes,
                            None if self.row_scale is None else self.row_scale.to(device))

    def c_struct(self) -> _lib.Stream:
        if self._c is None:
            self._c = _lib.Stream(self.grp_codes.data_ptr(), self.grp_cols.data_ptr(),
                                  self.grp_ptr.data_ptr(), self.n_groups,
                                  self.out_features // TILE, self.in_features // TILE, self.scale,
                                  None if self.row_scale is None else self.row_scale.data_ptr())
        return self._c
