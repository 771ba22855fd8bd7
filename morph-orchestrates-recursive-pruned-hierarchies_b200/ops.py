"""Torch-facing operators of the MORTAR path.  Every function launches the hand-written
sm_100a kernels through the C ABI on the current CUDA stream; CPU tensors are rejected
(there is no fallback, as with the reference's CUDA-only ``morph_stk::dds`` op,
morph/sparse/stk/backend/custom_ops.py:35).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .format import TILE, BlockSched, GemvBlocks, MortarMatrix, SchedMatrix, StreamMatrix, TopologyDev

_launches = 0      # kernels launched by this module (bench.py reports it)
_kernel_counts: dict = {}   # the same, per kernel family


def launch_count() -> int:
    return _launches


def kernel_counts() -> dict:
    """Launches so far per kernel family: "act_prep", "bcsr_stream" (the streaming linear / SwiGLU
    kernel), "prefill_panel" (tcgen05 / tensor memory), "stack_decode", "route_flags", "router".
    Tests use the deltas to tell which kernel an operator or module forward ran."""
    return dict(_kernel_counts)


def _count(name: str, n: int = 1) -> None:
    global _launches
    _launches += n
    _kernel_counts[name] = _kernel_counts.get(name, 0) + n


def _stream_ptr() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise NotImplementedError(
            f"{name} is on {t.device}: the MORTAR operators are CUDA-only (sm_100a), no CPU path")


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _lib.F32
    if t.dtype == torch.bfloat16:
        return _lib.BF16
    raise ValueError(f"unsupported dtype {t.dtype}: expected float32 or bfloat16")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _rows2d(x: torch.Tensor, features: int, name: str) -> torch.Tensor:
    if x.shape[-1] != features:
        raise ValueError(f"{name} has last dim {x.shape[-1]}, expected {features}")
    x2 = x.reshape(-1, features)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    return x2


def act_prep(x: torch.Tensor, n_planes: int = 3, rms_weight: Optional[torch.Tensor] = None,
             eps: float = 1e-6) -> torch.Tensor:
    """x[rows, cols] -> bf16 planes [n_planes, rows, cols] whose sum is x (after the optional
    RMSNorm (x*rsqrt(mean x^2+eps))*w, fused_decode_step.py:293-321)."""
    _require_cuda(x, "x")
    x2 = _rows2d(x, x.shape[-1], "x")
    rows, cols = x2.shape
    planes = torch.empty(n_planes, rows, cols, device=x.device, dtype=torch.bfloat16)
    if rows == 0:
        return planes
    w = None
    if rms_weight is not None:
        w = rms_weight.to(device=x.device, dtype=torch.float32).contiguous()
    _lib.check(_lib.lib().mortar_act_prep(_ptr(x2), _dtype_code(x2), rows, cols, x2.stride(0), _ptr(w),
                                          float(eps), _ptr(planes), n_planes, rows * cols, cols,
                                          _stream_ptr()), "mortar_act_prep")
    _count("act_prep")
    return planes


def linear_planes(w: StreamMatrix, planes: torch.Tensor, *, swiglu: bool = False,
                  out_dtype: torch.dtype = torch.float32, out_planes: int = 0,
                  round_bf16: bool = False, gates: Optional[torch.Tensor] = None,
                  cluster_size: int = 0, gates_on_input: bool = False,
                  row_act: Optional[torch.Tensor] = None, col_act: Optional[torch.Tensor] = None,
                  path: str = "auto"):
    """Block-sparse ternary linear on activation planes [P, rows, in]: returns [rows, out]
    (or [rows, out/2] = silu(gate)*up with ``swiglu``), as float32/bfloat16 or, with
    ``out_planes`` > 0, as planes [out_planes, rows, n].  ``path`` pins one of the kernel's
    paths ("plain", "staged", "persistent"); "auto" picks by matrix size and batch."""
    _require_cuda(planes, "planes")
    if planes.dim() != 3 or planes.dtype != torch.bfloat16 or not planes.is_contiguous():
        raise ValueError("planes must be a contiguous bfloat16 tensor [P, rows, in_features]")
    P, rows, cols = planes.shape
    if cols != w.in_features:
        raise ValueError(f"planes have {cols} columns, matrix expects {w.in_features}")
    n_out = w.out_features // 2 if swiglu else w.out_features
    dev = planes.device
    if out_planes:
        out = torch.empty(out_planes, rows, n_out, device=dev, dtype=torch.bfloat16)
        mode = _lib.OUT_PLANES
    elif out_dtype == torch.float32:
        out = torch.empty(rows, n_out, device=dev, dtype=torch.float32)
        mode = _lib.OUT_F32
    elif out_dtype == torch.bfloat16:
        out = torch.empty(rows, n_out, device=dev, dtype=torch.bfloat16)
        mode = _lib.OUT_BF16
    else:
        raise ValueError(f"unsupported out_dtype {out_dtype}")
    if rows == 0:
        return out
    flags = (_lib.FLAG_SWIGLU if swiglu else 0) | (_lib.FLAG_ROUND_BF16 if round_bf16 else 0) \
        | (_lib.FLAG_GATES_ON_INPUT if gates_on_input else 0) | _lib.PATH_FLAGS[path]
    if gates is not None:
        gates = gates.to(device=dev, dtype=torch.float32).reshape(rows, -1).contiguous()
    for name, a in (("row_act", row_act), ("col_act", col_act)):
        if a is not None and (a.dtype != torch.int32 or a.dim() != 2 or a.shape[0] != rows
                              or a.stride(1) != 1):
            raise ValueError(f"{name} must be int32 [rows, n] with unit inner stride")
    st = w.c_struct()
    _lib.check(_lib.lib().mortar_linear(
        C.byref(st), _ptr(planes), P, rows * cols, cols, rows, _ptr(out), mode, out_planes,
        rows * n_out, n_out, flags, _ptr(gates), gates.stride(0) if gates is not None else 0,
        int(cluster_size), _ptr(row_act), row_act.stride(0) if row_act is not None else 0,
        _ptr(col_act), col_act.stride(0) if col_act is not None else 0, _stream_ptr()),
        "mortar_linear")
    _count("bcsr_stream")
    return out


def gemv_xprep(planes: torch.Tensor) -> torch.Tensor:
    """Activation planes [P, rows, in] (bf16, rows * P <= 16) -> the activation operand of
    ``gemv_blocks``: in/16 tiles of 512 bytes."""
    _require_cuda(planes, "planes")
    if planes.dim() != 3 or planes.dtype != torch.bfloat16 or not planes.is_contiguous():
        raise ValueError("planes must be a contiguous bfloat16 tensor [P, rows, in_features]")
    P, rows, cols = planes.shape
    xb = torch.empty(cols // 16 * 512, device=planes.device, dtype=torch.uint8)
    _lib.check(_lib.lib().mortar_gemv_xprep(_ptr(planes), P, rows * cols, cols, rows, cols, _ptr(xb), _stream_ptr()),
               "mortar_gemv_xprep")
    _count("gemv_xprep")
    return xb


def gemv_xprep_swiglu(gate_up: torch.Tensor, n_planes: int = 3) -> torch.Tensor:
    """fp32 result of an unfused gate/up product [rows, 2 d_ff] -> activation operand of the down
    product: silu(gate) * up as ``n_planes`` exact bf16 planes in the layout of ``gemv_xprep``."""
    _require_cuda(gate_up, "gate_up")
    if gate_up.dim() != 2 or gate_up.dtype != torch.float32 or gate_up.stride(1) != 1:
        raise ValueError("gate_up must be float32 [rows, 2 d_ff] with unit inner stride")
    rows, two_f = gate_up.shape
    xb = torch.empty(two_f // 2 // 16 * 512, device=gate_up.device, dtype=torch.uint8)
    _lib.check(_lib.lib().mortar_gemv_xprep_swiglu(_ptr(gate_up), gate_up.stride(0), rows, two_f // 2, n_planes,
                                                   _ptr(xb), _stream_ptr()), "mortar_gemv_xprep_swiglu")
    _count("gemv_xprep")
    return xb


def gemv_blocks(w: GemvBlocks, xb: torch.Tensor, rows: int, n_planes: int, *,
                out_dtype: torch.dtype = torch.float32, out_planes: int = 0) -> torch.Tensor:
    """Decode GEMV on the tensor-memory path for a matrix carved in 128 x 128 blocks
    (``MortarMatrix.to_gemv_blocks``) against an activation operand from ``gemv_xprep``:
    [rows, out] (or [rows, out/2] = silu(gate)*up for a swiglu layout) as float32 / bfloat16, or
    with ``out_planes`` > 0 as exact bf16 planes [out_planes, rows, n]."""
    _require_cuda(xb, "xb")
    n_out = w.n_out
    dev = xb.device
    if xb.numel() != w.in_features // 16 * 512:
        raise ValueError("activation operand does not match the matrix")
    if out_planes:
        out, mode = torch.empty(out_planes, rows, n_out, device=dev, dtype=torch.bfloat16), _lib.OUT_PLANES
    elif out_dtype == torch.float32:
        out, mode = torch.empty(rows, n_out, device=dev, dtype=torch.float32), _lib.OUT_F32
    elif out_dtype == torch.bfloat16:
        out, mode = torch.empty(rows, n_out, device=dev, dtype=torch.bfloat16), _lib.OUT_BF16
    else:
        raise ValueError(f"unsupported out_dtype {out_dtype}")
    st = w.c_struct()
    _lib.check(_lib.lib().mortar_gemv_blocks(C.byref(st), _ptr(xb), rows, n_planes, _ptr(out), mode, out_planes,
                                             rows * n_out, n_out, _stream_ptr()), "mortar_gemv_blocks")
    _count("gemv_tc")
    return out


def gemv_blocks_error(reset: bool = True) -> int:
    """Error word of the tensor-memory decode GEMV (0 = none; synchronises the device)."""
    code = C.c_int32(0)
    _lib.check(_lib.lib().mortar_gemv_blocks_error(C.byref(code), int(reset)), "mortar_gemv_blocks_error")
    return code.value


def linear(x: torch.Tensor, w: StreamMatrix, *, n_planes: Optional[int] = None,
           out_dtype: Optional[torch.dtype] = None, round_bf16: Optional[bool] = None) -> torch.Tensor:
    """y = x @ W^T for x[..., in]; the drop-in for ``CMSBlockLinear._forward_mortar``
    (block_sparse.py:921-970).  bf16 input -> bf16 output with the reference's rounding;
    fp32 input -> fp32 output computed from exact 3-plane activations."""
    _require_cuda(x, "x")
    lead = x.shape[:-1]
    x2 = _rows2d(x, w.in_features, "x")
    is_bf16 = x2.dtype == torch.bfloat16
    if n_planes is None:
        n_planes = 1 if is_bf16 else 3
    if out_dtype is None:
        out_dtype = x2.dtype
    if round_bf16 is None:
        round_bf16 = is_bf16
    if is_bf16 and x2.is_contiguous():
        planes = x2.unsqueeze(0)
    else:
        planes = act_prep(x2, n_planes)
    y = linear_planes(w, planes, out_dtype=out_dtype, round_bf16=round_bf16)
    return y.reshape(*lead, w.out_features)


_workspaces: dict = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    """Scratch for the hidden activations of one MLP call when the caller passes none: one buffer
    per (device, stream), so calls on different streams never share it; it grows by
    reallocation, so code that captures CUDA graphs should pass its own ``workspace``."""
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), device=device, dtype=torch.uint8)
        _workspaces[key] = ws
    return ws


def mlp_decode(x: torch.Tensor, gate_up: StreamMatrix, down: StreamMatrix, *,
               rms_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
               gates: Optional[torch.Tensor] = None, n_clusters: int = 0,
               n_planes: int = 3, round_bf16: bool = False,
               out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
               accumulate: bool = False,
               workspace: Optional[torch.Tensor] = None, path: str = "auto") -> torch.Tensor:
    """One SwiGLU MLP application for a block of rows: [rmsnorm] -> gate_up -> silu(g)*u
    [*gates] -> down.  Mirrors StaticDecodeEngine._mlp_fn (morph/inference/engine.py:936-986)
    with ``n_planes=3`` (fp32 semantics) and ``_SwiGLUMortar.forward`` under autocast
    (morph/model/transformer.py:402-431) with ``n_planes=1, round_bf16=True``.  With
    ``accumulate`` the result is added into ``out`` (the residual carrier)."""
    _require_cuda(x, "x")
    d_model, d_ff = gate_up.in_features, gate_up.out_features // 2
    lead = x.shape[:-1]
    x2 = _rows2d(x, d_model, "x")
    rows = x2.shape[0]
    if out_dtype is None:
        out_dtype = x2.dtype
    if out is None:
        if accumulate:
            raise ValueError("accumulate needs an `out` tensor to add into")
        out = torch.empty(rows, d_model, device=x.device, dtype=out_dtype)
    elif out.shape[-1] != d_model or out.numel() != rows * d_model or out.stride(-1) != 1:
        raise ValueError("out has the wrong shape")
    out2 = out.reshape(rows, d_model)
    if rows == 0:
        return out.reshape(*lead, d_model)
    L = _lib.lib()
    need = L.mortar_mlp_workspace_bytes(rows, d_model, d_ff, n_planes)
    if need < 0:
        _lib.check(int(need), "mortar_mlp_workspace_bytes")
    if workspace is None:
        workspace = _workspace(x.device, need)
    w = None
    if rms_weight is not None:
        w = rms_weight.to(device=x.device, dtype=torch.float32).contiguous()
    g = None
    if gates is not None:
        g = gates.to(device=x.device, dtype=torch.float32).reshape(rows, -1).contiguous()
        if g.shape[1] != n_clusters:
            raise ValueError(f"gates have {g.shape[1]} clusters, n_clusters={n_clusters}")
    gu, dn = gate_up.c_struct(), down.c_struct()
    _lib.check(L.mortar_mlp_decode(
        C.byref(gu), C.byref(dn), _ptr(x2), _dtype_code(x2), x2.stride(0), rows, _ptr(w), float(eps),
        _ptr(g), g.stride(0) if g is not None else 0, int(n_clusters), _ptr(out2), _dtype_code(out2),
        out2.stride(0), int(n_planes),
        (_lib.FLAG_ROUND_BF16 if round_bf16 else 0) | (_lib.FLAG_ACCUMULATE if accumulate else 0)
        | _lib.PATH_FLAGS[path],
        _ptr(workspace), workspace.numel(), _stream_ptr()), "mortar_mlp_decode")
    direct = x2.dtype == torch.bfloat16 and rms_weight is None and x2.stride(0) % 2 == 0 \
        and x2.data_ptr() % 4 == 0
    if not direct:
        _count("act_prep")
    if g is not None and rows > 8:          # routed batch: per-row gather of the hidden tile rows
        _count("route_gather")
        _count("bcsr_gather")
        _count("bcsr_stream")
    else:
        _count("bcsr_stream", 2)
    return out.reshape(*lead, d_model)


def mlp_decode_static(x: torch.Tensor, gate_up: StreamMatrix, down: StreamMatrix, out: torch.Tensor, *,
                      rms_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                      gates: Optional[torch.Tensor] = None, n_clusters: int = 0,
                      n_planes: int = 3, round_bf16: bool = False, accumulate: bool = False) -> torch.Tensor:
    """``mlp_decode`` for callers that must not allocate: the activation planes go to an 8 MiB
    array built into the library instead of a workspace tensor, and the result is written to
    the caller's ``out``.  Every argument must already be a contiguous CUDA tensor of its final
    dtype (fp32 gates / rms_weight): this wrapper converts and allocates nothing.  Raises
    ``ValueError`` when the batch needs more than the built-in scratch.  Calls share the
    scratch, so run them one after another on a stream, not concurrently."""
    _require_cuda(x, "x")
    d_model, d_ff = gate_up.in_features, gate_up.out_features // 2
    if x.dim() != 2 or x.shape[1] != d_model or x.stride(1) != 1:
        raise ValueError("x must be [rows, d_model] with unit inner stride")
    if out.shape != x.shape or out.stride(1) != 1 or not out.is_cuda:
        raise ValueError("out must be a CUDA tensor shaped like x")
    for name, t in (("rms_weight", rms_weight), ("gates", gates)):
        if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous float32 CUDA tensor")
    if x.device.index != torch.cuda.current_device() or out.device != x.device:
        raise ValueError("x and out must live on the current CUDA device (its scratch array and stream are used)")
    rows = x.shape[0]
    if rows == 0:
        return out
    gu, dn = gate_up.c_struct(), down.c_struct()
    _lib.check(_lib.lib().mortar_mlp_decode_static(
        C.byref(gu), C.byref(dn), _ptr(x), _dtype_code(x), x.stride(0), rows, _ptr(rms_weight), float(eps),
        _ptr(gates), gates.stride(0) if gates is not None else 0, int(n_clusters), _ptr(out),
        _dtype_code(out), out.stride(0), int(n_planes),
        (_lib.FLAG_ROUND_BF16 if round_bf16 else 0) | (_lib.FLAG_ACCUMULATE if accumulate else 0),
        _stream_ptr()), "mortar_mlp_decode_static")
    direct = x.dtype == torch.bfloat16 and rms_weight is None and x.stride(0) % 2 == 0 and x.data_ptr() % 4 == 0
    if not direct:
        _count("act_prep")
    if gates is not None and rows > 8:
        _count("route_gather")
        _count("bcsr_gather")
        _count("bcsr_stream")
    else:
        _count("bcsr_stream", 2)
    return out


class _StackBlobs:
    """Per-(layer, cluster rank) weights of a stack for one cluster size, in two parts per rank:
    the stream layout of the rank's gate/up tile rows, and the stream layout of the matching
    K-slice of the down projection.  Each part = int32[8] header {n_groups, byte offsets of
    grp_ptr, grp_cols, grp_codes, scale bits, part bytes, byte offset of an fp32[d_model] norm
    weight or 0, 0} followed by the arrays (16-byte aligned)."""

    def __init__(self, layers, d_model, d_ff, cs, device, embed_norm_weights):
        import numpy as np
        F_ = d_ff // TILE
        U = F_ // cs
        blobs, table, off = [], np.zeros((len(layers), cs, 4), dtype=np.int32), 0
        for li, (gu, dn, w) in enumerate(layers):
            wb = b"" if (w is None or not embed_norm_weights) else \
                w.detach().float().cpu().numpy().astype(np.float32).tobytes()
            for c in range(cs):
                rows = list(range(c * U, (c + 1) * U)) + list(range(F_ + c * U, F_ + (c + 1) * U))
                subs = (gu.slice_tile_rows(rows), dn.slice_tile_cols(c * U, (c + 1) * U))
                for part, sub in enumerate(subs):
                    gp, gc, gcd, G = sub.build_stream_host()
                    arrays = [gp.tobytes(), gc[:max(G, 1) * 8].tobytes(), gcd[:max(G, 1) * 512].tobytes()]
                    if part == 0:
                        arrays.append(wb)
                    hdr = np.zeros(8, dtype=np.int32)
                    body, pos = [], 32
                    for k, raw in enumerate(arrays):
                        if k < 3:
                            hdr[1 + k] = pos
                        else:
                            hdr[6] = pos if raw else 0
                        pad = (-len(raw)) % 16
                        body.append(raw + b"\0" * pad)
                        pos += len(raw) + pad
                    hdr[0] = G
                    hdr[4] = np.float32(sub.scale).view(np.int32)
                    hdr[5] = pos
                    blob = hdr.tobytes() + b"".join(body)
                    table[li, c, 2 * part] = off // 16
                    table[li, c, 2 * part + 1] = len(blob)
                    blobs.append(blob)
                    off += len(blob)
        self.cs = cs
        self.max_a = (int(table[:, :, 1].max()) + 127) // 128 * 128
        self.max_b = (int(table[:, :, 3].max()) + 127) // 128 * 128
        self.blobs = torch.from_numpy(np.frombuffer(b"".join(blobs), dtype=np.uint8).copy()).to(device)
        self.table = torch.from_numpy(table.reshape(-1)).to(device)


class DecodeStack:
    """A list of MLP applications (the MLP sites of one decode step, in execution order) that
    one persistent launch walks: x <- x + MLP_i(rmsnorm_i(x)).  `layers` are (gate_up, down,
    rms_weight) triples of canonical ``MortarMatrix`` / fp32 tensor (or None); `order` indexes
    into them.  Every thread-block cluster rank gets its share of each layer as one blob: the
    gate/up tile rows of its hidden slice and the matching K-slice of the down projection.
    Blobs are built for clusters of 8 and, where the shapes divide, of 16 (used for small
    batches, where only a few clusters run and 16 SMs per row block halve the latency)."""

    def __init__(self, layers, order, device="cuda", cluster_sizes=(8, 16)):
        self.order = list(order)
        gu0, dn0, _ = layers[0]
        self.d_model, self.d_ff = gu0.in_features, gu0.out_features // 2
        for gu, dn, w in layers:
            if (gu.in_features, gu.out_features // 2) != (self.d_model, self.d_ff) or \
                    (dn.in_features, dn.out_features) != (self.d_ff, self.d_model):
                raise ValueError("every application of a stack must have the same d_model and d_ff")
        # norm weights: one [n_layers, d_model] array the kernel reads per application; only when
        # some layers have a weight and others none do the blobs carry their own copies instead
        have = [w is not None for _, _, w in layers]
        self.rms_weights = None
        if all(have):
            self.rms_weights = torch.stack([w.detach().float().cpu() for _, _, w in layers]).contiguous().to(device)
        embed = any(have) and not all(have)
        self.variants = {}
        for cs in cluster_sizes:
            if (self.d_ff // TILE) % cs == 0 and self.d_model % (TILE * cs) == 0:
                self.variants[cs] = _StackBlobs(layers, self.d_model, self.d_ff, cs, device, embed)
        if not self.variants:
            raise ValueError("d_ff/16 and d_model/16 must be divisible by the cluster size (8 or 16)")
        self.app_layer = torch.tensor(self.order, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.n_apps, self.n_layers = len(self.order), len(layers)

    def pick(self, rows: int) -> "_StackBlobs":
        # at most 4 clusters of 16 CTAs are co-resident on the 8 GPCs: use them for <= 32 rows
        if 16 in self.variants and (rows <= 32 or 8 not in self.variants):
            return self.variants[16]
        return self.variants[8] if 8 in self.variants else next(iter(self.variants.values()))

    def error(self, reset: bool = True) -> int:
        """Non-zero if a bounded wait inside the kernel expired (synchronises)."""
        v = int(self.status.item())
        if reset and v:
            self.status.zero_()
        return v


PLANES_HALF2 = 12      # MORTAR_PLANES_HALF2: two fp16 planes with exact per-row power-of-two scaling


def stack_decode(x: torch.Tensor, stack: DecodeStack, *, eps: float = 1e-6, n_planes: int = PLANES_HALF2,
                 cluster_size: Optional[int] = None) -> torch.Tensor:
    """In-place decode step of a whole MLP stack on the fp32 residual carrier x [rows, d_model]:
    one launch, every block of 8 rows walks all applications inside one thread-block cluster.
    ``n_planes``: 3 = three bf16 planes (fp32 activations represented exactly), ``PLANES_HALF2``
    (default) = two scaled fp16 planes (residual below 2^-22 of an element; a third fewer MMAs)."""
    _require_cuda(x, "x")
    if x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] != stack.d_model or x.stride(1) != 1:
        raise ValueError("x must be float32 [rows, d_model] with unit inner stride")
    rows = x.shape[0]
    v = stack.variants[cluster_size] if cluster_size else stack.pick(rows)
    _lib.check(_lib.lib().mortar_stack_decode(
        _ptr(v.blobs), _ptr(v.table), _ptr(stack.app_layer), _ptr(stack.rms_weights), stack.n_apps, stack.n_layers,
        stack.d_model, stack.d_ff, v.max_a, v.max_b, v.cs, _ptr(x), x.stride(0), rows,
        float(eps), int(n_planes), _ptr(stack.status), _stream_ptr()), "mortar_stack_decode")
    _count("stack_decode")
    return x


def _hc_struct(hres, hpost_row, carrier, out, term, n, C_):
    for name, t in (("hres", hres), ("hpost_row", hpost_row), ("carrier", carrier), ("out", out), ("term", term)):
        if t is not None and (t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous()):
            raise ValueError(f"{name} must be a contiguous float32 CUDA tensor")
    rows = carrier.numel() // (n * C_)
    if hres.numel() != rows * n * n or hpost_row.numel() != rows * n or out.shape != carrier.shape or \
            (term is not None and term.numel() != rows * C_):
        raise ValueError("hres [rows,n,n], hpost_row [rows,n], carrier/out [rows,n,C], term [rows,C] expected")
    return _lib.HcPost(hres.data_ptr(), hpost_row.data_ptr(), carrier.data_ptr(), out.data_ptr(),
                       None if term is None else term.data_ptr(), n), rows


def mlp_decode_hc(x: torch.Tensor, gate_up: StreamMatrix, down: StreamMatrix, hres: torch.Tensor,
                  hpost_row: torch.Tensor, carrier: torch.Tensor, *, term: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None, rms_weight: Optional[torch.Tensor] = None, eps: float = 1e-6,
                  gates: Optional[torch.Tensor] = None, n_clusters: int = 0, n_planes: int = 3,
                  workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The MLP site of the decode engine including the write the engine runs after it
    (morph/inference/engine.py:1001-1060): x [..., d_model] is the single-stream input the
    hyper-connection PRE map produced, ``carrier`` [..., n, d_model] the n-stream residual; the down
    projection's epilogue writes out[..., i, :] = sum_j hres[..., i, j] carrier[..., j, :] +
    hpost_row[..., i] * MLP(x) (+ term), the arithmetic of ``_hc_post_fwd_kernel``
    (morph/kernels/triton/fused_hyper_connection.py:933-977).  ``out`` defaults to a new tensor;
    passing ``carrier`` itself updates the carrier in place."""
    _require_cuda(x, "x")
    d_model, d_ff = gate_up.in_features, gate_up.out_features // 2
    x2 = _rows2d(x, d_model, "x")
    n = carrier.shape[-2]
    if carrier.shape[-1] != d_model:
        raise ValueError("carrier must be [..., n_streams, d_model]")
    if out is None:
        out = torch.empty_like(carrier)
    hc, rows = _hc_struct(hres, hpost_row, carrier, out, term, n, d_model)
    if rows != x2.shape[0]:
        raise ValueError("x and carrier disagree on the number of tokens")
    if rows == 0:
        return out
    L = _lib.lib()
    need = L.mortar_mlp_workspace_bytes(rows, d_model, d_ff, n_planes)
    if workspace is None:
        workspace = _workspace(x.device, need)
    w = None if rms_weight is None else rms_weight.to(device=x.device, dtype=torch.float32).contiguous()
    g = None
    if gates is not None:
        g = gates.to(device=x.device, dtype=torch.float32).reshape(rows, -1).contiguous()
    gu, dn = gate_up.c_struct(), down.c_struct()
    _lib.check(L.mortar_mlp_decode_hc(
        C.byref(gu), C.byref(dn), _ptr(x2), _dtype_code(x2), x2.stride(0), rows, _ptr(w), float(eps), _ptr(g),
        g.stride(0) if g is not None else 0, int(n_clusters), C.byref(hc), d_model, int(n_planes), 0,
        _ptr(workspace), workspace.numel(), _stream_ptr()), "mortar_mlp_decode_hc")
    _count("bcsr_stream", 2)
    return out


class RowScaledPack:
    """A stack of dense ternary projections with per-row scales in this library's stream layout
    (what ``ternary_gemv_rs`` consumes; built once per weight stack)."""

    def __init__(self, stream: StreamMatrix, out_features: int):
        self.stream, self.out_features = stream, int(out_features)


def ternary_pack_rs(codes: torch.Tensor, row_scale: torch.Tensor, device="cuda") -> RowScaledPack:
    """Strip-packed dense ternary rows [O, I/4] uint8 (byte j = columns j, j+I/4, j+I/2, j+3I/4;
    ``ternary_pack``, fused_decode_step.py:1181-1204) + fp32 row scales [O] -> stream layout.  Rows
    are padded to a multiple of 16 with zero codes; I must be a multiple of 16."""
    import numpy as np
    p = codes.detach().cpu().numpy().astype(np.uint8)
    O, I4 = p.shape
    I = 4 * I4
    if I % TILE:
        raise ValueError("in_features must be a multiple of 16")
    dense = np.zeros((O, 4, I4), dtype=np.int8)
    for st in range(4):
        dense[:, st] = ((p >> (2 * st)) & 3).astype(np.int8) - 1
    dense = dense.reshape(O, I)
    Opad = (O + TILE - 1) // TILE * TILE
    if Opad != O:
        dense = np.concatenate([dense, np.zeros((Opad - O, I), dtype=np.int8)])
    m = MortarMatrix.from_codes(dense, None, 1.0)
    s = m.to_stream(device)
    rs = torch.zeros(Opad, dtype=torch.float32)
    rs[:O] = row_scale.detach().float().cpu().reshape(-1)
    s.row_scale = rs.to(device)
    s._c = None
    return RowScaledPack(s, O)


def ternary_gemv_rs(x: torch.Tensor, pack: RowScaledPack) -> torch.Tensor:
    """Row-scaled dense ternary GEMV, the role of the reference ``ternary_gemv_rs(x, codes,
    row_scale)`` (fused_decode_step.py:1778-1791): x [B, I] fp32 -> [B, O] fp32 with exact +-x
    products (three bf16 planes), fp32 accumulation and the row's scale applied after the sum."""
    _require_cuda(x, "x")
    planes = act_prep(x.float().reshape(-1, x.shape[-1]), 3)
    y = linear_planes(pack.stream, planes, out_dtype=torch.float32)
    return y[:, :pack.out_features]


def stack_decode_raw(x: torch.Tensor, blobs: torch.Tensor, blob_table: torch.Tensor, app_layer: torch.Tensor,
                     rms_weights: Optional[torch.Tensor], status: torch.Tensor, n_layers: int, d_model: int,
                     d_ff: int, max_gate_up_bytes: int, max_down_bytes: int, cluster_size: int,
                     eps: float = 1e-6, n_planes: int = 3) -> torch.Tensor:
    """``mortar_stack_decode`` on raw tensors (what ``DecodeStack`` holds): in place on x
    [rows, d_model] fp32.  ``rms_weights`` [n_layers, d_model] fp32 serves layers whose blobs do
    not carry their own norm weight."""
    _require_cuda(x, "x")
    if x.dtype != torch.float32 or x.dim() != 2 or x.shape[1] != d_model or x.stride(1) != 1:
        raise ValueError("x must be float32 [rows, d_model] with unit inner stride")
    if rms_weights is not None and (rms_weights.dtype != torch.float32 or not rms_weights.is_contiguous()
                                    or tuple(rms_weights.shape) != (n_layers, d_model)):
        raise ValueError("rms_weights must be contiguous float32 [n_layers, d_model]")
    _lib.check(_lib.lib().mortar_stack_decode(
        _ptr(blobs), _ptr(blob_table), _ptr(app_layer), _ptr(rms_weights), int(app_layer.numel()),
        int(n_layers), int(d_model), int(d_ff), int(max_gate_up_bytes), int(max_down_bytes), int(cluster_size),
        _ptr(x), x.stride(0),
        x.shape[0], float(eps), int(n_planes), _ptr(status), _stream_ptr()), "mortar_stack_decode")
    _count("stack_decode")
    return x


def mlp_prefill(x: torch.Tensor, gate_up: StreamMatrix, down: StreamMatrix, *,
                gates: Optional[torch.Tensor] = None, n_clusters: int = 0,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``_SwiGLUMortar.forward`` for a block of tokens in the reference's autocast dtype:
    bf16 operands, fp32 accumulation, bf16 rounding after gate_up, silu, the product, the
    gate multiply and down (transformer.py:402-431; triton_kernels.py:203-226)."""
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    return mlp_decode(xb, gate_up, down, gates=gates, n_clusters=n_clusters, n_planes=1,
                      round_bf16=True, out_dtype=torch.bfloat16, out=out)


def linear_tc(x: torch.Tensor, w: SchedMatrix, *, gates: Optional[torch.Tensor] = None,
              cluster_size: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Tensor-memory (tcgen05) block-sparse linear for token blocks: bf16 x[rows, in] ->
    bf16 [rows, out] (or [rows, out/2] = silu(gate)*up for a swiglu schedule), with the
    reference's prefill rounding (stk dds, triton_kernels.py:203-226)."""
    _require_cuda(x, "x")
    if x.dtype != torch.bfloat16:
        raise ValueError("linear_tc takes bfloat16 activations")
    lead = x.shape[:-1]
    x2 = _rows2d(x, w.in_features, "x")
    rows = x2.shape[0]
    if x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    n_out = w.n_out
    if out is None:
        out = torch.empty(rows, n_out, device=x.device, dtype=torch.bfloat16)
    out2 = out.reshape(rows, n_out)
    if rows == 0:
        return out.reshape(*lead, n_out)
    g = None
    if gates is not None:
        g = gates.to(device=x.device, dtype=torch.float32).reshape(rows, -1).contiguous()
    st = w.c_struct()
    _lib.check(_lib.lib().mortar_linear_tc(C.byref(st), _ptr(x2), x2.stride(0), rows, _ptr(out2),
                                           out2.stride(0), _ptr(g), g.stride(0) if g is not None else 0,
                                           int(cluster_size), _stream_ptr()), "mortar_linear_tc")
    _count("prefill_panel")
    return out.reshape(*lead, n_out)


def mlp_prefill_tc(x: torch.Tensor, gate_up: SchedMatrix, down: SchedMatrix, *,
                   gates: Optional[torch.Tensor] = None, n_clusters: int = 0,
                   out: Optional[torch.Tensor] = None,
                   workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``_SwiGLUMortar.forward`` on a token block through the tcgen05 kernels: bf16 in, bf16
    out, the reference's autocast rounding points (transformer.py:402-431)."""
    _require_cuda(x, "x")
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    d_model, d_ff = gate_up.in_features, gate_up.out_features // 2
    lead = xb.shape[:-1]
    x2 = _rows2d(xb, d_model, "x")
    rows = x2.shape[0]
    if x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty(rows, d_model, device=x.device, dtype=torch.bfloat16)
    out2 = out.reshape(rows, d_model)
    if rows == 0:
        return out.reshape(*lead, d_model)
    need = rows * d_ff * 2
    if workspace is None:
        workspace = _workspace(x.device, need)
    g = None
    if gates is not None:
        g = gates.to(device=x.device, dtype=torch.float32).reshape(rows, -1).contiguous()
        if g.shape[1] != n_clusters:
            raise ValueError(f"gates have {g.shape[1]} clusters, n_clusters={n_clusters}")
    gu, dn = gate_up.c_struct(), down.c_struct()
    _lib.check(_lib.lib().mortar_mlp_prefill(
        C.byref(gu), C.byref(dn), _ptr(x2), x2.stride(0), rows, _ptr(g),
        g.stride(0) if g is not None else 0, int(n_clusters), _ptr(out2), out2.stride(0),
        _ptr(workspace), workspace.numel(), _stream_ptr()), "mortar_mlp_prefill")
    _count("prefill_panel", 2)
    return out.reshape(*lead, d_model)


BLOCKS_MODES = {"auto": 0, "single": 1, "pairs": 2}


def linear_blocks_mode(mode: str) -> str:
    """Chooses the kernel of the block path process-wide: "auto" (the default: CTA pairs, tcgen05
    cta_group::2, from 129 rows on), "single" or "pairs".  Returns the previous mode."""
    prev = _lib.lib().mortar_linear_blocks_mode(BLOCKS_MODES[mode])
    _lib.check(min(prev, 0), "mortar_linear_blocks_mode")
    return {v: k for k, v in BLOCKS_MODES.items()}[prev]


def linear_blocks(x: torch.Tensor, w: BlockSched, *, gates: Optional[torch.Tensor] = None,
                  cluster_size: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``linear_tc`` on the block path: the matrix as expanded 128 x 128 blocks (``MortarMatrix.to_blocks``),
    bf16 x[rows, in] -> bf16 [rows, out] (or [rows, out/2] = silu(gate)*up for a swiglu layout), the
    reference's prefill rounding (stk dds at its own granularity, triton_kernels.py:203-226)."""
    _require_cuda(x, "x")
    if x.dtype != torch.bfloat16:
        raise ValueError("linear_blocks takes bfloat16 activations")
    lead = x.shape[:-1]
    x2 = _rows2d(x, w.in_features, "x")
    rows = x2.shape[0]
    if x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    n_out = w.n_out
    if out is None:
        out = torch.empty(rows, n_out, device=x.device, dtype=torch.bfloat16)
    out2 = out.reshape(rows, n_out)
    if rows == 0:
        return out.reshape(*lead, n_out)
    g = None
    if gates is not None:
        g = gates.to(device=x.device, dtype=torch.float32).reshape(rows, -1).contiguous()
    st = w.c_struct()
    _lib.check(_lib.lib().mortar_linear_blocks(C.byref(st), _ptr(x2), x2.stride(0), rows, _ptr(out2),
                                               out2.stride(0), _ptr(g), g.stride(0) if g is not None else 0,
                                               int(cluster_size), _stream_ptr()), "mortar_linear_blocks")
    _count("prefill_blocks")
    return out.reshape(*lead, n_out)


def mlp_prefill_blocks(x: torch.Tensor, gate_up: BlockSched, down: BlockSched, *,
                       gates: Optional[torch.Tensor] = None, n_clusters: int = 0,
                       out: Optional[torch.Tensor] = None,
                       workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``_SwiGLUMortar.forward`` on a token block through the block path of the tcgen05 kernels
    (transformer.py:402-431): bf16 in, bf16 out, the reference's autocast rounding points."""
    _require_cuda(x, "x")
    xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
    d_model, d_ff = gate_up.in_features, gate_up.out_features // 2
    lead = xb.shape[:-1]
    x2 = _rows2d(xb, d_model, "x")
    rows = x2.shape[0]
    if x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    if out is None:
        out = torch.empty(rows, d_model, device=x.device, dtype=torch.bfloat16)
    out2 = out.reshape(rows, d_model)
    if rows == 0:
        return out.reshape(*lead, d_model)
    if workspace is None:
        workspace = _workspace(x.device, rows * d_ff * 2)
    g = None
    if gates is not None:
        g = gates.to(device=x.device, dtype=torch.float32).reshape(rows, -1).contiguous()
        if g.shape[1] != n_clusters:
            raise ValueError(f"gates have {g.shape[1]} clusters, n_clusters={n_clusters}")
    gu, dn = gate_up.c_struct(), down.c_struct()
    _lib.check(_lib.lib().mortar_mlp_prefill_blocks(
        C.byref(gu), C.byref(dn), _ptr(x2), x2.stride(0), rows, _ptr(g),
        g.stride(0) if g is not None else 0, int(n_clusters), _ptr(out2), out2.stride(0),
        _ptr(workspace), workspace.numel(), _stream_ptr()), "mortar_mlp_prefill_blocks")
    _count("prefill_blocks", 2)
    return out.reshape(*lead, d_model)


def quantize_rows(x: torch.Tensor):
    """Per-row symmetric int8 quantisation of bf16 activations [rows, cols] on the device:
    (q int8 [rows, cols], scale fp32 [rows]) with scale = max|row| / 127."""
    _require_cuda(x, "x")
    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise ValueError("quantize_rows takes a 2-D bfloat16 tensor")
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    rows, cols = x.shape
    ldq = (cols + 15) // 16 * 16
    q = torch.empty(rows, ldq, device=x.device, dtype=torch.int8)
    scale = torch.empty(rows, device=x.device, dtype=torch.float32)
    _lib.check(_lib.lib().mortar_quantize_rows(_ptr(x), x.stride(0), rows, cols, _ptr(q), ldq, _ptr(scale),
                                               _stream_ptr()), "mortar_quantize_rows")
    _count("quantize_rows")
    return q[:, :cols], scale


def linear_tc_i8(x: torch.Tensor, w: SchedMatrix, *, gates: Optional[torch.Tensor] = None,
                 cluster_size: int = 0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``linear_tc`` on the 8-bit tensor-core path: the bf16 activations are quantised per row to
    int8, the products run as tcgen05 kind::i8 with int32 accumulators.  NOT the reference's
    arithmetic (activation quantisation error of about 1% of an output's typical magnitude);
    opt-in only.  ``w`` is a ``SchedMatrix(..., arith="i8")``."""
    _require_cuda(x, "x")
    if x.dtype != torch.bfloat16:
        raise ValueError("linear_tc_i8 takes bfloat16 activations")
    if w.arith != "i8":
        raise ValueError("linear_tc_i8 needs a schedule built with arith='i8'")
    lead = x.shape[:-1]
    x2 = _rows2d(x, w.in_features, "x")
    rows = x2.shape[0]
    n_out = w.n_out
    if out is None:
        out = torch.empty(rows, n_out, device=x.device, dtype=torch.bfloat16)
    out2 = out.reshape(rows, n_out)
    if rows == 0:
        return out.reshape(*lead, n_out)
    q, xs = quantize_rows(x2)
    g = None
    if gates is not None:
        g = gates.to(device=x.device, dtype=torch.float32).reshape(rows, -1).contiguous()
    st = w.c_struct()
    _lib.check(_lib.lib().mortar_linear_tc_i8(C.byref(st), _ptr(q), q.stride(0), _ptr(xs), rows, _ptr(out2),
                                              out2.stride(0), _ptr(g), g.stride(0) if g is not None else 0,
                                              int(cluster_size), _stream_ptr()), "mortar_linear_tc_i8")
    _count("prefill_panel_i8")
    return out.reshape(*lead, n_out)


def mlp_prefill_tc_i8(x: torch.Tensor, gate_up: SchedMatrix, down: SchedMatrix, *,
                      gates: Optional[torch.Tensor] = None, n_clusters: int = 0) -> torch.Tensor:
    """The SwiGLU block on the 8-bit path: quantise x, gate/up product with the SwiGLU epilogue
    (bf16 hidden block), quantise the hidden block, down product.  Four launches; opt-in."""
    d_ff = gate_up.out_features // 2
    h = linear_tc_i8(x, gate_up, gates=gates, cluster_size=(d_ff // n_clusters) if gates is not None else 0)
    return linear_tc_i8(h, down)


SDD_BLOCK_MIN_ROWS = 512      # token blocks of at least this many rows take the tensor-memory block kernel


def sdd_error(reset: bool = True) -> int:
    """Error word of the block weight-gradient kernel (0 = none; synchronises the device)."""
    code = C.c_int32(0)
    _lib.check(_lib.lib().mortar_sdd_error(C.byref(code), int(reset)), "mortar_sdd_error")
    return code.value


def sdd_tiles(dy: torch.Tensor, x: torch.Tensor, topo: TopologyDev, out_dtype: torch.dtype = torch.float32,
              path: Optional[str] = None) -> torch.Tensor:
    """Weight gradient on the topology: [nnz, 16, 16] with tile (r, c) = dy[:, 16r:16r+16]^T @
    x[:, 16c:16c+16] (bf16 operands, fp32 accumulation) -- ``morph_stk::sdd_at_b`` at tile 16
    (morph/sparse/stk/backend/custom_ops.py:68-89).  ``path``: "blocks" (whole 128 x 128 blocks on
    the tensor-memory path, the default from ``SDD_BLOCK_MIN_ROWS`` rows), "tiles" (one kept tile
    per warp), None = by row count."""
    _require_cuda(dy, "dy")
    d2 = _rows2d(dy.to(torch.bfloat16), topo.tile_rows * TILE, "dy")
    x2 = _rows2d(x.to(torch.bfloat16), topo.tile_cols * TILE, "x")
    if d2.shape[0] != x2.shape[0]:
        raise ValueError("dy and x disagree on the number of rows")
    if d2.stride(0) % 8 or d2.data_ptr() % 16:
        d2 = d2.contiguous()
    if x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    out = torch.empty(topo.nnz, TILE, TILE, device=dy.device, dtype=out_dtype)
    if topo.nnz == 0:
        return out
    if d2.shape[0] == 0:
        return out.zero_()
    rows = d2.shape[0]
    if path not in (None, "blocks", "tiles"):
        raise ValueError(f"unknown path {path!r}")
    if path == "blocks" or (path is None and rows >= SDD_BLOCK_MIN_ROWS):
        # enough CTAs for two waves of the GPU, each with at least four 64-token stages
        splits = max(1, min(16, -(-2 * 148 // topo.n_blocks), rows // 256))
        scratch = None
        if splits > 1 or out_dtype != torch.float32:
            scratch = _workspace(dy.device, splits * topo.nnz * 256 * 4)
        _lib.check(_lib.lib().mortar_sdd_blocks(
            _ptr(d2), d2.stride(0), _ptr(x2), x2.stride(0), rows, topo.tile_rows * TILE, topo.tile_cols * TILE,
            _ptr(topo.blk_rc), _ptr(topo.blk_tiles), topo.n_blocks, splits, topo.nnz, _ptr(scratch),
            scratch.numel() // 4 if scratch is not None else 0, _ptr(out), _dtype_code(out), _stream_ptr()),
            "mortar_sdd_blocks")
        _count("sdd_blocks", 1 if scratch is None else 2)
        return out
    _lib.check(_lib.lib().mortar_sdd_tiles(
        _ptr(d2), d2.stride(0), _ptr(x2), x2.stride(0), d2.shape[0], _ptr(topo.row_ptr), _ptr(topo.col_idx),
        topo.tile_rows, topo.tile_cols, _ptr(topo.item_row), _ptr(topo.item_first), topo.n_items, _ptr(out),
        _dtype_code(out), _stream_ptr()), "mortar_sdd_tiles")
    _count("sdd_tiles")
    return out


def linear_error(reset: bool = True) -> int:
    """Error word of the staged / persistent paths of ``mortar_linear`` (0 = none; synchronises)."""
    code = C.c_int32(0)
    _lib.check(_lib.lib().mortar_linear_error(C.byref(code), int(reset)), "mortar_linear_error")
    return code.value


def prefill_error(reset: bool = True) -> int:
    """Error word of the tcgen05 kernel (0 = none; synchronises the device)."""
    code = C.c_int32(0)
    _lib.check(_lib.lib().mortar_prefill_error(C.byref(code), int(reset)), "mortar_prefill_error")
    return code.value


def route_flags(gates: torch.Tensor, rlo: torch.Tensor, rhi: torch.Tensor, clo: torch.Tensor,
                chi: torch.Tensor, ract: torch.Tensor, cact: torch.Tensor) -> None:
    """Same contract as the reference ``route_flags`` (fused_decode_step.py:1913-1927): gates
    [B, n_clusters] fp32; rlo/rhi [NR], clo/chi [NC] int32 cluster spans; ract [B, NR] /
    cact [B, NC] int32 outputs (may be sliced views of a wider scratch)."""
    _require_cuda(gates, "gates")
    B = gates.shape[0]
    _lib.check(_lib.lib().mortar_route_flags(
        _ptr(gates), B, gates.stride(0), _ptr(rlo), _ptr(rhi), rlo.numel(), _ptr(clo), _ptr(chi),
        clo.numel(), _ptr(ract), ract.stride(0), _ptr(cact), cact.stride(0), _stream_ptr()),
        "mortar_route_flags")
    _count("route_flags")


def route_gather(gates: torch.Tensor, cluster_size: int, units: int):
    """Per hidden tile row (16 neurons; ``units`` of them) the ascending list of rows whose gate over
    the clusters it spans is positive: returns (cnt int32 [units], rows int32 [units, n_rows]); only
    the first cnt[u] entries of rows[u] are defined.  The per-stream activity of the reference's
    decode kernel (fused_decode_step.py:1371-1390) as a schedule for a whole batch."""
    _require_cuda(gates, "gates")
    g = gates.to(torch.float32).reshape(-1, gates.shape[-1])
    if g.stride(1) != 1:
        g = g.contiguous()
    n = g.shape[0]
    cnt = torch.empty(units, device=g.device, dtype=torch.int32)
    lst = torch.empty(units, max(n, 1), device=g.device, dtype=torch.int32)
    _lib.check(_lib.lib().mortar_route_gather(_ptr(g), n, g.stride(0), int(cluster_size), int(units), _ptr(cnt),
                                              _ptr(lst), lst.stride(0), _stream_ptr()), "mortar_route_gather")
    _count("route_gather")
    return cnt, lst


ROUTER_GEMM_MIN_ROWS = 256      # token blocks of at least this many rows project through a library GEMM


def router_gates(x: torch.Tensor, router, iter_idx: int = 0, out: Optional[torch.Tensor] = None,
                 scratch: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gates [rows, n_groups] (fp32) of a ReMoE router for activations x[..., d_model]: the
    projection, LayerNorm, product-key logits and the relu(logit - k-th) * k / sum rule of
    ``TileRouter.forward`` (morph/model/routing.py:159-284) in two launches, the role of the
    reference's ``fused_router`` (morph/kernels/triton/fused_router.py:101-139) for any number of
    rows.  ``router`` is anything with the reference router's parameters (``query_proj.weight``,
    ``iter_embed``, ``query_norm``, ``sub_keys_a/b``, ``group_bias``, ``activation_k``,
    ``n_sub_keys``, ``n_tile_groups``) in fp32 on the device of x.

    Token blocks of ``ROUTER_GEMM_MIN_ROWS`` rows or more run the dense d x d projection as a
    plain library GEMM (fp32; bf16 under autocast, as ``nn.Linear`` does in the reference) and
    only the second launch of the kernel path; smaller batches run both launches."""
    _require_cuda(x, "x")
    d = router.d_model
    x2 = _rows2d(x, d, "x")
    if x2.dtype != torch.float32:
        x2 = x2.float()
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    G, nsk = int(router.n_tile_groups), int(router.n_sub_keys)
    params = [router.query_proj.weight, router.iter_embed, router.query_norm.weight, router.query_norm.bias,
              router.sub_keys_a, router.sub_keys_b, router.group_bias]
    for t in params:
        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError("router parameters must be contiguous float32 CUDA tensors")
    it = max(0, min(int(iter_idx), router.iter_embed.shape[0] - 1))
    if out is None:
        out = torch.empty(rows, G, device=x.device, dtype=torch.float32)
    if scratch is None:
        scratch = torch.empty(max(rows, 1) * d, device=x.device, dtype=torch.float32)
    if rows == 0:
        return out
    wq, n_launch = router.query_proj.weight, 2
    if rows >= ROUTER_GEMM_MIN_ROWS:
        with torch.no_grad():
            if torch.is_autocast_enabled():
                dt = torch.get_autocast_dtype("cuda")
                q = torch.nn.functional.linear(x2.to(dt), wq.detach().to(dt)).float()
                q += router.iter_embed[it]
            else:
                q = torch.addmm(router.iter_embed[it], x2, wq.detach().t())
        scratch, wq, n_launch = q.contiguous(), None, 1
    _lib.check(_lib.lib().mortar_router_gates(
        _ptr(x2), x2.stride(0), rows, d, _ptr(wq), _ptr(router.iter_embed[it]),
        _ptr(router.query_norm.weight), _ptr(router.query_norm.bias), float(router.query_norm.eps),
        _ptr(router.sub_keys_a), _ptr(router.sub_keys_b), nsk, _ptr(router.group_bias), G,
        int(router.activation_k), _ptr(scratch), _ptr(out), out.stride(0), _stream_ptr()),
        "mortar_router_gates")
    _count("router", n_launch)
    return out


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 RMSNorm over the last dim (fused_decode_step.py:305-321), evaluated by the
    activation-prep kernel and re-assembled from its three exact planes."""
    planes = act_prep(x, 3, rms_weight=weight, eps=eps)
    return planes.float().sum(0).reshape(x.shape)


# ---- reference-signature shims ---------------------------------------------------------

class MortarPack:
    """What ``mortar_pack_strips`` returns here: the stream-format matrix plus the block size
    the caller's activity flags are expressed in."""

    def __init__(self, stream: StreamMatrix, matrix: MortarMatrix, flag_blocking: int):
        self.stream, self.matrix, self.flag_blocking = stream, matrix, int(flag_blocking)
        self.out_features = matrix.out_features


def mortar_pack_strips(cms, device="cuda") -> MortarPack:
    """Counterpart of the reference ``mortar_pack_strips(cms)`` (fused_decode_step.py:1465):
    converts a carved+packed ``CMSBlockLinear`` into this library's stream layout."""
    m = MortarMatrix.from_reference_cms(cms)
    return MortarPack(m.to_stream(device), m, int(cms._mortar_blocking))


def _expand_flags(act: Optional[torch.Tensor], blocking: int, first_half: bool):
    if act is None:
        return None
    if act.dim() == 1:
        act = act.unsqueeze(0)
    if first_half:
        act = act[:, : act.shape[1] // 2]
    rep = blocking // TILE
    if rep > 1:
        act = act.repeat_interleave(rep, dim=1)
    return act.to(torch.int32).contiguous()


def mortar_gemv(x: torch.Tensor, pack: MortarPack, swiglu_x: bool = False, swiglu_out: bool = False,
                row_act: Optional[torch.Tensor] = None, col_act: Optional[torch.Tensor] = None,
                gates: Optional[torch.Tensor] = None, cluster_size: int = 0) -> torch.Tensor:
    """Same signature and result as the reference ``mortar_gemv``
    (fused_decode_step.py:1502-1547): x [B, I] fp32 -> [B, O] fp32, or [B, O/2] =
    silu(g)*u (x cluster gate) with ``swiglu_out``; ``swiglu_x`` takes the packed [B, 2F]
    gate_up output and forms silu(g)*u on load.  Activity flags are per block of the
    pack's original blocking, [B, n_blocks] or [n_blocks]."""
    if swiglu_x and swiglu_out:
        raise AssertionError("swiglu_x and swiglu_out are mutually exclusive")
    _require_cuda(x, "x")
    xf = x.float()
    if swiglu_x:
        F_ = xf.shape[-1] // 2
        g, u = xf[..., :F_], xf[..., F_:]
        xf = g * torch.sigmoid(g) * u
    planes = act_prep(xf.reshape(-1, xf.shape[-1]), 3)
    B = planes.shape[1]
    ra = _expand_flags(row_act, pack.flag_blocking, first_half=swiglu_out)
    ca = _expand_flags(col_act, pack.flag_blocking, first_half=False)
    if ra is not None and ra.shape[0] == 1 and B > 1:
        ra = ra.expand(B, -1).contiguous()
    if ca is not None and ca.shape[0] == 1 and B > 1:
        ca = ca.expand(B, -1).contiguous()
    return linear_planes(pack.stream, planes, swiglu=swiglu_out, out_dtype=torch.float32,
                         gates=gates if swiglu_out else None, cluster_size=cluster_size,
                         row_act=ra, col_act=ca)
