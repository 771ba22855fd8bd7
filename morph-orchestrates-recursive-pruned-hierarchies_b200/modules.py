"""Drop-in mirrors of the reference's module API for the carved MLP
(morph/model/sparsity.py:33-166 ``MortarLinear``; morph/model/transformer.py:319-431
``_SwiGLUMortar``).  Same attribute names, argument meaning and error behaviour; the
forward runs the sm_100a kernels of this package.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from . import ops
from .format import TILE, MortarMatrix, StreamMatrix


class MortarLinear(nn.Module):
    """Carved (post-``carve``) ``MortarLinear``: y = x @ W^T over the kept 16x16 ternary
    tiles.  Built from a canonical matrix or from a reference layer with ``from_reference``;
    the dense pre-carve phase belongs to training and is not part of this package."""

    def __init__(self, matrix: MortarMatrix, bias: Optional[torch.Tensor] = None,
                 tile_size: int = TILE, device="cuda"):
        super().__init__()
        if tile_size != TILE:
            raise ValueError(f"tile_size must be {TILE}")
        self.in_features = matrix.in_features
        self.out_features = matrix.out_features
        self.tile_size = tile_size
        self.matrix = matrix
        self.stream: StreamMatrix = matrix.to_stream(device)
        # the stream tensors ride state_dict as buffers
        self.register_buffer("mortar_grp_ptr", self.stream.grp_ptr)
        self.register_buffer("mortar_grp_cols", self.stream.grp_cols)
        self.register_buffer("mortar_grp_codes", self.stream.grp_codes)
        self.register_buffer("mortar_scale", torch.tensor(matrix.scale, dtype=torch.float32))
        if bias is not None:
            self._bias = nn.Parameter(bias.detach().to(device))
        else:
            self.register_parameter("_bias", None)

    @classmethod
    def from_reference(cls, layer, device="cuda") -> "MortarLinear":
        """`layer` is a reference ``MortarLinear`` or its ``CMSBlockLinear`` after carve()."""
        cms = getattr(layer, "_cms", layer)
        return cls(MortarMatrix.from_reference_cms(cms), bias=cms.bias, device=device)

    @property
    def is_compact(self) -> bool:
        return True

    @property
    def bias(self):
        return self._bias

    def carve(self, blocking: int = 128) -> int:
        raise AssertionError("carve() already applied")

    def get_density(self) -> float:
        return self.matrix.density

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = ops.linear(x, self.stream)
        if self._bias is not None:
            y = y + self._bias.to(y.dtype)
        return y

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, tile={self.tile_size}, "
                f"density={self.get_density():.2f}, mode=mortar")


class SwiGLUMortar(nn.Module):
    """``_SwiGLUMortar``: gate_up -> chunk (gate first) -> silu(gate)*up -> [* cluster
    gates] -> down, evaluated by the fused kernels.  bf16 inputs follow the reference's
    autocast rounding points; fp32 inputs follow the decode engine's fp32 algebra."""

    def __init__(self, gate_up: MortarMatrix, down: MortarMatrix, device="cuda"):
        super().__init__()
        if gate_up.out_features != 2 * down.in_features or gate_up.in_features != down.out_features:
            raise ValueError("gate_up must be [2*d_ff, d_model] and down [d_model, d_ff]")
        self.d_model = gate_up.in_features
        self.d_ff = down.in_features
        self.gate_up = MortarLinear(gate_up, device=device)
        self.down = MortarLinear(down, device=device)
        self.router: Optional[nn.Module] = None
        self.n_clusters = 0
        self._last_aux_loss = None
        self._aux_detach_input = True

    @classmethod
    def from_reference(cls, mlp, device="cuda") -> "SwiGLUMortar":
        """`mlp` is a carved reference ``_SwiGLUMortar`` (its router, if any, is reused)."""
        new = cls(MortarMatrix.from_reference_cms(mlp.gate_up._cms),
                  MortarMatrix.from_reference_cms(mlp.down._cms), device=device)
        if getattr(mlp, "router", None) is not None:
            new.attach_router(mlp.router.to(device), int(mlp.n_clusters))
        return new

    def attach_router(self, router: nn.Module, n_clusters: int) -> None:
        """`router(x, iter_idx=...) -> (gates[..., n_clusters], aux)` as ``TileRouter.forward``
        (morph/model/routing.py:159)."""
        self.router = router
        self.n_clusters = int(n_clusters)
        base, rem = divmod(self.d_ff, self.n_clusters)
        sizes = torch.tensor([base + (1 if c < rem else 0) for c in range(self.n_clusters)])
        h2c = torch.repeat_interleave(torch.arange(self.n_clusters), sizes)
        self.register_buffer("hidden_to_cluster", h2c.to(self.gate_up.mortar_grp_ptr.device))

    def enable_routing(self, n_clusters: int = 16, activation_ratio: float = 0.5,
                       aux_loss_coeff: float = 1e-2, n_iters: int = 1, n_sub_keys: int = 0,
                       detach_input: bool = True) -> None:
        from .router import TileRouter
        self._aux_detach_input = bool(detach_input)
        dev = self.gate_up.mortar_grp_ptr.device
        self.attach_router(TileRouter(n_clusters, self.d_model, activation_ratio, n_sub_keys,
                                      aux_loss_coeff, n_iters).to(dev), n_clusters)

    def forward(self, x: torch.Tensor, iter_idx: int = 0) -> torch.Tensor:
        gates = None
        if self.router is not None:
            if self.d_ff % self.n_clusters:
                raise NotImplementedError("uneven clusters are not supported by the fused kernels")
            _rx = x.detach() if self._aux_detach_input else x
            gates, aux = self.router(_rx, iter_idx=iter_idx)
            self._last_aux_loss = aux
        if x.dtype == torch.bfloat16:
            return ops.mlp_prefill(x, self.gate_up.stream, self.down.stream, gates=gates,
                                   n_clusters=self.n_clusters)
        return ops.mlp_decode(x, self.gate_up.stream, self.down.stream, gates=gates,
                              n_clusters=self.n_clusters, n_planes=3)
