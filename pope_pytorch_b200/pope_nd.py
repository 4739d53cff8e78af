"""Axial (N-d) PoPE: each grid axis owns a slice of the rotated features.

API-compatible with PoPE_pytorch/pope_nd.py:23-106 of the reference, including the
``state_dict`` keys (``bias``, ``inv_freqs.<axis>``).  The resulting phase table is dense and not
an outer product of one position vector, which is why the kernels take ``freqs`` as an opaque
table.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch
from torch import Tensor, nn

from .pope import TWO_PI, FactoredPolarEmbed, PolarEmbedReturn, apply_pope_to_qk


class AxialPoPE(nn.Module):
    apply_pope_to_qk = staticmethod(apply_pope_to_qk)

    def __init__(self, dim: int, *, heads: int, axial_dims: Optional[Tuple[int, ...]] = None, theta: float = 10000,
                 bias_uniform_init: bool = False):
        super().__init__()
        axial_dims = (dim,) if axial_dims is None else tuple(axial_dims)
        assert sum(axial_dims) == dim, f"sum of axial_dims {axial_dims} must be equal to dim {dim}"
        self.dim, self.heads, self.axial_dims = dim, heads, axial_dims
        self.inv_freqs = nn.ParameterList(
            nn.Parameter(theta ** -(torch.arange(n).float() / n), requires_grad=False) for n in axial_dims)
        self.bias = nn.Parameter(torch.zeros(heads, dim))
        if bias_uniform_init:
            with torch.no_grad():
                self.bias.uniform_(-TWO_PI, 0.0)

    @property
    def device(self):
        return self.bias.device

    @staticmethod
    def get_grid_positions(*dims: int, device=None) -> Tensor:
        """All grid points, row-major over ``dims``; column 0 holds the LAST (fastest) axis."""
        coords = torch.cartesian_prod(*[torch.arange(n, device=device).float() for n in dims])
        if len(dims) == 1:
            coords = coords.unsqueeze(-1)
        return coords.flip(-1)

    @torch.autocast("cuda", enabled=False)
    def forward(self, pos_or_dims: Union[Tensor, Tuple[int, ...]]) -> PolarEmbedReturn:
        positions = self.get_grid_positions(*pos_or_dims, device=self.device) \
            if isinstance(pos_or_dims, tuple) else pos_or_dims
        assert positions.shape[-1] == len(self.axial_dims)
        per_axis = [positions[..., axis, None] * inv for axis, inv in enumerate(self.inv_freqs)]
        freqs, bias = torch.cat(per_axis, dim=-1), self.bias.clamp(-TWO_PI, 0.0)
        if positions.ndim == 2 and positions.dtype == torch.float32:
            axis_of = torch.cat([torch.full((n,), axis, dtype=torch.int32, device=freqs.device)
                                 for axis, n in enumerate(self.axial_dims)])
            inv_flat = torch.cat([inv.detach().float() for inv in self.inv_freqs])
            return FactoredPolarEmbed(freqs, bias, positions.contiguous(), inv_flat, axis_of)
        return PolarEmbedReturn(freqs, bias)
