"""PoPE embedding module and the pure-PyTorch transform.

API-compatible with PoPE_pytorch/pope.py of the reference: ``PolarEmbedReturn`` (:18),
``apply_pope_to_qk`` (:30-86) and ``PoPE`` (:90-147) keep their names, argument order, defaults
and ``state_dict`` keys (``bias``, ``inv_freqs``).  The module only PRODUCES the inputs of the
fused kernels (a phase table and a clamped per-head phase); the kernels themselves are reached
through ``attention.py``.
"""
from __future__ import annotations

import math
from collections import namedtuple
from typing import Optional, Sequence, Union

import torch
import torch.nn.functional as F
from torch import Tensor, nn

PolarEmbedReturn = namedtuple("PolarEmbedReturn", ("freqs", "bias"))


class FactoredPolarEmbed(PolarEmbedReturn):
    """The ``(freqs, bias)`` pair of the reference (it unpacks and indexes like PolarEmbedReturn) that
    also remembers how the table was built: ``freqs[p, c] = positions[p, axis_of[c]] * inv_freqs[c]``.
    Kernels that derive their own phase tables recompute the phases from the 4-byte positions
    (bit-identical: it is the same single fp32 multiply) instead of loading the fp32 table.  The
    factors also ride on the ``freqs`` tensor itself, so they survive ``freqs, bias = pos_emb``."""

    def __new__(cls, freqs, bias, positions=None, inv_freqs=None, axis_of=None):
        self = super().__new__(cls, freqs, bias)
        self.positions, self.inv_freqs, self.axis_of = positions, inv_freqs, axis_of
        if positions is not None and freqs.ndim == 2:
            freqs._pope_factored = (positions, inv_freqs, axis_of)
        return self

TWO_PI = 2.0 * math.pi


def _interleave_polar(magnitude: Tensor, phase: Tensor) -> Tensor:
    """(.., r) magnitude and phase -> (.., 2r) laid out as [m0 cos, m0 sin, m1 cos, m1 sin, ...]."""
    pair = torch.stack((magnitude * torch.cos(phase), magnitude * torch.sin(phase)), dim=-1)
    return pair.reshape(*pair.shape[:-2], -1)


@torch.autocast("cuda", enabled=False)
def apply_pope_to_qk(pope, q: Tensor, k: Tensor, to_magnitude=F.softplus, return_complex: bool = False):
    """Expand head-first q (b,h,i,d) and k (b,hk,j,d) to their polar form of width 2r + (d - r).

    Rotated features (the first r = freqs.shape[-1]) become magnitude * (cos, sin) of the
    position phase -- plus the per-head bias on the key side -- and the remaining features pass
    through.  A query block shorter than the keys sits at the END of the position range (decode).
    Same contract as PoPE_pytorch/pope.py:30-86; runs on any device in plain PyTorch.
    """
    freqs, bias = pope
    n_q, n_k, d, r = q.shape[-2], k.shape[-2], q.shape[-1], freqs.shape[-1]
    assert n_q <= n_k and r <= d

    if to_magnitude is F.softplus and not return_complex:
        from . import _native          # CUDA tensors: one fused pass in the native library (no fallback when it is present)
        if _native.apply_qk_supported(q, k, freqs, bias):
            return _native.apply_qk(q, k, freqs, bias)

    if freqs.ndim == 3:                       # (b, n, r) -> (b, 1, n, r)
        freqs = freqs.unsqueeze(1)
    key_phase = freqs + bias.unsqueeze(-2)    # (.., h, n, r)
    query_phase = freqs.narrow(-2, freqs.shape[-2] - n_q, n_q)

    q_mag, k_mag = to_magnitude(q[..., :r]), to_magnitude(k[..., :r])
    q_rest, k_rest = q[..., r:], k[..., r:]

    if return_complex:
        q_out, k_out = torch.polar(q_mag, query_phase.expand_as(q_mag).contiguous()), \
            torch.polar(k_mag, key_phase.expand_as(k_mag).contiguous())
        if r < d:
            q_out = torch.cat((q_out, torch.polar(q_rest, torch.zeros_like(q_rest))), dim=-1)
            k_out = torch.cat((k_out, torch.polar(k_rest, torch.zeros_like(k_rest))), dim=-1)
        return q_out, k_out

    q_out, k_out = _interleave_polar(q_mag, query_phase), _interleave_polar(k_mag, key_phase)
    if r < d:
        q_out = torch.cat((q_out, q_rest), dim=-1)
        k_out = torch.cat((k_out, k_rest), dim=-1)
    return q_out, k_out


class PoPE(nn.Module):
    """Polar positional embedding: one frequency per rotated feature, theta^(-c/dim), and a
    learned per-head key phase kept in [-2pi, 0]."""

    apply_pope_to_qk = staticmethod(apply_pope_to_qk)

    def __init__(self, dim: int, *, heads: int, theta: float = 10000, bias_uniform_init: bool = False,
                 inv_freqs: Optional[Union[Tensor, Sequence[float]]] = None):
        super().__init__()
        if inv_freqs is None:
            inv_freqs = theta ** -(torch.arange(dim).float() / dim)
        elif not torch.is_tensor(inv_freqs):
            inv_freqs = torch.tensor(inv_freqs, dtype=torch.float32)
        self.register_buffer("inv_freqs", inv_freqs)
        self.bias = nn.Parameter(torch.zeros(heads, dim))
        if bias_uniform_init:
            with torch.no_grad():
                self.bias.uniform_(-TWO_PI, 0.0)

    @property
    def device(self):
        return self.inv_freqs.device

    @torch.autocast("cuda", enabled=False)
    def forward(self, pos_or_seq_len: Union[Tensor, int], offset=0) -> PolarEmbedReturn:
        if torch.is_tensor(pos_or_seq_len):
            positions = pos_or_seq_len
        else:
            positions = torch.arange(pos_or_seq_len, device=self.device, dtype=self.inv_freqs.dtype)
        positions = positions + offset
        freqs = positions.unsqueeze(-1) * self.inv_freqs          # (..., n, dim)
        bias = self.bias.clamp(-TWO_PI, 0.0)
        if positions.ndim == 1 and positions.dtype == torch.float32 and self.inv_freqs.dtype == torch.float32:
            return FactoredPolarEmbed(freqs, bias, positions.contiguous(), self.inv_freqs.contiguous())
        return PolarEmbedReturn(freqs, bias)
