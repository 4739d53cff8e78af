"""CPU oracle for the PoPE hot path.  TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch CPU code, the algorithm of the reference
project's pure-PyTorch path (lucidrains/PoPE-pytorch v0.0.15).  It exists so the CUDA
kernels can be checked against it.  Only the test-suite, the smoke check and the CPU
baseline leg of the benchmark may import it; no product code path does.

Parity pin: every function here is compared against outputs of the reference package
itself (imported with a stand-in for its one missing third-party helper) by
``tests/golden/make_golden.py``; the resulting vectors are committed under
``tests/golden/`` and re-checked by ``tests/test_oracle_golden.py``.

Each function cites the reference file:line it follows (paths inside the reference
project).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


# --------------------------------------------------------------------------------------
# producing (freqs, bias)
# --------------------------------------------------------------------------------------

def pope_inv_freqs(dim: int, theta: float = 10000.0) -> torch.Tensor:
    """One inverse frequency per rotated feature: theta^(-c/dim).  PoPE_pytorch/pope.py:106-107."""
    return theta ** -(torch.arange(dim).float() / dim)


def pope_freqs(positions: torch.Tensor, inv_freqs: torch.Tensor, offset: float = 0) -> torch.Tensor:
    """freqs[..., i, c] = (pos[..., i] + offset) * inv_freq[c].  PoPE_pytorch/pope.py:131-141."""
    pos = positions + offset
    return pos[..., :, None] * inv_freqs


def pope_clamped_bias(bias_param: torch.Tensor) -> torch.Tensor:
    """The learned per-head phase is clamped to [-2pi, 0] on every forward.  PoPE_pytorch/pope.py:145."""
    return bias_param.clamp(-2.0 * math.pi, 0.0)


def axial_grid_positions(*dims: int) -> torch.Tensor:
    """Flattened 'ij' mesh with the axes reversed, so column 0 is the fastest-varying
    (last) grid axis.  PoPE_pytorch/pope_nd.py:65-68."""
    axes = [torch.arange(d).float() for d in dims]
    grid = torch.meshgrid(*axes, indexing="ij")
    return torch.stack([g.flatten() for g in reversed(grid)], dim=-1)


def axial_freqs(positions: torch.Tensor, axial_dims: Sequence[int], theta: float = 10000.0) -> torch.Tensor:
    """Per-axis pos x inv_freq tables concatenated along features.  PoPE_pytorch/pope_nd.py:48-52,88-100."""
    assert positions.shape[-1] == len(axial_dims)
    parts = []
    for axis, adim in enumerate(axial_dims):
        inv = pope_inv_freqs(adim, theta)
        parts.append(positions[..., axis, None] * inv)
    return torch.cat(parts, dim=-1)


# --------------------------------------------------------------------------------------
# the transform
# --------------------------------------------------------------------------------------

def apply_pope(freqs: torch.Tensor, bias: torch.Tensor, q: torch.Tensor, k: torch.Tensor
               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Expanded q', k' of width 2r + (d - r), head-first layout (b, h, n, d).

    Follows PoPE_pytorch/pope.py:37-86 step by step: split rotated / pass-through
    features (:43-47); a 3-D freqs table gets a head axis (:53-54); the key phase is
    freqs + bias[h] (:56); magnitudes are softplus (:60); queries use the TRAILING q_len
    rows of freqs (:64); each rotated feature becomes the interleaved pair
    (a cos, a sin) (:69-70, :77-78); pass-through features are appended (:82-84).
    """
    q_len, k_len, d, r = q.shape[-2], k.shape[-2], q.shape[-1], freqs.shape[-1]
    assert q_len <= k_len and r <= d

    q_rot, q_rest = q[..., :r], q[..., r:]
    k_rot, k_rest = k[..., :r], k[..., r:]

    if freqs.ndim == 3:
        freqs = freqs[:, None]
    key_phase = freqs + bias[:, None, :]

    aq, ak = F.softplus(q_rot), F.softplus(k_rot)

    n_rows = freqs.shape[-2]
    query_phase = freqs[..., n_rows - q_len:, :]

    def polar(mag, phase):
        pair = torch.stack((mag * phase.cos(), mag * phase.sin()), dim=-1)
        return pair.flatten(-2)

    q_out, k_out = polar(aq, query_phase), polar(ak, key_phase)
    if r < d:
        q_out = torch.cat((q_out, q_rest.expand(*q_out.shape[:-1], d - r)), dim=-1)
        k_out = torch.cat((k_out, k_rest.expand(*k_out.shape[:-1], d - r)), dim=-1)
    return q_out, k_out


def _repeat_kv_heads(t: torch.Tensor, groups: int) -> torch.Tensor:
    """Grouped-query repeat, group-major: query head g*Hk + h reads key head h.
    PoPE_pytorch/attention.py:44-45,118-120."""
    if groups == 1:
        return t
    return t.repeat(1, groups, *([1] * (t.ndim - 2)))


# --------------------------------------------------------------------------------------
# similarity and attention
# --------------------------------------------------------------------------------------

def similarity(q: torch.Tensor, k: torch.Tensor, freqs: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """sim[b,h,i,j] = <q'_i, k'_j>; no scale, no mask, no softmax.  PoPE_pytorch/attention.py:30-47."""
    qe, ke = apply_pope(freqs, bias, q, k)
    ke = _repeat_kv_heads(ke, qe.shape[1] // ke.shape[1])
    return torch.einsum("bhid,bhjd->bhij", qe, ke)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, freqs: torch.Tensor, bias: torch.Tensor,
              mask: Optional[torch.Tensor] = None, causal: bool = False,
              softmax_scale: Optional[float] = None, return_lse: bool = False):
    """PoPE attention on head-first (b, h, n, d) tensors in the dtype of the inputs
    (tests pass fp32 copies of the rounded low-precision inputs).

    apply_pope (above) -> einsum -> * softmax_scale (default d^-0.5 with d the ORIGINAL
    head dim, PoPE_pytorch/attention.py:88) -> key-padding mask, True = keep
    (attention.py:129-131) and/or TOP-LEFT aligned causal mask (the alignment of
    F.scaled_dot_product_attention's is_causal used at attention.py:133-138 and of the
    fused kernel, triton_pope_flash_attn.py:64,87) -> softmax -> einsum with v.
    A row with no visible key yields zeros (triton_pope_flash_attn.py:96-98,114).
    The reference's SDPA call cannot take mask and is_causal together, hence the explicit
    composition here.
    """
    d = q.shape[-1]
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    qe, ke = apply_pope(freqs, bias, q, k)
    groups = qe.shape[1] // ke.shape[1]
    ke, vv = _repeat_kv_heads(ke, groups), _repeat_kv_heads(v, groups)
    s = torch.einsum("bhid,bhjd->bhij", qe, ke) * scale
    nq, nk = s.shape[-2:]
    visible = torch.ones(nq, nk, dtype=torch.bool)
    if causal:
        visible = torch.tril(visible)
    visible = visible[None, None]
    if mask is not None:
        visible = visible & mask[:, None, None, :].bool()
    s = s.masked_fill(~visible, float("-inf"))
    row_max = s.amax(dim=-1, keepdim=True)
    row_max = torch.where(torch.isinf(row_max), torch.zeros_like(row_max), row_max)
    p = torch.exp(s - row_max)
    denom = p.sum(dim=-1, keepdim=True)
    attn = p / torch.where(denom == 0, torch.ones_like(denom), denom)
    out = torch.einsum("bhij,bhjd->bhid", attn, vv.to(attn.dtype))
    if return_lse:
        lse = (row_max + torch.log(denom)).squeeze(-1)
        return out, lse
    return out


def attention_with_grads(q, k, v, freqs, bias, dout, mask=None, causal=False, softmax_scale=None,
                         want_dfreqs: bool = False):
    """Forward + autograd backward of ``attention`` in fp32.  Returns a dict with out, dq,
    dk, dv, dbias (and dfreqs).  Gradient definitions match what
    triton_pope_flash_attn.py:199-210 accumulates."""
    q, k, v = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    freqs = freqs.detach().float().requires_grad_(want_dfreqs)
    bias = bias.detach().float().requires_grad_(True)
    out = attention(q, k, v, freqs, bias, mask=mask, causal=causal, softmax_scale=softmax_scale)
    out.backward(dout.float())
    res = dict(out=out.detach(), dq=q.grad, dk=k.grad, dv=v.grad, dbias=bias.grad)
    if want_dfreqs:
        res["dfreqs"] = freqs.grad
    return res


def similarity_with_grads(q, k, freqs, bias, dsim, want_dfreqs: bool = False):
    """Forward + autograd backward of ``similarity`` (what triton_pope.py:290-362 returns)."""
    q, k = (t.detach().float().requires_grad_(True) for t in (q, k))
    freqs = freqs.detach().float().requires_grad_(want_dfreqs)
    bias = bias.detach().float().requires_grad_(True)
    sim = similarity(q, k, freqs, bias)
    sim.backward(dsim.float())
    res = dict(sim=sim.detach(), dq=q.grad, dk=k.grad, dbias=bias.grad)
    if want_dfreqs:
        res["dfreqs"] = freqs.grad
    return res
