"""Dispatchers with the signatures of PoPE_pytorch/attention.py:30-145.

CUDA tensors go to the sm_100a kernels in libpope_b200.so through ``_native`` (there is no
Triton, no second backend and no silent fallback: a CUDA call without a loadable library
raises).  CPU tensors keep the reference's behaviour of running the pure-PyTorch composition,
as does an explicit ``fused=False``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _native
from .pope import apply_pope_to_qk

# Name kept from the reference (PoPE_pytorch/attention.py:21-26), where it reports whether the
# fused kernels can be imported.  Here it reports whether the native library is present.
TRITON_AVAILABLE = _native.is_available()
NATIVE_AVAILABLE = TRITON_AVAILABLE


def _repeat_heads(t, groups):
    """Group-major repeat: query head g*Hk + h uses key head h."""
    return t if groups == 1 else t.repeat(1, groups, 1, 1)


def _head_first(t, head_dimension_at_first):
    return t if head_dimension_at_first else t.transpose(1, 2)


def compute_attn_similarity_non_fused(q, k, pope, head_dimension_at_first=True):
    """Pure-PyTorch similarity: expand with apply_pope_to_qk, then q' k'^T."""
    q, k = _head_first(q, head_dimension_at_first), _head_first(k, head_dimension_at_first)
    q, k = apply_pope_to_qk(pope, q, k, to_magnitude=F.softplus)
    k = _repeat_heads(k, q.shape[1] // k.shape[1])
    return torch.einsum("bhid,bhjd->bhij", q, k)


def compute_attn_similarity(q, k, pope, allow_tf32=True, head_dimension_at_first=True):
    """sim (b, h, i, j) = <q'_i, k'_j> without materialising the expanded operands.

    No scale, mask or softmax is applied.  ``allow_tf32`` is accepted for compatibility; the
    native kernel always meets fp32 accuracy.
    """
    head_axis = 1 if head_dimension_at_first else 2
    assert q.shape[head_axis] % k.shape[head_axis] == 0
    freqs, bias = pope
    head_dim = q.shape[-1]
    assert head_dim in {32, 48, 64, 128, 256}, f"head_dim {head_dim} not in common sizes"

    if q.is_cuda and k.is_cuda and freqs.is_cuda and bias.is_cuda:
        q, k = _head_first(q, head_dimension_at_first), _head_first(k, head_dimension_at_first)
        return _native.similarity(q, k, freqs, bias, allow_tf32)
    return compute_attn_similarity_non_fused(q, k, pope, head_dimension_at_first=head_dimension_at_first)


def flash_attn_with_pope(q, k, v, pos_emb=None, mask=None, causal=False, softmax_scale=None, fused=None,
                         head_dimension_at_first=True):
    """PoPE attention.  q, k, v are (b, h, n, d) -- or (b, n, h, d) with
    ``head_dimension_at_first=False``; both layouts are read in place.  ``mask`` is a (b, n_k)
    boolean key-padding mask, True = keep; ``causal`` is top-left aligned; the default scale is
    d^-0.5 of the ORIGINAL head dim."""
    if fused is None:
        fused = q.is_cuda
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    freqs, bias = pos_emb

    if fused:
        qh, kh, vh = (_head_first(t, head_dimension_at_first) for t in (q, k, v))
        out = _native.flash_attn(qh, kh, vh, freqs, bias, mask=mask, causal=causal, softmax_scale=softmax_scale)
        return _head_first(out, head_dimension_at_first)

    # pure-PyTorch composition (reference: attention.py:106-145)
    qh, kh, vh = (_head_first(t, head_dimension_at_first) for t in (q, k, v))
    qe, ke = apply_pope_to_qk(pos_emb, qh, kh, to_magnitude=F.softplus)
    groups = qe.shape[1] // ke.shape[1]
    ke, vh = _repeat_heads(ke, groups), _repeat_heads(vh, groups)
    out = F.scaled_dot_product_attention(qe, ke, vh.to(qe.dtype),
                                         attn_mask=None if mask is None else mask[:, None, None, :],
                                         is_causal=causal, scale=softmax_scale).to(v.dtype)
    return _head_first(out, head_dimension_at_first)
