"""Sharding of PoPE attention over the GPUs of one box.

The (batch, head) units of attention are independent in forward and backward (every reference
kernel indexes one (b, h) per program: PoPE_pytorch/triton_pope_flash_attn.py:38-39,145-146),
so ranks take disjoint blocks of units and the attention path needs NO collective.  Outputs
stay resident on their rank.  Two optional exchanges exist around the path:
  * gather_units      -- all-gather the per-rank outputs when a caller wants the full tensor
  * reduce_bias_grad  -- the phase-bias gradient sums over the batch
                         (triton_pope_flash_attn.py:210); when the shard cuts the batch axis each rank
                         holds a partial (H, r) sum that one small all-reduce completes
One process per GPU; the process group is whatever torch.distributed backend the caller
initialised (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .attention import flash_attn_with_pope


@dataclass(frozen=True)
class ShardPlan:
    axis: str          # "heads" or "batch"
    world: int
    rank: int
    start: int         # first index of this rank's block along `axis`
    size: int          # block length

    @property
    def dim(self) -> int:
        return 1 if self.axis == "heads" else 0


def plan_shard(batch: int, heads: int, kv_heads: int, rank: int, world: int) -> ShardPlan:
    """Cut the head axis when every rank can own whole query AND key heads, else the batch axis."""
    if world == 1:
        return ShardPlan("heads", 1, 0, 0, heads)
    if heads % world == 0 and kv_heads == heads:
        size = heads // world
        return ShardPlan("heads", world, rank, rank * size, size)
    if batch % world == 0:
        size = batch // world
        return ShardPlan("batch", world, rank, rank * size, size)
    raise ValueError(f"cannot split batch={batch} x heads={heads} (kv heads {kv_heads}) evenly over {world} ranks")


def take_block(t: Optional[torch.Tensor], plan: ShardPlan, dim: int) -> Optional[torch.Tensor]:
    return None if t is None else t.narrow(dim, plan.start, plan.size)


def shard_attention_inputs(q, k, v, pos_emb, mask, plan: ShardPlan):
    """Views of this rank's block: q/k/v (b,h,n,d) head-first, bias rows with the heads, the
    key-padding mask with the batch.  A batched (b,n,r) / (b,h,n,r) phase table follows its axes."""
    freqs, bias = pos_emb
    ql, kl, vl = (take_block(t, plan, plan.dim) for t in (q, k, v))
    if plan.axis == "heads":
        bias_l = take_block(bias, plan, 0)
        freqs_l = take_block(freqs, plan, 1) if freqs.ndim == 4 and freqs.shape[1] > 1 else freqs
        mask_l = mask
    else:
        bias_l = bias
        freqs_l = take_block(freqs, plan, 0) if freqs.ndim >= 3 and freqs.shape[0] > 1 else freqs
        mask_l = take_block(mask, plan, 0)
    return ql, kl, vl, (freqs_l, bias_l), mask_l


def sharded_flash_attn(q, k, v, pos_emb, mask=None, causal=False, softmax_scale=None, *, rank: int, world: int,
                       fused=None) -> Tuple[torch.Tensor, ShardPlan]:
    """Run this rank's block of units.  q, k, v are the FULL head-first tensors (or any tensors of
    the full shape whose local block is valid on this rank); returns (local_out, plan)."""
    plan = plan_shard(q.shape[0], q.shape[1], k.shape[1], rank, world)
    ql, kl, vl, emb_l, mask_l = shard_attention_inputs(q, k, v, pos_emb, mask, plan)
    out = flash_attn_with_pope(ql, kl, vl, pos_emb=emb_l, mask=mask_l, causal=causal, softmax_scale=softmax_scale,
                               fused=fused)
    return out, plan


def gather_units(local: torch.Tensor, plan: ShardPlan, group=None) -> torch.Tensor:
    """All-gather the per-rank blocks back into the full tensor (only when a caller asks for it)."""
    if plan.world == 1:
        return local
    parts = [torch.empty_like(local.contiguous()) for _ in range(plan.world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=plan.dim)


def reduce_bias_grad(dbias_local: torch.Tensor, plan: ShardPlan, group=None) -> torch.Tensor:
    """Complete the (H, r) phase-bias gradient: sum over ranks when the batch was cut, concatenate
    the per-rank head rows when the heads were cut."""
    if plan.world == 1:
        return dbias_local
    if plan.axis == "batch":
        total = dbias_local.clone()
        dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
        return total
    parts = [torch.empty_like(dbias_local.contiguous()) for _ in range(plan.world)]
    dist.all_gather(parts, dbias_local.contiguous(), group=group)
    return torch.cat(parts, dim=0)
