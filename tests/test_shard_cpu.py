"""World-size-2 gloo test of the batch x heads sharding around the attention path (CPU)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import pope_oracle as O
from pope_pytorch_b200 import PoPE
from pope_pytorch_b200 import shard as S


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(b, h, hk, n, d, r):
    g = torch.Generator().manual_seed(123)
    q = torch.randn(b, h, n, d, generator=g)
    k, v = torch.randn(b, hk, n, d, generator=g), torch.randn(b, hk, n, d, generator=g)
    do = torch.randn(b, h, n, d, generator=g)
    freqs = PoPE(r, heads=hk)(n).freqs
    bias = -torch.rand(hk, r, generator=g) * 6
    lens = torch.tensor([n, n - 5][:b] + [n] * max(0, b - 2))
    mask = torch.arange(n)[None, :] < lens[:, None]
    return q, k, v, do, freqs, bias, mask


def _worker(rank, world, port, shape, out_dir):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, k, v, do, freqs, bias, mask = _inputs(*shape)
        bias = bias.clone().requires_grad_(True)
        q = q.clone().requires_grad_(True)
        out, plan = S.sharded_flash_attn(q, k, v, (freqs, bias), mask=mask, causal=False, rank=rank, world=world,
                                         fused=False)
        out.backward(S.take_block(do, plan, plan.dim))
        full = S.gather_units(out.detach(), plan)
        dbias_local = bias.grad if plan.axis == "batch" else S.take_block(bias.grad, plan, 0)
        dbias = S.reduce_bias_grad(dbias_local, plan)
        if rank == 0:
            torch.save(dict(out=full, dbias=dbias, axis=plan.axis, dq=q.grad), os.path.join(out_dir, "r0.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("shape,axis", [((2, 4, 4, 24, 32, 16), "heads"), ((2, 3, 3, 24, 32, 16), "batch"),
                                        ((2, 4, 2, 24, 32, 16), "batch")])
def test_two_rank_shard_matches_single_process(tmp_path, shape, axis):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, shape, str(tmp_path)), nprocs=2, join=True)
    got = torch.load(os.path.join(tmp_path, "r0.pt"))
    assert got["axis"] == axis
    q, k, v, do, freqs, bias, mask = _inputs(*shape)
    ref = O.attention_with_grads(q, k, v, freqs, bias, do, mask=mask)
    assert torch.allclose(got["out"], ref["out"], atol=2e-5)
    assert torch.allclose(got["dbias"], ref["dbias"], atol=1e-4, rtol=1e-4)


def test_plan_rejects_uneven_split():
    with pytest.raises(ValueError):
        S.plan_shard(3, 5, 5, 0, 2)
    p = S.plan_shard(8, 32, 32, 3, 8)
    assert (p.axis, p.start, p.size) == ("heads", 12, 4)
