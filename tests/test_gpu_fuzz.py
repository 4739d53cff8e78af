"""Randomised shapes through the tensor-core attention kernels, forward and backward, against the exact-arithmetic CUDA
family fed the same 16-bit inputs as fp32: ragged lengths, Nq < Nk, grouped heads, key-padding masks, every head width
and rotate width the tensor-core family takes.  Tolerance: 3e-2 of the largest entry (16-bit operands and outputs)."""
import random

import pytest
import torch

from pope_pytorch_b200 import PoPE, _native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cases(seed, count):
    rnd = random.Random(seed)
    out = []
    for it in range(count):
        d = rnd.choice([64, 96, 128])
        r = rnd.choice([x for x in (0, 16, 32, 64, 96, 128) if x <= d])
        hk = rnd.choice([1, 2, 4])
        h = hk * rnd.choice([1, 1, 2, 4])
        b = rnd.choice([1, 2, 3])
        nk = rnd.choice([64, 100, 128, 129, 200, 256, 257, 384, 500, 640, 1000, 1536])
        nq = min(nk, rnd.choice([nk, nk, max(64, nk // 2), max(64, nk - 37)]))
        out.append((it, b, h, hk, nq, nk, d, r, rnd.random() < 0.6, rnd.random() < 0.4,
                    rnd.choice([torch.bfloat16, torch.bfloat16, torch.float16])))
    return out


@pytest.mark.parametrize("it,b,h,hk,nq,nk,d,r,causal,masked,dtype", _cases(1, 24))
def test_random_shape_tc_vs_exact_family(it, b, h, hk, nq, nk, d, r, causal, masked, dtype):
    gen = torch.Generator().manual_seed(it)
    q = torch.randn(b, h, nq, d, generator=gen).to(dtype)
    k, v = (torch.randn(b, hk, nk, d, generator=gen).to(dtype) for _ in range(2))
    do = torch.randn(b, h, nq, d, generator=gen).to(dtype)
    if r > 0:
        freqs = PoPE(r, heads=hk)(nk).freqs.detach().contiguous().to(DEV)
        bias = (-torch.rand(hk, r, generator=gen) * 6).to(DEV)
    else:
        freqs, bias = torch.empty(nk, 0, device=DEV), torch.empty(hk, 0, device=DEV)
    mask = None
    if masked:
        mask = torch.rand(b, nk, generator=gen) > 0.3
        mask[:, 0] = True
        mask = mask.to(DEV)
    scale = d ** -0.5

    def run(dt):
        qq, kk, vv, dd = (t.to(DEV).to(dt) for t in (q, k, v, do))
        out, lse = _native.attn_forward(qq, kk, vv, freqs, bias, mask, causal, scale)
        path = _native.last_path()
        grads = _native.attn_backward(dd, qq, kk, vv, out, lse, freqs, bias, mask, causal, scale, False, r > 0)
        return out, lse, grads, path, _native.last_path()

    out, lse, grads, p_fwd, p_bwd = run(dtype)
    ref_out, ref_lse, ref_grads, _, _ = run(torch.float32)
    assert p_fwd == "tcgen05" and p_bwd == "tcgen05"
    assert _native.device_status() == 0

    def rel(a, ref):
        return float((a.float() - ref.float()).abs().max()) / max(1.0, float(ref.float().abs().max()))

    assert rel(out, ref_out) < 3e-2
    finite = torch.isfinite(ref_lse)
    assert torch.equal(torch.isfinite(lse), finite)
    if finite.any():
        assert float((lse[finite] - ref_lse[finite]).abs().max()) < 3e-2
    for name, a, ref in zip(("dq", "dk", "dv", "dfreqs", "dbias"), grads, ref_grads):
        if a is not None and ref is not None and a.numel():
            assert rel(a, ref) < 3e-2, name
