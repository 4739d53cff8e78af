"""The tcgen05 / TMEM kernels: they are the path taken for the benchmark shapes, they agree
with the exact-arithmetic CUDA family on full-size inputs, and their bounded waits never fired."""
import os

import pytest
import torch

from pope_pytorch_b200 import PoPE, _native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _fwd(q, k, v, emb, mask, causal, force_simt):
    os.environ["POPE_B200_FORCE_SIMT"] = "1" if force_simt else "0"
    try:
        out, lse = _native.attn_forward(q, k, v, emb[0], emb[1], mask, causal, q.shape[-1] ** -0.5)
        return out, lse, _native.last_path()
    finally:
        os.environ["POPE_B200_FORCE_SIMT"] = "0"


@pytest.mark.parametrize("b,h,n,d,r,causal,masked,dtype", [
    (2, 8, 1024, 64, 32, True, True, torch.bfloat16),      # forward config: causal + key padding
    (1, 4, 4096, 128, 128, True, False, torch.bfloat16),   # training shape (4 of its 64 units)
    (2, 8, 2048, 96, 96, False, False, torch.bfloat16),    # axial video shape
    (1, 2, 8192, 128, 64, True, False, torch.bfloat16),    # long-context shape, shortened
    (2, 2, 300, 64, 64, True, True, torch.float16),        # ragged tails, fp16
    (1, 2, 257, 128, 0, False, True, torch.bfloat16),      # no rotated dims
])
def test_forward_tc_matches_exact_family(b, h, n, d, r, causal, masked, dtype):
    g = torch.Generator().manual_seed(n + d)
    q, k, v = (torch.randn(b, h, n, d, generator=g).to(dtype).to(DEV) for _ in range(3))
    pope = PoPE(r, heads=h) if r > 0 else None
    if pope is not None:
        with torch.no_grad():
            pope.bias.uniform_(-6.0, 0.0, generator=g)
        e = pope(n)
        emb = (e.freqs.to(DEV), e.bias.detach().to(DEV))
    else:
        emb = (torch.empty(n, 0, device=DEV), torch.empty(h, 0, device=DEV))
    mask = None
    if masked:
        lens = torch.randint(n // 2, n + 1, (b,), generator=g)
        mask = (torch.arange(n)[None, :] < lens[:, None]).to(DEV)
    o_tc, lse_tc, path_tc = _fwd(q, k, v, emb, mask, causal, force_simt=False)
    o_ex, lse_ex, path_ex = _fwd(q, k, v, emb, mask, causal, force_simt=True)
    assert path_tc == "tcgen05" and path_ex == "simt"
    assert _native.device_status() == 0
    assert float((o_tc.float() - o_ex.float()).abs().max()) <= 2e-2
    finite = torch.isfinite(lse_ex)
    assert torch.equal(finite, torch.isfinite(lse_tc))
    assert float((lse_tc[finite] - lse_ex[finite]).abs().max()) <= 2e-2


def test_short_query_blocks_take_the_exact_family():
    q = torch.randn(1, 2, 1, 64, device=DEV, dtype=torch.bfloat16)
    k = torch.randn(1, 2, 512, 64, device=DEV, dtype=torch.bfloat16)
    e = PoPE(32, heads=2)(512)
    _native.attn_forward(q, k, k, e.freqs.to(DEV), e.bias.detach().to(DEV), None, False, 0.125)
    assert _native.last_path() == "simt"


def _bwd(do, q, k, v, out, lse, emb, mask, causal, force_simt, want_dfreqs=True):
    os.environ["POPE_B200_FORCE_SIMT"] = "1" if force_simt else "0"
    try:
        res = _native.attn_backward(do, q, k, v, out, lse, emb[0], emb[1], mask, causal, q.shape[-1] ** -0.5,
                                    want_dfreqs, True)
        return res, _native.last_path()
    finally:
        os.environ["POPE_B200_FORCE_SIMT"] = "0"


@pytest.mark.parametrize("b,h,hk,n,d,r,causal,masked,dtype", [
    (2, 8, 8, 1024, 64, 32, True, True, torch.bfloat16),
    (1, 4, 4, 4096, 128, 128, True, False, torch.bfloat16),
    (2, 4, 4, 2048, 96, 96, False, False, torch.bfloat16),
    (1, 2, 2, 2048, 128, 64, True, False, torch.bfloat16),
    (2, 2, 2, 300, 64, 64, True, True, torch.float16),
    (1, 2, 2, 257, 128, 0, False, True, torch.bfloat16),
    (1, 4, 2, 320, 64, 32, True, False, torch.bfloat16),     # grouped heads
])
def test_backward_tc_matches_exact_family(b, h, hk, n, d, r, causal, masked, dtype):
    g = torch.Generator().manual_seed(n + d + 1)
    q = torch.randn(b, h, n, d, generator=g).to(dtype).to(DEV)
    k, v = (torch.randn(b, hk, n, d, generator=g).to(dtype).to(DEV) for _ in range(2))
    do = torch.randn(b, h, n, d, generator=g).to(dtype).to(DEV)
    if r > 0:
        pope = PoPE(r, heads=hk)
        with torch.no_grad():
            pope.bias.uniform_(-6.0, 0.0, generator=g)
        e = pope(n)
        emb = (e.freqs.to(DEV), e.bias.detach().to(DEV))
    else:
        emb = (torch.empty(n, 0, device=DEV), torch.empty(hk, 0, device=DEV))
    mask = None
    if masked:
        lens = torch.randint(n // 2, n + 1, (b,), generator=g)
        mask = (torch.arange(n)[None, :] < lens[:, None]).to(DEV)
    out, lse, _ = _fwd(q, k, v, emb, mask, causal, force_simt=True)
    (dq1, dk1, dv1, df1, db1), path1 = _bwd(do, q, k, v, out, lse, emb, mask, causal, force_simt=False)
    (dq0, dk0, dv0, df0, db0), path0 = _bwd(do, q, k, v, out, lse, emb, mask, causal, force_simt=True)
    assert path1 == "tcgen05" and path0 == "simt"
    assert _native.device_status() == 0
    for name, a1, a0 in (("dq", dq1, dq0), ("dk", dk1, dk0), ("dv", dv1, dv0)):
        err = float((a1.float() - a0.float()).abs().max())
        # both sides are stored in 16 bits: two roundings of nearly equal values may land one ulp apart,
        # which is up to 2^-7 of the magnitude in bf16
        assert err <= max(2e-2, 2.0 ** -7 * float(a0.float().abs().max())), f"{name}: {err}"
    if r > 0:
        for name, a1, a0 in (("dbias", db1, db0), ("dfreqs", df1, df0)):
            rel = float((a1 - a0).abs().max() / a0.abs().max().clamp_min(1.0))
            assert rel <= 2e-2, f"{name}: {rel}"


@pytest.mark.parametrize("n,d,r,dtype", [(1024, 64, 64, torch.float32), (776, 64, 32, torch.float32),
                                          (512, 128, 64, torch.float32), (1024, 64, 64, torch.bfloat16)])
def test_similarity_tc_matches_exact_family(n, d, r, dtype):
    """The split-precision tensor-core similarity against the fp32 FMA kernel: 1e-4 of max|sim| for fp32."""
    g = torch.Generator().manual_seed(n + d + r)
    q, k = (torch.randn(1, 8, n, d, generator=g).to(dtype).to(DEV) for _ in range(2))
    pope = PoPE(r, heads=8)
    with torch.no_grad():
        pope.bias.uniform_(-6.0, 0.0, generator=g)
    e = pope(n)
    freqs, bias = e.freqs.to(DEV), e.bias.detach().to(DEV)
    os.environ["POPE_B200_FORCE_SIMT"] = "0"
    s_tc = _native.sim_forward(q, k, freqs, bias)
    path_tc = _native.last_path()
    os.environ["POPE_B200_FORCE_SIMT"] = "1"
    try:
        s_ex = _native.sim_forward(q, k, freqs, bias)
        path_ex = _native.last_path()
    finally:
        os.environ["POPE_B200_FORCE_SIMT"] = "0"
    assert path_tc == "tcgen05" and path_ex == "simt" and _native.device_status() == 0
    tol = 1e-4 if dtype == torch.float32 else 1e-2
    assert float((s_tc.float() - s_ex.float()).abs().max()) <= tol * float(s_ex.float().abs().max())


@pytest.mark.parametrize("b,h,hk,nq,nk,d,r,causal,masked,dtype", [
    (2, 8, 8, 1024, 1024, 64, 32, True, True, torch.bfloat16),
    (2, 8, 2, 1024, 1024, 96, 96, False, False, torch.bfloat16),
    (1, 4, 4, 777, 1500, 128, 64, True, True, torch.float16),
])
def test_tensor_core_step_is_bitwise_reproducible(b, h, hk, nq, nk, d, r, causal, masked, dtype):
    """out, lse, dq, dk, dv carry no atomics and no order-dependent reduction: repeated calls agree to the bit (a race
    between the roles of a kernel would show up here); the phase-bias gradient is summed by fp32 atomics and may differ
    in the last bits."""
    g = torch.Generator().manual_seed(5)
    q = torch.randn(b, h, nq, d, generator=g).to(dtype).to(DEV)
    k, v = (torch.randn(b, hk, nk, d, generator=g).to(dtype).to(DEV) for _ in range(2))
    do = torch.randn(b, h, nq, d, generator=g).to(dtype).to(DEV)
    f = PoPE(r, heads=hk).to(DEV)(nk).freqs.detach().contiguous()
    bias = (-torch.rand(hk, r, generator=g) * 6).to(DEV)
    mask = None
    if masked:
        mask = torch.rand(b, nk, generator=g) > 0.3
        mask[:, 0] = True
        mask = mask.to(DEV)
    ref = None
    for _ in range(8):
        out, lse = _native.attn_forward(q, k, v, f, bias, mask, causal, d ** -0.5)
        assert _native.last_path() == "tcgen05"
        dq, dk, dv, _, db = _native.attn_backward(do, q, k, v, out, lse, f, bias, mask, causal, d ** -0.5, False, True)
        cur = (out, lse, dq, dk, dv)
        if ref is None:
            ref, db_ref = [t.clone() for t in cur], db.clone()
            continue
        for name, a, c in zip(("out", "lse", "dq", "dk", "dv"), cur, ref):
            assert torch.equal(a, c), name
        assert float((db - db_ref).abs().max()) <= 1e-5 * float(db_ref.abs().max())
    assert _native.device_status() == 0
