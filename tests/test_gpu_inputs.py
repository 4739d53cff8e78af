"""GPU parity on the input forms the hot path must accept beyond the benchmark configurations:
batched phase tables (3-D ``(b, n, r)`` and 4-D ``(b, h, n, r)`` freqs, PoPE_pytorch/pope.py:53-56),
multi-tile similarity gradients, strided (non-contiguous) q / k / v / upstream gradients
(tests/test_triton.py:56-85 of the reference), broadcast key / value heads, adversarial softmax
inputs, plain attention through the inner seam (``freqs=None``,
PoPE_pytorch/triton_pope_flash_attn.py:364-373), the bounded-wait give-up path, and the
batch x heads shard helper driving the CUDA kernels.  Everything is compared with the CPU oracle
on identical seeded inputs, through the public API (which calls the C ABI).
"""
import math

import pytest
import torch

from oracle import pope_oracle as O
from pope_pytorch_b200 import PoPE, compute_attn_similarity, flash_attn_with_pope, _native
from pope_pytorch_b200.shard import plan_shard, sharded_flash_attn

from test_gpu_parity import REL_TOL, assert_close32, check16, gen, maxerr, record_errors, rel_err

pytestmark = pytest.mark.gpu
DEV = "cuda"


def batched_freqs(kind, b, h, n, r, g):
    """Random opaque phase tables of the three ranks the API accepts."""
    if kind == "2d":
        return torch.rand(n, r, generator=g) * 50.0
    if kind == "3d":
        return torch.rand(b, n, r, generator=g) * 50.0
    return torch.rand(b, h, n, r, generator=g) * 50.0


# ------------------------------------------------------------------------------------------
# batched phase tables
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("kind", ["3d", "4d"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq", [160, 1])
def test_attention_batched_freqs(kind, dtype, nq):
    b, h, nk, d, r = 2, 4, 160, 64, 32
    g = torch.Generator().manual_seed(70 + nq + (kind == "4d"))
    q, k, v, dout = gen((b, h, nq, d), g, dtype), gen((b, h, nk, d), g, dtype), gen((b, h, nk, d), g, dtype), gen((b, h, nq, d), g, dtype)
    freqs, bias = batched_freqs(kind, b, h, nk, r, g), -torch.rand(h, r, generator=g) * 6.0
    causal = nq > 1
    ref = O.attention_with_grads(q.float(), k.float(), v.float(), freqs, bias, dout.float(), causal=causal, want_dfreqs=True)
    qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    fg, bg = freqs.to(DEV).requires_grad_(True), bias.to(DEV).requires_grad_(True)
    out = flash_attn_with_pope(qg, kg, vg, pos_emb=(fg, bg), causal=causal)
    if dtype == torch.bfloat16 and nq >= 64:      # batched tables are served by the tensor-core kernels too
        assert _native.last_path() == "tcgen05"
    out.backward(dout.to(DEV))
    if dtype == torch.bfloat16 and nq >= 64:
        assert _native.last_path() == "tcgen05" and _native.device_status() == 0
    assert fg.grad.shape == freqs.shape
    errs = {}
    for name, got in (("out", out), ("dq", qg.grad), ("dk", kg.grad), ("dv", vg.grad)):
        if dtype == torch.float32:
            assert_close32(got, ref[name], name)
        else:
            check16(name, got, ref[name], dtype, errs=errs)
    assert rel_err(bg.grad, ref["dbias"]) <= (1e-3 if dtype == torch.float32 else REL_TOL)
    assert rel_err(fg.grad, ref["dfreqs"]) <= (1e-3 if dtype == torch.float32 else REL_TOL)
    if errs:
        record_errors(f"batched_freqs_{kind}_nq{nq}_bf16", errs)


@pytest.mark.parametrize("kind", ["3d", "4d"])
def test_similarity_batched_freqs(kind):
    b, h, nq, nk, d, r = 2, 4, 96, 200, 64, 32
    g = torch.Generator().manual_seed(81 + (kind == "4d"))
    q, k, dsim = gen((b, h, nq, d), g), gen((b, h, nk, d), g), gen((b, h, nq, nk), g)
    freqs, bias = batched_freqs(kind, b, h, nk, r, g), -torch.rand(h, r, generator=g) * 6.0
    ref = O.similarity_with_grads(q, k, freqs, bias, dsim, want_dfreqs=True)
    qg, kg = q.to(DEV).requires_grad_(True), k.to(DEV).requires_grad_(True)
    fg, bg = freqs.to(DEV).requires_grad_(True), bias.to(DEV).requires_grad_(True)
    sim = compute_attn_similarity(qg, kg, (fg, bg), allow_tf32=False)
    assert maxerr(sim, ref["sim"]) <= 1e-4 * float(ref["sim"].abs().max())
    sim.backward(dsim.to(DEV))
    assert_close32(qg.grad, ref["dq"], "dq"), assert_close32(kg.grad, ref["dk"], "dk")
    assert_close32(bg.grad, ref["dbias"], "dbias", atol=1e-3), assert_close32(fg.grad, ref["dfreqs"], "dfreqs", atol=1e-3)


# ------------------------------------------------------------------------------------------
# similarity gradients beyond one tile
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("b,h,hk,nq,nk,d,r", [(1, 8, 8, 1024, 1024, 64, 64),     # benchmark configuration 1
                                              (2, 4, 2, 300, 520, 64, 32)])     # ragged, grouped heads, partial rotation
@pytest.mark.parametrize("allow_tf32", [True, False])
def test_similarity_multi_tile_forward_and_gradients(b, h, hk, nq, nk, d, r, allow_tf32):
    g = torch.Generator().manual_seed(nq + nk + d)
    q, k, dsim = gen((b, h, nq, d), g), gen((b, hk, nk, d), g), gen((b, h, nq, nk), g)
    freqs = PoPE(r, heads=hk)(nk).freqs
    bias = -torch.rand(hk, r, generator=g) * 6.0
    ref = O.similarity_with_grads(q, k, freqs, bias, dsim, want_dfreqs=True)
    qg, kg = q.to(DEV).requires_grad_(True), k.to(DEV).requires_grad_(True)
    fg, bg = freqs.to(DEV).requires_grad_(True), bias.to(DEV).requires_grad_(True)
    sim = compute_attn_similarity(qg, kg, (fg, bg), allow_tf32=allow_tf32)
    scale = float(ref["sim"].abs().max())
    errs = dict(sim_rel=maxerr(sim, ref["sim"]) / scale)
    assert errs["sim_rel"] <= 1e-4
    sim.backward(dsim.to(DEV))
    assert _native.last_path() == "tcgen05" and _native.device_status() == 0   # forward AND backward on the tensor cores
    # gradients are sums over up to 1024 score gradients of magnitude ~1: the reference's own bound
    # (rtol 1e-3, atol 1e-4) applies to unit-scale entries, so the absolute part scales with the largest entry
    for name, got in (("dq", qg.grad), ("dk", kg.grad), ("dbias", bg.grad), ("dfreqs", fg.grad)):
        mag = max(1.0, float(ref[name].abs().max()))
        errs[name + "_rel"] = maxerr(got, ref[name]) / mag
        assert_close32(got, ref[name], name, rtol=1e-3, atol=1e-4 * mag)
    record_errors(f"similarity_{b}x{h}x{nq}x{nk}_d{d}_r{r}_tf32{int(allow_tf32)}", errs)


# ------------------------------------------------------------------------------------------
# strided inputs
# ------------------------------------------------------------------------------------------

def test_attention_row_sliced_inputs_and_upstream_gradient():
    """q, k, v and dout as every second row of larger buffers (feature axis contiguous, row stride 2d)."""
    from test_gpu_parity import run_case
    run_case(2, 4, 4, 320, 320, 64, 32, torch.bfloat16, causal=True, masked=False, seed=91, row_sliced_dout=True)
    b, h, n, d, r = 1, 4, 192, 128, 64
    g = torch.Generator().manual_seed(92)
    big = [gen((b, h, 2 * n, d), g, torch.bfloat16) for _ in range(4)]
    q, k, v, dout = (t[:, :, ::2] for t in big)
    freqs, bias = PoPE(r, heads=h)(n).freqs, -torch.rand(h, r, generator=g) * 6.0
    ref = O.attention_with_grads(q.float(), k.float(), v.float(), freqs, bias, dout.float(), causal=True)
    bg = [t.to(DEV) for t in big]
    qg, kg, vg = (t[:, :, ::2].requires_grad_(True) for t in bg[:3])
    assert not qg.is_contiguous()
    out = flash_attn_with_pope(qg, kg, vg, pos_emb=(freqs.to(DEV), bias.to(DEV)), causal=True)
    out.backward(bg[3][:, :, ::2])
    for name, got in (("out", out), ("dq", qg.grad), ("dk", kg.grad), ("dv", vg.grad)):
        check16(name, got, ref[name], torch.bfloat16)


def test_attention_key_value_heads_given_as_broadcast_views():
    """One key / value head expanded over all query heads (stride 0 on the head axis), as a caller
    doing multi-query attention by hand passes them."""
    b, h, n, d, r = 2, 4, 256, 64, 32
    g = torch.Generator().manual_seed(93)
    q, k1, v1 = gen((b, h, n, d), g, torch.bfloat16), gen((b, 1, n, d), g, torch.bfloat16), gen((b, 1, n, d), g, torch.bfloat16)
    freqs, bias1 = PoPE(r, heads=1)(n).freqs, -torch.rand(1, r, generator=g) * 6.0
    bias = bias1.expand(h, r).contiguous()
    ref = O.attention(q.float(), k1.expand(b, h, n, d).float(), v1.expand(b, h, n, d).float(), freqs, bias, causal=True)
    kx, vx = k1.to(DEV).expand(b, h, n, d), v1.to(DEV).expand(b, h, n, d)
    assert kx.stride(1) == 0
    out = flash_attn_with_pope(q.to(DEV), kx, vx, pos_emb=(freqs.to(DEV), bias.to(DEV)), causal=True)
    check16("out", out, ref, torch.bfloat16)
    assert _native.device_status() == 0


# ------------------------------------------------------------------------------------------
# softmax under adversarial scores
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("r", [0, 48])
def test_softmax_late_outlier_and_equal_scores(r):
    """The forward keeps a stale running maximum while the true one is within 2^8 of it.  A score
    that jumps by +30 (natural-log units) in the LAST key tile, and rows whose scores are all
    equal, must still come out within the bf16 bound."""
    b, h, n, d = 1, 2, 1024, 64
    g = torch.Generator().manual_seed(94 + r)
    q, k, v = (gen((b, h, n, d), g, torch.bfloat16) for _ in range(3))
    q, k = q * 0.25, k * 0.25
    # pass-through feature d-1 carries the outlier: q = 8, last-tile key = 30  ->  8 * 30 * d^-0.5 = +30
    q[..., d - 1] = 8.0
    k[..., d - 1] = 0.0
    k[:, :, n - 5, d - 1] = 30.0
    if r > 0:
        freqs, bias = PoPE(r, heads=h)(n).freqs, -torch.rand(h, r, generator=g) * 6.0
    else:
        freqs, bias = torch.empty(n, 0), torch.empty(h, 0)
    for causal in (False, True):
        ref = O.attention(q.float(), k.float(), v.float(), freqs, bias, causal=causal)
        out = flash_attn_with_pope(q.to(DEV), k.to(DEV), v.to(DEV), pos_emb=(freqs.to(DEV), bias.to(DEV)), causal=causal)
        assert _native.last_path() == "tcgen05"
        check16(f"outlier causal={causal}", out, ref, torch.bfloat16)
    # all keys identical: every visible score of a row is the same, the output is the running mean of v
    k_same = k[:, :, :1].expand(b, h, n, d).contiguous()
    k_same[..., d - 1] = 0.0
    if r > 0:   # identical scores need identical phases too: one repeated table row
        freqs = freqs[:1].expand(n, -1).contiguous()
    ref = O.attention(q.float(), k_same.float(), v.float(), freqs, bias, causal=True)
    out = flash_attn_with_pope(q.to(DEV), k_same.to(DEV), v.to(DEV), pos_emb=(freqs.to(DEV), bias.to(DEV)), causal=True)
    check16("equal scores", out, ref, torch.bfloat16)
    mean = v.float().cumsum(dim=2) / torch.arange(1, n + 1)[None, None, :, None]
    assert maxerr(out, mean) <= 2e-2


# ------------------------------------------------------------------------------------------
# plain attention through the inner seam
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype,n", [(torch.bfloat16, 512), (torch.float32, 100)])
def test_inner_seam_without_freqs_is_plain_attention(dtype, n):
    g = torch.Generator().manual_seed(95)
    q, k, v, dout = (gen((2, 4, n, 64), g, dtype) for _ in range(4))
    ref = O.attention_with_grads(q.float(), k.float(), v.float(), torch.empty(n, 0), torch.empty(4, 0), dout.float(), causal=True)
    qg, kg, vg = (t.to(DEV).requires_grad_(True) for t in (q, k, v))
    out = _native.flash_attn(qg, kg, vg, causal=True)
    out.backward(dout.to(DEV))
    for name, got in (("out", out), ("dq", qg.grad), ("dk", kg.grad), ("dv", vg.grad)):
        if dtype == torch.float32:
            assert_close32(got, ref[name], name)
        else:
            check16(name, got, ref[name], dtype)


# ------------------------------------------------------------------------------------------
# a bounded wait that runs out
# ------------------------------------------------------------------------------------------

def test_bounded_wait_gives_up_and_the_device_stays_usable():
    assert _native.device_status() == 0
    _native.selftest_bounded_wait()
    assert _native.device_status() & 1 == 1          # the give-up path ran and reported
    _native.clear_device_status()
    assert _native.device_status() == 0
    # tensor memory was freed and the context is healthy: a tensor-core call right after is correct
    g = torch.Generator().manual_seed(96)
    q, k, v = (gen((1, 2, 256, 64), g, torch.bfloat16) for _ in range(3))
    freqs, bias = PoPE(32, heads=2)(256).freqs, torch.zeros(2, 32)
    ref = O.attention(q.float(), k.float(), v.float(), freqs, bias, causal=True)
    out = flash_attn_with_pope(q.to(DEV), k.to(DEV), v.to(DEV), pos_emb=(freqs.to(DEV), bias.to(DEV)), causal=True)
    assert _native.last_path() == "tcgen05" and _native.device_status() == 0
    check16("out", out, ref, torch.bfloat16)


# ------------------------------------------------------------------------------------------
# batch x heads shards on the CUDA kernels
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("b,h,hk", [(1, 8, 8), (2, 4, 2), (4, 1, 1)])
def test_two_shards_run_one_after_the_other_equal_the_unsharded_call(b, h, hk):
    n, d, r = 256, 64, 32
    g = torch.Generator().manual_seed(97 + b)
    q, k, v = gen((b, h, n, d), g, torch.bfloat16).to(DEV), gen((b, hk, n, d), g, torch.bfloat16).to(DEV), gen((b, hk, n, d), g, torch.bfloat16).to(DEV)
    pope = PoPE(r, heads=hk)
    with torch.no_grad():
        pope.bias.uniform_(-2 * math.pi, 0.0, generator=g)
    e = pope(n)
    emb = (e.freqs.to(DEV), e.bias.detach().to(DEV))
    whole = flash_attn_with_pope(q, k, v, pos_emb=emb, causal=True)
    parts = []
    for rank in range(2):
        out, plan = sharded_flash_attn(q, k, v, emb, causal=True, rank=rank, world=2, fused=True)
        assert plan == plan_shard(b, h, hk, rank, 2)
        parts.append(out)
    assert torch.equal(torch.cat(parts, dim=plan.dim), whole)


# ------------------------------------------------------------------------------------------
# single-token decode on the streaming kernel
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("b,h,hk,nk,d,r,dtype,masked,seq_first", [
    (2, 4, 4, 4096, 128, 64, torch.bfloat16, False, False),
    (1, 8, 2, 1500, 128, 128, torch.bfloat16, True, False),     # ragged key count, grouped heads, full rotation
    (2, 4, 4, 2048, 64, 32, torch.float16, True, True),         # (b, n, h, d) layout: rows arrive one copy each
    (1, 4, 4, 3000, 96, 96, torch.bfloat16, False, False),
    (1, 2, 2, 1024, 64, 0, torch.bfloat16, False, False),       # no rotated dims
    (3, 2, 2, 1111, 128, 8, torch.bfloat16, True, True),
])
def test_decode_stream_matches_oracle(b, h, hk, nk, d, r, dtype, masked, seq_first):
    g = torch.Generator().manual_seed(nk + d + r)
    q, k, v = gen((b, h, 1, d), g, dtype), gen((b, hk, nk, d), g, dtype), gen((b, hk, nk, d), g, dtype)
    freqs = PoPE(r, heads=hk)(nk).freqs if r > 0 else torch.empty(nk, 0)
    bias = -torch.rand(hk, r, generator=g) * 6.0
    mask = None
    if masked:
        lens = torch.randint(nk // 2, nk + 1, (b,), generator=g)
        mask = torch.arange(nk)[None, :] < lens[:, None]
    ref = O.attention(q.float(), k.float(), v.float(), freqs, bias, mask=mask)
    qg, kg, vg = q.to(DEV), k.to(DEV), v.to(DEV)
    if seq_first:
        qg, kg, vg = (t.transpose(1, 2).contiguous() for t in (qg, kg, vg))
    out = flash_attn_with_pope(qg, kg, vg, pos_emb=(freqs.to(DEV), bias.to(DEV)), mask=None if mask is None else mask.to(DEV),
                               head_dimension_at_first=not seq_first)
    assert _native.last_path() == "decode_stream" and _native.device_status() == 0
    if seq_first:
        out = out.transpose(1, 2)
    check16("out", out, ref, dtype)


# ------------------------------------------------------------------------------------------
# the stand-alone transform (apply_pope_to_qk) as one fused pass
# ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("b,h,hk,nq,nk,d,r,dtype,kind", [
    (1, 8, 8, 1024, 1024, 64, 64, torch.float32, "2d"),       # shapes of the reference's own test (tests/test_pope.py:6-29)
    (1, 8, 8, 1, 1024, 64, 32, torch.float32, "2d"),          # decode: the query sits at the last position
    (2, 4, 2, 96, 200, 128, 64, torch.bfloat16, "3d"),
    (2, 4, 4, 33, 33, 48, 16, torch.float16, "4d"),
    (1, 2, 2, 50, 50, 32, 0, torch.float32, "2d"),
])
def test_apply_pope_to_qk_fused_forward_and_gradients(b, h, hk, nq, nk, d, r, dtype, kind):
    from pope_pytorch_b200 import apply_pope_to_qk
    g = torch.Generator().manual_seed(nq + nk + d + r)
    q, k = gen((b, h, nq, d), g, dtype), gen((b, hk, nk, d), g, dtype)
    freqs = batched_freqs(kind, b, hk, nk, r, g)
    bias = -torch.rand(hk, r, generator=g) * 6.0
    gq, gk = gen((b, h, nq, d + r), g), gen((b, hk, nk, d + r), g)
    # oracle: its own restatement of the transform, gradients by autograd, all in fp32 on the rounded inputs
    qr, kr = q.float().clone().requires_grad_(True), k.float().clone().requires_grad_(True)
    fr, br = freqs.clone().requires_grad_(True), bias.clone().requires_grad_(True)
    qe, ke = O.apply_pope(fr, br, qr, kr)   # a table without a head axis serves any number of query heads
    (qe * gq).sum().backward(retain_graph=True)
    (ke * gk).sum().backward()
    qg, kg = q.to(DEV).requires_grad_(True), k.to(DEV).requires_grad_(True)
    fg, bg = freqs.to(DEV).requires_grad_(True), bias.to(DEV).requires_grad_(True)
    q_out, k_out = apply_pope_to_qk((fg, bg), qg, kg)
    assert q_out.dtype == torch.float32 and q_out.shape == (b, h, nq, d + r) and k_out.shape == (b, hk, nk, d + r)
    assert_close32(q_out, qe, "q'", rtol=1e-5, atol=1e-5), assert_close32(k_out, ke, "k'", rtol=1e-5, atol=1e-5)
    (q_out * gq.to(DEV)).sum().backward(retain_graph=True)
    (k_out * gk.to(DEV)).sum().backward()
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-2, atol=1e-2)
    assert_close32(qg.grad, qr.grad, "dq", **tol), assert_close32(kg.grad, kr.grad, "dk", **tol)
    if r > 0:
        mag = max(1.0, float(br.grad.abs().max()))
        assert_close32(bg.grad, br.grad, "dbias", rtol=1e-4, atol=1e-4 * mag)
        assert_close32(fg.grad, fr.grad, "dfreqs", rtol=1e-4, atol=1e-4 * max(1.0, float(fr.grad.abs().max())))


# ------------------------------------------------------------------------------------------
# factored phase tables: positions x inverse frequencies recomputed inside the table builders
# ------------------------------------------------------------------------------------------

def test_factored_embeds_give_bitwise_the_results_of_the_plain_table():
    from pope_pytorch_b200 import AxialPoPE, FactoredPolarEmbed
    g = torch.Generator().manual_seed(98)
    n, d = 1024, 64
    q, k, v = (gen((1, 4, n, d), g, torch.bfloat16).to(DEV) for _ in range(3))
    for module, arg in ((PoPE(32, heads=4).to(DEV), n), (AxialPoPE(48, heads=4, axial_dims=(16, 16, 16)).to(DEV), (4, 16, 16))):
        emb = module(arg)
        assert isinstance(emb, FactoredPolarEmbed) and _native._factors_of(emb.freqs) is not None
        freqs, bias = emb                                      # unpacking keeps the factors on the tensor
        plain = (freqs.detach().clone(), bias.detach())        # a copy of the table carries none
        assert _native._factors_of(plain[0]) is None
        a = flash_attn_with_pope(q, k, v, pos_emb=(freqs, bias.detach()), causal=True)
        b = flash_attn_with_pope(q, k, v, pos_emb=plain, causal=True)
        assert _native.last_path() == "tcgen05" and torch.equal(a, b)
        a = flash_attn_with_pope(q[:, :, -1:], k, v, pos_emb=(freqs, bias.detach()))
        b = flash_attn_with_pope(q[:, :, -1:], k, v, pos_emb=plain)
        assert _native.last_path() == "decode_stream" and torch.equal(a, b)
        a = compute_attn_similarity(q.float(), k.float(), (freqs, bias.detach()))
        b = compute_attn_similarity(q.float(), k.float(), plain)
        assert _native.last_path() == "tcgen05" and torch.equal(a, b)
    # a module called with an offset, and gradients through the factored path
    pope = PoPE(32, heads=4).to(DEV)
    qg = q.clone().requires_grad_(True)
    out = flash_attn_with_pope(qg, k, v, pos_emb=pope(n, offset=7), causal=True)
    out.float().square().sum().backward()
    qp = q.clone().requires_grad_(True)
    pe = pope(n, offset=7)
    out_p = flash_attn_with_pope(qp, k, v, pos_emb=(pe.freqs.detach().clone(), pe.bias), causal=True)
    out_p.float().square().sum().backward()
    assert torch.equal(out, out_p) and torch.equal(qg.grad, qp.grad)
