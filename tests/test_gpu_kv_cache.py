"""Paged key / value cache on the GPU: append + decode through the C ABI against the oracle on the gathered keys."""
import pytest
import torch

from oracle import pope_oracle as O
from pope_pytorch_b200 import PagedKVCache, PoPE, _native
from pope_pytorch_b200.attention import flash_attn_with_pope

pytestmark = pytest.mark.gpu
DEV = "cuda"


def oracle_decode(q_row, k, v, freqs, bias, scale):
    """q_row (h, d), k / v (hk, n, d) fp32 on the CPU -> (h, d): the query at the last position."""
    out = O.attention(q_row[None, :, None, :].float(), k[None].float(), v[None].float(), freqs[: k.shape[1]].float(), bias.float(),
                      mask=None, causal=False, softmax_scale=scale)
    return out[0, :, 0]


def build_cache(lens, h, hk, d, r, dtype, page_size, seed, shuffle_pages=True):
    g = torch.Generator().manual_seed(seed)
    b = len(lens)
    need = sum(-(-(n + 8) // page_size) for n in lens) + 2
    cache = PagedKVCache(b, hk, d, num_pages=need, page_size=page_size, max_seq_len=max(lens) + 64, dtype=dtype, device=DEV)
    if shuffle_pages:   # physical pages in a scrambled order, so that logical != physical
        perm = torch.randperm(need, generator=g).tolist()
        cache.alloc.free = perm
    ks, vs = [], []
    for i, n in enumerate(lens):
        k = torch.randn(hk, n, d, generator=g).to(dtype)
        v = torch.randn(hk, n, d, generator=g).to(dtype)
        # two pieces, so that an append starts in the middle of a page
        cut = n // 3
        if cut:
            cache.append_to(i, k[:, :cut].to(DEV), v[:, :cut].to(DEV))
        cache.append_to(i, k[:, cut:].to(DEV), v[:, cut:].to(DEV))
        ks.append(k), vs.append(v)
    return cache, ks, vs, g


@pytest.mark.parametrize("lens,h,hk,d,r,dtype,page_size", [
    ([1000, 37, 2049], 4, 2, 128, 64, torch.bfloat16, 256),
    ([300, 300], 2, 2, 64, 64, torch.float16, 64),
    ([5000, 1], 8, 2, 96, 48, torch.bfloat16, 128),
    ([700], 2, 1, 128, 0, torch.bfloat16, 256),
])
def test_paged_decode_matches_the_oracle(lens, h, hk, d, r, dtype, page_size):
    cache, ks, vs, g = build_cache(lens, h, hk, d, r, dtype, page_size, seed=sum(lens) + d)
    assert cache.lens == lens
    for i in range(len(lens)):          # what append wrote is what was given
        gk, gv = cache.gather(i)
        assert torch.equal(gk.cpu(), ks[i]) and torch.equal(gv.cpu(), vs[i])
    q = torch.randn(len(lens), h, 1, d, generator=g).to(dtype)
    nmax = max(lens)
    if r > 0:
        emb = PoPE(r, heads=hk)(nmax)
        freqs, bias = emb.freqs.detach(), -torch.rand(hk, r, generator=g) * 6.0
    else:
        freqs, bias = torch.empty(nmax, 0), torch.empty(hk, 0)
    scale = d ** -0.5
    out, lse = cache.decode(q.to(DEV), (freqs.to(DEV), bias.to(DEV)), return_lse=True)
    assert _native.last_path() == "decode_stream_paged" and _native.device_status() == 0
    for i, n in enumerate(lens):
        ref = oracle_decode(q[i, :, 0], ks[i], vs[i], freqs, bias, scale)
        err = (out[i, :, 0].float().cpu() - ref).abs().max().item()
        assert err <= 2e-2, (i, n, err)
    assert torch.isfinite(lse).all()


def test_decode_loop_appends_one_token_at_a_time_and_equals_the_contiguous_call():
    b, h, hk, d, r, n0, steps = 2, 4, 4, 128, 64, 1100, 5
    g = torch.Generator().manual_seed(7)
    cache = PagedKVCache(b, hk, d, num_pages=2 * 6, page_size=256, dtype=torch.bfloat16, device=DEV)
    pope = PoPE(r, heads=hk).to(DEV)
    k_all = torch.randn(b, hk, n0 + steps, d, generator=g).bfloat16().to(DEV)
    v_all = torch.randn(b, hk, n0 + steps, d, generator=g).bfloat16().to(DEV)
    cache.append(k_all[:, :, :n0], v_all[:, :, :n0])
    for t in range(steps):
        n = n0 + t + 1
        cache.append(k_all[:, :, n - 1:n], v_all[:, :, n - 1:n])
        q = torch.randn(b, h, 1, d, generator=g).bfloat16().to(DEV)
        emb = pope(n)
        out = cache.decode(q, (emb.freqs.detach(), emb.bias.detach()))
        ref = flash_attn_with_pope(q, k_all[:, :, :n], v_all[:, :, :n], pos_emb=(emb.freqs.detach(), emb.bias.detach()), fused=True)
        assert cache.lens == [n, n]
        # the same kernel on the same keys: only the split of the key range may differ
        assert (out.float() - ref.float()).abs().max().item() <= 4e-3
    assert _native.device_status() == 0


def test_empty_sequence_gives_zeros_and_bad_page_is_reported_not_dereferenced():
    cache = PagedKVCache(2, 2, 64, num_pages=4, page_size=64, dtype=torch.bfloat16, device=DEV)
    g = torch.Generator().manual_seed(3)
    k = torch.randn(2, 100, 64, generator=g).bfloat16().to(DEV)
    cache.append_to(0, k, k)
    q = torch.randn(2, 2, 1, 64, generator=g).bfloat16().to(DEV)
    emb = PoPE(32, heads=2).to(DEV)(128)
    out, lse = cache.decode(q, (emb.freqs.detach(), emb.bias.detach()), return_lse=True)
    assert torch.count_nonzero(out[1]) == 0 and torch.isinf(lse[1]).all() and torch.isfinite(out[0]).all()
    assert _native.device_status() == 0
    cache.page_table[0, 1] = 77                      # outside the pool of 4 pages
    cache.decode(q, (emb.freqs.detach(), emb.bias.detach()))
    assert _native.device_status() & 2
    _native.clear_device_status()
    assert _native.device_status() == 0
