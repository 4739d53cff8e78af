"""Generate the golden vectors under tests/golden/ by running the UNMODIFIED reference package.

Run once, where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/PoPE-pytorch

The reference imports one helper from an uninstalled third-party package; the stand-in in
``_standin/`` (trailing-slice, no arithmetic) is put on sys.path for this script only.
Every case stores its inputs next to the reference's outputs, so the checks that consume
``pope_golden.npz`` need neither the reference nor any particular RNG.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(HERE, "_standin"))
    sys.path.insert(0, ref_root)
    import PoPE_pytorch  # the reference
    from PoPE_pytorch import PoPE, AxialPoPE, apply_pope_to_qk, compute_attn_similarity, flash_attn_with_pope
    assert os.path.abspath(PoPE_pytorch.__file__).startswith(os.path.abspath(ref_root))

    out = {}

    def put(name, t):
        out[name] = t.detach().cpu().numpy() if torch.is_tensor(t) else np.asarray(t)

    # ---- module forward: freqs / bias (offset, clamp), axial grid ---------------------
    torch.manual_seed(11)
    pope = PoPE(16, heads=4)
    with torch.no_grad():
        pope.bias.copy_(torch.empty(4, 16).uniform_(-8.0, 1.5))     # exercises the clamp
    pe = pope(24)
    put("mod/bias_param", pope.bias), put("mod/freqs24", pe.freqs), put("mod/bias_clamped", pe.bias)
    put("mod/freqs_off7", pope(8, offset=7).freqs)
    pos = torch.tensor([[0.0, 2.0, 5.0], [1.0, 1.0, 9.0]])
    put("mod/pos_b", pos), put("mod/freqs_posb", pope(pos).freqs)

    ax = AxialPoPE(24, heads=2, axial_dims=(8, 8, 8))
    put("axial/grid_2_3_4", AxialPoPE.get_grid_positions(2, 3, 4))
    put("axial/freqs_2_3_4", ax((2, 3, 4)).freqs)
    ax2 = AxialPoPE(32, heads=2, axial_dims=(16, 16))
    put("axial/freqs_4_5", ax2((4, 5)).freqs)

    # ---- apply_pope_to_qk ------------------------------------------------------------
    def transform_case(tag, b, hq, hk, nq, nk, d, r, freqs_ndim=2, seed=0):
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(b, hq, nq, d, generator=g)
        k = torch.randn(b, hk, nk, d, generator=g)
        if freqs_ndim == 2:
            freqs = torch.rand(nk, r, generator=g) * 50.0
        else:
            freqs = torch.rand(b, nk, r, generator=g) * 50.0
        bias = -torch.rand(hk, r, generator=g) * 6.0
        rq, rk = apply_pope_to_qk((freqs, bias), q, k)
        for n, t in (("q", q), ("k", k), ("freqs", freqs), ("bias", bias), ("rq", rq), ("rk", rk)):
            put(f"xform/{tag}/{n}", t)

    transform_case("full", 1, 2, 2, 12, 12, 8, 8, seed=1)
    transform_case("partial", 2, 2, 2, 12, 12, 8, 4, seed=2)
    transform_case("decode", 1, 2, 2, 1, 12, 8, 4, seed=3)
    transform_case("freqs3d", 2, 2, 2, 5, 12, 8, 8, freqs_ndim=3, seed=4)
    transform_case("r0", 1, 2, 2, 6, 6, 8, 0, seed=5)

    # ---- similarity (the CPU path of compute_attn_similarity) with gradients -------------
    def sim_case(tag, b, hq, hk, nq, nk, d, r, seed, random_table=False):
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(b, hq, nq, d, generator=g, requires_grad=True)
        k = torch.randn(b, hk, nk, d, generator=g, requires_grad=True)
        if random_table:
            freqs = torch.randn(nk, r, generator=g)
            bias = torch.randn(hk, r, generator=g)
        else:
            freqs = PoPE(r, heads=hk)(nk).freqs.detach() if r > 0 else torch.empty(nk, 0)
            bias = -torch.rand(hk, r, generator=g) * 6.0
        freqs.requires_grad_(True), bias.requires_grad_(True)
        sim = compute_attn_similarity(q, k, (freqs, bias))
        dsim = torch.randn(sim.shape, generator=g)
        sim.backward(dsim)
        for n, t in (("q", q), ("k", k), ("freqs", freqs), ("bias", bias), ("sim", sim), ("dsim", dsim),
                     ("dq", q.grad), ("dk", k.grad), ("dbias", bias.grad), ("dfreqs", freqs.grad)):
            if t is not None:
                put(f"sim/{tag}/{n}", t)

    sim_case("square", 2, 2, 2, 24, 24, 32, 16, seed=21)
    sim_case("decode", 1, 4, 4, 3, 40, 32, 32, seed=22)
    sim_case("gqa", 1, 4, 2, 16, 16, 32, 16, seed=23)
    sim_case("table", 1, 2, 2, 20, 20, 32, 16, seed=24, random_table=True)
    sim_case("r0", 1, 2, 2, 8, 8, 32, 0, seed=25)

    # ---- attention: the manual (fused=False) branch of flash_attn_with_pope, with gradients --
    def attn_case(tag, b, hq, hk, nq, nk, d, r, seed, causal=False, masked=False, layout_head_first=True):
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(b, hq, nq, d, generator=g, requires_grad=True)
        k = torch.randn(b, hk, nk, d, generator=g, requires_grad=True)
        v = torch.randn(b, hk, nk, d, generator=g, requires_grad=True)
        freqs = PoPE(r, heads=hk)(nk).freqs.detach().requires_grad_(True)
        bias = (-torch.rand(hk, r, generator=g) * 6.0).requires_grad_(True)
        mask = None
        if masked:
            lens = torch.randint(nk // 2, nk + 1, (b,), generator=g)
            mask = torch.arange(nk)[None, :] < lens[:, None]
        args = (q, k, v) if layout_head_first else tuple(t.transpose(1, 2) for t in (q, k, v))
        o = flash_attn_with_pope(*args, pos_emb=(freqs, bias), mask=mask, causal=causal, fused=False,
                                 head_dimension_at_first=layout_head_first)
        if not layout_head_first:
            o = o.transpose(1, 2)
        do = torch.randn(o.shape, generator=g)
        o.backward(do)
        for n, t in (("q", q), ("k", k), ("v", v), ("freqs", freqs), ("bias", bias), ("out", o), ("dout", do),
                     ("dq", q.grad), ("dk", k.grad), ("dv", v.grad), ("dbias", bias.grad), ("dfreqs", freqs.grad)):
            put(f"attn/{tag}/{n}", t)
        if mask is not None:
            put(f"attn/{tag}/mask", mask)
        put(f"attn/{tag}/causal", np.array(int(causal)))

    attn_case("plain", 2, 2, 2, 24, 24, 32, 16, seed=31)
    attn_case("causal", 1, 2, 2, 40, 40, 32, 32, seed=32, causal=True)
    attn_case("masked", 2, 2, 2, 24, 24, 32, 16, seed=33, masked=True)
    attn_case("decode", 1, 2, 2, 1, 40, 32, 16, seed=34)
    attn_case("short_q", 1, 2, 2, 5, 24, 32, 16, seed=35, causal=True)
    attn_case("gqa", 1, 4, 2, 16, 16, 32, 16, seed=36)
    attn_case("seq_first", 1, 2, 2, 16, 16, 32, 16, seed=37, layout_head_first=False)

    path = os.path.join(HERE, "pope_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
