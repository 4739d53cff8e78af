"""Pins the CPU oracle to vectors produced by the reference package itself (tests/golden/)."""
import pytest
import torch

from oracle import pope_oracle as O

XFORM = ["full", "partial", "decode", "freqs3d", "r0"]
SIM = ["square", "decode", "gqa", "table", "r0"]
ATTN = ["plain", "causal", "masked", "decode", "short_q", "gqa", "seq_first"]


def close(a, b, tol=2e-6):
    scale = max(1.0, float(b.abs().max())) if b.numel() else 1.0
    assert a.shape == b.shape
    assert float((a - b).abs().max()) <= tol * scale if b.numel() else True


def test_module_forward_vectors(golden):
    g = golden.case("mod")
    inv = O.pope_inv_freqs(16)
    close(O.pope_freqs(torch.arange(24).float(), inv), g["freqs24"])
    close(O.pope_freqs(torch.arange(8).float(), inv, offset=7), g["freqs_off7"])
    close(O.pope_freqs(g["pos_b"], inv), g["freqs_posb"])
    close(O.pope_clamped_bias(g["bias_param"]), g["bias_clamped"])


def test_axial_vectors(golden):
    g = golden.case("axial")
    grid = O.axial_grid_positions(2, 3, 4)
    assert torch.equal(grid, g["grid_2_3_4"])
    close(O.axial_freqs(grid, (8, 8, 8)), g["freqs_2_3_4"])
    close(O.axial_freqs(O.axial_grid_positions(4, 5), (16, 16)), g["freqs_4_5"])


@pytest.mark.parametrize("tag", XFORM)
def test_transform_vectors(golden, tag):
    g = golden.case(f"xform/{tag}")
    rq, rk = O.apply_pope(g["freqs"], g["bias"], g["q"], g["k"])
    close(rq, g["rq"]), close(rk, g["rk"])


@pytest.mark.parametrize("tag", SIM)
def test_similarity_vectors(golden, tag):
    g = golden.case(f"sim/{tag}")
    res = O.similarity_with_grads(g["q"], g["k"], g["freqs"], g["bias"], g["dsim"], want_dfreqs=True)
    close(res["sim"], g["sim"], 1e-5)
    for name in ("dq", "dk", "dbias", "dfreqs"):
        if name in g:
            close(res[name], g[name], 1e-5)


@pytest.mark.parametrize("tag", ATTN)
def test_attention_vectors(golden, tag):
    g = golden.case(f"attn/{tag}")
    res = O.attention_with_grads(g["q"], g["k"], g["v"], g["freqs"], g["bias"], g["dout"],
                                 mask=g.get("mask"), causal=bool(int(g["causal"])), want_dfreqs=True)
    for name in ("out", "dq", "dk", "dv", "dbias", "dfreqs"):
        close(res[name], g[name], 2e-5)


def test_golden_inventory(golden):
    assert golden.tags("xform") == sorted(XFORM)
    assert golden.tags("sim") == sorted(SIM)
    assert golden.tags("attn") == sorted(ATTN)


def test_fully_masked_row_is_zero():
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 1, 4, 8), torch.randn(1, 1, 4, 8), torch.randn(1, 1, 4, 8)
    freqs, bias = torch.rand(4, 8), torch.zeros(1, 8)
    mask = torch.zeros(1, 4, dtype=torch.bool)
    out, lse = O.attention(q, k, v, freqs, bias, mask=mask, return_lse=True)
    assert torch.all(out == 0) and torch.all(torch.isinf(lse) & (lse < 0))


def test_decode_causal_is_top_left():
    # a single query with causal=True sees key 0 only (reference semantics)
    torch.manual_seed(0)
    q, k, v = torch.randn(1, 1, 1, 8), torch.randn(1, 1, 6, 8), torch.randn(1, 1, 6, 8)
    out = O.attention(q, k, v, torch.rand(6, 4), torch.zeros(1, 4), causal=True)
    assert torch.allclose(out[0, 0, 0], v[0, 0, 0])
