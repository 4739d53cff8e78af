"""CPU-side checks of the drop-in Python surface against vectors produced by the reference."""
import inspect

import pytest
import torch

import pope_pytorch_b200 as P
from pope_pytorch_b200 import AxialPoPE, PoPE, apply_pope_to_qk, compute_attn_similarity, flash_attn_with_pope


def close(a, b, tol=2e-6):
    assert a.shape == b.shape
    if b.numel():
        assert float((a - b).abs().max()) <= tol * max(1.0, float(b.abs().max()))


def test_exports_and_signatures():
    for name in ("PoPE", "AxialPoPE", "apply_pope_to_qk", "compute_attn_similarity", "flash_attn_with_pope"):
        assert hasattr(P, name)
    sig = inspect.signature(flash_attn_with_pope)
    assert list(sig.parameters) == ["q", "k", "v", "pos_emb", "mask", "causal", "softmax_scale", "fused",
                                    "head_dimension_at_first"]
    sig = inspect.signature(compute_attn_similarity)
    assert list(sig.parameters) == ["q", "k", "pope", "allow_tf32", "head_dimension_at_first"]
    assert sig.parameters["allow_tf32"].default is True
    sig = inspect.signature(apply_pope_to_qk)
    assert list(sig.parameters) == ["pope", "q", "k", "to_magnitude", "return_complex"]
    from pope_pytorch_b200 import attention
    assert isinstance(attention.TRITON_AVAILABLE, bool)


def test_module_vectors_and_state_dict(golden):
    g = golden.case("mod")
    pope = PoPE(16, heads=4)
    assert sorted(pope.state_dict()) == ["bias", "inv_freqs"]
    with torch.no_grad():
        pope.bias.copy_(g["bias_param"])
    emb = pope(24)
    close(emb.freqs, g["freqs24"]), close(emb.bias, g["bias_clamped"])
    close(pope(8, offset=7).freqs, g["freqs_off7"])
    close(pope(g["pos_b"]).freqs, g["freqs_posb"])
    emb.bias.sum().backward()      # gradient reaches the parameter through the clamp
    assert pope.bias.grad is not None


def test_axial_vectors_and_state_dict(golden):
    g = golden.case("axial")
    ax = AxialPoPE(24, heads=2, axial_dims=(8, 8, 8))
    assert sorted(ax.state_dict()) == ["bias", "inv_freqs.0", "inv_freqs.1", "inv_freqs.2"]
    assert torch.equal(AxialPoPE.get_grid_positions(2, 3, 4), g["grid_2_3_4"])
    close(ax((2, 3, 4)).freqs, g["freqs_2_3_4"])
    close(AxialPoPE(32, heads=2, axial_dims=(16, 16))((4, 5)).freqs, g["freqs_4_5"])
    assert AxialPoPE(96, heads=8, axial_dims=(32, 32, 32))((8, 16, 16)).freqs.shape == (2048, 96)
    with pytest.raises(AssertionError):
        AxialPoPE(24, heads=2, axial_dims=(8, 8))


@pytest.mark.parametrize("tag", ["full", "partial", "decode", "freqs3d", "r0"])
def test_apply_pope_vectors(golden, tag):
    g = golden.case(f"xform/{tag}")
    rq, rk = apply_pope_to_qk((g["freqs"], g["bias"]), g["q"], g["k"])
    close(rq, g["rq"]), close(rk, g["rk"])


def test_apply_pope_complex_matches_real():
    torch.manual_seed(0)
    q, k = torch.randn(1, 2, 3, 8), torch.randn(1, 2, 5, 8)
    emb = (torch.rand(5, 4) * 9, -torch.rand(2, 4))
    rq, rk = apply_pope_to_qk(emb, q, k)
    cq, ck = apply_pope_to_qk(emb, q, k, return_complex=True)
    sim_real = torch.einsum("bhid,bhjd->bhij", rq, rk)
    sim_cplx = torch.einsum("bhid,bhjd->bhij", cq, ck.conj()).real
    close(sim_cplx, sim_real, 1e-5)


@pytest.mark.parametrize("tag", ["square", "decode", "gqa", "table", "r0"])
def test_cpu_similarity_vectors(golden, tag):
    g = golden.case(f"sim/{tag}")
    close(compute_attn_similarity(g["q"], g["k"], (g["freqs"], g["bias"])), g["sim"], 1e-5)


@pytest.mark.parametrize("tag", ["plain", "causal", "masked", "decode", "short_q", "gqa"])
def test_cpu_manual_attention_vectors(golden, tag):
    g = golden.case(f"attn/{tag}")
    out = flash_attn_with_pope(g["q"], g["k"], g["v"], pos_emb=(g["freqs"], g["bias"]), mask=g.get("mask"),
                               causal=bool(int(g["causal"])), fused=False)
    close(out, g["out"], 2e-5)


def test_asserts_match_reference_conventions():
    q, k = torch.randn(1, 3, 4, 32), torch.randn(1, 2, 4, 32)
    with pytest.raises(AssertionError):
        compute_attn_similarity(q, k, (torch.rand(4, 8), torch.zeros(2, 8)))       # 3 % 2 != 0
    with pytest.raises(AssertionError):
        compute_attn_similarity(torch.randn(1, 2, 4, 40), torch.randn(1, 2, 4, 40), (torch.rand(4, 8), torch.zeros(2, 8)))
    with pytest.raises(AssertionError):
        apply_pope_to_qk((torch.rand(4, 8), torch.zeros(2, 8)), torch.randn(1, 2, 5, 32), k)  # q longer than k
