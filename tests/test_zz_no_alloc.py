"""The allocation-free forward entry point, exercised through the C ABI.

Some hosts of this library are not allowed to allocate device memory at the moment they need
attention: an inference server whose memory plan is frozen after start-up, a plugin that is given
nothing but input and output buffers, a latency-critical thread that may not wait on an
allocator.  ``pope_b200_attn_fwd_noalloc`` serves them: the caller passes inputs and outputs, and
the kernel's scratch sits in a fixed array inside the library.  Here it is checked against the
regular entry point (caller-allocated workspace) on two calls in a row with different inputs and
shapes, since every call reuses the same scratch.  The file name keeps it last in collection
order, so a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

from pope_pytorch_b200 import PoPE, _native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(seed, b, h, n, d, r, causal, masked):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(b, h, n, d, generator=g).bfloat16().to(DEV) for _ in range(3))
    pope = PoPE(r, heads=h)
    with torch.no_grad():
        pope.bias.uniform_(-6.0, 0.0, generator=g)
    e = pope(n)
    freqs, bias = e.freqs.to(DEV).contiguous(), e.bias.detach().to(DEV).contiguous()
    mask = None
    if masked:
        lens = torch.randint(n // 2, n + 1, (b,), generator=g)
        mask = (torch.arange(n)[None, :] < lens[:, None]).to(DEV)
    return q, k, v, freqs, bias, mask, causal, d ** -0.5


def _check_pair(args):
    q, k, v, freqs, bias, mask, causal, scale = args
    want_out, want_lse = _native.attn_forward(q, k, v, freqs, bias, mask, causal, scale)
    assert _native.last_path() == "tcgen05"
    out = torch.full_like(q, float("nan"))
    lse = torch.full((q.shape[0], q.shape[1], q.shape[2]), float("nan"), device=DEV)
    _native.attn_forward_noalloc(q, k, v, freqs, bias, mask, causal, scale, out, lse)
    torch.cuda.synchronize()
    # same kernel, same table contents: the tolerance of the bf16 tests (2e-2) is far from needed
    assert float((out.float() - want_out.float()).abs().max()) <= 2e-2
    finite = torch.isfinite(want_lse)
    assert torch.equal(finite, torch.isfinite(lse))
    assert float((lse[finite] - want_lse[finite]).abs().max()) <= 2e-2
    assert torch.equal(out, want_out)


def test_noalloc_forward_matches_regular_entry_point_twice_in_a_row():
    _check_pair(_case(1, 2, 4, 1024, 64, 32, True, True))
    _check_pair(_case(2, 1, 2, 2048, 128, 128, False, False))   # different shape reuses the scratch
    _check_pair(_case(3, 2, 4, 1024, 64, 32, True, True))
    assert _native.device_status() == 0


def test_noalloc_rejects_what_it_cannot_serve():
    lib = _native.load_library()
    q, k, v, freqs, bias, mask, causal, scale = _case(4, 1, 1, 16640, 128, 128, True, False)  # 8.1 MiB of tables + 8.1 MiB of K' tiles
    out, lse = torch.empty_like(q), torch.empty(1, 1, 16640, device=DEV)
    with pytest.raises(RuntimeError, match="capacity"):
        _native.attn_forward_noalloc(q, k, v, freqs, bias, mask, causal, scale, out, lse)
    q32 = torch.randn(1, 1, 128, 64, device=DEV)                     # fp32: not a tensor-core shape
    with pytest.raises(RuntimeError, match="unsupported"):
        _native.attn_forward_noalloc(q32, q32, q32, freqs[:128, :32].contiguous(), bias[:, :32].contiguous(), None, False,
                                     0.125, torch.empty_like(q32), torch.empty(1, 1, 128, device=DEV))
    lib.pope_b200_attn_fwd_noalloc.restype = C.c_int
    lib.pope_b200_attn_fwd_noalloc.argtypes = [C.c_void_p, C.c_void_p]
    assert lib.pope_b200_attn_fwd_noalloc(None, None) == -1
