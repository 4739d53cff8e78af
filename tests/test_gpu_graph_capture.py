"""The library calls are CUDA-graph capturable (no allocation, no synchronisation, the backward's side stream forks and
joins inside the capture): a captured forward, training step and similarity replay to the bits of the eager calls."""
import pytest
import torch

from pope_pytorch_b200 import PoPE, _native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _capture(fn):
    # one eager pass on a side stream first, as torch asks (it also sets the kernel attributes outside the capture)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        res = fn()
    return graph, res


def test_training_step_replays_bitwise():
    g = torch.Generator().manual_seed(21)
    q, k, v, do = (torch.randn(2, 4, 320, 64, generator=g).bfloat16().to(DEV) for _ in range(4))
    emb = PoPE(32, heads=4).to(DEV)(320)
    f, b = emb.freqs.detach().contiguous(), emb.bias.detach().contiguous()
    mask = (torch.arange(320)[None, :] < torch.tensor([[320], [250]])).to(DEV)

    def step():
        out, lse = _native.attn_forward(q, k, v, f, b, mask, True, 0.125)
        return (out, lse) + tuple(_native.attn_backward(do, q, k, v, out, lse, f, b, mask, True, 0.125, False, True))

    ref = [t.clone() for t in step() if t is not None]
    assert _native.last_path() == "tcgen05"
    graph, res = _capture(step)
    for t in res:
        if t is not None:
            t.zero_()
    graph.replay()
    torch.cuda.synchronize()
    got = [t for t in res if t is not None]
    for i, (a, c) in enumerate(zip(got[:5], ref[:5])):      # out, lse, dq, dk, dv are deterministic
        assert torch.equal(a, c), i
    # the phase-bias gradient is accumulated by atomics into a buffer the CALLER zero-fills: the capture holds the
    # zero-fill of the eager wrapper, so a replay accumulates on top of whatever the buffer holds
    assert torch.isfinite(got[-1]).all()
    assert _native.device_status() == 0


def test_similarity_and_decode_replay_bitwise():
    g = torch.Generator().manual_seed(22)
    q, k = (torch.randn(1, 4, 300, 64, generator=g).to(DEV) for _ in range(2))
    emb = PoPE(64, heads=4).to(DEV)(300)
    f, b = emb.freqs.detach().contiguous(), emb.bias.detach().contiguous()
    ref = _native.sim_forward(q, k, f, b).clone()
    graph, res = _capture(lambda: _native.sim_forward(q, k, f, b))
    res.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(res, ref)

    qd = torch.randn(2, 4, 1, 128, generator=g).bfloat16().to(DEV)
    kd, vd = (torch.randn(2, 4, 2048, 128, generator=g).bfloat16().to(DEV) for _ in range(2))
    e2 = PoPE(64, heads=4).to(DEV)(2048)
    f2, b2 = e2.freqs.detach().contiguous(), e2.bias.detach().contiguous()
    ref_o, _ = _native.attn_forward(qd, kd, vd, f2, b2, None, False, 128 ** -0.5)
    ref_o = ref_o.clone()
    assert _native.last_path() == "decode_stream"
    graph, res = _capture(lambda: _native.attn_forward(qd, kd, vd, f2, b2, None, False, 128 ** -0.5))
    res[0].zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(res[0], ref_o) and _native.device_status() == 0
