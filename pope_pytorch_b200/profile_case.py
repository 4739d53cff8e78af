"""Run one operator of the library a few times on seeded synthetic inputs -- the small driver to put under
a profiler (`ncu -k regex:attn_fwd_tc ... python -m pope_pytorch_b200.profile_case --op fwd ...`) or to time
a single shape from the command line.

    python -m pope_pytorch_b200.profile_case --op fwd|bwd|step|sim|decode [--B 1 --H 16 --N 4096 --d 128 --r 128]
                                             [--causal] [--dtype bf16|fp16|fp32] [--iters 3] [--time]
"""
from __future__ import annotations

import argparse

import torch

from . import PoPE, _native


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="fwd", choices=["fwd", "bwd", "step", "sim", "decode"])
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--H", type=int, default=16)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--r", type=int, default=128)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--time", action="store_true", help="print CUDA-event milliseconds per iteration")
    a = ap.parse_args()

    dev = torch.device("cuda")
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    g = torch.Generator().manual_seed(0)
    nq = 1 if a.op == "decode" else a.N
    q = torch.randn(a.B, a.H, nq, a.d, generator=g).to(dtype).to(dev)
    k, v = (torch.randn(a.B, a.H, a.N, a.d, generator=g).to(dtype).to(dev) for _ in range(2))
    do = torch.randn(a.B, a.H, nq, a.d, generator=g).to(dtype).to(dev)
    emb = PoPE(a.r, heads=a.H).to(dev)(a.N)
    freqs, bias = emb.freqs.contiguous(), emb.bias.detach().contiguous()
    scale = a.d ** -0.5
    causal = a.causal and a.op != "decode"

    out, lse = _native.attn_forward(q, k, v, freqs, bias, None, causal, scale)

    def run():
        nonlocal out, lse
        if a.op in ("fwd", "decode"):
            out, lse = _native.attn_forward(q, k, v, freqs, bias, None, causal, scale)
        elif a.op == "bwd":
            _native.attn_backward(do, q, k, v, out, lse, freqs, bias, None, causal, scale, False, True)
        elif a.op == "step":
            out, lse = _native.attn_forward(q, k, v, freqs, bias, None, causal, scale)
            _native.attn_backward(do, q, k, v, out, lse, freqs, bias, None, causal, scale, False, True)
        else:
            _native.sim_forward(q, k, freqs, bias)

    run()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(a.iters):
        run()
    stop.record()
    torch.cuda.synchronize()
    print(f"{a.op} path={_native.last_path()} status={_native.device_status()}"
          + (f" ms/iter={start.elapsed_time(stop) / a.iters:.4f}" if a.time else ""))


if __name__ == "__main__":
    main()
