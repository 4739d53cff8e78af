"""Benchmark of the PoPE flash-attention training step (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload = the training-shape configuration the headline metric is quoted on: bf16, B=4, H=16,
N=4096, head dim 128, PoPE dim 128, causal, q,k,v,dO ~ N(0,1) (seeded, synthetic).  One step =
one forward + one backward over that batch.  With N > 1 GPUs every rank processes its own batch
of the same shape (batch x heads units are independent: weak scaling, no collective on the
path); the reported value is the sum over ranks divided by the slowest rank's time.

Prints ONE JSON line.  `value` is timed with inputs resident in HBM; `e2e` is timed through the
public API with pinned HOST buffers, copies inside the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = dict(name="train_fwd_bwd_B4_H16_N4096_d128_r128_causal_bf16", B=4, H=16, N=4096, d=128, r=128, causal=True)
METRIC = "pope_flash_attn_fwd_bwd_tflops_per_job"
UNIT = "TFLOP/s"


def algorithmic_flops(B, H, N, d, r, causal=True):
    """fwd 2*U*pairs*(2d+r) + bwd 2*U*pairs*(5d+3r); pairs = N^2/2 when causal; elementwise work counts 0."""
    pairs = N * N / 2 if causal else N * N
    return 2.0 * B * H * pairs * (7 * d + 4 * r)


def make_inputs(seed, w, device=None, pin=False):
    g = torch.Generator().manual_seed(seed)
    shape = (w["B"], w["H"], w["N"], w["d"])
    ts = [torch.randn(*shape, generator=g).bfloat16() for _ in range(4)]
    if pin:
        ts = [t.pin_memory() for t in ts]
    if device is not None:
        ts = [t.to(device) for t in ts]
    return ts


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(bf16_tflops=p["bf16_tflops"], bf16_tflops_sustained=p.get("bf16_tflops_sustained"),
                    hbm_gbs=p["hbm_gbs"], source="measured")
    return dict(bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.path = gpu_index, None, None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "20"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, reasons, mx = [], set(), None
        for line in open(self.path).read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), (mx := float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            sm.sort()
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))
        return out


# ---------------------------------------------------------------------------------------------
# CPU baseline: the oracle (a port of the reference's pure-PyTorch path) on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_baseline_run(w, units, threads):
    """Time forward+backward of `units` (b,h) slices of the workload with the CPU oracle.
    Returns seconds.  Units are independent, so whole-job time = this * (B*H / units)."""
    from oracle import pope_oracle as O      # checker / CPU baseline only
    from pope_pytorch_b200 import PoPE
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(77)
    N, d, r = w["N"], w["d"], w["r"]
    emb = PoPE(r, heads=1)(N)
    freqs, bias = emb.freqs.detach(), emb.bias.detach()
    total = 0.0
    for _ in range(units):
        q, k, v, do = (torch.randn(1, 1, N, d, generator=g).bfloat16().float() for _ in range(4))
        t0 = time.perf_counter()
        O.attention_with_grads(q, k, v, freqs, bias, do, causal=w["causal"])
        total += time.perf_counter() - t0
    return total


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's CPU implementation of the path (oracle port: the reference
    checkout is not present on the benchmark machine) on all host cores, bounded sample per step."""
    if rank != 0:
        return
    w = WORKLOAD
    threads = os.cpu_count() or 1
    units_per_step = 2
    U = w["B"] * w["H"]
    for _ in range(args.warmup):
        cpu_baseline_run(w, 1, threads)
    secs = [cpu_baseline_run(w, units_per_step, threads) for _ in range(args.steps)]
    per_step_job = sum(secs) / len(secs) * (U / units_per_step)      # one rank's whole batch
    flops = algorithmic_flops(**{k_: w[k_] for k_ in ("B", "H", "N", "d", "r", "causal")})
    value = flops / per_step_job / 1e12
    line = dict(metric=METRIC, value=value, unit=UNIT, impl="reference", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=per_step_job * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=w["name"], note="CPU path runs in fp32 on bf16-rounded inputs"),
                tokens_per_s=w["B"] * w["N"] / per_step_job,
                cpu_baseline=dict(value=value, unit=UNIT, cores=threads, kind="port",
                                  sample=f"{units_per_step} of {U} (b,h) units per step, fwd+bwd, scaled by {U // units_per_step}"),
                e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    from pope_pytorch_b200 import PoPE, flash_attn_with_pope, _native

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    _native.load_library()                      # fail loudly when the native library is missing
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    w = WORKLOAD
    B, H, N, d, r = w["B"], w["H"], w["N"], w["d"], w["r"]
    pope = PoPE(r, heads=H).to(dev)
    with torch.no_grad():
        pope.bias.uniform_(-6.0, 0.0)
    emb = pope(N)
    freqs, bias = emb.freqs.detach().contiguous(), emb.bias.detach().contiguous()
    scale = d ** -0.5
    q, k, v, do = make_inputs(2000 + rank, w, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3 * max(args.steps, 1))]

    def step(i=None):
        if i is not None:
            ev[3 * i].record()
        out, lse = _native.attn_forward(q, k, v, freqs, bias, None, True, scale)
        if i is not None:
            ev[3 * i + 1].record()
        grads = _native.attn_backward(do, q, k, v, out, lse, freqs, bias, None, True, scale, False, True)
        if i is not None:
            ev[3 * i + 2].record()
        return out, grads

    for _ in range(max(args.warmup, 3)):
        step()
    path = _native.last_path()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for i in range(args.steps):
        step(i)
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = max_over_ranks(t_start.elapsed_time(t_end))
    ms_per_step = total_ms / args.steps
    fwd_ms = sum(ev[3 * i].elapsed_time(ev[3 * i + 1]) for i in range(args.steps)) / args.steps
    bwd_ms = sum(ev[3 * i + 1].elapsed_time(ev[3 * i + 2]) for i in range(args.steps)) / args.steps

    flops_rank = algorithmic_flops(B, H, N, d, r, True)
    value = flops_rank * world / (ms_per_step * 1e-3) / 1e12
    # kernels of this library per step -- exact-arithmetic path: fwd, delta, dq, dkdv; tensor-core path:
    # phase table + operand images + fwd, then phase table + operand images + row statistics + dq + dkdv
    launches_per_step = 4 if path == "simt" else 8

    # ---- end to end: pinned host buffers -> public API -> results back on the host -------------
    hq, hk, hv, hdo = make_inputs(3000 + rank, w, pin=True)
    h_out = [torch.empty_like(hq).pin_memory() for _ in range(4)]
    h_dbias = torch.empty(H, r).pin_memory()

    # The step is cut along the batch axis and software-pipelined over three streams (host->device copies, compute,
    # device->host copies): PCIe is full duplex, so chunk c+1 arrives and chunk c-1 leaves while chunk c computes.
    # Everything still goes through the public API, one call per chunk; the phase-bias gradient is summed over chunks.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    chunks = B

    def e2e_step():
        main = torch.cuda.current_stream()
        keep = []                       # tensors stay referenced until the final synchronize (they cross streams)
        dbias_acc = torch.zeros(H, r, device=dev)
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        arrived = []
        for c in range(chunks):
            with torch.cuda.stream(s_in):
                xs = [t[c:c + 1].to(dev, non_blocking=True) for t in (hq, hk, hv, hdo)]
                ev = torch.cuda.Event()
                ev.record(s_in)
            arrived.append((xs, ev))
        for c in range(chunks):
            xs, ev = arrived[c]
            main.wait_event(ev)
            dq_, dk_, dv_ = (t.requires_grad_(True) for t in xs[:3])
            bias_p = bias.clone().requires_grad_(True)
            out = flash_attn_with_pope(dq_, dk_, dv_, pos_emb=(freqs, bias_p), causal=True)
            out.backward(xs[3])
            dbias_acc += bias_p.grad
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(h_out, (out.detach(), dq_.grad, dk_.grad, dv_.grad)):
                    dst[c:c + 1].copy_(src, non_blocking=True)
            keep.append((xs, out, dq_, dk_, dv_, bias_p))
        main.wait_stream(s_out)
        h_dbias.copy_(dbias_acc, non_blocking=True)
        main.synchronize()
        s_out.synchronize()

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(e2e_steps):
        e2e_step()
    e_end.record()
    barrier()
    e2e_ms = max_over_ranks(e_start.elapsed_time(e_end)) / e2e_steps
    e2e_value = flops_rank * world / (e2e_ms * 1e-3) / 1e12
    tensor_bytes = hq.numel() * hq.element_size()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    achieved = flops_rank / (ms_per_step * 1e-3) / 1e12
    pairs = N * N / 2
    bwd_flops = 2.0 * B * H * pairs * (5 * d + 3 * r)
    fwd_flops = 2.0 * B * H * pairs * (2 * d + r)
    bwd_achieved = bwd_flops / (bwd_ms * 1e-3) / 1e12
    peak_sus = pk["bf16_tflops_sustained"] or pk["bf16_tflops"]

    # secondary workloads of the same path (HBM-bound): fp32 similarity and single-token decode
    secondary = {}
    try:
        sq, sk = (torch.randn(1, 8, 4096, 64, device=dev) for _ in range(2))
        semb = PoPE(64, heads=8).to(dev)(4096)
        sf, sb = semb.freqs.contiguous(), semb.bias.detach().contiguous()
        dq1 = torch.randn(8, 32, 1, 128, device=dev).bfloat16()
        dk1, dv1 = (torch.randn(8, 32, 32768, 128, device=dev).bfloat16() for _ in range(2))
        demb = PoPE(64, heads=32).to(dev)(32768)
        df, db = demb.freqs.contiguous(), demb.bias.detach().contiguous()

        def timed(fn, iters=10):
            for _ in range(3):
                fn()
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a_.record()
            for _ in range(iters):
                fn()
            b_.record()
            torch.cuda.synchronize()
            return a_.elapsed_time(b_) / iters

        t_sim = timed(lambda: _native.sim_forward(sq, sk, sf, sb))
        sim_bytes = 8 * 4096 * 4096 * 4 + 2 * 8 * 4096 * 64 * 4 + 4096 * 64 * 4
        secondary["similarity_fp32_1x8x4096x64"] = dict(ms=t_sim, algorithmic_gb_s=sim_bytes / t_sim / 1e6,
                                                        frac_of_hbm_peak=sim_bytes / t_sim / 1e6 / pk["hbm_gbs"],
                                                        path=_native.last_path())
        t_dec = timed(lambda: _native.attn_forward(dq1, dk1, dv1, df, db, None, False, 128 ** -0.5), iters=5)
        dec_bytes = 2 * 8 * 32 * 32768 * 128 * 2
        secondary["decode_bf16_8x32x32768x128_r64"] = dict(ms=t_dec, algorithmic_gb_s=dec_bytes / t_dec / 1e6,
                                                           frac_of_hbm_peak=dec_bytes / t_dec / 1e6 / pk["hbm_gbs"],
                                                           path=_native.last_path())
        del dk1, dv1
    except Exception as exc:  # the headline line must still print
        secondary["error"] = repr(exc)
    line = dict(
        metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
        ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
        data="synthetic",
        config=dict(workload=w["name"], per_gpu_batch=B, global_batch=B * world, heads=H, seq_len=N, head_dim=d,
                    rotate_dim=r, causal=True, sharding=f"batch x heads units, {world} rank(s), no collective",
                    l2="per-step working set (inputs, outputs and operand images: 0.9 GB) exceeds the 126 MB L2; no explicit flush", kernel_path=path),
        tokens_per_s=B * N * world / (ms_per_step * 1e-3),
        fwd_ms=fwd_ms, bwd_ms=bwd_ms,
        pct_of_nominal_bf16_peak=100.0 * achieved / 2250.0,
        roofline=dict(bound="tensor", achieved=bwd_achieved, peak=peak_sus, unit="TFLOP/s", frac=bwd_achieved / peak_sus,
                      traffic=4 * (101.2e6 + 8.6e6 + 101.3e6 + 16.1e6),
                      kernel="backward pass = attn_bwd_dkdv_tc_kernel + attn_bwd_dq_tc_kernel (90 % of its time; the rest "
                             "is its pre-pass: operand images, row statistics, phase tables; one C-ABI call launches all "
                             "of it, timed together with CUDA events on the launch stream)",
                      peak_source=f"{pk['source']} sustained bf16 GEMM (kernels timed inside a long step)",
                      algorithmic_flops_per_launch=bwd_flops,
                      traffic_note="dram read+write bytes of the dq and dkdv launches of one ncu capture at B=1 (109.8 MB dq, "
                                   "117.4 MB dkdv), scaled by 4: traffic is proportional to the number of (b,h) units",
                      forward=dict(achieved=fwd_flops / (fwd_ms * 1e-3) / 1e12, frac=fwd_flops / (fwd_ms * 1e-3) / 1e12 / peak_sus,
                                   what="forward call (tables + images + attn_fwd_tc_kernel), algorithmic flops 2*U*pairs*(2d+r)"),
                      step=dict(achieved=achieved, frac=achieved / peak_sus, frac_of_burst_peak=achieved / pk["bf16_tflops"],
                                what="forward + backward of one step, algorithmic flops 2*U*pairs*(7d+4r)")),
        secondary=secondary,
        e2e=dict(value=e2e_value, unit=UNIT, ms_per_step=e2e_ms, h2d_bytes_per_step=4 * tensor_bytes,
                 d2h_bytes_per_step=4 * tensor_bytes + h_dbias.numel() * 4, steps=e2e_steps,
                 api="flash_attn_with_pope(...).backward() per batch element, pipelined over copy-in / compute / copy-out streams; pinned host q,k,v,dO in; out,dq,dk,dv,dbias back to host"),
        gpu_launches=launches_per_step * args.steps,
        clocks=clocks,
    )
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        units = 4
        cpu_baseline_run(w, 1, threads)
        secs = cpu_baseline_run(w, units, threads)
        job = secs * (B * H / units)
        line["cpu_baseline"] = dict(value=flops_rank / job / 1e12, unit=UNIT, cores=threads, kind="port",
                                    ms_per_step=job * 1e3,
                                    sample=f"{units} of {B * H} (b,h) units, fwd+bwd in fp32 via the CPU oracle, scaled by {B * H // units}")
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
