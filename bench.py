"""Benchmark of the PoPE flash-attention training step (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case fwd|bwd|step|sim|sim_bwd|decode [--B 1 --H 16 --N 4096 --d 128 --r 128 --causal
                    --dtype bf16 --iters 1 --time]          # one operator on one shape, for profilers

Workload = the training-shape configuration the headline metric is quoted on: bf16, B=4, H=16,
N=4096, head dim 128, PoPE dim 128, causal, q,k,v,dO ~ N(0,1) (seeded, synthetic).  One step =
one forward + one backward over that batch.  With N > 1 GPUs every rank processes its own batch
of the same shape (batch x heads units are independent: weak scaling, no collective on the
path); the reported value is the sum over ranks divided by the slowest rank's time.  The same
line carries, under `long_context`, the long-context causal forward (B=8, H=32, N=32768, d=128,
PoPE dim 64) with its 256 units block-partitioned over the ranks (strong scaling, tokens/s).

Prints ONE JSON line.  `value` is timed with inputs resident in HBM; `e2e` is timed through the
public API with pinned HOST buffers, copies inside the timed region.

`--impl reference` times the reference's own CPU implementation of the path (its pure-PyTorch
branch, imported unmodified from baseline/_ref when that install is present, else the CPU oracle
port) on all host cores; it imports nothing of the product package.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
REF_DIR = os.path.join(ROOT, "baseline", "_ref")

WORKLOAD = dict(name="train_fwd_bwd_B4_H16_N4096_d128_r128_causal_bf16", B=4, H=16, N=4096, d=128, r=128, causal=True)
LONG = dict(name="long_context_fwd_B8_H32_N32768_d128_r64_causal_bf16", B=8, H=32, N=32768, d=128, r=64)
METRIC = "pope_flash_attn_fwd_bwd_tflops_per_job"
UNIT = "TFLOP/s"

# DRAM bytes (read + write) per launch of each kernel of one training step at B=1 (16 units), from the ncu
# captures summarised under profiles/ (dram__bytes_read.sum + dram__bytes_write.sum); traffic is proportional to
# the number of (batch, head) units, so a B=4 launch moves 4x these.  Constants, not live measurements.
NCU_TRAFFIC_B1 = {
    "fwd": {"expand_image_kernel": 18.9e6, "attn_fwd_tc_kernel": 71.2e6},
    "bwd": {"bwd_rowstat_kernel": 33.8e6, "expand_image_kernel": 45.9e6, "attn_bwd_dq_tc_kernel": 106.1e6,
            "attn_bwd_dkdv_tc_kernel": 113.9e6},
}


def fwd_flops(B, H, N, d, r, causal=True):
    pairs = N * N / 2 if causal else N * N
    return 2.0 * B * H * pairs * (2 * d + r)


def bwd_flops(B, H, N, d, r, causal=True):
    pairs = N * N / 2 if causal else N * N
    return 2.0 * B * H * pairs * (5 * d + 3 * r)


def algorithmic_flops(B, H, N, d, r, causal=True):
    """fwd 2*U*pairs*(2d+r) + bwd 2*U*pairs*(5d+3r); pairs = N^2/2 when causal; elementwise work counts 0."""
    return fwd_flops(B, H, N, d, r, causal) + bwd_flops(B, H, N, d, r, causal)


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
        self.gpu_index, self.proc, self.path, self.skip = gpu_index, None, None, 0

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "20"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def wait_running(self, timeout_s=3.0):
        """Block until nvidia-smi has written its first sample (it needs a few hundred ms to start), then remember
        how many idle samples to discard: only samples taken from here on count."""
        if self.proc is None:
            return
        t_end = time.time() + timeout_s
        while time.time() < t_end:
            try:
                n = sum(1 for _ in open(self.path))
            except OSError:
                n = 0
            if n > 0:
                self.skip = n
                return
            time.sleep(0.02)

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
        for line in open(self.path).read().splitlines()[self.skip:]:
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


def event_times(fn, iters, warmup=3, flush=None):
    """Per-iteration CUDA-event milliseconds of fn() on the current stream.  `flush` (a tensor larger than L2) is
    overwritten before every timed iteration when the working set would otherwise stay L2-resident."""
    for _ in range(warmup):
        fn()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in evs:
        if flush is not None:
            flush.zero_()
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in evs]


def med_best(ts):
    return dict(ms=statistics.median(ts), ms_best=min(ts), iters=len(ts))


# ---------------------------------------------------------------------------------------------
# the reference's CPU path on the host cores (no import of the product package)
# ---------------------------------------------------------------------------------------------

def _reference_module():
    """The unmodified reference package from baseline/_ref, or None when that install is absent."""
    if not os.path.isdir(os.path.join(REF_DIR, "PoPE_pytorch")):
        return None
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        import PoPE_pytorch as ref
        return ref
    except Exception:
        return None


def cpu_baseline_run(w, units, threads):
    """Time forward+backward of `units` (b,h) slices of the workload on the host cores with the reference's
    pure-PyTorch path (`fused=False`) when the reference install is present, else with the CPU oracle port.
    Returns (seconds, kind).  Units are independent, so whole-job time = this * (B*H / units)."""
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(77)
    N, d, r = w["N"], w["d"], w["r"]
    ref = _reference_module()
    total = 0.0
    if ref is not None:
        pope = ref.PoPE(r, heads=1)
        for _ in range(units):
            q, k, v, do = (torch.randn(1, 1, N, d, generator=g).bfloat16().float() for _ in range(4))
            q, k, v = (t.requires_grad_(True) for t in (q, k, v))
            t0 = time.perf_counter()
            out = ref.flash_attn_with_pope(q, k, v, pos_emb=pope(N), causal=w["causal"], fused=False)
            out.backward(do)
            total += time.perf_counter() - t0
        return total, "reference"
    from oracle import pope_oracle as O      # CPU baseline only
    freqs = O.pope_freqs(torch.arange(N, dtype=torch.float32), O.pope_inv_freqs(r))
    bias = torch.zeros(1, r)
    for _ in range(units):
        q, k, v, do = (torch.randn(1, 1, N, d, generator=g).bfloat16().float() for _ in range(4))
        t0 = time.perf_counter()
        O.attention_with_grads(q, k, v, freqs, bias, do, causal=w["causal"])
        total += time.perf_counter() - t0
    return total, "port"


def run_reference_arm(args, rank, world):
    """`--impl reference`: the reference's CPU implementation of the path on all host cores, a bounded sample of
    the workload per step (2 of its 64 units, scaled: the units are independent)."""
    if rank != 0:
        return
    w = WORKLOAD
    threads = os.cpu_count() or 1
    units_per_step = 2
    U = w["B"] * w["H"]
    kind = "port"
    for _ in range(args.warmup):
        cpu_baseline_run(w, 1, threads)
    secs = []
    for _ in range(args.steps):
        s, kind = cpu_baseline_run(w, units_per_step, threads)
        secs.append(s)
    per_step_job = sum(secs) / len(secs) * (U / units_per_step)      # one rank's whole batch
    flops = algorithmic_flops(**{k_: w[k_] for k_ in ("B", "H", "N", "d", "r", "causal")})
    value = flops / per_step_job / 1e12
    line = dict(metric=METRIC, value=value, unit=UNIT, impl="reference", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=per_step_job * 1e3, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=w["name"], note="CPU path runs in fp32 on bf16-rounded inputs"),
                tokens_per_s=w["B"] * w["N"] / per_step_job,
                cpu_baseline=dict(value=value, unit=UNIT, cores=threads, kind=kind,
                                  sample=f"{units_per_step} of {U} (b,h) units per step, fwd+bwd, scaled by {U // units_per_step}"),
                e2e=dict(value=value, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------
# the reference's own Triton kernels on the same GPU (child process, bounded)
# ---------------------------------------------------------------------------------------------

def reference_triton_child():
    """Runs in a child process: the unmodified reference, `fused=True`, on the training shape (fwd+bwd) and on
    the fp32 similarity configuration; first (JIT-compiling) call excluded.  Prints one JSON object."""
    ref = _reference_module()
    if ref is None:
        print(json.dumps(dict(unavailable="reference install baseline/_ref not present")))
        return
    dev = torch.device("cuda")
    w = WORKLOAD
    B, H, N, d, r = w["B"], w["H"], w["N"], w["d"], w["r"]
    res = {}
    try:
        q, k, v, do = make_inputs(2000, w, device=dev)
        pope = ref.PoPE(r, heads=H).to(dev)

        def step():
            qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
            out = ref.flash_attn_with_pope(qq, kk, vv, pos_emb=pope(N), causal=True, fused=True)
            out.backward(do)

        def fwd():
            with torch.no_grad():
                ref.flash_attn_with_pope(q, k, v, pos_emb=pope(N), causal=True, fused=True)

        step()
        torch.cuda.synchronize()
        ts = event_times(step, 5, warmup=1)
        tf = event_times(fwd, 5, warmup=1)
        fl = algorithmic_flops(B, H, N, d, r, True)
        res["train_step"] = dict(**med_best(ts), tflops=fl / (statistics.median(ts) * 1e-3) / 1e12,
                                 fwd_ms=statistics.median(tf))
    except Exception as exc:
        res["train_step"] = dict(unavailable=repr(exc)[:300])
    try:
        g = torch.Generator().manual_seed(1001)
        sq, sk = (torch.randn(1, 8, 1024, 64, generator=g).to(dev) for _ in range(2))
        spope = ref.PoPE(64, heads=8).to(dev)
        sim = lambda: ref.compute_attn_similarity(sq, sk, spope(1024))
        with torch.no_grad():
            sim()
            torch.cuda.synchronize()
            ts = event_times(sim, 20, warmup=2)
        res["similarity_fp32_1x8x1024x64"] = med_best(ts)
    except Exception as exc:
        res["similarity_fp32_1x8x1024x64"] = dict(unavailable=repr(exc)[:300])
    print(json.dumps(res))


def reference_triton(timeout_s=420):
    if not os.path.isdir(os.path.join(REF_DIR, "PoPE_pytorch")):
        return dict(unavailable="reference install baseline/_ref not present (python baseline/install_ref.py <checkout>)")
    try:
        out = subprocess.run([sys.executable, os.path.abspath(__file__), "--case", "reference_triton"], capture_output=True,
                             text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return dict(unavailable=f"reference Triton run exceeded {timeout_s} s")
    for line in reversed(out.stdout.strip().splitlines()):
        if line.startswith("{"):
            try:
                return json.loads(line)
            except ValueError:
                break
    tail = (out.stderr or out.stdout).strip().splitlines()
    return dict(unavailable=(tail[-1] if tail else f"exit code {out.returncode}")[:300])


# ---------------------------------------------------------------------------------------------
# one operator on one shape (the entry point to put under a profiler)
# ---------------------------------------------------------------------------------------------

def run_case(a):
    if a.case == "reference_triton":
        reference_triton_child()
        return
    from pope_pytorch_b200 import PoPE, _native
    dev = torch.device("cuda")
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    g = torch.Generator().manual_seed(0)
    nq = 1 if a.case in ("decode", "decode_paged") else a.N
    q = torch.randn(a.B, a.H, nq, a.d, generator=g).to(dtype).to(dev)
    k, v = (torch.randn(a.B, a.H, a.N, a.d, generator=g).to(dtype).to(dev) for _ in range(2))
    do = torch.randn(a.B, a.H, nq, a.d, generator=g).to(dtype).to(dev)
    emb = PoPE(a.r, heads=a.H).to(dev)(a.N)
    freqs, bias = emb.freqs.contiguous(), emb.bias.detach().contiguous()
    scale = a.d ** -0.5
    causal = a.causal and a.case != "decode"
    out = lse = dsim = cache = None
    if a.case == "decode_paged":
        from pope_pytorch_b200 import PagedKVCache
        pages = a.B * (a.N // 256 + 2)
        cache = PagedKVCache(a.B, a.H, a.d, num_pages=pages, page_size=256, dtype=dtype, device=dev)
        cache.alloc.free = torch.randperm(pages, generator=g).tolist()
        cache.append(k, v)
    if a.case in ("fwd", "bwd", "step", "decode"):
        out, lse = _native.attn_forward(q, k, v, freqs, bias, None, causal, scale)
    if a.case == "sim_bwd":
        dsim = torch.randn(a.B, a.H, a.N, a.N, device=dev, dtype=dtype)

    def run():
        nonlocal out, lse
        if a.case in ("fwd", "decode"):
            out, lse = _native.attn_forward(q, k, v, freqs, bias, None, causal, scale)
        elif a.case == "bwd":
            _native.attn_backward(do, q, k, v, out, lse, freqs, bias, None, causal, scale, False, True)
        elif a.case == "step":
            out, lse = _native.attn_forward(q, k, v, freqs, bias, None, causal, scale)
            _native.attn_backward(do, q, k, v, out, lse, freqs, bias, None, causal, scale, False, True)
        elif a.case == "decode_paged":
            out = cache.decode(q, (freqs, bias), softmax_scale=scale)
        elif a.case == "sim":
            _native.sim_forward(q, k, freqs, bias)
        else:
            _native.sim_backward(dsim, q, k, freqs, bias, False, True)

    ts = event_times(run, a.iters, warmup=1)
    print(f"{a.case} path={_native.last_path()} status={_native.device_status()}"
          + (f" ms median={statistics.median(ts):.4f} best={min(ts):.4f}" if a.time else ""))


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------

def secondary_workloads(dev, pk, PoPE, AxialPoPE, _native):
    """The other configurations of the same path: latency of the small ones, HBM fraction of the memory-bound ones,
    tensor fraction of the compute-bound ones.  Every entry: median and best CUDA-event ms over its iterations."""
    sec = {}
    burst = pk["bf16_tflops"]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # larger than the 126 MB L2

    def guarded(name, fn):
        try:
            sec[name] = fn()
        except Exception as exc:      # the headline line must still print
            sec[name] = dict(error=repr(exc)[:300])
        torch.cuda.empty_cache()

    def sim_case(n, iters):
        def run():
            g = torch.Generator().manual_seed(1001)
            q, k = (torch.randn(1, 8, n, 64, generator=g).to(dev) for _ in range(2))
            emb = PoPE(64, heads=8).to(dev)(n)
            f, b = emb.freqs.contiguous(), emb.bias.detach().contiguous()
            ts = event_times(lambda: _native.sim_forward(q, k, f, b), iters, flush=flush)
            nbytes = 8 * n * n * 4 + 2 * 8 * n * 64 * 4 + n * 64 * 4 + 8 * 64 * 4
            gbs = nbytes / statistics.median(ts) / 1e6
            return dict(**med_best(ts), algorithmic_bytes=nbytes, algorithmic_gb_s=gbs, frac_of_hbm_peak=gbs / pk["hbm_gbs"],
                        path=_native.last_path(), l2="flushed between iterations")
        return run

    guarded("similarity_fp32_1x8x1024x64_config1", sim_case(1024, 20))
    guarded("similarity_fp32_1x8x4096x64", sim_case(4096, 10))
    guarded("similarity_fp32_1x8x8192x64", sim_case(8192, 5))

    def sim_bwd():
        n = 4096
        g = torch.Generator().manual_seed(1001)
        q, k = (torch.randn(1, 8, n, 64, generator=g).to(dev) for _ in range(2))
        dsim = torch.randn(1, 8, n, n, device=dev)
        emb = PoPE(64, heads=8).to(dev)(n)
        f, b = emb.freqs.contiguous(), emb.bias.detach().contiguous()
        ts = event_times(lambda: _native.sim_backward(dsim, q, k, f, b, False, True), 5, flush=flush)
        nbytes = 8 * n * n * 4
        gbs = nbytes / statistics.median(ts) / 1e6
        return dict(**med_best(ts), algorithmic_bytes=nbytes, algorithmic_gb_s=gbs, frac_of_hbm_peak=gbs / pk["hbm_gbs"],
                    what="dq, dk, dbias from dS (one read of dS counted)", path=_native.last_path())
    guarded("similarity_bwd_fp32_1x8x4096x64", sim_bwd)

    def config2():
        g = torch.Generator().manual_seed(1002)
        q, k, v = (torch.randn(2, 8, 1024, 64, generator=g).bfloat16().to(dev) for _ in range(3))
        emb = PoPE(32, heads=8).to(dev)(1024)
        f, b = emb.freqs.contiguous(), emb.bias.detach().contiguous()
        lens = torch.randint(512, 1025, (2,), generator=g)
        mask = (torch.arange(1024)[None, :] < lens[:, None]).to(dev)
        ts = event_times(lambda: _native.attn_forward(q, k, v, f, b, mask, True, 0.125), 50, flush=flush)
        pairs = sum(min(i + 1, int(l)) for l in lens for i in range(1024))
        fl = 2.0 * 8 * pairs * (2 * 64 + 32)
        return dict(**med_best(ts), algorithmic_tflops=fl / statistics.median(ts) / 1e9, note="latency-bound (2.7 GFLOP)",
                    path=_native.last_path())
    guarded("config2_fwd_2x8x1024x64_r32_causal_padding", config2)

    def config2_graph():
        # the same shape, forward + backward as ONE isolated call (idle GPU, warm L2): eager launches against the replay
        # of a CUDA graph that captured them (3 + 5 launches, the backward's side stream forked and joined inside)
        g = torch.Generator().manual_seed(1002)
        q, k, v, do = (torch.randn(2, 8, 1024, 64, generator=g).bfloat16().to(dev) for _ in range(4))
        emb = PoPE(32, heads=8).to(dev)(1024)
        f, b = emb.freqs.contiguous(), emb.bias.detach().contiguous()
        lens = torch.randint(512, 1025, (2,), generator=g)
        mask = (torch.arange(1024)[None, :] < lens[:, None]).to(dev)

        def step():
            out, lse = _native.attn_forward(q, k, v, f, b, mask, True, 0.125)
            return _native.attn_backward(do, q, k, v, out, lse, f, b, mask, True, 0.125, False, True)

        def isolated(fn, iters=30):
            ts = []
            for _ in range(iters):
                torch.cuda.synchronize()
                a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a_.record(); fn(); b_.record(); torch.cuda.synchronize()
                ts.append(a_.elapsed_time(b_))
            return ts
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        te, tg = isolated(step), isolated(graph.replay)
        return dict(eager_ms=statistics.median(te), graph_replay_ms=statistics.median(tg), eager_ms_best=min(te),
                    graph_replay_ms_best=min(tg), iters=30, status=_native.device_status(),
                    note="one fwd+bwd call on an idle GPU: launch-bound eager, the captured graph removes the host launches")
    guarded("config2_fwd_bwd_isolated_call_eager_vs_cuda_graph", config2_graph)

    def config4():
        g = torch.Generator().manual_seed(1004)
        q, k, v, do = (torch.randn(2, 8, 2048, 96, generator=g).bfloat16().to(dev) for _ in range(4))
        emb = AxialPoPE(96, heads=8, axial_dims=(32, 32, 32)).to(dev)((8, 16, 16))
        f, b = emb.freqs.contiguous(), emb.bias.detach().contiguous()
        sc = 96 ** -0.5

        def step():
            out, lse = _native.attn_forward(q, k, v, f, b, None, False, sc)
            _native.attn_backward(do, q, k, v, out, lse, f, b, None, False, sc, False, True)
        ts = event_times(step, 20, flush=flush)
        fl = algorithmic_flops(2, 8, 2048, 96, 96, False)
        tf = fl / statistics.median(ts) / 1e9
        return dict(**med_best(ts), algorithmic_tflops=tf, frac_of_burst_peak=tf / burst, path=_native.last_path())
    guarded("config4_axial_fwd_bwd_2x8x2048x96_r96", config4)

    def decode():
        g = torch.Generator().manual_seed(1005)
        q = torch.randn(8, 32, 1, 128, device=dev).bfloat16()
        k, v = (torch.randn(8, 32, 32768, 128, device=dev).bfloat16() for _ in range(2))
        emb = PoPE(64, heads=32).to(dev)(32768)
        f, b = emb.freqs.contiguous(), emb.bias.detach().contiguous()
        ts = event_times(lambda: _native.attn_forward(q, k, v, f, b, None, False, 128 ** -0.5), 10)
        nbytes = 2 * 8 * 32 * 32768 * 128 * 2
        gbs = nbytes / statistics.median(ts) / 1e6
        return dict(**med_best(ts), algorithmic_bytes=nbytes, algorithmic_gb_s=gbs, frac_of_hbm_peak=gbs / pk["hbm_gbs"],
                    path=_native.last_path(), l2="K + V = 4.3 GB per iteration, far beyond L2")
    guarded("decode_bf16_8x32x32768x128_r64", decode)

    def decode_paged():
        # the same decode over a paged cache: 8 sequences of 32768 keys in 256-key pages handed out in a scrambled order
        from pope_pytorch_b200 import PagedKVCache
        g = torch.Generator().manual_seed(1005)
        cache = PagedKVCache(8, 32, 128, num_pages=8 * 129, page_size=256, max_seq_len=32768 + 256, dtype=torch.bfloat16, device=dev)
        cache.alloc.free = torch.randperm(8 * 129, generator=g).tolist()
        for c0 in range(0, 32768, 8192):
            k, v = (torch.randn(8, 32, 8192, 128, device=dev).bfloat16() for _ in range(2))
            cache.append(k, v)
        k1, v1 = (torch.randn(8, 32, 1, 128, device=dev).bfloat16() for _ in range(2))
        q = torch.randn(8, 32, 1, 128, device=dev).bfloat16()
        emb = PoPE(64, heads=32).to(dev)(32768 + 64)
        f, b = emb.freqs.contiguous(), emb.bias.detach().contiguous()
        ts = event_times(lambda: cache.decode(q, (f, b)), 10)
        nbytes = 2 * 8 * 32 * 32768 * 128 * 2
        gbs = nbytes / statistics.median(ts) / 1e6
        path = _native.last_path()
        ta = event_times(lambda: cache.append(k1, v1), 10)     # ten single-token appends (the cache grows to 32778)
        return dict(**med_best(ts), algorithmic_bytes=nbytes, algorithmic_gb_s=gbs, frac_of_hbm_peak=gbs / pk["hbm_gbs"], path=path,
                    append_one_token_ms=statistics.median(ta), page_size=256, status=_native.device_status(),
                    l2="K + V = 4.3 GB per iteration, far beyond L2")
    guarded("decode_paged_bf16_8x32x32768x128_r64", decode_paged)
    return sec


def long_context_leg(dev, rank, world, pk, PoPE, _native, plan_shard, barrier, max_over_ranks):
    """Long-context causal forward, B=8 H=32 N=32768 d=128 PoPE dim 64: the 256 (batch, head) units are
    block-partitioned over the ranks by `plan_shard` (strong scaling, no collective on the path); every rank
    generates only its own block.  tokens/s = B * N / slowest rank's time."""
    w = LONG
    plan = plan_shard(w["B"], w["H"], w["H"], rank, world)
    bl, hl = (w["B"], plan.size) if plan.axis == "heads" else (plan.size, w["H"])
    g = torch.Generator(device=dev).manual_seed(5000 + rank)
    q, k, v = (torch.randn(bl, hl, w["N"], w["d"], device=dev, generator=g).bfloat16() for _ in range(3))
    emb = PoPE(w["r"], heads=w["H"]).to(dev)(w["N"])
    freqs = emb.freqs.contiguous()
    bias = emb.bias.detach()[plan.start:plan.start + plan.size].contiguous() if plan.axis == "heads" else emb.bias.detach().contiguous()
    sc = w["d"] ** -0.5
    run = lambda: _native.attn_forward(q, k, v, freqs, bias, None, True, sc)
    for _ in range(2):
        run()
    barrier()
    iters = 3
    a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a_.record()
    for _ in range(iters):
        run()
    b_.record()
    barrier()
    ms = max_over_ranks(a_.elapsed_time(b_)) / iters
    fl = fwd_flops(w["B"], w["H"], w["N"], w["d"], w["r"], True)
    tf = fl / (ms * 1e-3) / 1e12
    return dict(workload=w["name"], scaling="strong", units_total=w["B"] * w["H"], units_per_rank=bl * hl,
                shard_axis=plan.axis, ms=ms, tokens_per_s=w["B"] * w["N"] / (ms * 1e-3), algorithmic_tflops=tf,
                frac_of_burst_peak_per_gpu=tf / world / pk["bf16_tflops"], path=_native.last_path())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary workloads and the reference Triton leg")
    ap.add_argument("--case", default=None, choices=["fwd", "bwd", "step", "sim", "sim_bwd", "decode", "decode_paged", "reference_triton"])
    ap.add_argument("--B", type=int, default=1)
    ap.add_argument("--H", type=int, default=16)
    ap.add_argument("--N", type=int, default=4096)
    ap.add_argument("--d", type=int, default=128)
    ap.add_argument("--r", type=int, default=128)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--time", action="store_true", help="--case: print CUDA-event milliseconds per iteration")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.case is not None:
        run_case(args)
        return
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch.distributed as dist
    from pope_pytorch_b200 import AxialPoPE, PoPE, flash_attn_with_pope, _native
    from pope_pytorch_b200.shard import plan_shard, reduce_bias_grad

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

    # the clock sampler runs from the first warm-up step on (every sample is taken under the same load); it is started
    # early because nvidia-smi takes longer to deliver its first sample than the whole timed region lasts
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        sampler.wait_running()
    barrier()
    for _ in range(max(args.warmup, 3)):
        step()
    path = _native.last_path()
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
    fwd_t = [ev[3 * i].elapsed_time(ev[3 * i + 1]) for i in range(args.steps)]
    bwd_t = [ev[3 * i + 1].elapsed_time(ev[3 * i + 2]) for i in range(args.steps)]
    fwd_ms, bwd_ms = sum(fwd_t) / len(fwd_t), sum(bwd_t) / len(bwd_t)

    flops_rank = algorithmic_flops(B, H, N, d, r, True)
    value = flops_rank * world / (ms_per_step * 1e-3) / 1e12
    # kernels of this library per step -- exact-arithmetic path: fwd, delta, dq, dkdv; tensor-core path:
    # phase table + operand images + fwd, then row statistics + phase table + operand images + dq + dkdv
    launches_per_step = 4 if path == "simt" else 8

    # ---- long-context forward, units sharded over the ranks (strong scaling) --------------------
    pk = peaks()
    try:
        long_context = long_context_leg(dev, rank, world, pk, PoPE, _native, plan_shard, barrier, max_over_ranks)
    except Exception as exc:
        long_context = dict(error=repr(exc)[:300])
    torch.cuda.empty_cache()

    # ---- the one exchange around the path: phase-bias gradient partial sums when the shard cuts the batch ----
    bias_reduce = None
    if world > 1:
        plan_b = plan_shard(world, 1, 1, rank, world)               # one batch element per rank: the batch axis is cut
        part = torch.full((H, r), float(rank + 1), device=dev)
        for _ in range(3):
            reduce_bias_grad(part, plan_b)
        barrier()
        a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_.record()
        for _ in range(20):
            total = reduce_bias_grad(part, plan_b)
        b_.record()
        barrier()
        ok = bool(torch.all(total == world * (world + 1) / 2))
        bias_reduce = dict(what="NCCL all-reduce of the (H, r) fp32 phase-bias gradient partial sums", bytes=H * r * 4,
                           us=max_over_ranks(a_.elapsed_time(b_)) / 20 * 1e3, correct=ok)

    # ---- end to end: pinned host buffers -> public API -> results back on the host -------------
    hq, hk, hv, hdo = make_inputs(3000 + rank, w, pin=True)
    h_out = [torch.empty_like(hq).pin_memory() for _ in range(4)]
    h_dbias = torch.empty(H, r).pin_memory()

    # The step is cut into (batch entry, half of the heads) chunks and software-pipelined over three streams (host->device
    # copies, compute, device->host copies): PCIe is full duplex, so chunk c+1 arrives and chunk c-1 leaves while chunk c
    # computes, and a small last chunk keeps the un-overlapped tail (its compute and its copy back) short.
    # Everything still goes through the public API, one call per chunk; the phase-bias gradient is summed over chunks.
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    hsplit = 2 if H % 2 == 0 else 1
    chunks = B * hsplit
    hpc = H // hsplit

    def chunk_of(t, c):      # (1, hpc, N, d) view of chunk c: contiguous in a (B, H, N, d) tensor
        b_i, h0 = c // hsplit, (c % hsplit) * hpc
        return t[b_i:b_i + 1, h0:h0 + hpc]

    def e2e_step(keep):
        # `keep`: tensors stay referenced until the caller's synchronize (they cross streams).  Nothing here waits for the
        # previous step: its results are still leaving on s_out while this step's inputs arrive on s_in.
        main = torch.cuda.current_stream()
        dbias_acc = torch.zeros(H, r, device=dev)
        arrived = []
        for c in range(chunks):
            with torch.cuda.stream(s_in):
                xs = [chunk_of(t, c).to(dev, non_blocking=True) for t in (hq, hk, hv, hdo)]
                ev_ = torch.cuda.Event()
                ev_.record(s_in)
            arrived.append((xs, ev_))
        for c in range(chunks):
            xs, ev_ = arrived[c]
            main.wait_event(ev_)
            dq_, dk_, dv_ = (t.requires_grad_(True) for t in xs[:3])
            h0 = (c % hsplit) * hpc
            bias_p = bias[h0:h0 + hpc].clone().requires_grad_(True)
            out = flash_attn_with_pope(dq_, dk_, dv_, pos_emb=(freqs, bias_p), causal=True)
            out.backward(xs[3])
            dbias_acc[h0:h0 + hpc] += bias_p.grad
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                for dst, src in zip(h_out, (out.detach(), dq_.grad, dk_.grad, dv_.grad)):
                    chunk_of(dst, c).copy_(src, non_blocking=True)
            keep.append((xs, out, dq_, dk_, dv_, bias_p))
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            h_dbias.copy_(dbias_acc, non_blocking=True)
        keep.append(dbias_acc)

    def e2e_run(n):
        # n steps back to back, every one with its own copies in and out.  The host waits for step s - 1 to have left
        # completely only after it has enqueued step s (then drops that step's tensors, so the allocator reuses their
        # memory): two steps are in flight at most, and the copies out of one overlap the copies in of the next.
        main = torch.cuda.current_stream()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        pending = []
        for _ in range(n):
            keep = []
            e2e_step(keep)
            left = torch.cuda.Event()
            left.record(s_out)
            pending.append((left, keep))
            if len(pending) > 1:
                ev0, keep0 = pending.pop(0)
                ev0.synchronize()
                keep0.clear()
        for ev0, keep0 in pending:
            ev0.synchronize()
            keep0.clear()
        main.wait_stream(s_in)
        main.wait_stream(s_out)
        main.synchronize()

    e2e_steps = max(3, min(args.steps, 10))
    e2e_run(4)
    barrier()
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    e2e_run(e2e_steps)
    e_end.record()
    barrier()
    e2e_ms = max_over_ranks(e_start.elapsed_time(e_end)) / e2e_steps
    e2e_value = flops_rank * world / (e2e_ms * 1e-3) / 1e12
    tensor_bytes = hq.numel() * hq.element_size()
    del hq, hk, hv, hdo, h_out

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    achieved = flops_rank / (ms_per_step * 1e-3) / 1e12
    bfl, ffl = bwd_flops(B, H, N, d, r), fwd_flops(B, H, N, d, r)
    bwd_achieved = bfl / (bwd_ms * 1e-3) / 1e12
    # the denominator follows the length of the timed region: the burst GEMM rate for a region shorter than two
    # seconds (the clocks have not settled under the power cap), the sustained rate for a longer one
    sustained = total_ms >= 2000.0 and pk["bf16_tflops_sustained"]
    peak = pk["bf16_tflops_sustained"] if sustained else pk["bf16_tflops"]
    peak_name = "sustained" if sustained else "burst"
    traffic = {ph: sum(kv.values()) * B for ph, kv in NCU_TRAFFIC_B1.items()} if path != "simt" else None

    secondary = {}
    if not args.no_secondary:
        del q, k, v, do
        torch.cuda.empty_cache()
        secondary = secondary_workloads(dev, pk, PoPE, AxialPoPE, _native)
        secondary["reference_triton"] = reference_triton() if world == 1 else dict(skipped="timed at N=1 only")
        rt = secondary["reference_triton"].get("train_step", {})
        if "ms" in rt:
            secondary["reference_triton"]["ratio_ours_over_reference"] = rt["ms"] / ms_per_step

    line = dict(
        metric=METRIC, value=value, unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
        ms_per_step=ms_per_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
        data="synthetic",
        config=dict(workload=w["name"], per_gpu_batch=B, global_batch=B * world, heads=H, seq_len=N, head_dim=d,
                    rotate_dim=r, causal=True, sharding=f"batch x heads units, {world} rank(s), no collective",
                    l2="per-step working set (inputs, outputs and operand images: 0.9 GB) exceeds the 126 MB L2; no explicit flush", kernel_path=path),
        tokens_per_s=B * N * world / (ms_per_step * 1e-3),
        fwd_ms=fwd_ms, bwd_ms=bwd_ms, fwd_ms_median=statistics.median(fwd_t), bwd_ms_median=statistics.median(bwd_t),
        fwd_ms_best=min(fwd_t), bwd_ms_best=min(bwd_t),
        pct_of_nominal_bf16_peak=100.0 * achieved / 2250.0,
        roofline=dict(bound="tensor", achieved=bwd_achieved, peak=peak, unit="TFLOP/s", frac=bwd_achieved / peak,
                      traffic=traffic["bwd"] if traffic else None,
                      kernel="backward call = bwd_rowstat_kernel + pope_trig_table_f32_kernel + expand_image_kernel + "
                             "attn_bwd_dq_tc_kernel + attn_bwd_dkdv_tc_kernel (the two attention kernels are 90 % of its "
                             "time); one C-ABI call launches all of it, timed together with CUDA events on the launch stream",
                      peak_source=f"{pk['source']} {peak_name} bf16 GEMM rate (timed region {total_ms:.0f} ms)",
                      algorithmic_flops_per_launch=bfl,
                      algorithmic_bytes_per_launch=(8 * B * H * N * d * 2),
                      traffic_note="CONSTANT from ncu captures at B=1 (profiles/), every launch of the backward call summed "
                                   "(pre-pass included) and scaled by 4: traffic is proportional to the number of (b,h) units; "
                                   "algorithmic bytes = q,k,v,out,dO read + dq,dk,dv written",
                      traffic_per_kernel_b1=NCU_TRAFFIC_B1 if traffic else None,
                      frac_of_burst_peak=bwd_achieved / pk["bf16_tflops"],
                      frac_of_sustained_peak=bwd_achieved / (pk["bf16_tflops_sustained"] or pk["bf16_tflops"]),
                      forward=dict(achieved=ffl / (fwd_ms * 1e-3) / 1e12, frac=ffl / (fwd_ms * 1e-3) / 1e12 / peak,
                                   traffic=traffic["fwd"] if traffic else None,
                                   what="forward call (tables + K' images + attn_fwd_tc_kernel), algorithmic flops 2*U*pairs*(2d+r); its K' image (33.5 MB at B=1) is still dirty in L2 when the pre-pass ends, which is why the pre-pass shows 19 MB"),
                      step=dict(achieved=achieved, frac=achieved / peak, frac_of_burst_peak=achieved / pk["bf16_tflops"],
                                what="forward + backward of one step, algorithmic flops 2*U*pairs*(7d+4r)")),
        long_context=long_context,
        bias_grad_reduce=bias_reduce,
        secondary=secondary,
        e2e=dict(value=e2e_value, unit=UNIT, ms_per_step=e2e_ms, h2d_bytes_per_step=4 * tensor_bytes,
                 d2h_bytes_per_step=4 * tensor_bytes + h_dbias.numel() * 4, steps=e2e_steps,
                 api="flash_attn_with_pope(...).backward() per (batch entry, half of the heads), pipelined over copy-in / compute / copy-out streams, consecutive steps back to back (two steps in flight at most: the copies out of step s overlap the copies in of step s+1); pinned host q,k,v,dO in and out,dq,dk,dv,dbias back to host EVERY step",
                 limiter="PCIe: 268 MB each way per step; the ranks of one box share the host's PCIe complex"),
        gpu_launches=launches_per_step * args.steps,
        clocks=clocks,
    )
    if not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        units = 4
        cpu_baseline_run(w, 1, threads)
        secs, kind = cpu_baseline_run(w, units, threads)
        job = secs * (B * H / units)
        line["cpu_baseline"] = dict(value=flops_rank / job / 1e12, unit=UNIT, cores=threads, kind=kind,
                                    ms_per_step=job * 1e3,
                                    sample=f"{units} of {B * H} (b,h) units, fwd+bwd in fp32 on the host cores, scaled by {B * H // units}")
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
