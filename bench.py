"""Benchmark of the three-way attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload: triple-dot-product trittention forward + backward, B=1, N=16 heads, T=2048,
D=128, bf16, causal with full windows, alpha = 1/D, inputs and upstream gradient
N(0,1)*0.5 from a fixed seed (synthetic; the reference uses no dataset).  The 16
(batch*head) slices are independent: with N GPUs every rank takes 16/N heads and there is no
data-path collective.  Total work is fixed, so scaling is "strong".

One JSON line is printed by rank 0.  `value` is algorithmic TFLOP/s (16*D flops per
attended (q, j, k) triple: two GEMM-shaped contractions forward, six backward) with inputs
resident in HBM; `e2e` is the same metric through the public autograd entry point with
host (pinned) inputs and results copied back, all copies inside the timed region.

`--impl reference` times the reference's algorithm on the host cores instead (the CPU
restatement in oracle/, all threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if not os.environ.get("TRITT_BENCH_REFERENCE_WORKER"):
    # (the child process that times the reference's own kernels must import the reference's package of the same
    #  name instead: see reference_kernel_worker)
    for _p in (ROOT, os.path.join(ROOT, "flash-3-way-attention_b200")):
        if _p not in sys.path:
            sys.path.insert(0, _p)

import torch  # noqa: E402

WORK = dict(B=1, N=16, T=2048, D=128, dtype="bf16", causal=True, scale_in=0.5, seed=0)
METRIC = "tdp_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(burst=float(d["bf16_tflops"]), sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm_gbs=6650.0, source="fallback")


def _flops(B, N, T, D, mode="fwd+bwd"):
    per = {"fwd": 4, "bwd": 12, "fwd+bwd": 16}[mode]
    return float(per * D * B * N * (T * (T + 1) * (2 * T + 1) // 6))


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def wait_first(self, timeout: float = 8.0):
        """Returns once the sampler has printed its first line (its start-up enumerates every GPU of the machine and
        can hold up kernel launches for hundreds of milliseconds, which must not fall into a timed region)."""
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < timeout and self.proc.poll() is None:
            time.sleep(0.02)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [x.strip() for x in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def _make_inputs(B, N, T, D, scale, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(B, N, T, D, generator=g, dtype=torch.float32) * scale).to(dtype) for _ in range(6)]


def cpu_reference_sample(threads=None, T_s=896, D=128):
    """The reference algorithm (CPU restatement) on one head at reduced T; returns TFLOP/s."""
    from oracle import trittention_oracle as orc

    if threads:
        torch.set_num_threads(threads)
    q, k1, k2, v1, v2, dz = orc.make_inputs(1, 1, T_s, D, scale=WORK["scale_in"], seed=WORK["seed"])
    t0 = time.perf_counter()
    orc.tdp_forward(q, k1, k2, v1, v2, 1.0 / D, True)
    orc.tdp_backward(q, k1, k2, v1, v2, dz, 1.0 / D, True)
    dt = time.perf_counter() - t0
    fl = _flops(1, 1, T_s, D)
    return fl / dt / 1e12, dt, f"B=1,N=1,T={T_s},D={D} fp32 causal fwd+bwd of the same distribution ({dt:.1f} s)"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    vals, sample = [], ""
    for i in range(args.warmup + args.steps):
        v, dt, sample = cpu_reference_sample(T_s=args.ref_T)
        if i >= args.warmup:
            vals.append((v, dt))
    value = sum(v for v, _ in vals) / len(vals)
    ms = 1e3 * sum(dt for _, dt in vals) / len(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "tdp fwd+bwd B=1 N=16 T=2048 D=128 causal (each step = a bounded sample, see cpu_baseline.sample)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _timed(fn, iters=5):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def other_workloads(dev):
    """Short CUDA-event timings of the other benchmark configurations on one GPU (not part of the headline
    value): config 2 forward, the shapes of the reference's own forward benchmark (b200/bench_b200.py there:
    2 x 8 x {512, 1024} x 64 fp16 full windows, 2 x 8 x 2048 x 64 with windows 128/128/32/32), narrow bands,
    a non-causal case, and config 3 (dot-product-sum) forward+backward."""
    from flash_trittention import flash_trittention
    from flash_trittention.dot_product_sum.trittention_triton import TrittentionTriton

    out = {}
    t = [x.to(dev) for x in _make_inputs(4, 8, 512, 64, 0.5, 2, torch.bfloat16)[:5]]
    with torch.no_grad():
        ms = _timed(lambda: flash_trittention(*t, 1 / 64, None, None, None, None, True))
    out["tdp_fwd_4x8x512x64_bf16"] = {"ms": ms, "tflops": _flops(4, 8, 512, 64, "fwd") / ms / 1e9}
    for T in (512, 1024):
        ins = [x.to(dev) for x in _make_inputs(2, 8, T, 64, 1.0, 3, torch.float16)]
        with torch.no_grad():
            ms = _timed(lambda: flash_trittention(*ins[:5], 1 / 8, None, None, None, None, True))
        out[f"tdp_fwd_2x8x{T}x64_fp16"] = {"ms": ms, "tflops": _flops(2, 8, T, 64, "fwd") / ms / 1e9}
        if T == 512:
            def tdp_step():
                leaves = [x.detach().requires_grad_(True) for x in ins[:5]]
                flash_trittention(*leaves, 1 / 8, None, None, None, None, True).backward(ins[5])

            ms = _timed(tdp_step)
            out["tdp_fwd_bwd_2x8x512x64_fp16"] = {"ms": ms, "tflops": _flops(2, 8, 512, 64) / ms / 1e9}
            # not causal: every (q, j, k) triple is attended, T^3 per head; the kernels execute exactly the
            # algorithmic products forward (T is a multiple of the 128-wide tiles) and 8 for 6 backward
            with torch.no_grad():
                ms = _timed(lambda: flash_trittention(*ins[:5], 1 / 8, None, None, None, None, False))
            fl = 4.0 * 64 * 2 * 8 * T ** 3
            out["tdp_fwd_2x8x512x64_fp16_noncausal"] = {"ms": ms, "tflops": fl / ms / 1e9,
                                                         "executed_over_algorithmic_flops": 1.0}

            def nc_step():
                leaves = [x.detach().requires_grad_(True) for x in ins[:5]]
                flash_trittention(*leaves, 1 / 8, None, None, None, None, False).backward(ins[5])

            ms = _timed(nc_step, iters=3)
            out["tdp_fwd_bwd_2x8x512x64_fp16_noncausal"] = {"ms": ms, "tflops": 4 * fl / ms / 1e9,
                                                             "executed_over_algorithmic_flops": (4 + 16) / 16.0}
    t = [x.to(dev) for x in _make_inputs(2, 8, 2048, 64, 1.0, 3, torch.float16)[:5]]
    with torch.no_grad():
        ms = _timed(lambda: flash_trittention(*t, 1 / 8, 32, 32, 128, 128, True))
        out["tdp_fwd_2x8x2048x64_fp16_windows_128_128_32_32"] = {"ms": ms}
        ms = _timed(lambda: flash_trittention(*t, 1 / 8, 4, 4, 8, 8, True))
        out["tdp_fwd_2x8x2048x64_fp16_windows_8_8_4_4"] = {"ms": ms}
    t = [x.to(dev) for x in _make_inputs(2, 8, 8192, 64, 1.0, 5, torch.float16)[:5]]
    with torch.no_grad():
        ms = _timed(lambda: flash_trittention(*t, 1 / 8, 32, 32, 128, 128, True), iters=3)
    out["tdp_fwd_2x8x8192x64_fp16_windows_128_128_32_32"] = {"ms": ms}
    del t
    ins = [x.to(dev) for x in _make_inputs(2, 8, 1024, 64, 1.0, 4, torch.float16)]
    mod = TrittentionTriton(causal=True, softmax_scale=1 / 8, k_diff=1024)

    def dps_step():
        leaves = [x.detach().requires_grad_(True) for x in ins[:5]]
        o, _ = mod(*leaves)
        o.backward(ins[5])

    out["dps_fwd_bwd_2x8x1024x64_fp16"] = {"ms": _timed(dps_step, iters=20)}
    with torch.no_grad():
        out["dps_fwd_2x8x1024x64_fp16"] = {"ms": _timed(lambda: mod(*ins[:5]), iters=20)}
    return out


REF_DIR = os.path.join(ROOT, "baseline", "_ref")


def reference_kernel_worker():
    """Runs in a child process whose import path holds the unmodified reference package (installed from its own
    pyproject into baseline/_ref, which is not part of the repository's history) and NOT this repository's package of
    the same name: times the reference's Triton kernels on this GPU on the shapes of its own forward benchmark
    (b200/bench_b200.py:107-150 there) and prints one JSON object."""
    import triton.testing as tt
    from b200.flash_trittention_b200 import flash_trittention_b200
    from flash_trittention.triple_dot_product.flash_trittention import flash_trittention as ref_ft

    dev = torch.device("cuda:0")
    res = {"triton": __import__("triton").__version__}

    def bench(fn, rep=60):
        return float(tt.do_bench(fn, warmup=10, rep=rep))

    for T, win, label in ((512, None, "full"), (1024, None, "full"), (2048, (128, 128, 32, 32), "windows_128_128_32_32")):
        ins = [x.to(dev) for x in _make_inputs(2, 8, T, 64, 1.0, 3, torch.float16)]
        w = win or (T, T, T, T)
        kw = dict(softmax_scale=1 / 8, k1_window=w[0], k2_window=w[1], kk_left=w[2], kk_right=w[3], causal=True)
        with torch.no_grad():
            a = ref_ft(*ins[:5], **kw)
            b = flash_trittention_b200(*ins[:5], **kw)
            res[f"fwd_2x8x{T}x64_fp16_{label}"] = {
                "generic_ms": bench(lambda: ref_ft(*ins[:5], **kw)),
                "b200_ms": bench(lambda: flash_trittention_b200(*ins[:5], **kw)),
                "generic_vs_b200_max_abs_diff": float((a.float() - b.float()).abs().max())}
        if T == 512:
            def step():
                leaves = [x.detach().requires_grad_(True) for x in ins[:5]]
                ref_ft(*leaves, **kw).backward(ins[5])

            step()
            torch.cuda.synchronize()
            res["fwd_bwd_2x8x512x64_fp16_full"] = {"generic_ms": _timed(step, iters=3)}
    # dot-product-sum, config 3 (the reference's TrittentionTriton module, forward and forward + backward)
    try:
        from flash_trittention import TrittentionTriton as RefDps

        ins = [x.to(dev) for x in _make_inputs(2, 8, 1024, 64, 1.0, 4, torch.float16)]
        mod = RefDps(causal=True, softmax_scale=1 / 8, k_diff=1024)

        def dps_step():
            leaves = [x.detach().requires_grad_(True) for x in ins[:5]]
            o, _ = mod(*leaves)
            o.backward(ins[5])

        dps_step()
        torch.cuda.synchronize()
        with torch.no_grad():
            fwd = bench(lambda: mod(*ins[:5]))
        res["dps_2x8x1024x64_fp16"] = {"fwd_ms": fwd, "fwd_bwd_ms": _timed(dps_step, iters=3)}
    except Exception as exc:  # the triple-dot-product timings above stand on their own
        res["dps_2x8x1024x64_fp16"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}
    print("REFJSON " + json.dumps(res), flush=True)


def reference_kernel_timings(timeout_s=420):
    """Times the reference's own GPU kernels beside ours (one GPU).  Returns a dict, or a one-line reason."""
    if not os.path.isdir(os.path.join(REF_DIR, "flash_trittention")):
        return {"unavailable": "reference tree not on GPU box (baseline/_ref is absent)"}
    env = dict(os.environ)
    env["PYTHONPATH"] = REF_DIR
    env["TRITT_BENCH_REFERENCE_WORKER"] = "1"
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--reference-kernel-worker"], env=env,
                           capture_output=True, text=True, timeout=timeout_s)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"reference kernels did not finish within {timeout_s} s"}
    for ln in r.stdout.splitlines():
        if ln.startswith("REFJSON "):
            return json.loads(ln[8:])
    tail = (r.stderr or r.stdout).strip().splitlines()[-1:] or ["no output"]
    return {"unavailable": f"reference kernels failed here (exit {r.returncode}): {tail[0][:200]}"}


def config5(dev, world, rank):
    """BASELINE config 5 (B=1, N=4, T=4096, D=64, bf16, causal, alpha = 1/D): on one GPU the plain entry point, on
    several the query-row-sharded path (interleaved rows, one NCCL all-reduce of the fp32 key-side partial sums,
    all-gathers of the output and dQ rows).  3 steps after 2 warm-ups, CUDA events, max over ranks; the all-reduce
    of a buffer of the partial sums' size is also timed by itself."""
    import torch.distributed as dist

    from flash_trittention import flash_trittention
    from flash_trittention.parallel import flash_trittention_query_sharded

    B, N, T, D = 1, 4, 4096, 64
    ins = [x.to(dev) for x in _make_inputs(B, N, T, D, 0.5, 11, torch.bfloat16)]

    def step():
        leaves = [x.detach().requires_grad_(True) for x in ins[:5]]
        if world > 1:
            out = flash_trittention_query_sharded(*leaves, 1.0 / D, True)
        else:
            out = flash_trittention(*leaves, 1.0 / D, None, None, None, None, True)
        out.backward(ins[5])

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        sync()
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            tt = torch.tensor([ms], device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        return ms

    for _ in range(2):
        step()
    ms = timed(step, 3)
    res = {"ms": ms, "tflops": _flops(B, N, T, D) / ms / 1e9, "n_gpus": world,
           "path": "flash_trittention_query_sharded" if world > 1 else "flash_trittention"}
    if world > 1:
        buf = torch.zeros(4 * B * N * T * D, device=dev)
        for _ in range(2):
            dist.all_reduce(buf)
        ar = timed(lambda: dist.all_reduce(buf), 5)
        res["allreduce_ms"] = ar
        res["allreduce_bytes"] = buf.numel() * 4
        res["allreduce_share_of_step"] = ar / ms
    return res


def run_ours(args):
    import torch.distributed as dist

    from flash_trittention import _native, flash_trittention

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch multi-GPU runs with torch.distributed.run (one process per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    B, N, T, D = WORK["B"], args.heads, args.seq, WORK["D"]
    dtype = torch.bfloat16
    heads = B * N
    if heads % world:
        raise SystemExit(f"{heads} heads do not divide over {world} ranks")
    per = heads // world
    alpha = 1.0 / D
    # every rank draws the same global tensors and keeps its slice of heads
    full = _make_inputs(B, N, T, D, WORK["scale_in"], WORK["seed"], dtype)
    host = [t.view(heads, T, D)[rank * per:(rank + 1) * per].reshape(1, per, T, D).contiguous().pin_memory() for t in full]
    del full
    dev_in = [t.to(dev) for t in host]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    host_out = [torch.empty(1, per, T, D, dtype=dtype).pin_memory() for _ in range(6)]

    def step_resident():
        leaves = [t.detach().requires_grad_(True) for t in dev_in[:5]]
        out = flash_trittention(*leaves, alpha, None, None, None, None, True)
        out.backward(dev_in[5])
        return out, leaves

    def step_e2e():
        ins = [t.to(dev, non_blocking=True) for t in host]
        leaves = [t.requires_grad_(True) for t in ins[:5]]
        out = flash_trittention(*leaves, alpha, None, None, None, None, True)
        out.backward(ins[5])
        host_out[0].copy_(out.detach(), non_blocking=True)
        for dst, leaf in zip(host_out[1:], leaves):
            dst.copy_(leaf.grad, non_blocking=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, bwd_events=None):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            flush.zero_()
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    warmup = max(args.warmup, 1)
    for _ in range(warmup):
        step_resident()
    torch.cuda.synchronize()

    # per-kernel-family timing of the dominant (backward) launch, CUDA events on the launching stream
    fwd_ms, bwd_ms = [], []
    for _ in range(3):
        leaves = [t.detach().requires_grad_(True) for t in dev_in[:5]]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        flush.zero_()
        ev[0].record()
        out = flash_trittention(*leaves, alpha, None, None, None, None, True)
        ev[1].record()
        out.backward(dev_in[5])
        ev[2].record()
        torch.cuda.synchronize()
        fwd_ms.append(ev[0].elapsed_time(ev[1]))
        bwd_ms.append(ev[1].elapsed_time(ev[2]))

    if rank == 0:
        sampler.wait_first()
        sampler.lines.clear()   # keep the samples of the timed regions only
    l0 = _native.lib().tritt_kernel_launches()
    ms_res = timed(step_resident, args.steps)
    launches = _native.lib().tritt_kernel_launches() - l0
    ms_e2e = None
    if not args.skip_e2e:
        for _ in range(2):
            step_e2e()
        ms_e2e = timed(step_e2e, args.steps)
    clocks = sampler.stop() if rank == 0 else None
    status = _native.read_status(dev)
    # config 5 after the headline measurement (every rank takes part in its collectives)
    c5 = None if args.skip_cpu else config5(dev, world, rank)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    total_flops = _flops(B, N, T, D)
    peaks = _peaks()
    bwd_med = statistics.median(bwd_ms)
    bwd_ach = _flops(1, per, T, D, "bwd") / bwd_med / 1e9
    cpu_v, cpu_dt, cpu_sample = (cpu_reference_sample(T_s=args.ref_T) if world == 1 and not args.skip_cpu
                                 else (None, None, None))
    nbytes = sum(t.numel() * t.element_size() for t in host)
    line = {
        "metric": METRIC, "value": total_flops / ms_res / 1e9, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_res, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "workload": f"triple-dot-product trittention fwd+bwd, B=1 N={N} T={T} D={D} bf16 causal full windows alpha=1/D",
            "sharding": f"{per} of {heads} (batch*head) slices per GPU, no collective",
            "flops_per_step": total_flops,
            "l2": "256 MiB memset between steps (inside the timed region) flushes the 126 MB L2",
            "fwd_ms": statistics.median(fwd_ms), "bwd_ms": bwd_med, "kernel_status": status,
        },
        "clocks": clocks,
        "e2e": None if ms_e2e is None else {
            "value": total_flops / ms_e2e / 1e9, "unit": UNIT, "ms_per_step": ms_e2e,
            "h2d_bytes_per_step": nbytes * world, "d2h_bytes_per_step": nbytes * world},
        "gpu_launches": int(launches),
        "roofline": {
            "bound": "tensor", "kernel": "tdp_bwd_kernel<128, bf16>", "achieved": bwd_ach, "peak": peaks["sustained"],
            "unit": "TFLOP/s", "frac": bwd_ach / peaks["sustained"], "peak_source": peaks["source"] + " sustained bf16 GEMM",
            "frac_of_burst_peak": bwd_ach / peaks["burst"], "frac_of_nominal_2250": bwd_ach / 2250.0,
            # 8 tensor-core products per tile for the 6 of the minimum schedule (S and dP are recomputed for the
            # second role), times the 128-wide tiles on the diagonal of the causal mask (ratio for T=2048)
            "executed_over_algorithmic_flops": (8.0 / 6.0) * 1.095,
            # dram__bytes_read+write of one backward launch: 15.9 MB captured at 2 heads (profiles/), scaled by heads
            "traffic": 7.93e6 * per, "traffic_unit": "bytes per launch (ncu at 2 heads, scaled by heads)",
        },
    }
    fwd_ach = _flops(1, per, T, D, "fwd") / statistics.median(fwd_ms) / 1e9
    line["roofline_forward"] = {
        "bound": "tensor", "kernel": "tdp_fwd_kernel<128, bf16>", "achieved": fwd_ach, "peak": peaks["sustained"],
        "unit": "TFLOP/s", "frac": fwd_ach / peaks["sustained"], "frac_of_burst_peak": fwd_ach / peaks["burst"],
        # 128-wide tiles on the diagonal of the causal mask (ratio for T=2048); no recomputation in the forward
        "executed_over_algorithmic_flops": 1.095,
    }
    if world == 1 and not args.skip_cpu:
        line["other_workloads"] = other_workloads(dev)
        line["other_workloads"]["reference_kernels_same_gpu"] = reference_kernel_timings()
    if c5 is not None:
        line.setdefault("other_workloads", {})["c5_query_sharded" if world > 1 else "c5_one_gpu"] = c5
    if cpu_v is not None:
        line["cpu_baseline"] = {"value": cpu_v, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                "sample": cpu_sample}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ref-T", type=int, default=896, help="sequence length of the CPU sample")
    ap.add_argument("--heads", type=int, default=WORK["N"], help="smaller head count, for profiler captures only")
    ap.add_argument("--seq", type=int, default=WORK["T"], help="other sequence length, for profiler captures only")
    ap.add_argument("--skip-e2e", action="store_true", help="profiler captures: no host-copy pass")
    ap.add_argument("--skip-cpu", action="store_true", help="profiler captures: no CPU baseline sample")
    ap.add_argument("--only-other", action="store_true",
                    help="profiler captures: only the short timings of the other configurations (one GPU)")
    ap.add_argument("--with-reference-kernels", action="store_true",
                    help="with --only-other: also time the reference's Triton kernels from baseline/_ref")
    ap.add_argument("--reference-kernel-worker", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.reference_kernel_worker:
        reference_kernel_worker()
    elif args.only_other:
        dev = torch.device("cuda:0")
        torch.cuda.set_device(dev)
        ow = other_workloads(dev)
        if args.with_reference_kernels:
            ow["reference_kernels_same_gpu"] = reference_kernel_timings()
        print(json.dumps({"other_workloads": ow}))
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
