"""Benchmark of the MORTAR sparse-MLP hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--quick]

Headline workload (N=1 and every N): the decode stack of the default 3+6xT+3 layout --
12 independent ternary MLP layers (d_model 768, d_ff 2048, 25% tile density, seeds
100..111), 42 MLP applications per token in engine order, 64 tokens per GPU per step.  One
step = one decode step of the whole stack: x <- x + MLP_i(rmsnorm_i(x)) for the 42
applications (the residual add makes the chain data-dependent; attention between the
applications is not part of this path).  `value` = tokens/s with inputs resident in HBM,
`e2e` = the same through pinned host buffers with the copies inside the timed region;
`parity_max_rel` = the launch's result against the CPU oracle on the same input.
Between timed steps a 256 MiB buffer is written to flush L2.  The JSON line also carries, each
with its own roofline and clock record: batch 1 / 8 decode, the single-layer configuration with
its CPU path timed beside it, cloud-shape prefill (through the module forward, device-resident
and end to end), the density / topology sweep, the ReMoE-routed configuration, the 30B-model
GEMV shape, the router, and a measured dense fp8 tensor peak.

Under torchrun (N>1) every rank runs the same stack on its own GPU with its own 64 tokens
(weights replicated, no collective on the data path); the aggregate is all tokens over
the slowest rank's device time.  The cloud prefill is run the same way (16384 tokens per rank).
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

LOCAL = dict(d_model=768, d_ff=2048, prelude=3, core=6, coda=3, T=6, seed0=100)
CLOUD = dict(d_model=2048, d_ff=5632, prelude=4, core=8, coda=4, T=8, seed0=200)
DENSITY = 0.25
DECODE_BATCH = 64
PREFILL_TOKENS = 16384
L2_FLUSH_BYTES = 256 << 20


def site_order(cfg) -> list[int]:
    """Layer index of every MLP application of one token, in the order of
    StaticDecodeEngine's site list (morph/inference/engine.py:207-213)."""
    p, c, d, T = cfg["prelude"], cfg["core"], cfg["coda"], cfg["T"]
    return (list(range(p)) + [p + i for _ in range(T) for i in range(c)]
            + [p + c + i for i in range(d)])


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["source"] = "measured"
        return d
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
            "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            f = [t.strip() for t in s.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def max_over_ranks(ms: float, device) -> float:
    """Whole-job time of a timed region = the slowest rank's summed device time."""
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def job_throughput(units_per_rank: int, world: int, slowest_ms: float) -> float:
    """Units processed by all ranks (weak scaling: the same count on each) per second."""
    return units_per_rank * world / (slowest_ms * 1e-3)


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------

class Stack:
    """Device-resident layers of one configuration."""

    def __init__(self, cfg, mb, device):
        self.cfg = cfg
        n_layers = cfg["prelude"] + cfg["core"] + cfg["coda"]
        self.layers = [mb.synth.make_layer(cfg["d_model"], cfg["d_ff"], DENSITY, seed=cfg["seed0"] + i)
                       for i in range(n_layers)]
        self.gu = [L.gate_up.to_stream(device) for L in self.layers]
        self.dn = [L.down.to_stream(device) for L in self.layers]
        gen = torch.Generator().manual_seed(cfg["seed0"] + 999)
        self.rms = [(1.0 + 0.05 * torch.randn(cfg["d_model"], generator=gen)).to(device)
                    for _ in range(n_layers)]
        self.order = site_order(cfg)
        self.decode_stack = mb.ops.DecodeStack(
            [(L.gate_up, L.down, w) for L, w in zip(self.layers, self.rms)], self.order, device) \
            if cfg is LOCAL else None
        self.matrix_bytes = [L.gate_up.algorithmic_bytes() + L.down.algorithmic_bytes()
                             for L in self.layers]
        self.tiles = [L.gate_up.nnz + L.down.nnz for L in self.layers]

    def algorithmic_bytes_per_step(self, batch: int) -> int:
        """per application: codes + column indices + row pointers + scales of both matrices,
        plus the bf16 activations in and out (2*d*batch*2 bytes)."""
        d = self.cfg["d_model"]
        return sum(self.matrix_bytes[i] + batch * 2 * d * 2 for i in self.order)

    def useful_flops_per_token(self) -> int:
        return sum(2 * 256 * self.tiles[i] for i in self.order)


def decode_step(mb, stack: Stack, x: torch.Tensor, ws: torch.Tensor) -> None:
    """x [B, d] fp32 residual carrier, updated in place through the 42 applications."""
    for i in stack.order:
        mb.ops.mlp_decode(x, stack.gu[i], stack.dn[i], rms_weight=stack.rms[i], eps=1e-6,
                          n_planes=3, out=x, accumulate=True, workspace=ws)


def time_steps(fn, steps: int, warmup: int, flush: torch.Tensor | None, pre=None, post=None):
    """Runs `fn` warmup+steps times; returns per-step device milliseconds (CUDA events on the
    current stream).  `pre`/`post` run inside the timed window (the host copies of the
    end-to-end measurement); the L2 flush runs outside it."""
    times = []
    for it in range(warmup + steps):
        if flush is not None:
            flush.fill_(float(it & 7))
        s = torch.cuda.Event(enable_timing=True)
        e = torch.cuda.Event(enable_timing=True)
        s.record()
        if pre is not None:
            pre()
        fn()
        if post is not None:
            post()
        e.record()
        e.synchronize()
        if it >= warmup:
            times.append(s.elapsed_time(e))
    return times


def capture(fn):
    """CUDA graph of `fn` (one warm call first so lazy allocations are outside the capture)."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        fn()
        stream.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            fn()
    torch.cuda.current_stream().wait_stream(stream)
    return g


def run_decode(mb, stack: Stack, batch: int, steps: int, warmup: int, flush, device, seed: int,
               mode: str = "stack"):
    """Times decode steps of the whole stack.  mode "stack": one persistent cluster launch per
    step (ops.stack_decode); mode "per_application": three launches per MLP application
    (ops.mlp_decode), the whole step captured in one CUDA graph."""
    d = stack.cfg["d_model"]
    x0 = mb.synth.make_activations(batch, d, seed=seed, dtype=torch.float32)
    x = x0.to(device)
    n0 = mb.ops.launch_count()
    if mode == "stack":
        step = lambda: mb.ops.stack_decode(x, stack.decode_stack)
        step()
        launches_per_step = mb.ops.launch_count() - n0
    else:
        ws = torch.empty(mb._lib.lib().mortar_mlp_workspace_bytes(batch, d, stack.cfg["d_ff"], 3) + 256,
                         device=device, dtype=torch.uint8)
        g = capture(lambda: decode_step(mb, stack, x, ws))
        launches_per_step = (mb.ops.launch_count() - n0) // 2
        step = g.replay
    xin = x0.to(device)

    def reset():
        x.copy_(xin)          # same input every step (outside the timed window)

    t_dev = []
    for it in range(warmup + steps):
        reset()
        t = time_steps(step, 1, 0, flush)
        if it >= warmup:
            t_dev += t
    # end to end through pinned host memory
    hx = x0.clone().pin_memory()
    hy = torch.empty_like(hx).pin_memory()
    t_e2e = time_steps(step, steps, warmup, flush,
                       pre=lambda: x.copy_(hx, non_blocking=True),
                       post=lambda: hy.copy_(x, non_blocking=True))
    # warm L2 (no flush), for reference
    reset()
    t_warm = time_steps(step, steps, warmup, None)
    err = stack.decode_stack.error() if mode == "stack" else 0
    reset()
    step()
    output = x.detach().cpu().clone()          # one step on the seeded input, for the parity check
    return dict(batch=batch, t_dev=t_dev, t_e2e=t_e2e, t_warm=t_warm, output=output,
                launches_per_step=launches_per_step, h2d=hx.numel() * 4, d2h=hy.numel() * 4,
                checksum=float(hy.double().abs().sum()), device_error_word=err)


def kernel_only(mb, stack: Stack, batch: int, reps: int, device):
    """Average duration of one launch of the block-sparse streaming kernel (the dominant
    kernel): gate_up and down launches of every application back to back, activations already
    in plane form, CUDA events around the whole run."""
    d, f = stack.cfg["d_model"], stack.cfg["d_ff"]
    xp = mb.ops.act_prep(mb.synth.make_activations(batch, d, seed=5, dtype=torch.float32).to(device), 3)
    hp = torch.empty(3, batch, f, device=device, dtype=torch.bfloat16)
    y = torch.empty(batch, d, device=device, dtype=torch.float32)
    L = mb._lib.lib()
    import ctypes as C

    def one(i):
        gu, dn = stack.gu[i].c_struct(), stack.dn[i].c_struct()
        st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        mb._lib.check(L.mortar_linear(C.byref(gu), C.c_void_p(xp.data_ptr()), 3, batch * d, d, batch,
                                      C.c_void_p(hp.data_ptr()), 2, 3, batch * f, f, 1, None, 0, 0,
                                      None, 0, None, 0, st), "mortar_linear")
        mb._lib.check(L.mortar_linear(C.byref(dn), C.c_void_p(hp.data_ptr()), 3, batch * f, f, batch,
                                      C.c_void_p(y.data_ptr()), 0, 0, 0, d, 0, None, 0, 0,
                                      None, 0, None, 0, st), "mortar_linear")

    def step():
        for i in stack.order:
            one(i)
    g = capture(step)
    t = time_steps(g.replay, reps, 3, None)
    launches = 2 * len(stack.order)
    return statistics.mean(t) / launches * 1e3     # microseconds per launch


def bench_config(world: int) -> dict:
    """The `config` object of the JSON line; identical for both arms."""
    return {"workload": "decode stack 3+6x6+3 (configs[1]): d_model 768, d_ff 2048, 12 ternary layers at "
                        "25% 16x16-tile density, 42 applications/token",
            "batch_per_gpu": DECODE_BATCH, "l2": "256 MiB flush between timed steps",
            "parallelism": f"dp{world} (token shards, replicated weights, no collective)"}


def cpu_reference_decode(batch: int, budget_s: float, cfg=LOCAL, seed: int = 1):
    """The reference's CPU path for this MLP (dense reconstruction of the effective weights
    + F.linear, fp32, all host threads; morph/inference/engine.py:74-84 and
    morph/model/transformer.py:402-431) on the same stack, for a bounded number of steps.
    Uses the oracle's own workload generator: the CUDA library is not loaded."""
    from oracle import workloads as wl
    torch.set_num_threads(os.cpu_count() or 1)
    n_layers = cfg["prelude"] + cfg["core"] + cfg["coda"]
    dense = [wl.dense_layer(cfg["d_model"], cfg["d_ff"], DENSITY, cfg["seed0"] + i)[:2] for i in range(n_layers)]
    rms = wl.norm_weights(n_layers, cfg["d_model"], cfg["seed0"] + 999)
    order = site_order(cfg)
    x0 = wl.activations(batch, cfg["d_model"], seed=seed, dtype=torch.float32)
    out = wl.decode_stack_step(x0.clone(), dense, rms, order)
    times = []
    t_start = time.perf_counter()
    while len(times) < 3 or (time.perf_counter() - t_start < budget_s and len(times) < 200):
        t0 = time.perf_counter()
        wl.decode_stack_step(x0.clone(), dense, rms, order)
        times.append(time.perf_counter() - t0)
    return dict(ms_per_step=1e3 * min(times), steps=len(times), cores=torch.get_num_threads(),
                tokens_per_s=batch / min(times), output=out)


def cpu_single_layer(tokens: int, reps: int = 3):
    """configs[0] on the host cores: one 768/2048 layer, 4 x 4096 tokens, the reference's dense
    reconstruction path under bf16 autocast rounding (and in fp32), best of `reps`."""
    from oracle import mortar_oracle as orc
    from oracle import workloads as wl
    torch.set_num_threads(os.cpu_count() or 1)
    wg, wd, _ = wl.dense_layer(LOCAL["d_model"], LOCAL["d_ff"], DENSITY, 0, bf16_scale=True)
    x = wl.activations(tokens, LOCAL["d_model"], seed=0).float()
    out = {"cores": torch.get_num_threads(), "torch": torch.__version__}
    for name, dt in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        ts = []
        for _ in range(reps + 1):
            t0 = time.perf_counter()
            orc.swiglu_mlp(x, wg, wd, dtype=dt)
            ts.append(time.perf_counter() - t0)
        out[f"{name}_ms"] = round(1e3 * min(ts[1:]), 2)
        out[f"{name}_tokens_per_s"] = round(tokens / min(ts[1:]), 1)
    return out


def measured_fp8_peak(device, n: int = 8192, reps: int = 10):
    """Dense fp8 (e4m3) tensor-core peak of this GPU through the library GEMM (torch._scaled_mm),
    burst figure, for the north star's 8-bit denominator.  Bench-only: nothing on the product path
    calls a library GEMM."""
    try:
        a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()     # column-major second operand
        one = torch.ones((), device=device)
        fn = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        t = time_steps(fn, reps, 3, None)
        return {"fp8_e4m3_tflops_burst": round(2 * n ** 3 / (min(t) * 1e-3) / 1e12, 1),
                "how": f"torch._scaled_mm {n}^3, best of {reps}"}
    except Exception as e:      # noqa: BLE001  (an absent kernel is reported, not fatal)
        return {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}


def measured_int8_peak(device, n: int = 8192, reps: int = 10):
    """Dense int8 tensor-core peak through the library GEMM (torch._int_mm), burst figure: the
    denominator of the opt-in 8-bit arm.  Bench-only."""
    try:
        a = torch.randint(-127, 128, (n, n), device=device, dtype=torch.int8)
        b = torch.randint(-127, 128, (n, n), device=device, dtype=torch.int8).t()
        t = time_steps(lambda: torch._int_mm(a, b), reps, 3, None)
        return {"int8_tops_burst": round(2 * n ** 3 / (min(t) * 1e-3) / 1e12, 1),
                "how": f"torch._int_mm {n}^3, best of {reps}"}
    except Exception as e:      # noqa: BLE001
        return {"unavailable": f"{type(e).__name__}: {str(e)[:160]}"}


def tensor_roofline(tf: float, pk: dict, fp8: dict | None = None) -> dict:
    r = {"bound": "tensor", "achieved": round(tf, 2), "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
         "frac": round(tf / pk["bf16_tflops_sustained"], 5), "peak_source": pk["source"] + " (bf16 sustained)"}
    if fp8 and "fp8_e4m3_tflops_burst" in fp8:
        r["frac_of_measured_fp8_burst"] = round(tf / fp8["fp8_e4m3_tflops_burst"], 5)
    return r


def run_ours(args, rank, world, local_rank):
    import mortar_b200 as mb
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    pk = peaks()
    stack = Stack(LOCAL, mb, device)
    flush = torch.empty(L2_FLUSH_BYTES, device=device, dtype=torch.uint8)
    steps, warmup = args.steps, max(args.warmup, 3)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sync_all()
    with ClockSampler(local_rank) as clk:
        # a second and a half of the same launch first, so the clock record holds tens of samples taken
        # under this load (the timed steps follow without a pause)
        soak = mb.synth.make_activations(DECODE_BATCH, LOCAL["d_model"], seed=1, dtype=torch.float32).to(device)
        t_end = time.perf_counter() + 1.5
        while time.perf_counter() < t_end:
            for _ in range(20):
                mb.ops.stack_decode(soak, stack.decode_stack)
            torch.cuda.synchronize()
        main = run_decode(mb, stack, DECODE_BATCH, steps, warmup, flush, device, seed=1 + rank)
    sync_all()

    def agg(times_ms):
        return max_over_ranks(sum(times_ms), device)

    tot_dev, tot_e2e, tot_warm = agg(main["t_dev"]), agg(main["t_e2e"]), agg(main["t_warm"])
    tokens = DECODE_BATCH * steps * world
    value = job_throughput(DECODE_BATCH * steps, world, tot_dev)
    e2e = job_throughput(DECODE_BATCH * steps, world, tot_e2e)

    # cloud prefill on every rank (weak scaling: 16384 tokens each)
    prefill = None
    if not args.quick:
        sync_all()
        with ClockSampler(local_rank) as pclk:
            prefill = run_prefill(mb, device, pk, flush, seed=7 + rank, reps=3 if world == 1 else 2)
        sync_all()
        slow = max_over_ranks(prefill["ms_per_pass"], device)
        slow_e2e = max_over_ranks(prefill["e2e_ms_per_pass"], device)
        prefill["clocks"] = pclk.summary()
        prefill["n_gpus"] = world
        prefill["tokens_per_s"] = round(job_throughput(prefill["tokens"], world, slow), 1)
        prefill["e2e"]["value"] = round(job_throughput(prefill["tokens"], world, slow_e2e), 1)

    extra = {}
    roof = None
    cpu = None
    parity = None
    if rank == 0:
        ms_step = statistics.mean(main["t_dev"])
        alg = stack.algorithmic_bytes_per_step(DECODE_BATCH)
        achieved = alg / (ms_step * 1e-3) / 1e9
        roof = {"bound": "hbm", "kernel": "stack_decode_kernel (one launch per decode step)",
                "achieved": round(achieved, 2), "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / pk["hbm_gbs"], 5), "peak_source": pk["source"],
                "us_per_launch": round(ms_step * 1e3, 2),
                "algorithmic_bytes_per_launch": int(alg),
                "traffic": profile_traffic("stack_decode_kernel_decode_stack_b64.md"),
                "note": "the 12 layers (3.6 MB packed) are L2-resident and every rank streams its "
                        "share into shared memory: this configuration is bound by on-SM instruction "
                        "issue and cluster synchronisation latency, not by HBM"}
        # the oracle on the very input of the headline launch (also the CPU baseline's timing run)
        c = cpu_reference_decode(DECODE_BATCH, budget_s=12.0 if world == 1 else 0.0, seed=1 + rank)
        parity = float((main["output"] - c["output"]).abs().max() / c["output"].abs().max())
        if world == 1:
            cpu = {"value": round(c["tokens_per_s"], 1), "unit": "tokens/s", "cores": c["cores"],
                   "kind": "port",
                   "sample": f"{c['steps']} decode steps of the same 42-application stack at batch "
                             f"{DECODE_BATCH}, fp32 dense reconstruction + F.linear, best step"}
        if world == 1 and not args.quick:
            fp8 = measured_fp8_peak(device)
            extra["measured_fp8_peak"] = fp8
            for b in (1, 8):
                with ClockSampler(local_rank) as sc:
                    r = run_decode(mb, stack, b, steps, warmup, flush, device, seed=11 + b)
                extra[f"decode_b{b}"] = {
                    "tokens_per_s": round(b * steps / (sum(r["t_dev"]) * 1e-3), 1),
                    "e2e_tokens_per_s": round(b * steps / (sum(r["t_e2e"]) * 1e-3), 1),
                    "ms_per_step": round(statistics.mean(r["t_dev"]), 4),
                    "hbm_frac_algorithmic": round(stack.algorithmic_bytes_per_step(b)
                                                  / (statistics.mean(r["t_dev"]) * 1e-3) / 1e9
                                                  / pk["hbm_gbs"], 5),
                    "clocks": sc.summary()}
            r = run_decode(mb, stack, DECODE_BATCH, steps, warmup, flush, device, seed=1,
                           mode="per_application")
            us_launch = kernel_only(mb, stack, DECODE_BATCH, max(steps, 10), device)
            extra["decode_b64_per_application_launches"] = {
                "tokens_per_s": round(DECODE_BATCH * steps / (sum(r["t_dev"]) * 1e-3), 1),
                "launches_per_step": r["launches_per_step"],
                "bcsr_stream_kernel_us_per_launch": round(us_launch, 3),
                "checksum": r["checksum"]}
            prefill["roofline"] = tensor_roofline(prefill["useful_tflops"], pk, fp8)
            extra["prefill_cloud"] = prefill
            with ClockSampler(local_rank) as sc:
                tp = run_prefill(mb, device, pk, flush, reps=2, tile_path=True)
            tp["roofline"] = tensor_roofline(tp["useful_tflops"], pk, fp8)
            tp["clocks"] = sc.summary()
            extra["prefill_cloud_tile_path"] = tp
            for name, fn in (("single_layer_c0", run_single_layer), ("prefill_cloud_blocks128", run_prefill_blocks128),
                             ("prefill_cloud_i8", run_prefill_i8), ("backward_gate_up_c0", run_backward), ("sweep_c3", run_sweep), ("remoe_c4", run_remoe),
                             ("gemv_large_b1", run_gemv_large)):
                with ClockSampler(local_rank) as sc:
                    extra[name] = fn(mb, device, pk, flush)
                extra[name]["clocks"] = sc.summary()
            extra["router"] = run_router(mb, device)
        elif prefill is not None:
            prefill["roofline"] = tensor_roofline(prefill["useful_tflops"], pk)
            extra["prefill_cloud"] = prefill
    if rank != 0:
        return
    ms_per_step = tot_dev / steps
    line = {
        "metric": "MORTAR MLP tokens/s (decode stack, 42 MLP applications per token)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "two scaled fp16 planes of the fp32 activations x ternary codes, fp32 accumulate",
        "data": "synthetic",
        "config": bench_config(world),
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": main["h2d"],
                "d2h_bytes_per_step": main["d2h"]},
        "gpu_launches": main["launches_per_step"] * steps,
        "launch": "one persistent cluster launch per decode step",
        "warm_l2_tokens_per_s": round(tokens / (tot_warm * 1e-3), 1),
        "clocks": clk.summary(),
        "roofline": roof,
        "cpu_baseline": cpu,
        "parity_max_rel": parity,
        "checksum": main["checksum"],
        "device_error_word": main["device_error_word"],
    }
    line.update(extra)
    print(json.dumps(line), flush=True)


def profile_traffic(name: str):
    """dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the line
    `dram_bytes_per_launch: N` of the ncu summary committed under profiles/ (None if absent)."""
    import re
    try:
        with open(os.path.join(ROOT, "profiles", name)) as f:
            m = re.search(r"dram_bytes_per_launch:\s*(\d+)", f.read())
        return int(m.group(1)) if m else None
    except OSError:
        return None


def cloud_modules(mb, device, n_layers=None, mask="topk_l2", density=DENSITY):
    cfg = CLOUD
    n_layers = n_layers or (cfg["prelude"] + cfg["core"] + cfg["coda"])
    layers = [mb.synth.make_layer(cfg["d_model"], cfg["d_ff"], density, seed=cfg["seed0"] + i, mask=mask)
              for i in range(n_layers)]
    mods = [mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=device) for L in layers]
    return layers, mods


def run_prefill(mb, device, pk, flush, tokens: int = PREFILL_TOKENS, reps: int = 3, seed: int = 7,
                tile_path: bool = False):
    """Cloud-shape prefill (configs[2]): 16 layers, 72 applications, 16384 tokens per GPU, bf16 with
    the reference's rounding points, through the MODULE forward (``SwiGLUMortar.__call__``, which
    sends token blocks to the tcgen05 / tensor-memory kernels).  Every application reads the same
    normalised token block (64 MB, plus a 176 MB hidden block: larger than L2).  `e2e`: the same
    pass with the token block copied in from pinned host memory and the last application's output
    copied back inside the timed window."""
    cfg = CLOUD
    layers, mods = cloud_modules(mb, device)
    order = site_order(cfg)
    d = cfg["d_model"]
    x0 = mb.synth.make_activations(tokens, d, seed=seed)
    x = x0.to(device)
    # the module picks the kernel by the fill of the touched 128 x 128 blocks (25% random tiles: the
    # block path); tile_path pins the per-tile kernel for comparison
    saved_fill = mb.format.BLOCK_PATH_MIN_FILL
    if tile_path:
        mb.format.BLOCK_PATH_MIN_FILL = 2.0
    counts0 = dict(mb.ops.kernel_counts())
    state = {}

    def fn():
        for i in order:
            state["y"] = mods[i](x)
    with torch.no_grad():
        t = time_steps(fn, reps, 1, flush)
        mb.format.BLOCK_PATH_MIN_FILL = saved_fill
        counts = mb.ops.kernel_counts()
        launched = {k: (counts.get(k, 0) - counts0.get(k, 0)) // (reps + 1) for k in ("prefill_panel", "prefill_blocks")}
        kernel = "prefill_blocks_kernel (tcgen05, dense 128x128 blocks)" if launched["prefill_blocks"] else \
            "prefill_panel_kernel (tcgen05, per tile)"
        launches = launched["prefill_blocks"] or launched["prefill_panel"]
        hx, hy = x0.clone().pin_memory(), torch.empty_like(x0).pin_memory()
        te = time_steps(fn, max(reps - 1, 1), 0, flush, pre=lambda: x.copy_(hx, non_blocking=True),
                        post=lambda: hy.copy_(state["y"], non_blocking=True))
    ms, ms_e2e = statistics.mean(t), statistics.mean(te)
    err = mb.ops.prefill_error()
    flops = sum(2 * 256 * (layers[i].gate_up.nnz + layers[i].down.nnz) for i in order) * tokens
    tf = flops / (ms * 1e-3) / 1e12
    return {"tokens_per_s": round(tokens / (ms * 1e-3), 1), "ms_per_pass": round(ms, 3),
            "e2e_ms_per_pass": round(ms_e2e, 3),
            "e2e": {"value": round(tokens / (ms_e2e * 1e-3), 1), "unit": "tokens/s",
                    "h2d_bytes_per_step": hx.numel() * 2, "d2h_bytes_per_step": hy.numel() * 2},
            "applications": len(order), "tokens": tokens, "through": "SwiGLUMortar.forward",
            "kernel": kernel, "launches_per_pass": launches,
            "useful_tflops": round(tf, 2), "dense_equivalent_tflops": round(tf / DENSITY, 2),
            "checksum": float(hy.double().abs().sum()), "device_error_word": err}


def run_single_layer(mb, device, pk, flush, reps: int = 5):
    """configs[0]: one 768/2048 layer at 25%, 4 x 4096 bf16 tokens, through the module forward on
    the GPU and through the reference's dense-reconstruction path on the host cores."""
    d, f, tokens = LOCAL["d_model"], LOCAL["d_ff"], 4 * 4096
    L = mb.synth.make_layer(d, f, DENSITY, seed=0)
    mlp = mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=device)
    x = mb.synth.make_activations(tokens, d, seed=0).reshape(4, 4096, d).to(device)
    with torch.no_grad():
        t = time_steps(lambda: mlp(x), reps, 3, flush)
    ms = statistics.median(t)
    flops = 2 * 256 * (L.gate_up.nnz + L.down.nnz) * tokens
    tf = flops / (ms * 1e-3) / 1e12
    return {"tokens": tokens, "ms": round(ms, 4), "tokens_per_s": round(tokens / (ms * 1e-3), 1),
            "useful_tflops": round(tf, 2), "roofline": tensor_roofline(tf, pk),
            "cpu_reference_path": cpu_single_layer(tokens), "device_error_word": mb.ops.prefill_error()}


def run_prefill_blocks128(mb, device, pk, flush, tokens: int = PREFILL_TOKENS, reps: int = 5):
    """One cloud-shape MLP whose 25% topology is made of ragged 128x128 blocks, the granularity the
    reference carves at in production (carve(blocking=128), block_sparse.py:810-907; 64 tiles per
    block after the split).  Vertically adjacent tiles fuse into N = 128 tensor-core runs, so this
    is the same kernel at the rate the tensor pipe gives wide MMAs; configs[2] with single-tile
    topology is the `prefill_cloud` entry."""
    d, f = CLOUD["d_model"], CLOUD["d_ff"]
    gu_m = mb.synth.make_block_matrix(2 * f, d, DENSITY, seed=11)
    dn_m = mb.synth.make_block_matrix(d, f, DENSITY, seed=12)
    mlp = mb.SwiGLUMortar.from_matrices(gu_m, dn_m, device=device)
    x = mb.synth.make_activations(tokens, d, seed=7).to(device)
    with torch.no_grad():
        t = time_steps(lambda: mlp(x), reps, 2, flush)
    ms = statistics.median(t)
    flops = 2 * 256 * (gu_m.nnz + dn_m.nnz) * tokens
    tf = flops / (ms * 1e-3) / 1e12
    return {"ms_per_application": round(ms, 3), "tokens": tokens, "useful_tflops": round(tf, 2),
            "roofline": tensor_roofline(tf, pk), "device_error_word": mb.ops.prefill_error()}


def run_prefill_i8(mb, device, pk, flush, tokens: int = PREFILL_TOKENS, reps: int = 5):
    """The opt-in 8-bit arm (tcgen05 kind::i8 on per-row quantised activations) beside the bf16 arm on
    one cloud-shape MLP, single-tile and 128-block topologies: time of the whole MLP (the two
    quantisation launches included) and its error against the bf16 arm's output -- relative to the
    output RMS, and the share of elements outside the bf16 element-wise tolerance, which is why the
    arm is not the default."""
    d, f = CLOUD["d_model"], CLOUD["d_ff"]
    x = mb.synth.make_activations(tokens, d, seed=7).to(device)
    peak = measured_int8_peak(device)
    out = {"tokens": tokens, "measured_int8_peak": peak, "default_arm": "bf16"}
    L = mb.synth.make_layer(d, f, DENSITY, seed=CLOUD["seed0"])
    cases = {"tile16": (L.gate_up, L.down),
             "blocks128": (mb.synth.make_block_matrix(2 * f, d, DENSITY, seed=11),
                           mb.synth.make_block_matrix(d, f, DENSITY, seed=12))}
    for name, (gu_m, dn_m) in cases.items():
        g16, d16 = gu_m.to_sched(True, device), dn_m.to_sched(False, device)
        g8, d8 = gu_m.to_sched(True, device, arith="i8"), dn_m.to_sched(False, device, arith="i8")
        ms16 = statistics.median(time_steps(lambda: mb.ops.mlp_prefill_tc(x, g16, d16), reps, 2, flush))
        ms8 = statistics.median(time_steps(lambda: mb.ops.mlp_prefill_tc_i8(x, g8, d8), reps, 2, flush))
        y16 = mb.ops.mlp_prefill_tc(x[:2048], g16, d16).float()
        y8 = mb.ops.mlp_prefill_tc_i8(x[:2048], g8, d8).float()
        err = (y8 - y16).abs()
        flops = 2 * 256 * (gu_m.nnz + dn_m.nnz) * tokens
        tf8 = flops / (ms8 * 1e-3) / 1e12
        cell = {"ms_bf16": round(ms16, 3), "ms_i8": round(ms8, 3), "useful_tops_i8": round(tf8, 1),
                "launches_i8": 4,
                "rms_error_over_rms_output": round(float(err.pow(2).mean().sqrt() / y16.pow(2).mean().sqrt()), 5),
                "fraction_outside_1e-2_rel_1e-3_abs": round(float((err > 1e-2 * y16.abs() + 1e-3).float().mean()), 5)}
        if "int8_tops_burst" in peak:
            cell["frac_of_measured_int8_burst"] = round(tf8 / peak["int8_tops_burst"], 5)
        out[name] = cell
    out["device_error_word"] = mb.ops.prefill_error()
    return out


def run_backward(mb, device, pk, flush, reps: int = 5):
    """Training backward of the gate/up matrix at the shape the reference profiled (x [16384, 768],
    W [4096, 768] at 25%; RTX 5090, 128x128 blocks: dW 445.7 us stock / 197 us tuned, dx 180.6 us,
    .agents/notes/implemented/process/2026-07-03-perf-pass-focus2-bcsr.md:22-46): the weight
    gradient on the topology (sdd_tiles_kernel) and the input gradient through the transposed
    matrix on the tensor-memory kernel, for single-tile and 128-block topologies."""
    d, f, tokens = LOCAL["d_model"], LOCAL["d_ff"], 4 * 4096
    from importlib import import_module
    fmt = import_module(mb.__name__ + ".format")
    out = {"tokens": tokens, "reference_published_us_rtx5090": {"dW_stock": 445.7, "dW_tuned": 197.0, "dx": 180.6}}
    x = mb.synth.make_activations(tokens, d, seed=5).to(device)
    dy = mb.synth.make_activations(tokens, 2 * f, seed=6).to(device)
    cases = {"tile16": mb.synth.make_layer(d, f, DENSITY, seed=0).gate_up,
             "blocks128": mb.synth.make_block_matrix(2 * f, d, DENSITY, seed=3)}
    for name, m in cases.items():
        topo = fmt.TopologyDev(m, device)
        # dx the way the registered operator's backward runs it: the transposed matrix on the block
        # path when its touched blocks are full enough, else per tile
        mT = m.transpose()
        if fmt.wants_block_path(mT, False):
            mt, dx_path = mT.to_blocks(False, device), "prefill_blocks_kernel"
            dx = lambda: mb.ops.linear_blocks(dy, mt)
        else:
            mt, dx_path = mT.to_sched(False, device), "prefill_panel_kernel"
            dx = lambda: mb.ops.linear_tc(dy, mt)
        t_dw = statistics.median(time_steps(lambda: mb.ops.sdd_tiles(dy, x, topo), reps, 2, flush))
        t_dw_tiles = statistics.median(time_steps(lambda: mb.ops.sdd_tiles(dy, x, topo, path="tiles"), reps, 1, flush))
        t_dx = statistics.median(time_steps(dx, reps, 2, flush))
        flops = 2 * 256 * m.nnz * tokens
        out[name] = {"dW_us": round(t_dw * 1e3, 1), "dW_tflops": round(flops / (t_dw * 1e-3) / 1e12, 1),
                     "dW_per_tile_kernel_us": round(t_dw_tiles * 1e3, 1),
                     "dx_us": round(t_dx * 1e3, 1), "dx_tflops": round(flops / (t_dx * 1e-3) / 1e12, 1),
                     "dx_kernel": dx_path}
    out["device_error_word"] = mb.ops.prefill_error() or mb.ops.sdd_error()
    return out


def run_sweep(mb, device, pk, flush, tokens: int = 8192, reps: int = 3):
    """configs[3]: one cloud-shape MLP, 8192 tokens, tile density 12.5 / 25 / 50 / 100% under the
    uniform-random and the Zipf(1.2) row-clustered mask generators; load balance shows in max /
    mean kept tiles per tile row."""
    import numpy as np
    d, f = CLOUD["d_model"], CLOUD["d_ff"]
    x = mb.synth.make_activations(tokens, d, seed=3).to(device)
    cells = {}
    for mask in ("uniform", "zipf_rows"):
        for rho in (0.125, 0.25, 0.5, 1.0):
            L = mb.synth.make_layer(d, f, rho, seed=300, mask=mask)
            mlp = mb.SwiGLUMortar.from_matrices(L.gate_up, L.down, device=device)
            with torch.no_grad():
                t = time_steps(lambda: mlp(x), reps, 1, flush)
            ms = statistics.median(t)
            tf = 2 * 256 * (L.gate_up.nnz + L.down.nnz) * tokens / (ms * 1e-3) / 1e12
            cells[f"{mask}_{rho}"] = {"ms": round(ms, 3), "useful_tflops": round(tf, 1),
                                      "frac_of_measured_bf16_sustained": round(tf / pk["bf16_tflops_sustained"], 4),
                                      "dense_equivalent_tflops": round(tf / rho, 1),
                                      "gate_up_tiles_per_row_max_mean": [int(np.diff(L.gate_up.row_ptr).max()),
                                                                         round(float(np.diff(L.gate_up.row_ptr).mean()), 1)],
                                      "down_tiles_per_row_max_mean": [int(np.diff(L.down.row_ptr).max()),
                                                                      round(float(np.diff(L.down.row_ptr).mean()), 1)]}
            del mlp
    return {"tokens": tokens, "cells": cells, "device_error_word": mb.ops.prefill_error()}


def run_remoe(mb, device, pk, flush, reps: int = 10):
    """configs[4]: cloud shape at 25%, 352 groups of 16 hidden neurons, k = 88 (87 active per
    token), 4096 tokens -- as 64-token decode batches (fp32 semantics; routed through the per-row
    tile gather vs unrouted) and as one prefill (bf16; the tensor-memory kernel with the gate
    multiply in its epilogue vs the gathered streaming kernel)."""
    d, f, ncls, k, tokens = CLOUD["d_model"], CLOUD["d_ff"], 352, 88, 4096
    L = mb.synth.make_layer(d, f, DENSITY, seed=200)
    gu, dn = L.gate_up.to_stream(device), L.down.to_stream(device)
    gs, ds = L.gate_up.to_sched(True, device), L.down.to_sched(False, device)
    gates = mb.synth.make_gates(tokens, L, ncls, k, seed=6).to(device)
    x32 = mb.synth.make_activations(tokens, d, seed=5, dtype=torch.float32).to(device)
    xb = x32.to(torch.bfloat16)
    out = {"tokens": tokens, "groups": ncls, "active_per_token": int((gates[0] > 0).sum())}
    cnt, _ = mb.ops.route_gather(gates, f // ncls, f // 16)
    listed = float(cnt.sum()) / (tokens * (f // 16))
    # gate/up tile MMAs follow the lists; down runs every tile for every block of 8 rows
    nnz_gu, nnz_dn = L.gate_up.nnz, L.down.nnz
    out["pairs_listed_frac"] = round(listed, 4)
    out["tile_mmas_skipped_frac_decode"] = round(1.0 - (nnz_gu * listed + nnz_dn) / (nnz_gu + nnz_dn), 4)
    B = DECODE_BATCH
    ws = torch.empty(mb._lib.lib().mortar_mlp_workspace_bytes(B, d, f, 3) + 256, device=device, dtype=torch.uint8)
    y = torch.empty(B, d, device=device)
    nb = tokens // B

    def decode_all(routed):
        for j in range(nb):
            sl = slice(j * B, (j + 1) * B)
            mb.ops.mlp_decode(x32[sl], gu, dn, gates=gates[sl] if routed else None, n_clusters=ncls if routed else 0,
                              n_planes=3, out=y, workspace=ws)
    for routed in (True, False):
        g = capture(lambda: decode_all(routed))
        t = time_steps(g.replay, reps, 3, flush)
        ms = statistics.median(t)
        out["decode_b64_routed" if routed else "decode_b64_unrouted"] = {
            "ms_per_4096_tokens": round(ms, 3), "tokens_per_s": round(tokens / (ms * 1e-3), 1),
            "us_per_batch": round(ms * 1e3 / nb, 2)}
    h = torch.empty(tokens, d, device=device, dtype=torch.bfloat16)
    wsp = torch.empty(max(tokens * f * 2, mb._lib.lib().mortar_mlp_workspace_bytes(tokens, d, f, 1)) + 256,
                      device=device, dtype=torch.uint8)
    bgs, bds = L.gate_up.to_blocks(True, device), L.down.to_blocks(False, device)
    for name, fn in (("prefill_blocks_gate_multiply", lambda: mb.ops.mlp_prefill_blocks(xb, bgs, bds, gates=gates, n_clusters=ncls, out=h, workspace=wsp)),
                     ("prefill_tc_gate_multiply", lambda: mb.ops.mlp_prefill_tc(xb, gs, ds, gates=gates, n_clusters=ncls, out=h, workspace=wsp)),
                     ("prefill_tc_unrouted", lambda: mb.ops.mlp_prefill_tc(xb, gs, ds, out=h, workspace=wsp)),
                     ("prefill_stream_gathered", lambda: mb.ops.mlp_decode(xb, gu, dn, gates=gates, n_clusters=ncls, n_planes=1,
                                                                        round_bf16=True, out=h, workspace=wsp))):
        t = time_steps(fn, 3, 1, flush)
        ms = statistics.median(t)
        out[name] = {"ms": round(ms, 3), "tokens_per_s": round(tokens / (ms * 1e-3), 1)}
    out["device_error_word"] = mb.ops.prefill_error()
    return out


def run_router(mb, device, reps: int = 20, calls: int = 16):
    """The two-launch ReMoE router (query projection + tail) at the decode shapes: d_model 768,
    16 groups, k = 8, fp32, batch 1 and 64; one CUDA graph of `calls` router calls, weights warm
    in L2 (2.4 MB of projection weights).  The reference's engine runs the same function as two
    Triton launches for one row (morph/kernels/triton/fused_router.py:101-139)."""
    from importlib import import_module
    router = import_module(mb.__name__ + ".router").TileRouter(16, LOCAL["d_model"], activation_ratio=0.5)
    router = router.to(device).eval()
    out = {}
    for b in (1, DECODE_BATCH):
        x = mb.synth.make_activations(b, LOCAL["d_model"], seed=9, dtype=torch.float32).to(device)
        gates = torch.empty(b, 16, device=device, dtype=torch.float32)
        scratch = torch.empty(b * LOCAL["d_model"], device=device, dtype=torch.float32)
        g = capture(lambda: [mb.ops.router_gates(x, router, out=gates, scratch=scratch) for _ in range(calls)])
        t = time_steps(g.replay, reps, 3, None)
        out[f"b{b}_us_per_call"] = round(statistics.median(t) * 1e3 / calls, 2)
    out["launches_per_call"] = 2
    # prefill scale (configs[4] routing: cloud shape, 352 groups, k = 88, 4096 tokens): the d x d
    # projection runs as a library GEMM, the rest as the router's second launch
    big = import_module(mb.__name__ + ".router").TileRouter(352, CLOUD["d_model"], activation_ratio=0.25)
    big = big.to(device).eval()
    xb = mb.synth.make_activations(4096, CLOUD["d_model"], seed=9, dtype=torch.float32).to(device)
    t32 = statistics.median(time_steps(lambda: mb.ops.router_gates(xb, big), 5, 2, None))
    with torch.autocast("cuda", dtype=torch.bfloat16):
        t16 = statistics.median(time_steps(lambda: mb.ops.router_gates(xb, big), 5, 2, None))
    out["cloud_4096_tokens_ms"] = {"fp32_projection": round(t32, 3), "bf16_autocast_projection": round(t16, 3)}
    return out


def run_gemv_large(mb, device, pk, flush, reps: int = 20, copies: int = 8):
    """The one shape with a reference-published per-kernel number (RTX 5090, 1.79 TB/s part;
    tile-prover/benchmarks/30b_gemv/report.json:18-19: gate_up 43.3 us, down 38.9 us): gate_up
    [43648, 8192] with fused silu(g)*u and down [8192, 21824], 25% ragged 128x128 blocks, batch
    1, fp32 activations (3 exact planes).

    Cold-cache timing without a flush inside the window: one CUDA graph walks `copies` device
    copies of the matrix, one launch each, and the L2 is flushed before every replay, so each
    launch streams weights that were never read since the flush; the event pair spans `copies`
    launches (a single launch is only a few ticks of the event clock)."""
    d, f = 8192, 21824
    gu_m = mb.synth.make_block_matrix(2 * f, d, DENSITY, seed=1)
    dn_m = mb.synth.make_block_matrix(d, f, DENSITY, seed=2)
    gus = [gu_m.to_stream(device) for _ in range(copies)]
    dns = [dn_m.to_stream(device) for _ in range(copies)]
    xp = mb.ops.act_prep(mb.synth.make_activations(1, d, seed=3, dtype=torch.float32).to(device), 3)
    hp = mb.ops.linear_planes(gus[0], xp, swiglu=True, out_planes=3)
    out = {}
    for name, m, ws, call in (
            ("gate_up", gu_m, gus, lambda w: mb.ops.linear_planes(w, xp, swiglu=True, out_planes=3)),
            ("down", dn_m, dns, lambda w: mb.ops.linear_planes(w, hp, out_dtype=torch.float32))):
        g = capture(lambda: [call(w) for w in ws])
        # between replays: flush, so the first launch of a replay is as cold as the others
        t = time_steps(g.replay, reps, 3, flush)
        us = statistics.median(t) * 1e3 / copies
        gbs = m.algorithmic_bytes() / (us * 1e-6) / 1e9
        out[name] = {"us": round(us, 2), "algorithmic_mb": round(m.algorithmic_bytes() / 1e6, 2),
                     "gb_per_s": round(gbs, 1), "frac_of_measured_hbm": round(gbs / pk["hbm_gbs"], 4),
                     "frac_of_8tbs_spec": round(gbs / 8000.0, 4)}
    # the tensor-memory GEMV (codes expanded straight into tensor memory; opt-in, not selected): same
    # matrices, gate/up as a plain product with the SwiGLU in the operand preparation of the down product
    dn_pad = mb.synth.make_block_matrix(d, f + 64, DENSITY, seed=2)      # hidden width padded to a multiple of 128
    tg = [gu_m.to_gemv_blocks(False, device) for _ in range(copies)]
    td = [dn_pad.to_gemv_blocks(False, device) for _ in range(copies)]
    xb = mb.ops.gemv_xprep(xp)
    g32 = mb.ops.gemv_blocks(tg[0], xb, 1, 3)
    hb = torch.zeros((f + 64) // 16 * 512, device=device, dtype=torch.uint8)
    hb[:f // 16 * 512] = mb.ops.gemv_xprep_swiglu(g32, 3)
    tm = {}
    for name, ws, call in (("gate_up", tg, lambda w: mb.ops.gemv_blocks(w, xb, 1, 3)),
                           ("down", td, lambda w: mb.ops.gemv_blocks(w, hb, 1, 3))):
        g = capture(lambda: [call(w) for w in ws])
        tm[name + "_us"] = round(statistics.median(time_steps(g.replay, reps, 3, flush)) * 1e3 / copies, 2)
    tm["device_error_word"] = mb.ops.gemv_blocks_error()
    out["tensor_memory_path_not_selected"] = tm
    del tg, td, gus, dns
    # the same layer as a token block (block path; d_ff = 21824 is not a multiple of 128, the step
    # lists exceed the kernel's shared-memory cache): one MLP over 4096 tokens
    tokens = 4096
    bg, bd = gu_m.to_blocks(True, device), dn_m.to_blocks(False, device)
    xt = mb.synth.make_activations(tokens, d, seed=4).to(device)
    yt = torch.empty(tokens, d, device=device, dtype=torch.bfloat16)
    wsp = torch.empty(tokens * f * 2 + 256, device=device, dtype=torch.uint8)
    t_pf = statistics.median(time_steps(lambda: mb.ops.mlp_prefill_blocks(xt, bg, bd, out=yt, workspace=wsp), 5, 2, flush))
    flops = 2.0 * 256 * (gu_m.nnz + dn_m.nnz) * tokens
    out["prefill_blocks_4096_tokens"] = {"ms": round(t_pf, 3), "useful_tflops": round(flops / (t_pf * 1e-3) / 1e12, 1),
                                         "frac_of_measured_bf16_sustained": round(flops / (t_pf * 1e-3) / 1e12 / pk["bf16_tflops_sustained"], 4),
                                         "device_error_word": mb.ops.prefill_error()}
    out["reference_published_us_rtx5090"] = {"gate_up": 43.3, "down": 38.9}
    # the reference's own Triton GEMV on this GPU: its source tree is not present on the machine this
    # benchmark runs on and may not be copied into this repository, so there is nothing to launch
    out["reference_triton_us_b200"] = {"unavailable": "the reference's Triton kernel source is not on this machine"}
    out["note"] = (f"kernel bcsr_stream_kernel; one CUDA graph of {copies} launches over {copies} "
                   f"distinct weight copies, L2 flushed before each replay; per-launch time = "
                   f"graph time / {copies} (includes the launch gaps inside the graph)")
    return out


# ---------------------------------------------------------------------------------------
# reference arm: the reference's CPU path on the host cores
# ---------------------------------------------------------------------------------------

def run_reference(args, rank, world):
    """The reference's own CPU implementation of the path (its carved kernels are CUDA/Triton-only,
    so its dense-reconstruction forward is its CPU path), restated by the oracle, on all host
    cores; rank 0 only.  Does not import the product package or load its library."""
    if rank != 0:
        return
    steps, warmup = args.steps, max(args.warmup, 1)
    c = cpu_reference_decode(DECODE_BATCH, budget_s=min(60.0, 2.0 * (steps + warmup)))
    line = {
        "impl": "reference",
        "metric": "MORTAR MLP tokens/s (decode stack, 42 MLP applications per token)",
        "value": round(c["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": round(c["ms_per_step"], 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(world),
        "cpu_baseline": {"value": round(c["tokens_per_s"], 1), "unit": "tokens/s", "cores": c["cores"],
                         "kind": "port",
                         "sample": f"{c['steps']} decode steps at batch {DECODE_BATCH}, dense "
                                   f"reconstruction + F.linear fp32 (the reference's CPU path; its "
                                   f"carved kernels are CUDA/Triton-only), best step"},
        "e2e": {"value": round(c["tokens_per_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_probe(name: str):
    """A few untimed launches of one kernel on a small case of its workload: the command the
    profiler captures (`ncu ... python bench.py --probe <name>`).  Prints nothing but "done"."""
    import mortar_b200 as mb
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    if name == "stack":              # stack_decode_kernel, the headline launch (batch 64)
        stack = Stack(LOCAL, mb, device)
        x = mb.synth.make_activations(DECODE_BATCH, LOCAL["d_model"], seed=1, dtype=torch.float32).to(device)
        x0 = x.clone()
        for _ in range(4):
            x.copy_(x0)
            mb.ops.stack_decode(x, stack.decode_stack)
    elif name == "decode":           # bcsr_stream_kernel, one MLP application at batch 64 (3 launches)
        L = mb.synth.make_layer(LOCAL["d_model"], LOCAL["d_ff"], DENSITY, seed=100)
        gu, dn = L.gate_up.to_stream(device), L.down.to_stream(device)
        x = mb.synth.make_activations(DECODE_BATCH, LOCAL["d_model"], seed=1, dtype=torch.float32).to(device)
        out = torch.empty_like(x)
        for _ in range(4):
            mb.ops.mlp_decode(x, gu, dn, n_planes=3, out_dtype=torch.float32, out=out)
    elif name == "gemv":             # bcsr_stream_kernel, 30B-model gate_up at batch 1, cold L2
        gu = mb.synth.make_block_matrix(2 * 21824, 8192, DENSITY, seed=1).to_stream(device)
        xp = mb.ops.act_prep(mb.synth.make_activations(1, 8192, seed=3, dtype=torch.float32).to(device), 3)
        flush = torch.empty(L2_FLUSH_BYTES, device=device, dtype=torch.uint8)
        for i in range(3):
            flush.fill_(i)
            mb.ops.linear_planes(gu, xp, swiglu=True, out_planes=3)
    elif name == "prefill":          # prefill_panel_kernel, one cloud-shape MLP on 4096 tokens
        L = mb.synth.make_layer(CLOUD["d_model"], CLOUD["d_ff"], DENSITY, seed=200)
        gu, dn = L.gate_up.to_sched(True, device), L.down.to_sched(False, device)
        x = mb.synth.make_activations(4096, CLOUD["d_model"], seed=2).to(device)
        h = torch.empty(4096, CLOUD["d_ff"], device=device, dtype=torch.bfloat16)
        y = torch.empty(4096, CLOUD["d_model"], device=device, dtype=torch.bfloat16)
        for _ in range(3):
            mb.ops.linear_tc(x, gu, out=h)
            mb.ops.linear_tc(h, dn, out=y)
    elif name == "prefill_blocks":   # prefill_blocks_kernel, one cloud-shape MLP carved in 128x128 blocks, 4096 tokens
        gu_m = mb.synth.make_block_matrix(2 * CLOUD["d_ff"], CLOUD["d_model"], DENSITY, seed=11)
        dn_m = mb.synth.make_block_matrix(CLOUD["d_model"], CLOUD["d_ff"], DENSITY, seed=12)
        gu, dn = gu_m.to_blocks(True, device), dn_m.to_blocks(False, device)
        x = mb.synth.make_activations(4096, CLOUD["d_model"], seed=2).to(device)
        h = torch.empty(4096, CLOUD["d_ff"], device=device, dtype=torch.bfloat16)
        y = torch.empty(4096, CLOUD["d_model"], device=device, dtype=torch.bfloat16)
        for _ in range(3):
            mb.ops.linear_blocks(x, gu, out=h)
            mb.ops.linear_blocks(h, dn, out=y)
    else:
        raise SystemExit(f"unknown probe {name}")
    torch.cuda.synchronize()
    print("done", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--quick", action="store_true", help="headline measurement only")
    ap.add_argument("--probe", default=None, choices=["stack", "decode", "gemv", "prefill", "prefill_blocks"],
                    help="run a few untimed launches of one kernel (small case) for a profiler capture")
    args = ap.parse_args()
    if args.probe:
        run_probe(args.probe)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
