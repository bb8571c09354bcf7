"""Benchmark of the W4A4 QuEST linear layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload linear|gemm|hadamard_quantize] [--m M --k K --n N --block B]

One "step" = one pass of the hot path over one batch of synthetic activations:
    fused Hadamard+scale+quantise+pack kernel  ->  int4 GEMM with fused dequant epilogue  (-> all-gather, N>1)
The default workload is the headline configuration M=2048, K=N=4096 (Llama-7B O-projection shape).
With N GPUs every rank owns N=4096 output columns of a layer that is N*4096 columns wide (weak scaling),
quantises the replicated activations itself and the column blocks are all-gathered.

Prints ONE JSON line (rank 0).  `value` is whole-layer TOPS = 2*M*N_total*K / step time with inputs resident
in HBM; `e2e` is the same metric through the public API with host buffers (pinned host -> device copy of the
activations and device -> host copy of the result inside the timed region); `roofline` describes the dominant
kernel (the GEMM) and `roofline_hadamard_quantize` the HBM-bound kernel; `cpu_baseline` times the CPU oracle
port of the reference's torch path on this host's cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "W4A4 QuEST linear TOPS (M=2048,K=N=4096); Had+quant HBM GB/s; 1/2/4/8 GPU"
L2_FLUSH_BYTES = 256 << 20  # > 126 MB L2


# ----------------------------------------------------------------------------------------------------
def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="linear", choices=["linear", "gemm", "hadamard_quantize", "prefill", "sweep"])
    ap.add_argument("--batch", type=int, default=16, help="prefill workload: sequences")
    ap.add_argument("--seq", type=int, default=1024, help="prefill workload: tokens per sequence")
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--n", type=int, default=4096, help="output columns PER GPU")
    ap.add_argument("--block", type=int, default=128)
    ap.add_argument("--exchange", default="push", choices=["push", "nccl"], help="N>1: how the column blocks are assembled")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch the step's kernels one by one instead of replaying a CUDA graph")
    return ap.parse_args()


def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def synthetic_inputs(m: int, k: int, n: int, seed: int = 0):
    """Llama-7B-shaped sweep inputs: activations Student-t(nu=4) scaled to unit RMS, weights N(0, 0.02)."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(m, k, generator=g)
    chi = torch.randn(4, m, k, generator=g).square().sum(0)
    x = z / (chi / 4).sqrt()
    x = (x / x.square().mean().sqrt()).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    return x, w


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.path = gpu_index, None, None

    def start(self):
        """Starts nvidia-smi and waits (up to 5 s) for its first sample, so that short runs are covered."""
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", "50"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
            t0 = time.time()
            while time.time() - t0 < 5.0 and os.path.getsize(self.path) == 0:
                time.sleep(0.02)
        except Exception:
            self.proc = None

    def stop(self) -> dict | None:
        if self.proc is None:
            return None
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return None
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------------
def cpu_reference_run(args, steps: int, warmup: int) -> dict:
    """The reference's torch CPU path for the same layer (oracle port: Hadamard as F.linear with the bf16
    Hadamard matrix, baseline scale/quantise, exact matmul of the codes, baseline epilogue)."""
    from oracle import quest_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m, k, n = args.m, args.k, args.n
    x, w = synthetic_inputs(m, k, n)
    wp, ws, wa, _ = O.preprocess_weight(w, use_hadamard=True)
    budget_s, times = 60.0, []
    t_begin = time.perf_counter()
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.linear_forward(x, wp, ws, wa, use_hadamard=True, block=args.block, reference_op=True)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
        if time.perf_counter() - t_begin > budget_s and len(times) >= 3:
            break
    t = sum(times) / len(times)
    return {"seconds_per_step": t, "tops": 2.0 * m * n * k / t / 1e12, "cores": torch.get_num_threads(),
            "steps_timed": len(times),
            "sample": f"full layer M={m} K={k} N={n} block={args.block}, {len(times)} timed passes after {warmup} warm-ups"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_reference_run(args, steps=min(args.steps, 10), warmup=min(args.warmup, 2))
    line = {
        "impl": "reference", "metric": METRIC, "value": r["tops"], "unit": "TOPS", "n_gpus": args.gpus,
        "steps": r["steps_timed"], "warmup": min(args.warmup, 2), "ms_per_step": r["seconds_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int4 codes, fp32 exact matmul (CPU)",
        "data": "synthetic",
        "config": {"workload": f"linear: W4A4 linear M={args.m} K={args.k} N={args.n} per GPU"
                               f" (N_total={args.n * args.gpus}), Hadamard block {args.block}",
                   "sample": "one GPU's share of the layer (all M rows, N columns) per step, on the host cores",
                   "inputs": "activations Student-t(nu=4) unit RMS bf16; weights N(0,0.02) quantised to packed int4"},
        "cpu_baseline": {"value": r["tops"], "unit": "TOPS", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": r["tops"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ----------------------------------------------------------------------------------------------------
def run_b200(args):
    import torch.distributed as dist
    import quest_b200 as quest
    from quest_b200.sharded import ShardedLinear4bit, shard_weight

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; quest_b200 has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # NCCL writes its version banner and debug output to stdout; stdout carries the one JSON line
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()

    m, k, n_local = args.m, args.k, args.n
    n_total = n_local * world
    x_host, w_local = synthetic_inputs(m, k, n_local, seed=rank)  # each rank builds only its own weight shard
    x_host, _ = synthetic_inputs(m, k, 8, seed=0)                 # activations are replicated: same seed everywhere
    x = x_host.to(dev)
    wp, ws, wa, _ = quest.preprocess_weight(w_local.to(dev), use_hadamard=True, block=args.block)
    layer = (ShardedLinear4bit((wp, ws, wa), n_total, rank, world, use_hadamard=True, block=args.block,
                               exchange=args.exchange) if world > 1 else None)
    if layer is not None and args.exchange == "push":
        # Symmetric memory needs peer access between the GPUs; if it cannot be set up, say so and use NCCL.
        try:
            layer.workspaces(m, k, dev, torch.bfloat16)
            ok = torch.ones(1, device=dev)
        except Exception as e:  # noqa: BLE001
            print(f"[rank {rank}] push exchange unavailable ({e!r}); using the NCCL all-gather", file=sys.stderr)
            ok = torch.zeros(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            args.exchange = "nccl"
            layer = ShardedLinear4bit((wp, ws, wa), n_total, rank, world, use_hadamard=True, block=args.block, exchange="nccl")
    flush = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=dev)

    a_scale = torch.empty(m, 1, dtype=torch.bfloat16, device=dev)
    a_packed = torch.empty(m, k // 2, dtype=torch.uint8, device=dev)
    a_rsum = torch.empty(m, 1, dtype=torch.int32, device=dev)
    out = torch.empty(m, n_local, dtype=torch.bfloat16, device=dev)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def step(timers=None, split=True):
        """One pass.  If `timers` is given, appends the event tuple (e0, e1, e2, e3): e0..e3 bracket the step; with
        `split` e1/e2 are recorded between its kernels (per-kernel times), otherwise they alias e0/e3 so that
        nothing sits between the quantiser and the GEMM (they are launched back to back, as a model would)."""
        e0, e3 = ev(), ev()
        e1, e2 = (ev(), ev()) if split else (None, None)

        def mark(e):
            if e is not None:
                e.record()

        if args.workload == "hadamard_quantize":
            e0.record()
            quest.hadamard_quantize_int4(x, args.block, a_packed, a_scale, a_rsum)
            mark(e1); mark(e2); e3.record()
        elif args.workload == "gemm":
            e0.record(); mark(e1)
            quest.fused_matmul_dequantize_int4_int4t_bf16(a_packed, wp, a_rsum, wa, a_scale, ws, out)
            mark(e2); e3.record()
        elif world == 1:
            e0.record()
            quest.hadamard_quantize_int4(x, args.block, a_packed, a_scale, a_rsum)
            mark(e1)
            quest.fused_matmul_dequantize_int4_int4t_bf16(a_packed, wp, a_rsum, wa, a_scale, ws, out)
            mark(e2); e3.record()
        elif args.exchange == "nccl":
            e0.record()
            lws = layer.workspaces(m, k, dev, torch.bfloat16)
            layer.quantize_activations(x, lws)
            mark(e1)
            quest.fused_matmul_dequantize_int4_int4t_bf16_into(lws["a_int_packed"], wp, lws["a_int_row_sum"], wa,
                                                               lws["a_scale"], ws, lws["local"][:, :n_local])
            mark(e2)
            dist.all_gather_into_tensor(lws["gathered"].view(-1), lws["local"].view(-1))
            lws["out"].view(m, world, -1).copy_(lws["gathered"].permute(1, 0, 2))
            e3.record()
        else:  # push: the GEMM epilogue stores its tiles into every rank's output; then one device-side barrier
            e0.record()
            lws = layer.workspaces(m, k, dev, torch.bfloat16)
            t, hdl, ptrs = lws["symm"][lws["parity"]]
            lws["parity"] ^= 1
            layer.quantize_activations(x, lws)
            mark(e1)
            off = layer.n0 * 2
            order = [rank] + [(rank + i) % world for i in range(1, world)]
            quest.fused_matmul_dequantize_int4_int4t_bf16_push(lws["a_int_packed"], wp, lws["a_int_row_sum"], wa,
                                                               lws["a_scale"], ws, [ptrs[r] + off for r in order], n_total)
            mark(e2)
            hdl.barrier(channel=0)
            e3.record()
        if timers is not None:
            timers.append((e0, e1 if split else e0, e2 if split else e3, e3))

    if args.workload == "gemm":  # the GEMM-only workload needs quantised activations once
        quest.hadamard_quantize_int4(x, args.block, a_packed, a_scale, a_rsum)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        flush.add_(1)
        step()
    barrier()
    # Single-GPU layer: the step's two launches are captured once into a CUDA graph and replayed (what a serving
    # loop does with a launch-bound step); the per-kernel pass below still launches them one by one.
    graph = None
    if world == 1 and args.workload == "linear" and not args.no_graph:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                quest.hadamard_quantize_int4(x, args.block, a_packed, a_scale, a_rsum)
                quest.fused_matmul_dequantize_int4_int4t_bf16(a_packed, wp, a_rsum, wa, a_scale, ws, out)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    barrier()  # rank 0 waited for the clock sampler's first sample: start the timed region together
    # Timed region 1: the K steps the headline value comes from; events only around the whole step.
    timers = []
    wall0 = time.perf_counter()
    for _ in range(args.steps):
        flush.add_(1)  # evict the previous step's tensors from L2 (outside the event brackets)
        if graph is not None:
            e0, e3 = ev(), ev()
            e0.record(); graph.replay(); e3.record()
            timers.append((e0, e0, e3, e3))
        else:
            step(timers, split=False)
    barrier()
    wall = time.perf_counter() - wall0
    # Timed region 2: the same K steps with events between the kernels, for the per-kernel (roofline) figures.
    split_timers = []
    for _ in range(args.steps):
        flush.add_(1)
        step(split_timers, split=True)
    barrier()
    clocks = sampler.stop() if sampler else None

    t_f1 = sum(e0.elapsed_time(e1) for e0, e1, _, _ in split_timers) / len(split_timers) * 1e-3
    t_gemm = sum(e1.elapsed_time(e2) for _, e1, e2, _ in split_timers) / len(split_timers) * 1e-3
    t_split_step = sum(e0.elapsed_time(e3) for e0, _, _, e3 in split_timers) / len(split_timers) * 1e-3
    t_step = sum(e0.elapsed_time(e3) for e0, _, _, e3 in timers) / len(timers) * 1e-3
    if os.environ.get("QB200_BENCH_DEBUG"):
        t_x = sum(e2.elapsed_time(e3) for _, _, e2, e3 in split_timers) / len(split_timers) * 1e-3
        print(f"[rank {rank}] step {t_step * 1e6:.1f} us (with inner events {t_split_step * 1e6:.1f} = f1 {t_f1 * 1e6:.1f} + gemm {t_gemm * 1e6:.1f} + exchange {t_x * 1e6:.1f});"
              f" wall/step {wall / args.steps * 1e6:.1f} us", file=sys.stderr, flush=True)
    if world > 1:
        tt = torch.tensor([t_step, t_f1, t_gemm], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t_step, t_f1, t_gemm = tt.tolist()

    # ---- end to end through the public API, host buffers in and out ----
    e2e = None
    if not args.no_e2e and args.workload == "linear":
        x_pin = x_host.pin_memory()
        y_pin = torch.empty(m, n_total, dtype=torch.bfloat16).pin_memory()
        x_dev = torch.empty_like(x)

        def e2e_step():
            x_dev.copy_(x_pin, non_blocking=True)
            if world == 1:
                y = quest.linear_forward(x_dev, wp, ws, wa, out=out, _a_scale=a_scale, _a_int_packed=a_packed,
                                         _a_int_row_sum=a_rsum, use_hadamard=True, block=args.block)
            else:
                y = layer(x_dev)
            y_pin.copy_(y, non_blocking=True)

        for _ in range(3):
            e2e_step()
        barrier()
        ets = []
        for _ in range(args.steps):
            flush.add_(1)
            s, e = ev(), ev()
            s.record(); e2e_step(); e.record()
            ets.append((s, e))
        barrier()
        t_e2e = sum(s.elapsed_time(e) for s, e in ets) / len(ets) * 1e-3
        if world > 1:
            tt = torch.tensor([t_e2e], dtype=torch.float64, device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t_e2e = tt.item()
        e2e = {"value": 2.0 * m * n_total * k / t_e2e / 1e12, "unit": "TOPS", "ms_per_step": t_e2e * 1e3,
               "h2d_bytes_per_step": x_pin.numel() * 2, "d2h_bytes_per_step": y_pin.numel() * 2,
               "api": "quest_b200.linear_forward" if world == 1 else "quest_b200.sharded.ShardedLinear4bit.forward",
               "mode": "one stream: copy in, layer, copy out, one step after the other"}

        if world == 1:
            # The same calls as a user would pipeline them: host->device copy, layer and device->host copy of
            # consecutive steps on three streams with two sets of buffers, so that the two PCIe directions and the
            # kernels overlap.  Every step still copies its input in and its result out inside the timed region.
            s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
            xb = [torch.empty_like(x) for _ in range(2)]
            ob = [torch.empty_like(out) for _ in range(2)]
            wsb = [(torch.empty_like(a_scale), torch.empty_like(a_packed), torch.empty_like(a_rsum)) for _ in range(2)]
            yb = [torch.empty(m, n_total, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
            cmp_done, out_done = [None, None], [None, None]

            def pipelined(nsteps):
                for i in range(nsteps):
                    b = i & 1
                    with torch.cuda.stream(s_in):
                        if cmp_done[b] is not None:
                            s_in.wait_event(cmp_done[b])      # the layer of step i-2 has consumed this input buffer
                        xb[b].copy_(x_pin, non_blocking=True)
                        e_in = torch.cuda.Event(); e_in.record(s_in)
                    with torch.cuda.stream(s_cmp):
                        s_cmp.wait_event(e_in)
                        if out_done[b] is not None:
                            s_cmp.wait_event(out_done[b])     # the result of step i-2 has left this output buffer
                        flush.add_(1)
                        sc, pk, rs = wsb[b]
                        quest.linear_forward(xb[b], wp, ws, wa, out=ob[b], _a_scale=sc, _a_int_packed=pk, _a_int_row_sum=rs,
                                             use_hadamard=True, block=args.block)
                        cmp_done[b] = torch.cuda.Event(); cmp_done[b].record(s_cmp)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(cmp_done[b])
                        yb[b].copy_(ob[b], non_blocking=True)
                        out_done[b] = torch.cuda.Event(); out_done[b].record(s_out)

            pipelined(4)
            torch.cuda.synchronize()
            t0, t1 = ev(), ev()
            t0.record(s_in)
            pipelined(args.steps)
            s_out.wait_stream(s_cmp); s_out.wait_stream(s_in)
            t1.record(s_out)
            torch.cuda.synchronize()
            t_pipe = t0.elapsed_time(t1) / args.steps * 1e-3
            e2e = {"value": 2.0 * m * n_total * k / t_pipe / 1e12, "unit": "TOPS", "ms_per_step": t_pipe * 1e3,
                   "h2d_bytes_per_step": x_pin.numel() * 2, "d2h_bytes_per_step": y_pin.numel() * 2,
                   "api": "quest_b200.linear_forward",
                   "mode": "three streams (copy in / layer / copy out), two buffer sets; L2 flushed before every layer call",
                   "one_stream": e2e}

    status = quest.device_status()
    if status != 0:
        raise RuntimeError(f"a kernel reported device status {status:#x}")

    if rank == 0:
        ops_total = 2.0 * m * n_total * k
        ops_gemm = 2.0 * m * n_local * k
        f1_bytes = 2.0 * m * k + m * k / 2 + 6.0 * m  # bf16 in + packed out + bf16 scale + int32 row sum
        int8_peak = 2.0 * peaks["bf16_tflops"]        # tcgen05 kind::i8 runs at twice the bf16 rate
        # DRAM traffic per launch: ncu captures of the headline-size launches showed the inputs read exactly once
        # (12.67 MB for the GEMM, 16.81 MB for the fused quantiser) and the outputs still in L2 at kernel end, so
        # traffic = input bytes read + output bytes written back later; only reported for the captured size.
        headline = (m, k, n_local) == (2048, 4096, 4096)
        gemm_traffic = 12.67e6 + 2.0 * m * n_local if headline else None
        f1_traffic = 16.81e6 + m * k / 2 + 6.0 * m if headline else None
        if args.workload == "hadamard_quantize":
            value, unit, t_main = f1_bytes / t_f1 / 1e9, "GB/s", t_f1
        elif args.workload == "gemm":
            value, unit, t_main = ops_gemm / t_gemm / 1e12, "TOPS", t_gemm
        else:
            value, unit, t_main = ops_total / t_step / 1e12, "TOPS", t_step
        launches_per_step = {"hadamard_quantize": 1, "gemm": 1}.get(args.workload, 2)
        line = {
            "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": t_main * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int4 operands, int8 tcgen05 MMA, int32 accumulate, bf16 out",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: W4A4 linear M={m} K={k} N={n_local} per GPU"
                                   f" (N_total={n_total}), Hadamard block {args.block}",
                       "l2": f"L2 flushed between timed steps by writing a {L2_FLUSH_BYTES >> 20} MiB buffer",
                       "parallelism": (f"N-sharded x{world}, " + ("epilogue pushes tiles to every GPU + barrier" if args.exchange == "push"
                                                                       else "NCCL all-gather + interleave copy")) if world > 1 else "single GPU",
                       "inputs": "activations Student-t(nu=4) unit RMS bf16; weights N(0,0.02) quantised to packed int4"},
            "roofline": {"kernel": "gemm_i4_wide_kernel / gemm_i4_kernel (TMA -> int4 unpack -> tcgen05 kind::i8, fused dequant epilogue;"
                                   " 256x256 tiles at the default shape)", "bound": "tensor",
                         "achieved": ops_gemm / t_gemm / 1e12 if t_gemm > 0 else None, "peak": int8_peak,
                         "unit": "TOPS", "frac": (ops_gemm / t_gemm / 1e12) / int8_peak if t_gemm > 0 else None,
                         "peak_source": f"2 x bf16_tflops ({peaks['bf16_tflops']}) of {peaks['source']}",
                         "traffic": gemm_traffic, "traffic_note": "12.67 MB read measured by ncu on this launch size plus the output"
                                                                   " bytes, which L2 writes back after the kernel (profiles/)",
                         "us_per_launch": t_gemm * 1e6},
            "roofline_hadamard_quantize": {"kernel": "fused Hadamard+scale+quantise+pack: hadamard_quant_tc_kernel (tcgen05) from 12 M elements,"
                                                     " hadamard_quant_mma_kernel below (the default shape)", "bound": "hbm",
                                           "achieved": f1_bytes / t_f1 / 1e9 if t_f1 > 0 else None,
                                           "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                           "frac": (f1_bytes / t_f1 / 1e9) / peaks["hbm_gbs"] if t_f1 > 0 else None,
                                           "peak_source": f"hbm_gbs of {peaks['source']}", "traffic": f1_traffic,
                                           "us_per_launch": t_f1 * 1e6, "algorithmic_bytes": f1_bytes},
            "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
            "timing": {"value_from": "K steps with events around the whole step only; the step's two launches are "
                                     + ("replayed from a CUDA graph" if graph is not None else "issued back to back"),
                       "roofline_from": "K further steps with events between the kernels",
                       "ms_per_step_with_inner_events": t_split_step * 1e3},
            "wall_s_timed_region": wall,
        }
        if not args.no_cpu_baseline and world == 1 and args.workload == "linear":
            r = cpu_reference_run(args, steps=5, warmup=1)
            line["cpu_baseline"] = {"value": r["tops"], "unit": "TOPS", "cores": r["cores"], "kind": "port",
                                    "sample": r["sample"], "ms_per_step": r["seconds_per_step"] * 1e3}
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_prefill(args):
    """End-to-end prefill of the 800M-shaped decoder (d=2048, 16 layers, 16 heads, SwiGLU 5632, vocab 32000) with
    random-init weights: bf16 linears vs W4A4 linears (with Hadamard) vs no-op linears, eager and CUDA graph."""
    from quest_b200.prefill import Decoder, DecoderConfig, swap_linears, prefill_time
    dev = torch.device("cuda", 0)
    cfg = DecoderConfig(sequence_length=max(1024, args.seq))
    out = {"metric": "prefill ms (batch x seq tokens through the decoder body)", "unit": "ms", "higher_is_better": False,
           "config": {"workload": f"prefill d={cfg.n_embd} L={cfg.n_layer} heads={cfg.n_head} ffn={cfg.ffn} "
                                  f"batch={args.batch} seq={args.seq}", "data": "uniform random token ids, random-init weights"}}
    for mode in ("bf16", "int4", "noop"):
        torch.manual_seed(0)
        model = swap_linears(Decoder(cfg).to(device=dev, dtype=torch.bfloat16).eval(), mode, use_hadamard=True)
        eager_ms, graph_ms, _ = prefill_time(model, args.batch, args.seq, n_warmup=args.warmup, n_iter=min(args.steps, 20))
        out[mode] = {"eager_ms": eager_ms, "graph_ms": graph_ms, "tokens_per_s": args.batch * args.seq / (min(eager_ms, graph_ms) * 1e-3)}
        del model
        torch.cuda.empty_cache()
    out["value"] = min(out["int4"]["eager_ms"], out["int4"]["graph_ms"])
    out["speedup_vs_bf16"] = min(out["bf16"]["eager_ms"], out["bf16"]["graph_ms"]) / out["value"]
    emit(out)


def run_sweep(args):
    """The single-GPU shape sweeps: W4A4 linear at K=4096, N in {4096, 11008, 12288}, M in {1, 16, 128, 2048, 8192}
    (fused quantiser + GEMM, each timed with events, L2 flushed between runs) and the Hadamard+quantise bandwidth
    sweep M in {1, 256, 4096, 65536} x K in {4096, 8192, 14336} x block in {64, 128, 256}.  One JSON object."""
    import quest_b200 as quest
    dev = torch.device("cuda", 0)
    peaks = measured_peaks()
    flush = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=dev)

    def timed(fn, iters=15, warm=4):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.add_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); fn(); e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e) * 1e-3)
        ts.sort()
        return ts[len(ts) // 2]

    g = torch.Generator().manual_seed(0)
    linear = []
    for n in (4096, 11008, 12288):
        w = (0.02 * torch.randn(n, 4096, generator=g)).to(torch.bfloat16).to(dev)
        wp, ws, wa, _ = quest.preprocess_weight(w, use_hadamard=True)
        for m in (1, 16, 128, 2048, 8192):
            x = torch.randn(m, 4096, generator=g).to(torch.bfloat16).to(dev)
            sc = torch.empty(m, 1, dtype=torch.bfloat16, device=dev)
            pk = torch.empty(m, 2048, dtype=torch.uint8, device=dev)
            rs = torch.empty(m, 1, dtype=torch.int32, device=dev)
            out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
            t_q = timed(lambda: quest.hadamard_quantize_int4(x, 128, pk, sc, rs))
            t_g = timed(lambda: quest.fused_matmul_dequantize_int4_int4t_bf16(pk, wp, rs, wa, sc, ws, out))
            ops = 2.0 * m * n * 4096
            gemm_bytes = m * 2048 + n * 2048 + 2.0 * m * n + 6.0 * (m + n)
            linear.append({"M": m, "N": n, "K": 4096, "quantize_us": t_q * 1e6, "gemm_us": t_g * 1e6,
                           "gemm_tops": ops / t_g / 1e12, "gemm_gbs": gemm_bytes / t_g / 1e9,
                           "layer_tops": ops / (t_q + t_g) / 1e12})
    hq = []
    for k in (4096, 8192, 14336):
        for m in (1, 256, 4096, 65536):
            x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(dev) if m * k < (1 << 28) else \
                torch.randn(m, k, device=dev).to(torch.bfloat16)
            sc = torch.empty(m, 1, dtype=torch.bfloat16, device=dev)
            pk = torch.empty(m, k // 2, dtype=torch.uint8, device=dev)
            rs = torch.empty(m, 1, dtype=torch.int32, device=dev)
            for block in (64, 128, 256):
                t = timed(lambda: quest.hadamard_quantize_int4(x, block, pk, sc, rs), iters=9, warm=3)
                nbytes = 2.0 * m * k + m * k / 2 + 6.0 * m
                hq.append({"M": m, "K": k, "block": block, "us": t * 1e6, "gbs": nbytes / t / 1e9,
                           "frac_of_hbm": nbytes / t / 1e9 / peaks["hbm_gbs"]})
            del x, pk
    emit({"workload": "sweep", "peaks": peaks, "linear": linear, "hadamard_quantize": hq})


_REAL_STDOUT = None


def keep_stdout_for_the_json_line():
    """Libraries (NCCL's version banner at NCCL_DEBUG=VERSION, for one) write to file descriptor 1.  The contract is
    ONE JSON line on stdout, so descriptor 1 is pointed at stderr for the whole run and the JSON line is written to a
    duplicate of the original stdout at the end."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _REAL_STDOUT if _REAL_STDOUT is not None else sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    args = parse_args()
    keep_stdout_for_the_json_line()
    if args.workload == "prefill":
        run_prefill(args)
        return
    if args.workload == "sweep":
        run_sweep(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
