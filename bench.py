"""Benchmark of the W4A4 QuEST linear layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload linear|gemm|hadamard_quantize|sweep|layers|c4|prefill] [--m M --k K --n N --block B]

One "step" = one pass of the hot path over one batch of synthetic activations:
    fused Hadamard+scale+quantise+pack kernel  ->  int4 GEMM with fused dequant epilogue  (-> exchange, N>1)
The default workload is the headline configuration M=2048, K=N=4096 (Llama-7B O-projection shape).
With N GPUs every rank owns N=4096 output columns of a layer that is N*4096 columns wide (weak scaling),
quantises the replicated activations itself and the column blocks are exchanged (pushed by the GEMM epilogue, or
all-gathered by NCCL).

Prints ONE JSON line (rank 0).  `value` is whole-layer TOPS = 2*M*N_total*K / step time with inputs resident
in HBM; `e2e` is the same metric through the public API with host buffers (pinned host -> device copy of the
activations and device -> host copy of the result inside the timed region); `roofline` describes the dominant
kernel (the GEMM), `roofline_hadamard_quantize` the HBM-bound kernel at the layer's shape and
`roofline_hadamard_quantize_large` the same kernel on an input far larger than L2; `cpu_baseline` times the CPU oracle
port of the reference's torch path on this host's cores.  With N > 1 the line also carries `parity`: every rank
recomputes every peer's columns on its own GPU with the single-GPU entry point and compares them bit for bit with what
the exchange delivered (the run exits non-zero on a mismatch).
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
sys.path.insert(0, ROOT)

METRIC = "W4A4 QuEST linear TOPS (M=2048,K=N=4096); Had+quant HBM GB/s; 1/2/4/8 GPU"
L2_FLUSH_BYTES = 256 << 20  # > 126 MB L2
L2_BYTES = 126 << 20

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture), keyed by kernel and launch
# shape; the file under profiles/ holds the capture's command and figures.  Only these shapes report `traffic`.
NCU_TRAFFIC = {
    # (kernel, M, K, N or None, int8-operand route?)
    ("gemm", 2048, 4096, 4096, True): (16.86e6 + 2.0 * 2048 * 4096, "profiles/gemm_i4_wide_kernel_fused_m2048_k4096_n4096.md (A8 column): 16.86 MB"
                                       " read by the kernel; its 16.78 MB of output are still in L2 when it ends and are written back afterwards"),
    ("gemm", 2048, 4096, 4096, False): (12.67e6 + 2.0 * 2048 * 4096, "profiles/gemm_i4_wide_kernel_fused_m2048_k4096_n4096.md (packed column): 12.67 MB"
                                        " read by the kernel; its 16.78 MB of output are still in L2 when it ends and are written back afterwards"),
    ("hadamard_quantize", 2048, 4096, None, True): (16.82e6 + 2048 * 4096 + 6.0 * 2048, "profiles/hadamard_quant_kernels_headline_and_large.md (first"
                                                    " column): the input is read exactly once, the outputs are written back after the kernel"),
    ("hadamard_quantize", 2048, 4096, None, False): (16.81e6 + 2048 * 4096 / 2 + 6.0 * 2048, "profiles/hadamard_quant_kernels_headline_and_large.md"
                                                     " (second column): the input is read exactly once, the outputs are written back after the kernel"),
}


# ----------------------------------------------------------------------------------------------------
def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="linear",
                    choices=["linear", "gemm", "hadamard_quantize", "prefill", "sweep", "layers", "c4"])
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


def synthetic_activations(m: int, k: int, seed: int = 0) -> torch.Tensor:
    """Llama-7B-shaped sweep activations: Student-t(nu=4) scaled to unit RMS, bf16 (CPU generator)."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(m, k, generator=g)
    chi = torch.randn(4, m, k, generator=g).square().sum(0)
    x = z / (chi / 4).sqrt()
    return (x / x.square().mean().sqrt()).to(torch.bfloat16)


def synthetic_weight(n: int, k: int, seed: int, std: float = 0.02) -> torch.Tensor:
    """Weights N(0, std) in bf16 (CPU generator; rank r's shard of the sharded layer is seed 1000 + r)."""
    g = torch.Generator().manual_seed(seed)
    return (std * torch.randn(n, k, generator=g)).to(torch.bfloat16)


def workload_config(args, world: int) -> dict:
    """The `config` object, identical in the GPU arm and the reference arm of the same command line."""
    return {"workload": f"{args.workload}: W4A4 linear M={args.m} K={args.k} N={args.n} per GPU"
                        f" (N_total={args.n * world}), Hadamard block {args.block}",
            "l2": "GPU arm: inputs larger than L2 - steps and per-kernel launches rotate through operand sets of more than"
                  f" 2.5 x L2 in total (isolated-step figures: L2 flushed by writing a {L2_FLUSH_BYTES >> 20} MiB buffer)."
                  " CPU arm: one GPU's share of the layer per step",
            "parallelism": (f"N-sharded x{world}, " + ("epilogue pushes tiles to every GPU + barrier" if args.exchange == "push"
                                                            else "NCCL all-gather + interleave copy")) if world > 1 else "single GPU",
            "inputs": "activations Student-t(nu=4) unit RMS bf16; weights N(0,0.02) quantised to packed int4"}


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


def ev():
    return torch.cuda.Event(enable_timing=True)


def rotating_sets_time(make_call, n_sets: int, reps: int, dev) -> float:
    """Seconds per launch of a kernel, measured over back-to-back launches: ``make_call(i)`` launches it on operand set
    i; ``reps`` cycles through the n_sets sets are captured into ONE CUDA graph (at most 512 launches per graph, more are
    covered by replaying it) and the graph is replayed between two events on the launching stream.  The sets occupy
    distinct memory and together exceed the L2 size, so every launch finds its operands in HBM, and no event or host
    gap sits between the launches."""
    make_call(0)  # first-call set-up (kernel attributes, scratch) outside the capture
    torch.cuda.synchronize()
    cycles = max(1, min(reps, 512 // n_sets))
    replays = max(1, -(-reps // cycles))
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(cycles):
                for i in range(n_sets):
                    make_call(i)
    torch.cuda.current_stream(dev).wait_stream(side)
    for _ in range(2):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (replays * cycles * n_sets)


def sets_for(bytes_per_set: float, cap_bytes: float = 6e9) -> int:
    """How many operand sets make consecutive launches cold in L2: their total is at least 2.5 x L2 (at least 3 sets,
    fewer only if that would exceed ``cap_bytes``; a set larger than L2 needs just 2)."""
    if bytes_per_set >= L2_BYTES:
        return 2
    n = max(3, int(2.5 * L2_BYTES / bytes_per_set) + 1)
    return max(2, min(n, int(cap_bytes / bytes_per_set), 256))  # at most 256 launches per graph: tiny operand sets stay L2-resident


# ----------------------------------------------------------------------------------------------------
def cpu_reference_run(args, steps: int, warmup: int, budget_s: float = 60.0) -> dict:
    """The reference's torch CPU path for the same layer (oracle port: Hadamard as F.linear with the bf16
    Hadamard matrix, baseline scale/quantise, exact matmul of the codes, baseline epilogue)."""
    from oracle import quest_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m, k, n = args.m, args.k, args.n
    x, w = synthetic_activations(m, k), synthetic_weight(n, k, 1000)
    wp, ws, wa, _ = O.preprocess_weight(w, use_hadamard=True)
    times = []
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
    """The reference arm: the reference's own CPU implementation of the path (its torch baseline functions, restated in
    oracle/ because the reference module cannot be imported here) on this host's cores; rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    # --steps / --warmup are honoured; only a run that would exceed five minutes is cut short (and says so in `steps`)
    r = cpu_reference_run(args, steps=args.steps, warmup=args.warmup, budget_s=300.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["tops"], "unit": "TOPS", "n_gpus": args.gpus,
        "steps": r["steps_timed"], "warmup": args.warmup, "ms_per_step": r["seconds_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int4 codes, fp32 exact matmul (CPU)",
        "data": "synthetic", "config": workload_config(args, world),
        "cpu_baseline": {"value": r["tops"], "unit": "TOPS", "cores": r["cores"], "kind": "port", "sample": r["sample"]},
        "e2e": {"value": r["tops"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ----------------------------------------------------------------------------------------------------
def check_exchange_parity(layer, x, n_local: int, block: int, exchanges, dev) -> dict:
    """Multi-GPU bit-identity: for every exchange mode, run the sharded layer once, then recompute EVERY rank's column
    block on this GPU with the single-GPU entry point (the peer's weight shard is regenerated from its seed) and compare
    bit for bit with what the exchange delivered.  Collective: every rank calls it with the same arguments."""
    import torch.distributed as dist
    import quest_b200 as quest
    from quest_b200.sharded import ShardedLinear4bit
    world, rank = layer.world, layer.rank
    m, k = x.shape
    res = {"equal": True, "columns_checked": 0, "exchanges": [], "checker": "single-GPU fused_matmul_dequantize on every rank's regenerated shard"}
    delivered = {}
    for exch in exchanges:
        lay = layer if exch == layer.exchange else ShardedLinear4bit((layer.w_int_packed, layer.w_scale, layer.w_add), layer.n_total,
                                                                     rank, world, use_hadamard=True, block=block, exchange=exch)
        try:
            delivered[exch] = lay(x).clone()
        except Exception as e:  # noqa: BLE001  (symmetric memory unavailable: reported, not fatal, if the other mode is checked)
            print(f"[rank {rank}] parity: exchange {exch} unavailable ({e!r})", file=sys.stderr)
            ok = torch.zeros(1, device=dev)
        else:
            ok = torch.ones(1, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() == 0:
            delivered.pop(exch, None)
    torch.cuda.synchronize()
    with quest.layer_launches():  # the quantiser kernel the layer itself chooses for this size
        pa, sa, ra = quest.hadamard_quantize_int4(x, block)
    for s in range(world):
        w_s = synthetic_weight(n_local, k, 1000 + s).to(dev)
        wp, ws, wa, _ = quest.preprocess_weight(w_s, use_hadamard=True, block=block)
        want = quest.fused_matmul_dequantize_int4_int4t_bf16(pa, wp, ra, wa, sa, ws)
        for exch, full in delivered.items():
            if not full[:, s * n_local:(s + 1) * n_local].equal(want):
                res["equal"] = False
                print(f"[rank {rank}] parity MISMATCH: exchange {exch}, columns of rank {s}", file=sys.stderr)
        del w_s, wp, want
    res["exchanges"] = sorted(delivered)
    res["columns_checked"] = world * n_local * len(delivered)
    flag = torch.tensor([1.0 if res["equal"] and delivered else 0.0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    res["equal"] = bool(flag.item() == 1.0)
    res["ranks"] = world
    return res


def run_b200(args):
    import torch.distributed as dist
    import quest_b200 as quest
    from quest_b200.sharded import ShardedLinear4bit

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
    x_host = synthetic_activations(m, k)                # activations are replicated: same seed everywhere
    w_local = synthetic_weight(n_local, k, 1000 + rank)  # each rank builds only its own weight shard
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

    # One GPU: the layer takes the route linear_forward takes.  Where the library prefers it (256 x 256 GEMM kernel and a
    # row length the tcgen05 quantiser tiles) the quantiser writes the GEMM's int8 operand instead of packed int4.
    use_a8 = world == 1 and args.block in (64, 128, 256) and k % args.block == 0 and quest.prefers_a8(m, k, n_local)
    a_scale = torch.empty(m, 1, dtype=torch.bfloat16, device=dev)
    a_packed = torch.empty(m, k if use_a8 else k // 2, dtype=torch.uint8, device=dev)

    def f1_op(x_, codes, sc_, rs_):
        if use_a8:
            quest.hadamard_quantize_a8(x_, args.block, codes, sc_, rs_)
        else:
            quest.hadamard_quantize_int4(x_, args.block, codes, sc_, rs_)

    def gemm_op(codes, w_, rs_, sc_, out_):
        if use_a8:
            quest.fused_matmul_dequantize_a8(codes, w_, rs_, wa, sc_, ws, out_)
        else:
            quest.fused_matmul_dequantize_int4_int4t_bf16(codes, w_, rs_, wa, sc_, ws, out_)

    def layer_op(x_, codes, sc_, rs_, w_, out_):
        """The layer as a user calls it: quest.linear_forward on caller-owned workspaces (one library call; the GEMM
        kernel is launched with a programmatic dependency on the quantiser)."""
        ws_kw = {"_a_int8": codes} if use_a8 else {"_a_int_packed": codes}
        quest.linear_forward(x_, w_, ws, wa, out=out_, _a_scale=sc_, _a_int_row_sum=rs_, use_hadamard=True,
                             block=args.block, **ws_kw)

    a_rsum = torch.empty(m, 1, dtype=torch.int32, device=dev)
    out = torch.empty(m, n_local, dtype=torch.bfloat16, device=dev)

    parity = None
    if world > 1:
        parity = check_exchange_parity(layer, x, n_local, args.block, ["push", "nccl"] if args.exchange == "push" else ["nccl"], dev)

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
            f1_op(x, a_packed, a_scale, a_rsum)
            mark(e1); mark(e2); e3.record()
        elif args.workload == "gemm":
            e0.record(); mark(e1)
            gemm_op(a_packed, wp, a_rsum, a_scale, out)
            mark(e2); e3.record()
        elif world == 1 and not split:
            e0.record()
            layer_op(x, a_packed, a_scale, a_rsum, wp, out)
            e3.record()
        elif world == 1:
            e0.record()
            f1_op(x, a_packed, a_scale, a_rsum)
            mark(e1)
            gemm_op(a_packed, wp, a_rsum, a_scale, out)
            mark(e2); e3.record()
        else:  # N > 1: the sharded layer (push: the GEMM epilogue stores its tiles into every rank's output, then one
            # device-side barrier; nccl: all-gather + interleaving copy); events at the layer's two stage boundaries
            e0.record()
            layer.forward(x, on_stage=lambda name: mark(e1 if name == "quantised" else e2))
            e3.record()
        if timers is not None:
            timers.append((e0, e1 if split else e0, e2 if split else e3, e3))

    if args.workload == "gemm":  # the GEMM-only workload needs quantised activations once
        f1_op(x, a_packed, a_scale, a_rsum)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        flush.add_(1)
        step()
    barrier()
    # Single-GPU layer: the step (one linear_forward call, two launches) is captured once into a CUDA graph and replayed (what a serving
    # loop does with a launch-bound step); the per-kernel pass below still launches them one by one.
    graph = None
    if world == 1 and args.workload == "linear" and not args.no_graph:
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                layer_op(x, a_packed, a_scale, a_rsum, wp, out)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    barrier()  # rank 0 waited for the clock sampler's first sample: start the timed region together
    # Timed region 1: the K steps the headline value comes from.
    # One GPU: exactly K steps back to back between two events, step i on operand set i mod n; the n sets (activations,
    # workspaces, a copy of the weights, output) occupy distinct memory and together exceed 2.5 x L2, so every step finds
    # its inputs in HBM.  Up to 256 consecutive steps are captured once into a CUDA graph (K itself for short runs), the
    # graph is replayed as often as it fits into K and the remaining steps are launched one by one inside the same bracket.
    timers = []
    t_step_b2b = None
    wall0 = time.perf_counter()
    if graph is not None:
        set_bytes = 2.0 * m * k + a_packed.numel() + n_local * k / 2 + 2.0 * m * n_local
        n_sets = min(sets_for(set_bytes), max(args.steps, 1))
        lsets = [(x.clone(), torch.empty_like(a_packed), torch.empty_like(a_scale), torch.empty_like(a_rsum), wp.clone(),
                  torch.empty_like(out)) for _ in range(n_sets)]

        def layer_step(i):
            xs, pk, sc, rs, wps, os_ = lsets[i]
            layer_op(xs, pk, sc, rs, wps, os_)

        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream())
        chain_steps = min(args.steps, max(n_sets, 256 // n_sets * n_sets))  # steps per graph: K itself for short runs
        with torch.cuda.stream(side):
            chain = torch.cuda.CUDAGraph()
            with torch.cuda.graph(chain, stream=side):
                for i in range(chain_steps):
                    layer_step(i % n_sets)
        torch.cuda.current_stream().wait_stream(side)
        for _ in range(max(2, -(-3 // chain_steps))):  # at least 3 more warm-up steps through the timed path
            chain.replay()
        torch.cuda.synchronize()
        e0, e3 = ev(), ev()
        wall0 = time.perf_counter()
        e0.record()
        for _ in range(args.steps // chain_steps):
            chain.replay()
        for i in range(args.steps % chain_steps):
            layer_step(i % n_sets)
        e3.record()
        barrier()
        t_step_b2b = e0.elapsed_time(e3) * 1e-3 / args.steps
        del lsets, chain
    elif world > 1 and args.workload == "linear":
        # N > 1: exactly K steps of the sharded layer back to back between two events (barrier + synchronise on both
        # sides), step i on activation set i mod n and on sibling layer i mod n (own copy of the weight shard, shared
        # output buffers), so that every step reads its activations and weights from HBM.  The ranks meet in every step's
        # exchange; the slowest rank's bracket is taken.
        set_bytes = 2.0 * m * k + m * k / 2 + n_local * k / 2
        n_sets = min(sets_for(set_bytes), max(args.steps, 1))
        sibs = [layer] + [layer.sibling((wp.clone(), ws.clone(), wa.clone())) for _ in range(n_sets - 1)]
        xs = [x.clone() for _ in range(n_sets)]
        for i in range(max(3, n_sets)):
            sibs[i % n_sets](xs[i % n_sets])
        barrier()
        e0, e3 = ev(), ev()
        wall0 = time.perf_counter()
        e0.record()
        for i in range(args.steps):
            sibs[i % n_sets](xs[i % n_sets])
        e3.record()
        barrier()
        t_step_b2b = e0.elapsed_time(e3) * 1e-3 / args.steps
        del sibs, xs
    wall = time.perf_counter() - wall0
    # Timed region 1b: the K steps one by one, each between its own pair of events with the L2 flushed before it (one
    # GPU: the step's two launches replayed from a graph).  This is the headline region for N > 1; on one GPU it is the
    # isolated-step figure reported beside the back-to-back one (an event pair around ~40 us of work adds launch gaps).
    wall1 = time.perf_counter()
    for _ in range(args.steps):
        flush.add_(1)  # evict the previous step's tensors from L2 (outside the event brackets)
        if graph is not None:
            e0, e3 = ev(), ev()
            e0.record(); graph.replay(); e3.record()
            timers.append((e0, e0, e3, e3))
        else:
            step(timers, split=False)
    barrier()
    if t_step_b2b is None:
        wall = time.perf_counter() - wall1
    # Timed region 2: the same K steps with events between the kernels (isolated per-kernel figures; each includes the
    # launch gap that an event between two launches costs).
    split_timers = []
    for _ in range(args.steps):
        flush.add_(1)
        step(split_timers, split=True)
    barrier()

    # Timed region 3 (per-kernel roofline figures): K launches of each kernel back to back on rotating operand sets.
    t_gemm_b2b = t_f1_b2b = None
    n_gemm_sets = n_f1_sets = 0
    if args.workload in ("linear", "gemm"):
        gemm_set_bytes = a_packed.numel() + n_local * k / 2 + 2.0 * m * n_local
        n_gemm_sets = sets_for(gemm_set_bytes)
        f1_op(x, a_packed, a_scale, a_rsum)
        gsets = [(a_packed.clone(), wp.clone(), torch.empty_like(out)) for _ in range(n_gemm_sets)]
        reps = max(1, -(-args.steps // n_gemm_sets))
        t_gemm_b2b = rotating_sets_time(
            lambda i: gemm_op(gsets[i][0], gsets[i][1], a_rsum, a_scale, gsets[i][2]), n_gemm_sets, reps, dev)
        del gsets
    if args.workload in ("linear", "hadamard_quantize"):
        f1_set_bytes = 2.0 * m * k + a_packed.numel()
        n_f1_sets = sets_for(f1_set_bytes)
        fsets = [(x.clone(), torch.empty_like(a_packed)) for _ in range(n_f1_sets)]
        reps = max(1, -(-args.steps // n_f1_sets))
        t_f1_b2b = rotating_sets_time(
            lambda i: f1_op(fsets[i][0], fsets[i][1], a_scale, a_rsum), n_f1_sets, reps, dev)
        del fsets
    # The fused quantiser on an input far larger than L2 (M=65536, K=8192: 1.07 GB in, 0.27 GB out), single GPU only.
    f1_large = None
    if world == 1 and args.workload == "linear":
        lm, lk = 65536, 8192
        xl = torch.empty(lm, lk, dtype=torch.bfloat16, device=dev)
        gl = torch.Generator(device=dev).manual_seed(1)
        for r0 in range(0, lm, 8192):  # Laplace(0,1), every hundredth column x50 (the bandwidth sweep's distribution)
            u = (torch.rand(8192, lk, generator=gl, device=dev) - 0.5) * 0.9999  # |u| < 0.5: finite
            v = -u.sign() * torch.log1p(-2 * u.abs())
            v[:, ::100] *= 50
            xl[r0:r0 + 8192] = v.to(torch.bfloat16)
            del u, v
        pl = torch.empty(lm, lk // 2, dtype=torch.uint8, device=dev)
        sl = torch.empty(lm, 1, dtype=torch.bfloat16, device=dev)
        rl = torch.empty(lm, 1, dtype=torch.int32, device=dev)
        n_large = min(max(args.steps, 5), 50)
        for _ in range(3):
            quest.hadamard_quantize_int4(xl, args.block, pl, sl, rl)
        torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(n_large):
            quest.hadamard_quantize_int4(xl, args.block, pl, sl, rl)
        e1.record()
        torch.cuda.synchronize()
        t_large = e0.elapsed_time(e1) * 1e-3 / n_large
        large_bytes = 2.0 * lm * lk + lm * lk / 2 + 6.0 * lm
        f1_large = {"kernel": "hadamard_quant_tc_kernel (tcgen05)", "bound": "hbm", "shape": f"M={lm} K={lk} block={args.block}",
                    "achieved": large_bytes / t_large / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": large_bytes / t_large / 1e9 / peaks["hbm_gbs"], "peak_source": f"hbm_gbs of {peaks['source']}",
                    "algorithmic_bytes": large_bytes, "us_per_launch": t_large * 1e6, "launches": n_large,
                    "traffic": None, "timing": "back-to-back launches between two events; the 1.3 GB working set is ten times L2"}
        del xl, pl, sl, rl
    clocks = sampler.stop() if sampler else None

    t_f1 = sum(e0.elapsed_time(e1) for e0, e1, _, _ in split_timers) / len(split_timers) * 1e-3
    t_gemm = sum(e1.elapsed_time(e2) for _, e1, e2, _ in split_timers) / len(split_timers) * 1e-3
    t_split_step = sum(e0.elapsed_time(e3) for e0, _, _, e3 in split_timers) / len(split_timers) * 1e-3
    t_step_isolated = sum(e0.elapsed_time(e3) for e0, _, _, e3 in timers) / len(timers) * 1e-3
    t_step = t_step_b2b if t_step_b2b is not None else t_step_isolated
    if os.environ.get("QB200_BENCH_DEBUG"):
        t_x = sum(e2.elapsed_time(e3) for _, _, e2, e3 in split_timers) / len(split_timers) * 1e-3
        print(f"[rank {rank}] step {t_step * 1e6:.1f} us, isolated {t_step_isolated * 1e6:.1f} us (with inner events {t_split_step * 1e6:.1f} = f1 {t_f1 * 1e6:.1f} + gemm {t_gemm * 1e6:.1f} + exchange {t_x * 1e6:.1f});"
              f" wall/step {wall / args.steps * 1e6:.1f} us", file=sys.stderr, flush=True)
    if world > 1:
        tt = torch.tensor([t_step, t_f1, t_gemm, t_gemm_b2b or 0.0, t_f1_b2b or 0.0, t_step_isolated], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        t_step, t_f1, t_gemm, tg, tf, t_step_isolated = tt.tolist()
        t_gemm_b2b = tg if t_gemm_b2b is not None else None
        t_f1_b2b = tf if t_f1_b2b is not None else None

    # ---- end to end through the public API, host buffers in and out ----
    e2e = None
    if not args.no_e2e and args.workload == "linear":
        x_pin = x_host.pin_memory()
        # N > 1: every rank copies the (replicated) activations in; the assembled [M, N_total] result goes back to the
        # host ONCE, split by rows over the ranks' PCIe links (rank r reads rows r*M/N .. of its own assembled copy).
        rows_per_rank = -(-m // world)
        r0, r1 = min(m, rank * rows_per_rank), min(m, (rank + 1) * rows_per_rank)
        y_pin = torch.empty(r1 - r0, n_total, dtype=torch.bfloat16).pin_memory()
        x_dev = torch.empty_like(x)

        def e2e_step():
            x_dev.copy_(x_pin, non_blocking=True)
            if world == 1:
                y = quest.linear_forward(x_dev, wp, ws, wa, out=out, _a_scale=a_scale, _a_int_row_sum=a_rsum, use_hadamard=True,
                                         block=args.block, **({"_a_int8": a_packed} if use_a8 else {"_a_int_packed": a_packed}))
            else:
                y = layer(x_dev)[r0:r1]
            y_pin.copy_(y, non_blocking=True)

        for _ in range(3):
            e2e_step()
        barrier()
        n_e2e = min(args.steps, 200)
        ets = []
        for _ in range(n_e2e):
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
        api = "quest_b200.linear_forward" if world == 1 else "quest_b200.sharded.ShardedLinear4bit.forward"
        one_stream = {"value": 2.0 * m * n_total * k / t_e2e / 1e12, "unit": "TOPS", "ms_per_step": t_e2e * 1e3,
                      "h2d_bytes_per_step": x_pin.numel() * 2, "d2h_bytes_per_step": y_pin.numel() * 2, "api": api,
                      "mode": "one stream: copy in, layer, copy out, one step after the other"}

        # The same calls as a user would pipeline them: host->device copy, layer and device->host copy of
        # consecutive steps on three streams with two sets of buffers, so that the two PCIe directions and the
        # kernels overlap.  Every step still copies its input in and its result out inside the timed region.  With
        # N > 1 the layer's result lives in buffers its peers write into, so the compute stream first copies it to a
        # private staging buffer (inside the timed region) and the copy-out stream reads that.
        s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        xb = [torch.empty_like(x) for _ in range(2)]
        ob = [torch.empty(r1 - r0, n_total, dtype=torch.bfloat16, device=dev) for _ in range(2)]
        wsb = [(torch.empty_like(a_scale), torch.empty_like(a_packed), torch.empty_like(a_rsum)) for _ in range(2)]
        yb = [torch.empty(r1 - r0, n_total, dtype=torch.bfloat16).pin_memory() for _ in range(2)]
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
                    if world == 1:
                        sc, pk, rs = wsb[b]
                        quest.linear_forward(xb[b], wp, ws, wa, out=ob[b], _a_scale=sc, _a_int_row_sum=rs, use_hadamard=True,
                                             block=args.block, **({"_a_int8": pk} if use_a8 else {"_a_int_packed": pk}))
                    else:
                        ob[b].copy_(layer(xb[b])[r0:r1])
                    cmp_done[b] = torch.cuda.Event(); cmp_done[b].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(cmp_done[b])
                    yb[b].copy_(ob[b], non_blocking=True)
                    out_done[b] = torch.cuda.Event(); out_done[b].record(s_out)

        pipelined(4)
        barrier()
        t0, t1 = ev(), ev()
        t0.record(s_in)
        pipelined(n_e2e)
        s_out.wait_stream(s_cmp); s_out.wait_stream(s_in)
        t1.record(s_out)
        barrier()
        t_pipe = t0.elapsed_time(t1) / n_e2e * 1e-3
        if world > 1:
            tt = torch.tensor([t_pipe], dtype=torch.float64, device=dev)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            t_pipe = tt.item()
        e2e = {"value": 2.0 * m * n_total * k / t_pipe / 1e12, "unit": "TOPS", "ms_per_step": t_pipe * 1e3,
               "h2d_bytes_per_step": x_pin.numel() * 2, "d2h_bytes_per_step": y_pin.numel() * 2, "api": api, "steps": n_e2e,
               "mode": "three streams (copy in / layer / copy out), two buffer sets; L2 flushed before every layer call"
                       + ("; every rank copies the activations in; the assembled [M, N_total] result is read back once, split by rows over"
                          " the ranks (h2d/d2h bytes are per rank)" if world > 1 else ""),
               "one_stream": one_stream}

    status = quest.device_status()
    if status != 0:
        raise RuntimeError(f"a kernel reported device status {status:#x}")

    if rank == 0:
        ops_total = 2.0 * m * n_total * k
        ops_gemm = 2.0 * m * n_local * k
        f1_bytes = 2.0 * m * k + a_packed.numel() + 6.0 * m  # bf16 in + codes out (packed int4, or the int8 operand) + bf16 scale + int32 row sum
        int8_peak = 2.0 * peaks["bf16_tflops"]        # tcgen05 kind::i8 runs at twice the bf16 rate
        gemm_traffic = NCU_TRAFFIC.get(("gemm", m, k, n_local, bool(use_a8)))
        f1_traffic = NCU_TRAFFIC.get(("hadamard_quantize", m, k, None, bool(use_a8)))
        t_gemm_roof = t_gemm_b2b if t_gemm_b2b else t_gemm
        t_f1_roof = t_f1_b2b if t_f1_b2b else t_f1
        if args.workload == "hadamard_quantize":
            value, unit, t_main = f1_bytes / t_f1_roof / 1e9, "GB/s", t_f1_roof
        elif args.workload == "gemm":
            value, unit, t_main = ops_gemm / t_gemm_roof / 1e12, "TOPS", t_gemm_roof
        else:
            value, unit, t_main = ops_total / t_step / 1e12, "TOPS", t_step
        launches_per_step = {"hadamard_quantize": 1, "gemm": 1}.get(args.workload, 2)
        b2b_note = ("K launches back to back (one CUDA graph of {n} launches on {n} rotating operand sets, {mb:.0f} MB in total, "
                    "replayed between two events): every launch finds its operands in HBM and no event sits between launches")
        line = {
            "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": t_main * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int4 operands, int8 tcgen05 MMA, int32 accumulate, bf16 out",
            "data": "synthetic", "config": workload_config(args, world),
            "roofline": {"kernel": "gemm_i4_wide_kernel / gemm_i4_kernel (TMA -> int4 unpack -> tcgen05 kind::i8, fused dequant epilogue;"
                                   " 256x256 tiles at the default shape, last tile of a CTA stored with bulk tensor stores)", "bound": "tensor",
                         "achieved": ops_gemm / t_gemm_roof / 1e12 if t_gemm_roof > 0 else None, "peak": int8_peak,
                         "unit": "TOPS", "frac": (ops_gemm / t_gemm_roof / 1e12) / int8_peak if t_gemm_roof > 0 else None,
                         "peak_source": f"2 x bf16_tflops ({peaks['bf16_tflops']}) of {peaks['source']}",
                         "traffic": gemm_traffic[0] if gemm_traffic else None,
                         "traffic_source": gemm_traffic[1] if gemm_traffic else None,
                         "us_per_launch": t_gemm_roof * 1e6,
                         "us_per_launch_isolated": t_gemm * 1e6 if t_gemm > 0 else None,
                         "route": ("int8 operand: the quantiser writes 16 x code as int8 in the GEMM's operand order, the 256x256 kernel copies A"
                                   " with TMA and unpacks only B (the library's default where both kernels apply; QB200_A8=0 for packed A)")
                         if use_a8 else "packed int4 A and B, both unpacked in the kernel",
                         "timing": b2b_note.format(n=n_gemm_sets, mb=n_gemm_sets * (a_packed.numel() + n_local * k / 2 + 2.0 * m * n_local) / 1e6)
                         if t_gemm_b2b else "events between the step's kernels",
                         "isolated_note": "us_per_launch_isolated: one launch between two events inside the step, launch gap included"},
            "roofline_hadamard_quantize": {"kernel": ("fused Hadamard+scale+quantise: hadamard_quant_tc_kernel (tcgen05), writing the GEMM's int8 operand"
                                                      if use_a8 else
                                                      "fused Hadamard+scale+quantise+pack: hadamard_quant_tc_kernel (tcgen05) from ~12 M elements,"
                                                      " hadamard_quant_mma_kernel below and for row lengths the tcgen05 tiling refuses"), "bound": "hbm",
                                           "achieved": f1_bytes / t_f1_roof / 1e9 if t_f1_roof > 0 else None,
                                           "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                           "frac": (f1_bytes / t_f1_roof / 1e9) / peaks["hbm_gbs"] if t_f1_roof > 0 else None,
                                           "peak_source": f"hbm_gbs of {peaks['source']}",
                                           "traffic": f1_traffic[0] if f1_traffic else None,
                                           "traffic_source": f1_traffic[1] if f1_traffic else None,
                                           "us_per_launch": t_f1_roof * 1e6,
                                           "us_per_launch_isolated": t_f1 * 1e6 if t_f1 > 0 else None,
                                           "algorithmic_bytes": f1_bytes,
                                           "output": "int8 operand [M, K] (see roofline.route)" if use_a8 else "packed int4 [M, K/2]",
                                           "timing": b2b_note.format(n=n_f1_sets, mb=n_f1_sets * (2.0 * m * k + a_packed.numel()) / 1e6)
                                           if t_f1_b2b else "events between the step's kernels"},
            "e2e": e2e,
            "gpu_launches": launches_per_step * args.steps,
            "gpu_launches_note": "launches inside timed region 1 (the region `value` comes from); the per-kernel regions launch"
                                 " the same kernels again",
            "clocks": clocks,
            "timing": {"value_from": ("exactly K steps back to back between two events, on operand sets that rotate through more than"
                                      " 2.5 x L2 (a CUDA graph of the sets, replayed; the remainder launched one by one)")
                                     if t_step_b2b is not None and world == 1 else
                                     ("exactly K steps of the sharded layer back to back between two events, on activation sets and sibling"
                                      " layers (own weight copies) that rotate through more than 2.5 x L2; max over ranks")
                                     if t_step_b2b is not None else
                                     "K steps, each between its own pair of events with the L2 flushed before it; max over ranks",
                       "roofline_from": "K launches of each kernel back to back on rotating operand sets (see roofline.timing)",
                       "ms_per_step_isolated": t_step_isolated * 1e3,
                       "isolated_note": "one step between two events, L2 flushed before it (launch gaps included)",
                       "ms_per_step_with_inner_events": t_split_step * 1e3},
            "wall_s_timed_region": wall,
        }
        if f1_large is not None:
            line["roofline_hadamard_quantize_large"] = f1_large
        if parity is not None:
            line["parity"] = parity
        if not args.no_cpu_baseline and world == 1 and args.workload == "linear":
            r = cpu_reference_run(args, steps=5, warmup=1)
            line["cpu_baseline"] = {"value": r["tops"], "unit": "TOPS", "cores": r["cores"], "kind": "port",
                                    "sample": r["sample"], "ms_per_step": r["seconds_per_step"] * 1e3}
        emit(line)
    bad_parity = parity is not None and not parity["equal"]
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if bad_parity:
        sys.exit(3)


# ----------------------------------------------------------------------------------------------------
def run_c4(args):
    """The 70B-shaped layers, column-sharded over the GPUs of this run: (K=8192, N=28672), (K=8192, N=10240),
    (K=28672, N=8192) x M in {16, 2048, 8192}.  Per shape and rank count: the shard GEMM alone, the replicated fused
    quantiser alone, and the whole step (quantiser + GEMM + exchange) for the push and the NCCL exchange, each as the
    max over ranks of a device-timed mean; plus the bit-identity check of the assembled output.  One JSON object."""
    import torch.distributed as dist
    import quest_b200 as quest
    from quest_b200.sharded import ShardedLinear4bit, shard_bounds

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    peaks = measured_peaks()
    flush = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.int32, device=dev)
    iters = min(max(args.steps, 5), 30)

    def maxr(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def timed(fn):
        for _ in range(3):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.add_(1)
            s, e = ev(), ev()
            s.record(); fn(); e.record()
            ts.append((s, e))
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        return maxr(sum(s.elapsed_time(e) for s, e in ts) / len(ts) * 1e-3)

    rows = []
    all_equal = True
    for (k, n_total) in ((8192, 28672), (8192, 10240), (28672, 8192)):
        n0, n1 = shard_bounds(n_total, rank, world)
        n_local = n1 - n0
        # every rank can regenerate every shard: device generator seeded by the shard's owner
        def shard(s):
            a, b = shard_bounds(n_total, s, world)
            g = torch.Generator(device=dev).manual_seed(7000 + 31 * s + k)
            w = (0.01 * torch.randn(b - a, k, generator=g, device=dev)).to(torch.bfloat16)
            return quest.preprocess_weight(w, use_hadamard=True, block=args.block)[:3]
        wp, ws, wa = shard(rank)
        for m in (16, 2048, 8192):
            gx = torch.Generator(device=dev).manual_seed(m + k)
            x = torch.randn(m, k, generator=gx, device=dev).to(torch.bfloat16)
            pk = torch.empty(m, k // 2, dtype=torch.uint8, device=dev)
            sc = torch.empty(m, 1, dtype=torch.bfloat16, device=dev)
            rs = torch.empty(m, 1, dtype=torch.int32, device=dev)
            local = torch.empty(m, n_local, dtype=torch.bfloat16, device=dev)
            t_f1 = timed(lambda: quest.hadamard_quantize_int4(x, args.block, pk, sc, rs))
            t_gemm = timed(lambda: quest.fused_matmul_dequantize_int4_int4t_bf16(pk, wp, rs, wa, sc, ws, local))
            row = {"M": m, "K": k, "N_total": n_total, "N_per_gpu": n_local, "gpus": world,
                   "gemm_us": t_gemm * 1e6, "gemm_tops_per_gpu": 2.0 * m * n_local * k / t_gemm / 1e12,
                   "gemm_frac_int8_peak": 2.0 * m * n_local * k / t_gemm / 1e12 / (2 * peaks["bf16_tflops"]),
                   "gemm_weight_gbs": n_local * k / 2 / t_gemm / 1e9,
                   "f1_us": t_f1 * 1e6, "f1_gbs": (2.5 * m * k + 6.0 * m) / t_f1 / 1e9,
                   "gemm_plus_f1_us": (t_gemm + t_f1) * 1e6,
                   "aggregate_tops_gemm_plus_f1": 2.0 * m * n_total * k / (t_gemm + t_f1) / 1e12}
            if world == 1:
                # the whole layer as linear_forward runs it on one GPU: the route the library prefers for the shape (int8
                # operand with balanced tile columns where the 256-row kernel applies), one call, dependent launches
                a8 = quest.prefers_a8(m, k, n_local)
                codes = torch.empty(m, k if a8 else k // 2, dtype=torch.uint8, device=dev)
                ws_kw = {"_a_int8": codes} if a8 else {"_a_int_packed": codes}
                t_layer = timed(lambda: quest.linear_forward(x, wp, ws, wa, out=local, _a_scale=sc, _a_int_row_sum=rs,
                                                             use_hadamard=True, block=args.block, **ws_kw))
                row["layer_us"] = t_layer * 1e6
                row["layer_route"] = "int8 operand" if a8 else "packed int4"
                row["aggregate_tops_layer"] = 2.0 * m * n_total * k / t_layer / 1e12
                del codes
            if world > 1:
                delivered = {}
                for exch in ("push", "nccl"):
                    try:
                        lay = ShardedLinear4bit((wp, ws, wa), n_total, rank, world, use_hadamard=True, block=args.block, exchange=exch)
                        lay.workspaces(m, k, dev, torch.bfloat16)
                        ok = torch.ones(1, device=dev)
                    except Exception as e:  # noqa: BLE001
                        print(f"[rank {rank}] c4: exchange {exch} unavailable ({e!r})", file=sys.stderr)
                        ok = torch.zeros(1, device=dev)
                    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                    if ok.item() == 0:
                        continue
                    t_full = timed(lambda: lay(x))
                    delivered[exch] = lay(x).clone()
                    recv = 2.0 * m * (n_total - n_local)
                    row[f"step_{exch}_us"] = t_full * 1e6
                    row[f"aggregate_tops_{exch}"] = 2.0 * m * n_total * k / t_full / 1e12
                    row[f"exchange_{exch}_us"] = (t_full - t_gemm - t_f1) * 1e6
                    row["recv_bytes_per_gpu"] = recv
                    row["nvlink_floor_us"] = recv / 770e9 * 1e6
                    del lay
                torch.cuda.synchronize()
                with quest.layer_launches():  # the quantiser kernel the layer itself chooses for this size
                    quest.hadamard_quantize_int4(x, args.block, pk, sc, rs)
                equal = bool(delivered)
                for s in range(world):
                    a, b = shard_bounds(n_total, s, world)
                    wps, wss, was = shard(s)
                    want = quest.fused_matmul_dequantize_int4_int4t_bf16(pk, wps, rs, was, sc, wss)
                    for exch, full in delivered.items():
                        equal = equal and full[:, a:b].equal(want)
                    del wps, want
                flag = torch.tensor([1.0 if equal else 0.0], device=dev)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                row["parity_equal"] = bool(flag.item() == 1.0)
                row["parity_exchanges"] = sorted(delivered)
                all_equal = all_equal and row["parity_equal"]
                del delivered
            rows.append(row)
            del x, pk, local
            torch.cuda.empty_cache()
        del wp, ws, wa
    status = quest.device_status()
    if rank == 0:
        emit({"workload": "c4: Llama-2-70B-shaped layers, column-sharded", "n_gpus": world, "peaks": peaks, "iters": iters,
              "timing": "CUDA events around each call, L2 flushed between calls, mean over iters, max over ranks",
              "inputs": "activations N(0,1) bf16, weights N(0,0.01) quantised to packed int4 (device generators)",
              "parity": {"equal": all_equal, "ranks": world} if world > 1 else None, "device_status": status, "rows": rows})
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not all_equal or status != 0:
        sys.exit(3)


def run_prefill(args):
    """End-to-end prefill of the 800M-shaped decoder (d=2048, 16 layers, 16 heads, SwiGLU 5632, vocab 32000) with
    random-init weights: bf16 linears vs W4A4 linears (with Hadamard) vs no-op linears, eager and CUDA graph."""
    from quest_b200.prefill import Decoder, DecoderConfig, swap_linears, prefill_time
    dev = torch.device("cuda", 0)
    cfg = DecoderConfig(sequence_length=max(1024, args.seq))
    out = {"metric": "prefill ms (batch x seq tokens through the decoder body)", "unit": "ms", "higher_is_better": False,
           "config": {"workload": f"prefill d={cfg.n_embd} L={cfg.n_layer} heads={cfg.n_head} ffn={cfg.ffn} "
                                  f"batch={args.batch} seq={args.seq}", "data": "uniform random token ids, random-init weights"}}
    modes = ("bf16", "int4", "int4_fused", "noop") if hasattr(sys.modules.get("quest_b200.prefill"), "FUSED_MODES") else ("bf16", "int4", "noop")
    for mode in modes:
        torch.manual_seed(0)
        model = swap_linears(Decoder(cfg).to(device=dev, dtype=torch.bfloat16).eval(), mode, use_hadamard=True)
        eager_ms, graph_ms, _ = prefill_time(model, args.batch, args.seq, n_warmup=args.warmup, n_iter=min(args.steps, 20))
        out[mode] = {"eager_ms": eager_ms, "graph_ms": graph_ms, "tokens_per_s": args.batch * args.seq / (min(eager_ms, graph_ms) * 1e-3)}
        del model
        torch.cuda.empty_cache()
    best = "int4_fused" if "int4_fused" in out else "int4"
    out["value"] = min(out[best]["eager_ms"], out[best]["graph_ms"])
    out["speedup_vs_bf16"] = min(out["bf16"]["eager_ms"], out["bf16"]["graph_ms"]) / out["value"]
    emit(out)


def run_layers(args):
    """Per-layer table in the reference's form (gemm-quest/benchmarks/bench_layer.py:12-54): for every layer shape of the
    800M and 7B models and batch sizes 32..16384, seconds per layer of a 20-layer chain (min of eager and CUDA graph) for
    the bf16 cuBLAS linear, the W4A4 layer without and with the Hadamard transform."""
    import quest_b200 as quest
    from quest_b200.harness import do_bench_network
    dev = torch.device("cuda", 0)
    dtype = torch.bfloat16
    hidden_sizes = [(6144, 2048), (2048, 2048), (11264, 2048), (2048, 5632), (12288, 4096), (4096, 4096), (22016, 4096), (4096, 11008)]
    batch_sizes = [2 ** i for i in range(5, 15)]
    if args.steps < 20:  # a short run: a subset
        hidden_sizes, batch_sizes = [(4096, 4096), (2048, 5632)], [32, 2048, 16384]
    table = []
    for n, k in hidden_sizes:
        g = torch.Generator(device=dev).manual_seed(n + k)
        weight = (0.02 * torch.randn(n, k, generator=g, device=dev)).to(dtype)
        wp, ws, wa, _ = quest.preprocess_weight(weight, use_hadamard=True)
        for m in batch_sizes:
            a_scale = torch.empty(m, 1, dtype=dtype, device=dev)
            a_packed = torch.empty(m, k // 2, dtype=torch.uint8, device=dev)
            a_rsum = torch.empty(m, 1, dtype=torch.int32, device=dev)
            t_base = do_bench_network(lambda a_in, a_out: torch.matmul(a_in, weight.t(), out=a_out), m, k, n, dtype, dev)
            t_kernel = do_bench_network(
                lambda a_in, a_out: quest.linear_forward(a_in, wp, ws, wa, out=a_out, _a_scale=a_scale, _a_int_packed=a_packed,
                                                         _a_int_row_sum=a_rsum, use_hadamard=False), m, k, n, dtype, dev)
            # with the Hadamard transform the layer takes the route the library prefers for the shape
            a8 = quest.prefers_a8(m, k, n)
            had_ws = {"_a_int8": torch.empty(m, k, dtype=torch.uint8, device=dev)} if a8 else {"_a_int_packed": a_packed}
            t_had = do_bench_network(
                lambda a_in, a_out: quest.linear_forward(a_in, wp, ws, wa, out=a_out, _a_scale=a_scale, _a_int_row_sum=a_rsum,
                                                         use_hadamard=True, **had_ws), m, k, n, dtype, dev)
            del had_ws
            table.append({"N": n, "K": k, "M": m, "route": "int8 operand" if a8 else "packed int4", "bf16_us": t_base * 1e6, "int4_us": t_kernel * 1e6, "int4_hadamard_us": t_had * 1e6,
                          "speedup_int4": t_base / t_kernel, "speedup_int4_hadamard": t_base / t_had,
                          "int4_hadamard_tops": 2.0 * m * n * k / t_had / 1e12})
        del weight, wp
    emit({"workload": "layers: 20 chained equal layers, min(eager, CUDA graph) per layer; bf16 = torch.matmul (cuBLAS)",
          "note": "the chain's activations (<= 0.4 GB) and weights are re-used layer after layer, so small shapes run from L2, as in the reference's harness",
          "table": table})


def run_sweep(args):
    """The single-GPU shape sweeps: W4A4 linear at K=4096, N in {4096, 11008, 12288}, M in {1, 16, 128, 2048, 8192}
    and the Hadamard+quantise bandwidth sweep M in {1, 256, 4096, 65536} x K in {4096, 8192, 14336} x block in
    {64, 128, 256}.  Every figure is the time per launch over back-to-back launches on operand sets that rotate
    through more than the L2 size (see rotating_sets_time), so small launches are not padded by event overhead."""
    import quest_b200 as quest
    dev = torch.device("cuda", 0)
    peaks = measured_peaks()
    g = torch.Generator(device=dev).manual_seed(0)
    linear = []
    for n in (4096, 11008, 12288):
        w = (0.02 * torch.randn(n, 4096, generator=g, device=dev)).to(torch.bfloat16)
        wp, ws, wa, _ = quest.preprocess_weight(w, use_hadamard=True)
        for m in (1, 16, 128, 2048, 8192):
            x = torch.randn(m, 4096, generator=g, device=dev).to(torch.bfloat16)
            sc = torch.empty(m, 1, dtype=torch.bfloat16, device=dev)
            rs = torch.empty(m, 1, dtype=torch.int32, device=dev)
            a8 = quest.prefers_a8(m, 4096, n)  # the route linear_forward takes for this shape
            code_bytes = m * (4096 if a8 else 2048)
            gemm_bytes = code_bytes + n * 2048 + 2.0 * m * n + 6.0 * (m + n)
            ns = sets_for(gemm_bytes)
            sets = [(x.clone(), torch.empty(m, 4096 if a8 else 2048, dtype=torch.uint8, device=dev), wp.clone(),
                     torch.empty(m, n, dtype=torch.bfloat16, device=dev)) for _ in range(ns)]
            f1 = quest.hadamard_quantize_a8 if a8 else quest.hadamard_quantize_int4
            mm = quest.fused_matmul_dequantize_a8 if a8 else quest.fused_matmul_dequantize_int4_int4t_bf16
            for s in sets:
                f1(s[0], 128, s[1], sc, rs)
            reps = max(1, 40 // ns)
            t_q = rotating_sets_time(lambda i: f1(sets[i][0], 128, sets[i][1], sc, rs), ns, reps, dev)
            t_g = rotating_sets_time(lambda i: mm(sets[i][1], sets[i][2], rs, wa, sc, ws, sets[i][3]), ns, reps, dev)

            def both(i):  # the layer as linear_forward runs it (one library call, the GEMM launched behind the quantiser)
                ws_kw = {"_a_int8": sets[i][1]} if a8 else {"_a_int_packed": sets[i][1]}
                quest.linear_forward(sets[i][0], sets[i][2], ws, wa, out=sets[i][3], _a_scale=sc, _a_int_row_sum=rs,
                                     use_hadamard=True, **ws_kw)
            t_l = rotating_sets_time(both, ns, reps, dev)
            ops = 2.0 * m * n * 4096
            linear.append({"M": m, "N": n, "K": 4096, "route": "int8 operand" if a8 else "packed int4", "quantize_us": t_q * 1e6, "gemm_us": t_g * 1e6, "layer_us": t_l * 1e6,
                           "gemm_tops": ops / t_g / 1e12, "gemm_frac_int8_peak": ops / t_g / 1e12 / (2 * peaks["bf16_tflops"]),
                           "gemm_gbs": gemm_bytes / t_g / 1e9, "gemm_frac_hbm": gemm_bytes / t_g / 1e9 / peaks["hbm_gbs"],
                           "layer_tops": ops / t_l / 1e12, "sets": ns})
            del sets
        del w, wp
    hq = []
    for k in (4096, 8192, 14336):
        for m in (1, 256, 4096, 65536):
            nbytes = 2.0 * m * k + m * k / 2 + 6.0 * m
            ns = sets_for(nbytes)
            xs = []
            for _ in range(ns):
                u = (torch.rand(m, k, generator=g, device=dev) - 0.5) * 0.9999  # |u| < 0.5: finite
                v = -u.sign() * torch.log1p(-2 * u.abs())
                v[:, ::100] *= 50
                xs.append(v.to(torch.bfloat16))
                del u, v
            sc = torch.empty(m, 1, dtype=torch.bfloat16, device=dev)
            rs = torch.empty(m, 1, dtype=torch.int32, device=dev)
            pks = [torch.empty(m, k // 2, dtype=torch.uint8, device=dev) for _ in range(ns)]
            for block in (64, 128, 256):
                reps = max(1, 30 // ns)
                t = rotating_sets_time(lambda i: quest.hadamard_quantize_int4(xs[i], block, pks[i], sc, rs), ns, reps, dev)
                hq.append({"M": m, "K": k, "block": block, "us": t * 1e6, "gbs": nbytes / t / 1e9,
                           "frac_of_hbm": nbytes / t / 1e9 / peaks["hbm_gbs"], "sets": ns})
            del xs, pks
            torch.cuda.empty_cache()
    emit({"workload": "sweep", "peaks": peaks,
          "timing": "time per launch over back-to-back launches in one CUDA graph on operand sets rotating through > 2.5 x L2",
          "inputs": "linear: activations N(0,1), weights N(0,0.02); hadamard_quantize: Laplace(0,1) with every hundredth column x50",
          "linear": linear, "hadamard_quantize": hq})


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
    elif args.workload == "sweep":
        run_sweep(args)
    elif args.workload == "layers":
        run_layers(args)
    elif args.workload == "c4":
        run_c4(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
