"""Timing harness for chained layers: the reference's ``do_bench`` / ``do_bench_network``
(gemm-quest/benchmarks/utils.py:787-835) with device-side timing.

``do_bench_network`` runs ``n_layers`` calls of ``f(activation_in, activation_out)`` back to back on views of one
workspace - what a model's stack of equal layers looks like to the GPU: no host gap, no event between the layers -
once launched one by one and once replayed from a CUDA graph, and returns the smaller time per layer.  The reference
measures with the host clock around a device synchronisation; here CUDA events on the launching stream bracket the
chain, which removes the host's share without changing what is compared.
"""
from __future__ import annotations

import torch


@torch.inference_mode()
def do_bench(f, n_iter: int = 100, n_warmup: int = 10) -> float:
    """Seconds per call of ``f`` (mean over ``n_iter`` back-to-back calls after ``n_warmup``)."""
    for _ in range(n_warmup):
        f()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(n_iter):
        f()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) * 1e-3 / n_iter


@torch.inference_mode()
def do_bench_network(f, M: int, K: int, N: int, dtype: torch.dtype, device: torch.device, n_layers: int = 20,
                     n_warmup: int = 3, n_iter: int = 5, details: bool = False):
    """Seconds per layer of a chain of ``n_layers`` calls ``f(activation_in [M,K], activation_out [M,N])``:
    min(eager, CUDA graph), as the reference does.  ``details`` also returns (eager, graph) seconds per layer."""
    workspace = torch.empty(M * max(K, N), dtype=dtype, device=device)
    activation_in = workspace[:M * K].reshape(M, K)
    activation_out = workspace[:M * N].reshape(M, N)

    def network():
        for _ in range(n_layers):
            f(activation_in, activation_out)

    tf = do_bench(network, n_iter=n_iter, n_warmup=n_warmup)
    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream(device)
    s.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(s):
        for _ in range(n_warmup):
            network()
    torch.cuda.current_stream(device).wait_stream(s)
    with torch.cuda.graph(graph):
        network()
    tg = do_bench(graph.replay, n_iter=n_iter, n_warmup=n_warmup)
    t = min(tf, tg) / n_layers
    return (t, tf / n_layers, tg / n_layers) if details else t
