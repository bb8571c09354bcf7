"""Activation-side workspaces of the W4A4 linear, kept between calls.

The reference's ``linear_forward`` takes caller-owned workspaces (``_a_scale``, ``_a_int_packed``, ``_a_int_row_sum``;
gemm-quest/benchmarks/utils.py:63-66, 92-99) so that a benchmark or a CUDA graph allocates nothing per call, but its
``Linear4bit`` passes none and allocates three tensors on every forward.  Here the module takes them from a cache:
one set per (device, stream, M, K), shared by every layer that runs on that stream - layers of a model execute one
after the other in stream order, and each consumes its quantised activations before it returns, so one set is enough.
In the steady state a forward allocates only its output.  Entries created while a stream is being captured belong to
that graph's memory pool; the cache keeps them alive, so the graph and later eager calls may both use them.
"""
from __future__ import annotations

import torch


class WorkspaceCache:
    def __init__(self):
        self._sets: dict = {}

    def get(self, m: int, k: int, device: torch.device, dtype: torch.dtype = torch.bfloat16, int8_operand: bool = False) -> dict:
        """{'_a_scale': [M,1] dtype, '_a_int_row_sum': [M,1] int32, and '_a_int_packed': [M,K/2] uint8 or, with
        ``int8_operand``, '_a_int8': [M,K] uint8} for the current stream of ``device``."""
        stream = torch.cuda.current_stream(device).cuda_stream
        key = (device.index, stream, m, k, dtype, bool(int8_operand))
        ws = self._sets.get(key)
        if ws is None:
            ws = {"_a_scale": torch.empty(m, 1, dtype=dtype, device=device),
                  "_a_int_row_sum": torch.empty(m, 1, dtype=torch.int32, device=device)}
            if int8_operand:
                ws["_a_int8"] = torch.empty(m, k, dtype=torch.uint8, device=device)
            else:
                ws["_a_int_packed"] = torch.empty(m, k // 2, dtype=torch.uint8, device=device)
            self._sets[key] = ws
        return ws

    def clear(self) -> None:
        self._sets.clear()

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for ws in self._sets.values() for t in ws.values())


default_cache = WorkspaceCache()
