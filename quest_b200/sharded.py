"""Column-sharded (N-sharded) W4A4 linear across the GPUs of one node.

Each rank owns the weight rows [n0, n0 + N/g) (packed codes, per-row scales and offsets slice exactly,
no re-quantisation), every rank quantises the replicated activations itself (cheap and deterministic,
so all ranks hold identical codes), runs the fused GEMM for its N/g output columns and the column
blocks are assembled with one all-gather.  Per element the arithmetic is the single-GPU arithmetic, so
the assembled output is bit-identical to the 1-GPU result.  The reference has no multi-GPU inference
path; this is the exchange step the sharding needs and nothing more.

Two exchange modes:
  "push"  the GEMM epilogue stores every finished tile straight into the [M, N_total] output buffer of every GPU
          (buffers in symmetric memory, plain peer stores over NVLink, issued while later tiles are still being
          computed), followed by one device-side barrier.  No collective kernel, no interleaving copy.
  "nccl"  each rank computes into a local block, NCCL all-gathers the blocks and one copy interleaves them.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

import quest_b200 as quest


def shard_bounds(n_total: int, rank: int, world: int, align: int = 8) -> tuple[int, int]:
    """[n0, n1) of the output columns owned by ``rank``.  Columns are dealt in multiples of ``align``
    (16-byte bf16 stores) and the remainder goes to the last ranks one ``align`` block at a time."""
    if n_total % align != 0:
        raise ValueError(f"N={n_total} must be a multiple of {align} to be column-sharded")
    blocks = n_total // align
    base, extra = divmod(blocks, world)
    counts = [base + (1 if r >= world - extra else 0) for r in range(world)]
    n0 = sum(counts[:rank]) * align
    return n0, n0 + counts[rank] * align


def shard_weight(w_int_packed: torch.Tensor, w_scale: torch.Tensor, w_add: torch.Tensor, rank: int, world: int):
    """Row slices of preprocess_weight's outputs for ``rank`` (contiguous copies)."""
    n0, n1 = shard_bounds(w_int_packed.size(0), rank, world)
    return (w_int_packed[n0:n1].contiguous(), w_scale[n0:n1].contiguous(), w_add[n0:n1].contiguous())


class ShardedLinear4bit:
    """One rank's part of a column-sharded W4A4 linear layer.

    forward(x) returns the full [M, N_total] bf16 output on every rank.  Buffers are allocated once per
    M (workspaces are reused across calls, so the steady state launches only kernels and one collective).
    """

    def __init__(self, w_shard: tuple[torch.Tensor, torch.Tensor, torch.Tensor], n_total: int, rank: int, world: int,
                 group=None, use_hadamard: bool = True, block: int = 128, exchange: str = "nccl"):
        if exchange not in ("nccl", "push"):
            raise ValueError(f"unknown exchange mode {exchange!r}")
        self.exchange = exchange
        self.w_int_packed, self.w_scale, self.w_add = w_shard
        self.n_total, self.rank, self.world, self.group = n_total, rank, world, group
        self.use_hadamard, self.block = use_hadamard, block
        self.n0, self.n1 = shard_bounds(n_total, rank, world)
        if self.w_int_packed.size(0) != self.n1 - self.n0:
            raise ValueError("weight shard does not match this rank's column range")
        self.widths = [shard_bounds(n_total, r, world)[1] - shard_bounds(n_total, r, world)[0] for r in range(world)]
        self.width_max = max(self.widths)  # uneven splits gather equal-sized (padded) blocks
        self._ws = {}

    # -- compute for this rank's columns (CUDA kernels; overridden by the CPU tests of the host logic) --
    _stage = None  # set by forward() while a caller wants to be told about stage boundaries

    def sibling(self, w_shard: tuple[torch.Tensor, torch.Tensor, torch.Tensor]) -> "ShardedLinear4bit":
        """Another layer of the same shape and sharding with its own weights that shares this layer's workspaces and
        output buffers (layers of a model run one after the other; no new collective set-up is needed)."""
        import copy
        other = copy.copy(self)
        other.w_int_packed, other.w_scale, other.w_add = w_shard
        if other.w_int_packed.shape != self.w_int_packed.shape:
            raise ValueError("a sibling layer must have this layer's shard shape")
        return other

    def compute_shard(self, x: torch.Tensor, out_cols: torch.Tensor, ws: dict) -> None:
        # quantiser and GEMM as one layer (same choice of quantiser kernel and of dependent launches as linear_forward)
        with quest.layer_launches() if self.use_hadamard else contextlib.nullcontext():
            self.quantize_activations(x, ws)
            if self._stage is not None:
                self._stage("quantised")
            quest.fused_matmul_dequantize_int4_int4t_bf16_into(ws["a_int_packed"], self.w_int_packed, ws["a_int_row_sum"],
                                                               self.w_add, ws["a_scale"], self.w_scale, out_cols)

    def quantize_activations(self, x: torch.Tensor, ws: dict) -> None:
        if self.use_hadamard:
            quest.hadamard_quantize_int4(x, self.block, ws["a_int_packed"], ws["a_scale"], ws["a_int_row_sum"])
        else:
            quest.find_scale_int4(x, ws["a_scale"])
            quest.quantize_int4(x, ws["a_scale"], None, ws["a_int_packed"], ws["a_int_row_sum"])

    def symmetric_outputs(self, m: int, device, dtype) -> list:
        """Two [M, N_total] output buffers in symmetric memory (alternated call by call, so that one barrier per
        call is enough: a buffer is rewritten only after every rank has passed the barrier of the call in between,
        which in stream order lies behind that rank's readers of the older result).  Collective: every rank must
        make its first call with a given M together."""
        import torch.distributed._symmetric_memory as symm_mem
        group = self.group if self.group is not None else dist.group.WORLD
        out = []
        for _ in range(2):
            t = symm_mem.empty((m, self.n_total), dtype=dtype, device=device)
            hdl = symm_mem.rendezvous(t, group)
            ptrs = [int(p) for p in hdl.buffer_ptrs]
            if len(ptrs) != self.world:
                raise RuntimeError("symmetric memory group does not match the sharding world size")
            try:  # every rank's buffer as a tensor in this process (used for the small-M exchange)
                views = [hdl.get_buffer(r, (m, self.n_total), dtype) for r in range(self.world)]
            except Exception:  # noqa: BLE001  (older symmetric-memory API: the push kernel handles every M)
                views = None
            out.append((t, hdl, ptrs, views))
        return out

    def workspaces(self, m: int, k: int, device, dtype) -> dict:
        key = (m, k, str(device))
        if key not in self._ws:
            self._ws[key] = dict(
                symm=self.symmetric_outputs(m, device, dtype) if (self.exchange == "push" and self.world > 1) else None,
                parity=0,
                a_scale=torch.empty(m, 1, dtype=dtype, device=device),
                a_int_packed=torch.empty(m, k // 2, dtype=torch.uint8, device=device),
                a_int_row_sum=torch.empty(m, 1, dtype=torch.int32, device=device),
                local=torch.zeros(m, self.width_max, dtype=dtype, device=device),
                gathered=torch.empty(self.world, m, self.width_max, dtype=dtype, device=device),
                out=torch.empty(m, self.n_total, dtype=dtype, device=device),
            )
        return self._ws[key]

    SMALL_M = 16  # up to this many rows the single-GPU small-M kernels compute the shard and plain copies deliver it

    def forward(self, x: torch.Tensor, gather: bool = True, on_stage=None) -> torch.Tensor:
        """``on_stage(name)``, if given, is called after the activations are quantised ("quantised") and after this
        rank's columns are computed and on their way ("computed"): a benchmark records events there."""
        stage = on_stage if on_stage is not None else (lambda name: None)
        m, k = x.shape
        ws = self.workspaces(m, k, x.device, x.dtype)
        out = ws["out"]
        if self.world == 1:
            self.compute_shard(x, out, ws)
            return out
        if not gather:
            self.compute_shard(x, out[:, self.n0:self.n1], ws)
            return out
        if self.exchange == "push":
            t, hdl, ptrs, views = ws["symm"][ws["parity"]]
            ws["parity"] ^= 1
            small = m <= self.SMALL_M and views is not None
            if small:
                # Few rows: the weight-streaming kernels (dp4a, split-K) are several times faster than a tensor-core
                # tile kernel that walks K serially, and the block to deliver is tiny - compute it into the local buffer
                # and copy it into every peer's.
                mine = t[:, self.n0:self.n1]
                self._stage = stage
                self.compute_shard(x, mine, ws)
                self._stage = None
                theirs = [views[(self.rank + i) % self.world][:, self.n0:self.n1] for i in range(1, self.world)]
                if not quest.copy_block_to_peers(mine, theirs):  # one launch for all peers where the block is 16-byte tiled
                    for dst in theirs:
                        dst.copy_(mine)
            else:
                off = self.n0 * t.element_size()
                order = [self.rank] + [(self.rank + i) % self.world for i in range(1, self.world)]
                if self.use_hadamard:
                    # quantiser and push GEMM as one layer: the GEMM sets itself up and requests its first weights while the
                    # quantiser's last blocks run, and the quantiser starts while the kernel before it drains
                    with quest.layer_launches():
                        self.quantize_activations(x, ws)
                        stage("quantised")
                        quest.fused_matmul_dequantize_int4_int4t_bf16_push(
                            ws["a_int_packed"], self.w_int_packed, ws["a_int_row_sum"], self.w_add, ws["a_scale"], self.w_scale,
                            [ptrs[r] + off for r in order], self.n_total)
                else:
                    self.quantize_activations(x, ws)
                    stage("quantised")
                    quest.fused_matmul_dequantize_int4_int4t_bf16_push(
                        ws["a_int_packed"], self.w_int_packed, ws["a_int_row_sum"], self.w_add, ws["a_scale"], self.w_scale,
                        [ptrs[r] + off for r in order], self.n_total)
            stage("computed")
            hdl.barrier(channel=0)  # every rank's tiles have landed everywhere
            return t
        # NCCL all-gather wants one contiguous, equal-sized block per rank: gather [g, M, width], then
        # interleave the column blocks into the row-major [M, N_total] result.
        self._stage = stage
        self.compute_shard(x, ws["local"][:, :self.n1 - self.n0], ws)
        self._stage = None
        stage("computed")
        dist.all_gather_into_tensor(ws["gathered"].view(-1), ws["local"].view(-1), group=self.group)
        if self.width_max * self.world == self.n_total:
            out.view(m, self.world, -1).copy_(ws["gathered"].permute(1, 0, 2))
        else:
            for r, w in enumerate(self.widths):
                a, _ = shard_bounds(self.n_total, r, self.world)
                out[:, a:a + w].copy_(ws["gathered"][r, :, :w])
        return out

    __call__ = forward
