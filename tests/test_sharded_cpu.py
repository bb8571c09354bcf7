"""Host-side logic of the column-sharded layer on CPU: shard bounds, weight slicing and the all-gather +
interleave assembly, run as two gloo ranks.  The per-shard compute is replaced by the CPU oracle here (the
CUDA kernels are covered by the GPU tests); the assembled output must equal the unsharded oracle output."""
from __future__ import annotations

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, make_activations


def test_shard_bounds_cover_and_align():
    from quest_b200.sharded import shard_bounds
    for n, g in [(4096, 8), (28672, 8), (10240, 4), (8192, 2), (264, 4), (8, 2)]:
        spans = [shard_bounds(n, r, g) for r in range(g)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0
        assert all(a % 8 == 0 and b % 8 == 0 and b >= a for a, b in spans)
    with pytest.raises(ValueError):
        shard_bounds(100, 0, 2)


def _worker(rank: int, world: int, port: int, n_total: int, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import quest_oracle as O
        from quest_b200.sharded import ShardedLinear4bit, shard_weight

        class OracleShard(ShardedLinear4bit):
            def compute_shard(self, x, out_cols, ws):
                out_cols.copy_(O.linear_forward(x, self.w_int_packed, self.w_scale, self.w_add,
                                                use_hadamard=self.use_hadamard, block=self.block))

        m, k = 24, 256
        x = make_activations("randn", m, k, seed=1)
        w = make_activations("randn", n_total, k, seed=2)
        wp, ws, wa, _ = O.preprocess_weight(w, use_hadamard=True)
        layer = OracleShard(shard_weight(wp, ws, wa, rank, world), n_total, rank, world, use_hadamard=True)
        y = layer(x)
        ref = O.linear_forward(x, wp, ws, wa, use_hadamard=True)
        ok = y.equal(ref)
        # a second call reuses the workspaces and must give the same bits
        ok = ok and layer(x).equal(ref)
        # a rank with a mismatched shard is refused on the host, before any collective
        try:
            OracleShard((wp, ws, wa), n_total, rank, world)
            ok = False
        except ValueError:
            pass
        q.put((rank, ok))
    except Exception as e:  # report instead of leaving the parent waiting on the queue
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_total", [64, 72])  # 72 = uneven split (40 + 32): non-uniform gather path
def test_two_rank_gather_assembles_full_output(n_total):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000) + n_total
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n_total, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, True), (1, True)]
