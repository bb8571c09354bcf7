"""GPU parity at the sizes the benchmarks are quoted on: the down-projection row lengths (K = 5632, 11008) and the other
7B / 70B row lengths for the fused Hadamard+quantise kernels, launches of 4096 and 65536 rows, and the int4 GEMM at the
corners of the 7B sweep and on the column shards of the 70B layers.

Small and medium cases are compared with the CPU oracle directly.  Where the oracle would need minutes (a full
8192 x 12288 x 4096 product) the exact int32 accumulators are compared with cuBLAS int8 on the unpacked codes plus
O(MK + NK) row/column checksums computed on the CPU, and the fused output with the oracle's epilogue expression
evaluated on those exact accumulators."""
from __future__ import annotations

import pytest
import torch

from oracle import quest_oracle as O
from conftest import make_activations

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import quest_b200 as quest
    DEV = torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    assert quest.device_status() == 0, "a kernel reported a bounded-wait timeout"


# Tolerated rate of +-1 code flips per element against the canonical ("exact sum, one rounding") oracle.  A flip needs a
# transform output that the kernel's fp32 summation rounds to the neighbouring bf16 value AND that sits beside a
# quantisation boundary; heavy-tailed rows (Laplace with x50 outlier columns) are the worst case measured, 8e-6.
FLIP_RATE = 2e-5


def hq_against_oracle(x: torch.Tensor, block: int, packed, scale, row_sum) -> tuple[int, int]:
    """Codes / scales / row sums of the rows ``x`` (CPU) against the canonical oracle.  Returns (code flips, scale flips)."""
    p_ref, s_ref, r_ref, _ = O.hadamard_quantize_int4(x, block)
    packed, scale, row_sum = packed.cpu(), scale.cpu(), row_sum.cpu()
    assert int(O.bf16_ulp_distance(scale, s_ref).max()) <= 1
    same = (scale == s_ref).view(-1)
    nflip, maxd = O.count_code_flips(packed[same], p_ref[same])
    assert maxd <= 1
    assert row_sum.equal(O.unpack_int4(packed).to(torch.int32).sum(-1, keepdim=True))
    return nflip, int((~same).sum())


# ------------------------------------------------------------------ Hadamard + quantise ----------------
# K = 5632 (44 blocks) and 11008 (86 blocks) are the down-projection row lengths: the tcgen05 kernel's tiling refuses
# them, so they run on hadamard_quant_mma_kernel; 10240 and 12288 are further 7B / 70B row lengths.
@pytest.mark.parametrize("block", [64, 128, 256])
@pytest.mark.parametrize("k", [5632, 11008, 10240, 12288])
@pytest.mark.parametrize("kind,m", [("student", 1), ("laplace", 33), ("randn", 300)])
@pytest.mark.parametrize("kernel", ["auto", "mma"])
def test_hadamard_quantize_down_projection_row_lengths(block, k, kind, m, kernel, monkeypatch):
    if kernel != "auto":
        monkeypatch.setenv("QB200_HQ_KERNEL", kernel)
    x = make_activations(kind, m, k, seed=block + m + k)
    packed, scale, row_sum = quest.hadamard_quantize_int4(x.to(DEV), block)
    nflip, sflip = hq_against_oracle(x, block, packed, scale, row_sum)
    assert nflip <= 1 + int(FLIP_RATE * m * k), (nflip, m * k)
    assert sflip <= max(1, m // 1000)


@pytest.mark.parametrize("k", [4096, 5632, 11008])
def test_hadamard_quantize_4096_rows(k):
    """A launch of 4096 tokens (the bandwidth sweep's middle size), every row against the oracle."""
    m = 4096
    x = make_activations("laplace", m, k, seed=k)
    packed, scale, row_sum = quest.hadamard_quantize_int4(x.to(DEV), 128)
    nflip, sflip = hq_against_oracle(x, 128, packed, scale, row_sum)
    assert nflip <= 1 + int(FLIP_RATE * m * k), (nflip, m * k)
    assert sflip <= max(1, m // 1000)


@pytest.mark.parametrize("k,block", [(4096, 128), (8192, 64), (14336, 256)])
def test_hadamard_quantize_65536_rows_sampled(k, block):
    """The largest launch of the bandwidth sweep (65536 tokens): 256 rows spread over the whole launch (first, last and
    a fixed stride in between) against the oracle, and the row sums of every row against the codes written."""
    m = 65536
    g = torch.Generator(device=DEV).manual_seed(k)
    x = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
    for r0 in range(0, m, 8192):  # Laplace(0, 1) with every hundredth column x50, generated on the device in slabs
        u = (torch.rand(8192, k, generator=g, device=DEV) - 0.5) * 0.9999  # |u| < 0.5: finite
        v = -u.sign() * torch.log1p(-2 * u.abs())
        v[:, ::100] *= 50
        x[r0:r0 + 8192] = v.to(torch.bfloat16)
        del u, v
    packed, scale, row_sum = quest.hadamard_quantize_int4(x, block)
    rows = torch.cat([torch.arange(0, m, 257), torch.tensor([m - 1])])[:256].to(DEV)
    nflip, sflip = hq_against_oracle(x[rows].cpu(), block, packed[rows], scale[rows], row_sum[rows])
    assert nflip <= 1 + int(FLIP_RATE * rows.numel() * k)
    assert sflip <= 1
    for r0 in range(0, m, 16384):
        codes = quest.unpack_int4(packed[r0:r0 + 16384])
        assert row_sum[r0:r0 + 16384].equal(codes.sum(-1, keepdim=True, dtype=torch.int32))
        del codes


def test_hadamard_quantize_real_down_projection_layer():
    """The 800M model's down projection (K = 5632 -> N = 2048) at 1024 tokens, layer output against the oracle layer."""
    m, k, n = 1024, 5632, 2048
    x = make_activations("student", m, k, seed=3)
    w = (0.02 * torch.randn(n, k, generator=torch.Generator().manual_seed(4))).to(torch.bfloat16)
    wp, ws, wa, _ = O.preprocess_weight(w, use_hadamard=True)
    y = quest.linear_forward(x.to(DEV), wp.to(DEV), ws.to(DEV), wa.to(DEV), use_hadamard=True).cpu()
    y_ref = O.linear_forward(x, wp, ws, wa, use_hadamard=True)
    pa, sa, _ = quest.hadamard_quantize_int4(x.to(DEV))
    pa_ref, sa_ref, _, _ = O.hadamard_quantize_int4(x)
    if pa.cpu().equal(pa_ref) and sa.cpu().equal(sa_ref):
        assert y.equal(y_ref)
    else:  # a tie flip of one activation code moves one row of outputs by at most a few ulp
        assert (y != y_ref).float().mean() < 0.02
        assert ((y.float() - y_ref.float()).norm() / y_ref.float().norm()).item() < 1e-3


# ------------------------------------------------------------------ int4 GEMM at the benchmark shapes ---
def random_packed_dev(rows: int, k: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, (rows, k // 2), generator=g, dtype=torch.uint8).to(DEV)  # every byte = two uniform codes


def epilogue_vectors(m: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    a_add = torch.randint(-8 * 64, 8 * 64, (m, 1), generator=g, dtype=torch.int32)
    b_add = torch.randint(-8 * 64, 8 * 64, (n, 1), generator=g, dtype=torch.int32)
    a_mul = (torch.rand(m, 1, generator=g) + 0.05).to(torch.bfloat16)
    b_mul = (0.02 * torch.rand(n, 1, generator=g) + 0.001).to(torch.bfloat16)
    return [t.to(DEV) for t in (a_add, a_mul, b_add, b_mul)]


def cublas_int8_product(ad: torch.Tensor, bd: torch.Tensor) -> torch.Tensor:
    a8 = quest.unpack_int4(ad)
    if a8.size(0) <= 16:  # torch._int_mm wants more than 16 rows
        a8 = torch.cat([a8, torch.zeros(32 - a8.size(0), a8.size(1), dtype=torch.int8, device=DEV)])
    return torch._int_mm(a8, quest.unpack_int4(bd).t().contiguous())[:ad.size(0)]


BENCH_GEMM_SHAPES = [
    # corners of the 7B sweep (K = 4096)
    (8192, 4096, 12288), (128, 4096, 11008), (2048, 4096, 11008), (8192, 4096, 4096), (1, 4096, 12288), (16, 4096, 11008),
    # column shards of the 70B layers: K = 8192 with N/g in {3584, 1280}, K = 28672 with N/g = 1024
    (16, 8192, 3584), (2048, 8192, 3584), (16, 8192, 1280), (2048, 8192, 1280), (16, 28672, 1024), (2048, 28672, 1024),
]


@pytest.mark.parametrize("m,k,n", BENCH_GEMM_SHAPES)
def test_gemm_benchmark_shapes_exact(m, k, n):
    ad, bd = random_packed_dev(m, k, m + k), random_packed_dev(n, k, n + k + 1)
    c = quest.matmul_int4_int4t_int32(ad, bd)
    ref = cublas_int8_product(ad, bd)
    assert c.equal(ref)
    # checksums against CPU arithmetic that never forms the product: sum_n C[m, n] = A[m, :] . (sum_n B[n, :])
    ai, bi = O.unpack_int4(ad.cpu()).to(torch.int64), O.unpack_int4(bd.cpu()).to(torch.int64)
    assert c.sum(dim=1, dtype=torch.int64).cpu().equal(ai @ bi.sum(dim=0))
    assert c.sum(dim=0, dtype=torch.int64).cpu().equal(bi @ ai.sum(dim=0))
    # fused output = the oracle's epilogue expression on those exact accumulators
    a_add, a_mul, b_add, b_mul = epilogue_vectors(m, n, m + n)
    want = O.add_mul_vv(a_add, a_mul, b_add, b_mul, ref, torch.empty(m, n, dtype=torch.bfloat16, device=DEV))
    got = quest.fused_matmul_dequantize_int4_int4t_bf16(ad, bd, a_add, b_add, a_mul, b_mul)
    assert got.equal(want)
    if m <= 256:  # small enough for the CPU oracle end to end
        cpu = O.fused_matmul_dequantize_int4_int4t_bf16(ad.cpu(), bd.cpu(), a_add.cpu(), b_add.cpu(), a_mul.cpu(), b_mul.cpu())
        assert got.cpu().equal(cpu)


@pytest.mark.parametrize("tile", ["auto", "128", "512"])
@pytest.mark.parametrize("m,k,n", [(300, 1024, 520), (256, 4096, 512), (2048, 512, 256)])
def test_fused_epilogue_with_large_add_vectors(tile, m, k, n, monkeypatch):
    """The add vectors are caller data: sums 2*acc + a_add + b_add far beyond the range a quantised layer produces,
    including beyond 2^24 where the int-to-float conversion itself rounds, must give the oracle's bits too."""
    if tile != "auto":
        monkeypatch.setenv("QB200_GEMM_TILE", tile)
    ad, bd = random_packed_dev(m, k, 21), random_packed_dev(n, k, 22)
    g = torch.Generator().manual_seed(23)
    a_add = torch.randint(-512, 512, (m, 1), generator=g, dtype=torch.int32)
    b_add = torch.randint(-512, 512, (n, 1), generator=g, dtype=torch.int32)
    a_add[::7] = torch.randint(-2 ** 23, 2 ** 23, (a_add[::7].numel(), 1), generator=g, dtype=torch.int32)   # rows beyond the bound
    a_add[3] = 2 ** 26 + 12345                                                                             # the conversion rounds
    b_add[40:44] = torch.randint(-2 ** 22, 2 ** 22, (4, 1), generator=g, dtype=torch.int32)               # one 32-column chunk
    b_add[n - 1] = -(2 ** 25) - 77
    a_mul = (torch.rand(m, 1, generator=g) + 0.05).to(torch.bfloat16)
    b_mul = (0.02 * torch.rand(n, 1, generator=g) + 0.001).to(torch.bfloat16)
    a_add, a_mul, b_add, b_mul = [t.to(DEV) for t in (a_add, a_mul, b_add, b_mul)]
    ref = O.add_mul_vv(a_add, a_mul, b_add, b_mul, cublas_int8_product(ad, bd), torch.empty(m, n, dtype=torch.bfloat16, device=DEV))
    got = quest.fused_matmul_dequantize_int4_int4t_bf16(ad, bd, a_add, b_add, a_mul, b_mul)
    assert got.equal(ref)
    cpu = O.fused_matmul_dequantize_int4_int4t_bf16(ad.cpu(), bd.cpu(), a_add.cpu(), b_add.cpu(), a_mul.cpu(), b_mul.cpu())
    assert got.cpu().equal(cpu)


def test_fused_matmul_dequantize_int4_bf16_switch():
    """The Python switch of the reference's layer code: debug_mode=True (int32 GEMM + add_mul_vv, with and without a
    caller-owned int32 workspace) and debug_mode=False (fused kernel) give the oracle's bits."""
    m, k, n = 160, 768, 224
    ad, bd = random_packed_dev(m, k, 1), random_packed_dev(n, k, 2)
    a_add, a_mul, b_add, b_mul = epilogue_vectors(m, n, 3)
    ref = O.fused_matmul_dequantize_int4_int4t_bf16(ad.cpu(), bd.cpu(), a_add.cpu(), b_add.cpu(), a_mul.cpu(), b_mul.cpu())
    d = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    c = torch.empty(m, n, dtype=torch.int32, device=DEV)
    out = quest.fused_matmul_dequantize_int4_bf16(ad, bd, a_add, b_add, a_mul, b_mul, d, _mat_c=c, debug_mode=True)
    assert out is d and d.cpu().equal(ref) and c.cpu().equal(O.matmul_int4_int4t_int32(ad.cpu(), bd.cpu()))
    out = quest.fused_matmul_dequantize_int4_bf16(ad, bd, a_add, b_add, a_mul, b_mul, None)  # the reference's default: debug
    assert out.dtype == torch.bfloat16 and out.cpu().equal(ref)
    d.zero_()
    quest.fused_matmul_dequantize_int4_bf16(ad, bd, a_add, b_add, a_mul, b_mul, d, debug_mode=False)
    assert d.cpu().equal(ref)


def test_split_k_graph_survives_a_larger_eager_request(monkeypatch):
    """A CUDA graph that captured a split-K launch keeps working after an eager call that needs far more split-K scratch:
    the per-device scratch buffer has a fixed size and is never freed or moved."""
    m, k, n = 16, 8192, 1024
    ad, bd = random_packed_dev(m, k, 5), random_packed_dev(n, k, 6)
    out = torch.zeros(m, n, dtype=torch.int32, device=DEV)
    ref = cublas_int8_product(ad, bd)
    monkeypatch.setenv("QB200_GEMM_SPLITS", "8")
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(2):
            quest.matmul_int4_int4t_int32(ad, bd, out=out)  # allocates the scratch outside the capture
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        quest.matmul_int4_int4t_int32(ad, bd, out=out)
    # 16 tiles x 8 ranges x 96 rows: six times the slabs of the captured launch
    big_a, big_b = random_packed_dev(96, 16384, 7), random_packed_dev(4096, 16384, 8)
    big = quest.matmul_int4_int4t_int32(big_a, big_b)
    assert big.equal(cublas_int8_product(big_a, big_b))
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert out.equal(ref)


def test_bounded_wait_runs_out_and_is_reported(monkeypatch):
    """A launch whose TMA producer issues nothing: every consumer wait runs out after the shortened limit, the kernel
    returns, the status word names a wait site of the GEMM, and the next ordinary call is exact with a clean status."""
    from quest_b200 import _lib
    m, k, n = 300, 1024, 520
    ad, bd = random_packed_dev(m, k, 9), random_packed_dev(n, k, 10)
    a_add, a_mul, b_add, b_mul = epilogue_vectors(m, n, 11)
    d = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    want = O.fused_matmul_dequantize_int4_int4t_bf16(ad.cpu(), bd.cpu(), a_add.cpu(), b_add.cpu(), a_mul.cpu(), b_mul.cpu())
    lib = _lib.load()
    for tile in ("128", "512"):  # the 128-row kernel and the 256 x 256 kernel
        monkeypatch.setenv("QB200_GEMM_TILE", tile)
        st = lib.quest_b200_test_bounded_wait_cuda(d.data_ptr(), ad.data_ptr(), bd.data_ptr(), a_add.data_ptr(),
                                                   b_add.data_ptr(), a_mul.data_ptr(), b_mul.data_ptr(), m, k, n,
                                                   4_000_000, torch.cuda.current_stream().cuda_stream)
        monkeypatch.delenv("QB200_GEMM_TILE")
        assert st == 0
        status = quest.device_status()
        assert status & 0xFF == 5, hex(status)            # QB200_ERR_DEVICE_TIMEOUT
        assert (status >> 8) in (4, 6, 7, 8), hex(status)  # MMA issuer, epilogue or unpack warps waiting for data
        assert quest.device_status() == 0                  # reading it cleared it
        assert float(d.abs().max()) == 0.0                 # nothing was written
        got = quest.fused_matmul_dequantize_int4_int4t_bf16(ad, bd, a_add, b_add, a_mul, b_mul)
        assert got.cpu().equal(want)
        assert quest.device_status() == 0


# ------------------------------------------------------------------ producer-fused quantisers ----------
def rmsnorm_reference(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """The model's RMSNorm (src/models/llama.py:64-76) in plain torch on the CPU."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).type_as(x) * weight


def producer_against_oracle(y_ref: torch.Tensor, block: int, packed, scale, row_sum):
    """Outputs of a producer-fused kernel against hadamard_quantize_int4 of the CPU-computed producer output.  The
    producer's fp32 arithmetic (summation order of the mean, exp and rsqrt) is not bit-identical between the CPU and the
    GPU; one bf16 ulp of difference in an input of the transform moves codes only next to a quantisation boundary."""
    m, k = y_ref.shape
    nflip, sflip = hq_against_oracle(y_ref, block, packed, scale, row_sum)
    assert nflip <= 2 + int(5 * FLIP_RATE * m * k), (nflip, m * k)
    assert sflip <= max(2, m // 200), sflip


@pytest.mark.parametrize("block", [64, 128, 256])
@pytest.mark.parametrize("m,k", [(1, 2048), (300, 2048), (77, 4096), (40, 5632), (33, 11008), (2048, 2048)])
def test_rmsnorm_hadamard_quantize_matches_the_composition(block, m, k):
    x = make_activations("student", m, k, seed=m + k) * 3
    x = x.to(torch.bfloat16)
    g = torch.Generator().manual_seed(k)
    w = (1.0 + 0.2 * torch.randn(k, generator=g)).to(torch.bfloat16)
    eps = 1e-5
    y_ref = rmsnorm_reference(x, w, eps)
    packed, scale, row_sum = quest.rmsnorm_hadamard_quantize_int4(x.to(DEV), w.to(DEV), eps, block)
    producer_against_oracle(y_ref, block, packed, scale, row_sum)
    # and against the two-kernel route on the GPU (torch RMSNorm, then the ordinary fused quantiser)
    y_gpu = rmsnorm_reference(x.to(DEV), w.to(DEV), eps)
    p2, s2, r2 = quest.hadamard_quantize_int4(y_gpu.contiguous(), block)
    same = (s2 == scale).view(-1)
    assert int((~same).sum()) <= max(2, m // 200)
    nflip, maxd = O.count_code_flips(packed[same].cpu(), p2[same].cpu())
    assert maxd <= 1 and nflip <= 2 + int(5 * FLIP_RATE * m * k)


@pytest.mark.parametrize("block", [64, 128, 256])
@pytest.mark.parametrize("m,k", [(1, 5632), (300, 5632), (64, 11008), (50, 2048), (1024, 5632)])
def test_silu_mul_hadamard_quantize_matches_the_composition(block, m, k):
    gate = (make_activations("randn", m, k, seed=m + k) * 2).to(torch.bfloat16)
    up = make_activations("student", m, k, seed=m + k + 1)
    y_ref = torch.nn.functional.silu(gate) * up
    packed, scale, row_sum = quest.silu_mul_hadamard_quantize_int4(gate.to(DEV), up.to(DEV), block)
    producer_against_oracle(y_ref, block, packed, scale, row_sum)
    y_gpu = torch.nn.functional.silu(gate.to(DEV)) * up.to(DEV)
    p2, s2, r2 = quest.hadamard_quantize_int4(y_gpu.contiguous(), block)
    same = (s2 == scale).view(-1)
    assert int((~same).sum()) <= max(2, m // 200)
    nflip, maxd = O.count_code_flips(packed[same].cpu(), p2[same].cpu())
    assert maxd <= 1 and nflip <= 2 + int(5 * FLIP_RATE * m * k)


def test_prefill_fused_blocks_track_the_unfused_model():
    """The decoder with producer-fused quantisers against the same decoder with one quantiser launch per linear: the
    same weights and codes up to tie flips, so the outputs agree to W4A4 noise; a CUDA-graph replay repeats the eager
    result bit for bit."""
    from quest_b200.prefill import Decoder, DecoderConfig, swap_linears, prefill_time
    torch.manual_seed(0)
    cfg = DecoderConfig(n_embd=256, n_layer=2, n_head=4, ffn=768, vocab_size=512, sequence_length=64)
    base = Decoder(cfg).to(device=DEV, dtype=torch.bfloat16).eval()
    a = Decoder(cfg).to(device=DEV, dtype=torch.bfloat16).eval()
    b = Decoder(cfg).to(device=DEV, dtype=torch.bfloat16).eval()
    a.load_state_dict(base.state_dict())
    b.load_state_dict(base.state_dict())
    swap_linears(a, "int4", use_hadamard=True)
    swap_linears(b, "int4_fused", use_hadamard=True)
    idx = torch.randint(0, cfg.vocab_size, (4, 64), generator=torch.Generator().manual_seed(1)).to(DEV)
    with torch.inference_mode():
        ya, yb = a(idx), b(idx)
    rel = ((ya.float() - yb.float()).norm() / ya.float().norm()).item()
    assert rel < 0.02, rel
    eager_ms, graph_ms, y_graph = prefill_time(b, 4, 64, n_warmup=2, n_iter=3, seed=1)
    assert y_graph.equal(yb)


# ------------------------------------------------------------------ the layer in one call (few rows) ---
@pytest.mark.parametrize("m", [1, 3, 16, 200, 2048])
@pytest.mark.parametrize("k,n", [(4096, 4096), (5632, 2048), (8192, 1280)])
def test_one_call_layer_equals_the_two_op_route(m, k, n):
    """linear_forward makes one library call whose GEMM kernel (dp4a, split-K, 128-row or 256-row tiles, by shape) is
    launched with a programmatic dependency on the quantiser: the workspaces and the output must hold exactly what the
    two ops called one after the other give, call after call, and also when the call is replayed from a CUDA graph."""
    x = make_activations("student", m, k, seed=m + k).to(DEV)
    w = (0.02 * torch.randn(n, k, generator=torch.Generator().manual_seed(n))).to(torch.bfloat16).to(DEV)
    wp, ws, wa, _ = quest.preprocess_weight(w, use_hadamard=True)
    with quest.layer_launches():  # the same choice of quantiser kernel as inside the one call (tcgen05 from 3 M elements on)
        p_ref, s_ref, r_ref = quest.hadamard_quantize_int4(x)
        y_ref = quest.fused_matmul_dequantize_int4_int4t_bf16(p_ref, wp, r_ref, wa, s_ref, ws)
    pk = torch.zeros(m, k // 2, dtype=torch.uint8, device=DEV)
    sc = torch.zeros(m, 1, dtype=torch.bfloat16, device=DEV)
    rs = torch.zeros(m, 1, dtype=torch.int32, device=DEV)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    for _ in range(3):
        out.zero_()
        y = quest.linear_forward(x, wp, ws, wa, out=out, _a_scale=sc, _a_int_packed=pk, _a_int_row_sum=rs, use_hadamard=True)
        assert y is out and out.equal(y_ref) and pk.equal(p_ref) and sc.equal(s_ref) and rs.equal(r_ref)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        quest.linear_forward(x, wp, ws, wa, out=out, _a_scale=sc, _a_int_packed=pk, _a_int_row_sum=rs, use_hadamard=True)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        quest.linear_forward(x, wp, ws, wa, out=out, _a_scale=sc, _a_int_packed=pk, _a_int_row_sum=rs, use_hadamard=True)
    x2 = make_activations("randn", m, k, seed=7).to(DEV)
    x.copy_(x2)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    with quest.layer_launches():
        p2, s2, r2 = quest.hadamard_quantize_int4(x2)
        y2 = quest.fused_matmul_dequantize_int4_int4t_bf16(p2, wp, r2, wa, s2, ws)
    assert out.equal(y2) and pk.equal(p2)


# ------------------------------------------------------------------ balanced tile columns (256-row GEMM kernel) ---
@pytest.mark.parametrize("m,k,n", [
    (2048, 256, 4096),    # 8 x 16 tiles of 256 columns -> 8 x 18 of 240 / 224
    (2048, 128, 4000),    # the same cut with a ragged last column
    (2048, 128, 4088),    # N no multiple of 16: the last column reaches past N and is clipped
    (1900, 128, 14336),   # 8 x 56 -> 8 x 74 columns of 208 / 192, four waves, ragged last tile row
    (8192, 128, 4096),    # four tiles per CTA, every one narrower
    (1024, 256, 8192),    # 4 x 32 -> 4 x 37 columns of 224 / 208
    (2048, 128, 2560),    # packed operands only: 8 x 10 -> 8 x 18 columns of 144 / 128
    (2048, 128, 5120),    # packed operands only: 8 x 20 -> 8 x 37 columns of 144 / 128, two waves
    (600, 128, 3000),     # too few tiles to fill the SMs with tiles of at least 128 columns: stays at 256
])
def test_gemm_with_balanced_tile_columns(m, k, n, monkeypatch):
    """Where more, narrower tile columns fill the same number of waves over the SMs, the 256-row GEMM kernel cuts N into
    columns of 128 ... 240 (packed operands) or 192 ... 240 (int8 operand) instead of 256 (widths multiples of 16; the last
    64-column piece of a tile overlaps the one before it; B rows beyond the width are not unpacked).  Whatever the cut and
    whichever way the tiles are stored, both routes give the bits of the uniform 256-column tiles with per-thread stores,
    which in turn are the int32 product put through the epilogue in torch."""
    g = torch.Generator(device=DEV).manual_seed(m + n)
    monkeypatch.setenv("QB200_GEMM_TILE", "512")  # the 256-row kernel at every shape (packed route)
    for rnd in range(2):
        packed = torch.randint(0, 256, (m, k // 2), dtype=torch.uint8, device=DEV, generator=g)
        wp = torch.randint(0, 256, (n, k // 2), dtype=torch.uint8, device=DEV, generator=g)
        a_add = torch.randint(-8 * k, 8 * k, (m, 1), dtype=torch.int32, device=DEV, generator=g)
        b_add = torch.randint(-8 * k, 8 * k, (n, 1), dtype=torch.int32, device=DEV, generator=g)
        a_mul = (0.01 + torch.rand(m, 1, device=DEV, generator=g)).to(torch.bfloat16)
        b_mul = (0.01 + torch.rand(n, 1, device=DEV, generator=g)).to(torch.bfloat16)
        codes = quest.unpack_int4(packed).view(m, k // 32, 16, 2)
        a8 = (torch.cat([codes[..., 0], codes[..., 1]], dim=-1).reshape(m, k) * 16).to(torch.int8).view(torch.uint8).contiguous()
        monkeypatch.setenv("QB200_GEMM_BALANCE", "0")
        monkeypatch.setenv("QB200_GEMM_TMA_STORE", "0")
        ref = quest.fused_matmul_dequantize_int4_int4t_bf16(packed, wp, a_add, b_add, a_mul, b_mul)
        acc = (quest.unpack_int4(packed).float() @ quest.unpack_int4(wp).float().t()).to(torch.int32)  # exact: |sums| < 2^24
        want = ((2 * acc + a_add + b_add.t()).float() * (0.5 * a_mul.float() * b_mul.float().t())).to(torch.bfloat16)
        assert ref.equal(want)
        for balance in ("0", "1"):
            monkeypatch.setenv("QB200_GEMM_BALANCE", balance)
            # every way a tile can leave: per-thread stores throughout (0), 64-column bulk stores for a CTA's last tile (1),
            # plus 16-column bulk stores for its earlier tiles on the int8-operand route (unset)
            for store in ("0", "1", None):
                if store is None:
                    monkeypatch.delenv("QB200_GEMM_TMA_STORE")
                else:
                    monkeypatch.setenv("QB200_GEMM_TMA_STORE", store)
                out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
                quest.fused_matmul_dequantize_int4_int4t_bf16(packed, wp, a_add, b_add, a_mul, b_mul, out)
                assert out.equal(ref), ("packed", balance, store)
                out.fill_(float("nan"))
                quest.fused_matmul_dequantize_a8(a8, wp, a_add, b_add, a_mul, b_mul, out=out)
                assert out.equal(ref), ("int8 operand", balance, store)
        monkeypatch.delenv("QB200_GEMM_BALANCE")
    assert quest.device_status() == 0



@pytest.mark.parametrize("m,k,n", [(2048, 4096, 4096), (1024, 4096, 14336), (4096, 8192, 1024)])
def test_one_call_layer_on_the_int8_operand_route(m, k, n):
    """The same for the int8-operand route: the 256-row GEMM kernel starts behind the tcgen05 quantiser, copies and
    unpacks its first weights and waits on the device before its first A copy and before reading the row sums."""
    if not quest.prefers_a8(m, k, n):
        pytest.skip("the library does not choose the int8 operand for this shape")
    w = (0.02 * torch.randn(n, k, generator=torch.Generator().manual_seed(n))).to(torch.bfloat16).to(DEV)
    wp, ws, wa, _ = quest.preprocess_weight(w, use_hadamard=True)
    a8 = torch.zeros(m, k, dtype=torch.uint8, device=DEV)
    sc = torch.zeros(m, 1, dtype=torch.bfloat16, device=DEV)
    rs = torch.zeros(m, 1, dtype=torch.int32, device=DEV)
    out = torch.zeros(m, n, dtype=torch.bfloat16, device=DEV)
    x = make_activations("student", m, k, seed=m + k).to(DEV)

    def two_ops(xx):
        q, s_, r_ = quest.hadamard_quantize_a8(xx, 128)
        return q, s_, r_, quest.fused_matmul_dequantize_a8(q, wp, r_, wa, s_, ws)

    q_ref, s_ref, r_ref, y_ref = two_ops(x)
    for _ in range(3):
        out.zero_()
        y = quest.linear_forward(x, wp, ws, wa, out=out, _a_scale=sc, _a_int8=a8, _a_int_row_sum=rs, use_hadamard=True)
        assert y is out and out.equal(y_ref) and a8.equal(q_ref) and sc.equal(s_ref) and rs.equal(r_ref)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        quest.linear_forward(x, wp, ws, wa, out=out, _a_scale=sc, _a_int8=a8, _a_int_row_sum=rs, use_hadamard=True)
    torch.cuda.current_stream().wait_stream(s)
    # Layers back to back on shared workspaces: the next layer's quantiser is launched with a programmatic dependency on
    # this layer's GEMM, so it must not overwrite the operand, scales or row sums before that GEMM has read them.
    xb = make_activations("student", m, k, seed=5).to(DEV)
    outs = [torch.zeros(m, n, dtype=torch.bfloat16, device=DEV) for _ in range(4)]
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i, o in enumerate(outs):
            quest.linear_forward(x if i % 2 == 0 else xb, wp, ws, wa, out=o, _a_scale=sc, _a_int8=a8, _a_int_row_sum=rs, use_hadamard=True)
    for seed in (7, 8):
        x.copy_(make_activations("randn", m, k, seed=seed).to(DEV))
        xb.copy_(make_activations("student", m, k, seed=seed + 10).to(DEV))
        for o in outs:
            o.zero_()
        graph.replay()
        torch.cuda.synchronize()
        ya, yb = two_ops(x)[3], two_ops(xb)
        assert outs[0].equal(ya) and outs[2].equal(ya) and outs[1].equal(yb[3]) and outs[3].equal(yb[3])
        assert a8.equal(yb[0]) and sc.equal(yb[1]) and rs.equal(yb[2])
    assert quest.device_status() == 0


# ------------------------------------------------------------------ few-row exchange of the sharded layer ---
@pytest.mark.parametrize("rows,cols,n_dst", [(16, 3584, 7), (1, 1280, 3), (5, 1024, 1), (16, 8, 2)])
def test_copy_block_to_peers_writes_exactly_the_block(rows, cols, n_dst):
    """One launch copies a column block into the same place of up to seven other buffers (here all on this GPU; in the
    sharded layer they are the peers' outputs) and touches nothing around it; views that are not 16-byte tiled are refused
    without a copy."""
    n_total, n0 = cols * 3 + 64, cols + 32
    g = torch.Generator(device=DEV).manual_seed(rows + cols)
    bufs = [torch.randn(rows, n_total, device=DEV, generator=g).to(torch.bfloat16) for _ in range(n_dst + 1)]
    before = [b.clone() for b in bufs]
    src = bufs[0][:, n0:n0 + cols]
    assert quest.copy_block_to_peers(src, [b[:, n0:n0 + cols] for b in bufs[1:]])
    torch.cuda.synchronize()
    assert bufs[0].equal(before[0])
    for b, old in zip(bufs[1:], before[1:]):
        assert b[:, n0:n0 + cols].equal(before[0][:, n0:n0 + cols])
        assert b[:, :n0].equal(old[:, :n0]) and b[:, n0 + cols:].equal(old[:, n0 + cols:])
    odd = [b[:, 3:3 + cols] for b in bufs]  # starts 6 bytes into a row: not 16-byte aligned
    assert not quest.copy_block_to_peers(odd[0], odd[1:])
    assert quest.device_status() == 0
