"""GPU parity tests: every op goes through the C-ABI library and is compared with the CPU oracle on the
same seeded inputs.  Integer outputs (codes, packed bytes, row sums, int32 accumulators) must be bit-exact;
bf16 outputs of the epilogue must be bit-exact given exact accumulators.  The only tolerated deviation is
the documented one for the Hadamard step: +-1 code flips at rounding ties (rate asserted below)."""
from __future__ import annotations

import pytest
import torch

from oracle import quest_oracle as O
from conftest import GOLDEN_CASES, load_golden, make_activations

pytestmark = pytest.mark.gpu

if torch.cuda.is_available():
    import quest_b200 as quest
    DEV = torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _device_status_clean():
    yield
    assert quest.device_status() == 0, "a kernel reported a bounded-wait timeout"


def random_packed(rows: int, k: int, seed: int, lo: int = -8, hi: int = 7) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(lo, hi + 1, (rows, k), generator=g, dtype=torch.int8)
    return O.pack_int4(codes)


# ------------------------------------------------------------------ scale / quantize ------------------
@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_scale_and_quantize_match_reference_golden(case):
    gd = load_golden(case)
    for tag, key in (("a", "activation"), ("w", "weight")):
        x = gd[key].to(DEV)
        scale = quest.find_scale_int4(x)
        assert scale.shape == (x.size(0), 1) and scale.dtype == torch.bfloat16
        assert scale.cpu().equal(gd[f"{tag}_scale"])
        x_int = torch.empty(x.shape, dtype=torch.int8, device=DEV)
        packed = torch.empty(x.size(0), x.size(1) // 2, dtype=torch.uint8, device=DEV)
        row_sum = torch.empty(x.size(0), 1, dtype=torch.int32, device=DEV)
        xd = x.clone()
        ret = quest.quantize_int4(xd, scale, x_int, packed, row_sum, do_dequantize=True)
        assert ret[0] is xd and ret[1] is x_int and ret[2] is packed and ret[3] is row_sum
        assert x_int.cpu().equal(gd[f"{tag}_int"])
        assert packed.cpu().equal(gd[f"{tag}_int_packed"])
        assert row_sum.cpu().equal(gd[f"{tag}_int_row_sum"])
        assert xd.cpu().equal(gd[f"{tag}_dq"])
        # None-output convention: absent outputs come back as None and x is untouched without dequantize
        x2 = x.clone()
        ret = quest.quantize_int4(x2, scale, x_int_packed=packed)
        assert ret[1] is None and ret[3] is None and x2.equal(x)
        assert packed.cpu().equal(gd[f"{tag}_int_packed"])
        assert quest.unpack_int4(packed).cpu().equal(gd[f"{tag}_int"])


@pytest.mark.parametrize("m", [1, 2, 17, 129])
@pytest.mark.parametrize("k", [256, 776, 4096, 5632, 11008, 14336, 28672])
def test_scale_and_quantize_shapes(m, k):
    """K = 776 is not a multiple of 32 (4-byte packed stores); K > 8192 uses several units per warp."""
    x = make_activations("outlier", m, k, seed=k + m)
    x[0, : k // 2] = 0  # a half-empty row
    if m > 1:
        x[1] = 0        # an all-zero row: scale = bf16(1e-8), codes 0
    xs = O.find_scale_int4(x)
    p_ref = torch.empty(m, k // 2, dtype=torch.uint8)
    r_ref = torch.empty(m, 1, dtype=torch.int32)
    O.quantize_int4(x, xs, None, p_ref, r_ref)
    xd = x.to(DEV)
    scale = quest.find_scale_int4(xd)
    mism = int((scale.cpu() != xs).sum())
    assert mism == 0, f"{mism} scale mismatches"
    _, _, packed, row_sum = quest.quantize_int4(xd, scale, None, torch.empty_like(p_ref, device=DEV),
                                                torch.empty_like(r_ref, device=DEV))
    assert packed.cpu().equal(p_ref)
    assert row_sum.cpu().equal(r_ref)


def test_quantize_generic_path_odd_shapes():
    """K % 8 != 0 and a misaligned base pointer take the scalar kernel; results must not change."""
    for k in (6, 100, 1022):
        x = make_activations("randn", 5, k, seed=k)
        xs = O.find_scale_int4(x)
        xi = torch.empty(5, k, dtype=torch.int8)
        p_ref = torch.empty(5, k // 2, dtype=torch.uint8)
        r_ref = torch.empty(5, 1, dtype=torch.int32)
        xq = x.clone()
        O.quantize_int4(xq, xs, xi, p_ref, r_ref, True)
        xd = x.to(DEV)
        scale = quest.find_scale_int4(xd)
        assert scale.cpu().equal(xs)
        out = quest.quantize_int4(xd, scale, torch.empty_like(xi, device=DEV), torch.empty_like(p_ref, device=DEV),
                                  torch.empty_like(r_ref, device=DEV), True)
        assert out[0].cpu().equal(xq) and out[1].cpu().equal(xi) and out[2].cpu().equal(p_ref) and out[3].cpu().equal(r_ref)
    # misaligned (but contiguous) view
    base = make_activations("randn", 1, 4 * 256 + 8, seed=9).view(-1).to(DEV)
    x = base[3:3 + 4 * 256].view(4, 256)
    assert x.is_contiguous() and x.data_ptr() % 16 != 0
    assert quest.find_scale_int4(x).cpu().equal(O.find_scale_int4(x.cpu()))


def test_exact_integer_quotients_floor_correctly():
    """x / scale is an exact integer for ~1 % of real data; build rows where it is for EVERY element."""
    scale = torch.tensor([[0.3125], [1.0], [3.0517578125e-05], [24.0]], dtype=torch.bfloat16)  # <= 3-bit mantissas
    n = torch.arange(-10, 10, dtype=torch.float32).repeat(13)[:256]
    x = (n.view(1, -1) * scale.float()).to(torch.bfloat16)
    assert ((x.float() / scale.float()) == n).all()
    p_ref = torch.empty(4, 128, dtype=torch.uint8)
    O.quantize_int4(x, scale, None, p_ref, None)
    got = quest.quantize_int4(x.to(DEV), scale.to(DEV), None, torch.empty_like(p_ref, device=DEV))[2]
    assert got.cpu().equal(p_ref)


# ------------------------------------------------------------------ fused Hadamard + quantize ---------
def check_hadamard_quantize(x: torch.Tensor, block: int) -> tuple[int, int, int]:
    p_ref, s_ref, r_ref, xh_ref = O.hadamard_quantize_int4(x, block)
    packed, scale, row_sum = quest.hadamard_quantize_int4(x.to(DEV), block)
    xh = quest.hadamard_transform(x.to(DEV), block)
    packed, scale, row_sum, xh = packed.cpu(), scale.cpu(), row_sum.cpu(), xh.cpu()
    # the transform itself: one bf16 ulp apart at rounding ties; where a block cancels to (nearly) zero the
    # fp32 summation error (<= 2^-20 of the block's absolute sum) can exceed an ulp of the tiny result
    ulp = O.bf16_ulp_distance(xh, xh_ref)
    abs_sum = x.float().abs().view(x.size(0), -1, block).sum(-1, keepdim=True).expand(-1, -1, block).reshape(x.shape)
    fp32_slack = abs_sum * O.hadamard_constant(block) * 2.0 ** -20
    assert bool(((ulp <= 1) | ((xh.float() - xh_ref.float()).abs() <= fp32_slack)).all())
    xh_mism = int((ulp != 0).sum())
    # rows whose bf16 scale agrees must have codes that differ only by +-1 tie flips
    same = (scale == s_ref).view(-1)
    scale_flips = int((~same).sum())
    assert int(O.bf16_ulp_distance(scale, s_ref).max()) <= 1
    nflip, maxd = O.count_code_flips(packed[same], p_ref[same])
    assert maxd <= 1
    # row sums are consistent with the codes actually written
    assert row_sum.equal(O.unpack_int4(packed).to(torch.int32).sum(-1, keepdim=True))
    return xh_mism, nflip, scale_flips


# "tc": the tcgen05 kernel where the shape fits its tiling (it must: the call fails otherwise); "mma": the CUDA-core
# kernel with mma.sync for the 16-point factor; "auto": what the library picks.
HQ_TC_SHAPES = [("student", 128, 4096), ("laplace", 64, 8192), ("randn", 33, 14336), ("outlier", 7, 2048),
                ("randn", 1, 256), ("student", 300, 512), ("laplace", 5, 16384), ("randn", 1000, 128),
                ("randn", 5, 28672), ("student", 3, 32768), ("laplace", 2, 65536)]  # tokens spanning 2 and 4 tiles


@pytest.mark.parametrize("block", [64, 128, 256])
@pytest.mark.parametrize("kind,m,k", HQ_TC_SHAPES)
def test_hadamard_quantize_tensor_core_kernel_matches_oracle(block, kind, m, k, monkeypatch):
    if k % block != 0:
        pytest.skip("K is not a multiple of the block")
    monkeypatch.setenv("QB200_HQ_KERNEL", "tc")
    x = make_activations(kind, m, k, seed=block + m)
    xh_mism, nflip, scale_flips = check_hadamard_quantize(x, block)
    n = m * k
    assert nflip <= 1 + int(5e-6 * n), (nflip, n)
    assert scale_flips <= max(1, m // 1000)


@pytest.mark.parametrize("block", [64, 128, 256])
def test_hadamard_quantize_kernels_agree_at_full_size(block, monkeypatch):
    """The two kernels on the headline activation shape: same scales, codes equal up to +-1 tie flips."""
    x = make_activations("student", 2048, 4096, seed=9).to(DEV)
    out = {}
    for kern in ("mma", "tc"):
        monkeypatch.setenv("QB200_HQ_KERNEL", kern)
        out[kern] = [t.cpu() for t in quest.hadamard_quantize_int4(x, block)]
    (p1, s1, r1), (p2, s2, r2) = out["mma"], out["tc"]
    assert int((s1 != s2).sum()) <= 2
    same = (s1 == s2).view(-1)
    nflip, maxd = O.count_code_flips(p1[same], p2[same])
    assert maxd <= 1 and nflip <= 1 + int(5e-6 * x.numel())
    assert r2.equal(O.unpack_int4(p2).to(torch.int32).sum(-1, keepdim=True))


@pytest.mark.parametrize("block", [64, 128, 256])
@pytest.mark.parametrize("kind,m,k", [("student", 128, 4096), ("laplace", 64, 8192), ("randn", 33, 14336),
                                      ("outlier", 7, 2048), ("randn", 3, 28672), ("randn", 1, 256)])
@pytest.mark.parametrize("kernel", ["auto", "mma"])
def test_hadamard_quantize_matches_oracle(block, kind, m, k, kernel, monkeypatch):
    if kernel != "auto":
        monkeypatch.setenv("QB200_HQ_KERNEL", kernel)
    x = make_activations(kind, m, k, seed=block + m)
    xh_mism, nflip, scale_flips = check_hadamard_quantize(x, block)
    n = m * k
    # documented tolerance: tie flips only.  Transform outputs differ from the exact-sum oracle where the
    # fp32 product sum * bf16(128^-0.5) is rounded twice (expected ~2^-15 of the elements for block 128,
    # none for the power-of-two constants of blocks 64/256); codes flip by +-1 at <~ 1e-6 per element.
    assert xh_mism <= 3 + int(1.5e-4 * n), (xh_mism, n)
    assert nflip <= 1 + int(5e-6 * n), (nflip, n)
    assert scale_flips <= max(1, m // 1000)


def test_hadamard_transform_weight_side_and_one_hot():
    w = (0.02 * torch.randn(96, 1024, generator=torch.Generator().manual_seed(2))).to(torch.bfloat16)
    ref = O.block_hadamard(w, 128, weight_side=True)
    got = quest.hadamard_transform(w.to(DEV), 128, weight_side=True).cpu()
    assert int(O.bf16_ulp_distance(got, ref).max()) <= 1 and (got != ref).float().mean() < 1e-4
    e = torch.zeros(2, 256, dtype=torch.bfloat16)
    e[0, 5] = 1
    e[1, 128 + 77] = -2
    got = quest.hadamard_transform(e.to(DEV), 128).cpu()
    assert got.equal(O.block_hadamard(e, 128))


# ------------------------------------------------------------------ int4 GEMM --------------------------
GEMM_SHAPES = [
    (160, 768, 224),      # the reference unit-test shape
    (1, 128, 8), (16, 4096, 264), (127, 160, 100), (129, 32, 257), (128, 256, 256), (300, 1024, 520),
    (256, 11008, 384),    # long K
    (64, 28672, 136),     # longest K of the 70B-shaped layers
    (1024, 512, 1024),    # many tiles per CTA: exercises the double-buffered accumulators
]


@pytest.mark.parametrize("m,k,n", GEMM_SHAPES)
def test_matmul_int4_exact(m, k, n):
    a = random_packed(m, k, seed=m + k)
    b = random_packed(n, k, seed=n + k + 1)
    c = quest.matmul_int4_int4t_int32(a.to(DEV), b.to(DEV))
    assert c.dtype == torch.int32 and c.shape == (m, n)
    assert c.cpu().equal(O.matmul_int4_int4t_int32(a, b))


def test_matmul_int4_extreme_values():
    """All codes -8: every accumulator equals 64 * K, the largest magnitude possible."""
    m, k, n = 130, 28672, 72
    a = torch.full((m, k // 2), 0x88, dtype=torch.uint8, device=DEV)
    b = torch.full((n, k // 2), 0x88, dtype=torch.uint8, device=DEV)
    c = quest.matmul_int4_int4t_int32(a, b)
    assert int(c.min()) == 64 * k and int(c.max()) == 64 * k
    b7 = torch.full((n, k // 2), 0x77, dtype=torch.uint8, device=DEV)
    c = quest.matmul_int4_int4t_int32(a, b7)
    assert int(c.min()) == -56 * k and int(c.max()) == -56 * k


def test_matmul_int4_nibble_order():
    """A one-hot code at column j of A and 1..K at B's columns picks out B[n, j]: checks nibble/K order."""
    k, n = 256, 16
    g = torch.Generator().manual_seed(5)
    b_codes = torch.randint(-8, 8, (n, k), generator=g, dtype=torch.int8)
    a_codes = torch.zeros(k, k, dtype=torch.int8)
    a_codes[torch.arange(k), torch.arange(k)] = 1
    c = quest.matmul_int4_int4t_int32(O.pack_int4(a_codes).to(DEV), O.pack_int4(b_codes).to(DEV))
    assert c.cpu().equal(b_codes.t().to(torch.int32))


def test_matmul_int4_output_reuse_and_out_argument():
    a, b = random_packed(64, 512, 1), random_packed(96, 512, 2)
    out = torch.full((64, 96), 12345, dtype=torch.int32, device=DEV)
    ret = quest.matmul_int4_int4t_int32(a.to(DEV), b.to(DEV), out=out)
    assert ret is out and out.cpu().equal(O.matmul_int4_int4t_int32(a, b))


def test_matmul_full_size_checksums():
    """Headline shape (M=2048, K=N=4096): row/column checksums against O(MK+NK) CPU arithmetic, and the
    full result against cuBLAS int8 on the unpacked codes."""
    m, k, n = 2048, 4096, 4096
    a, b = random_packed(m, k, 11), random_packed(n, k, 12)
    ad, bd = a.to(DEV), b.to(DEV)
    c = quest.matmul_int4_int4t_int32(ad, bd)
    ai, bi = O.unpack_int4(a).to(torch.int64), O.unpack_int4(b).to(torch.int64)
    assert c.sum(dim=1).cpu().to(torch.int64).equal(ai @ bi.sum(dim=0))
    assert c.sum(dim=0).cpu().to(torch.int64).equal(bi @ ai.sum(dim=0))
    ref = torch._int_mm(quest.unpack_int4(ad), quest.unpack_int4(bd).t().contiguous())
    assert c.equal(ref)


# ------------------------------------------------------------------ epilogue ---------------------------
def epilogue_inputs(m: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    a_add = torch.randint(-8 * 64, 8 * 64, (m, 1), generator=g, dtype=torch.int32)
    b_add = torch.randint(-8 * 64, 8 * 64, (n, 1), generator=g, dtype=torch.int32)
    a_mul = (torch.rand(m, 1, generator=g) + 0.05).to(torch.bfloat16)
    b_mul = (0.02 * torch.rand(n, 1, generator=g) + 0.001).to(torch.bfloat16)
    return a_add, a_mul, b_add, b_mul


@pytest.mark.parametrize("m,n", [(160, 224), (3, 8), (33, 100), (1, 7), (257, 4104)])
def test_add_mul_vv_bit_exact(m, n):
    a_add, a_mul, b_add, b_mul = epilogue_inputs(m, n, m + n)
    c = torch.randint(-2 ** 20, 2 ** 20, (m, n), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    ref = O.add_mul_vv(a_add, a_mul, b_add, b_mul, c)
    got = quest.add_mul_vv(a_add.to(DEV), a_mul.to(DEV), b_add.to(DEV), b_mul.to(DEV), c.to(DEV))
    assert got.cpu().equal(ref)


@pytest.mark.parametrize("m,k,n", [(160, 768, 224), (16, 4096, 264), (129, 8192, 257), (300, 1024, 520), (1, 256, 4)])
def test_fused_matmul_dequantize_bit_exact(m, k, n):
    a, b = random_packed(m, k, 21), random_packed(n, k, 22)
    a_add, a_mul, b_add, b_mul = epilogue_inputs(m, n, 23)
    ref = O.fused_matmul_dequantize_int4_int4t_bf16(a, b, a_add, b_add, a_mul, b_mul)
    got = quest.fused_matmul_dequantize_int4_int4t_bf16(a.to(DEV), b.to(DEV), a_add.to(DEV), b_add.to(DEV),
                                                        a_mul.to(DEV), b_mul.to(DEV))
    assert got.dtype == torch.bfloat16 and got.cpu().equal(ref)


@pytest.mark.parametrize("tile", [64, 128, 256, 512])
@pytest.mark.parametrize("m,k,n", [(300, 1024, 520), (129, 256, 257), (256, 512, 256), (1, 128, 8), (1100, 384, 1544)])
def test_every_tile_shape_is_bit_exact(tile, m, k, n, monkeypatch):
    """QB200_GEMM_TILE forces one tile shape (512 = the 256 x 256 kernel): each must give the same bits on full,
    ragged and many-tiles-per-CTA shapes, for the int32 and the fused entry points."""
    monkeypatch.setenv("QB200_GEMM_TILE", str(tile))
    a, b = random_packed(m, k, 41), random_packed(n, k, 42)
    ad, bd = a.to(DEV), b.to(DEV)
    assert quest.matmul_int4_int4t_int32(ad, bd).cpu().equal(O.matmul_int4_int4t_int32(a, b))
    a_add, a_mul, b_add, b_mul = epilogue_inputs(m, n, 43)
    ref = O.fused_matmul_dequantize_int4_int4t_bf16(a, b, a_add, b_add, a_mul, b_mul)
    got = quest.fused_matmul_dequantize_int4_int4t_bf16(ad, bd, a_add.to(DEV), b_add.to(DEV), a_mul.to(DEV), b_mul.to(DEV))
    assert got.cpu().equal(ref)


def test_wide_tile_kernel_full_size_against_cublas(monkeypatch):
    """The 256 x 256 kernel at a size with several tiles per CTA (M=4096, K=2048, N=10240 -> 640 tiles)."""
    monkeypatch.setenv("QB200_GEMM_TILE", "512")
    m, k, n = 4096, 2048, 10240
    ad, bd = random_packed(m, k, 51).to(DEV), random_packed(n, k, 52).to(DEV)
    c = quest.matmul_int4_int4t_int32(ad, bd)
    ref = torch._int_mm(quest.unpack_int4(ad), quest.unpack_int4(bd).t().contiguous())
    assert c.equal(ref)


@pytest.mark.parametrize("splits", [2, 3, 8])
@pytest.mark.parametrize("m,k,n", [(1, 4096, 512), (16, 1024, 264), (128, 2048, 1024), (130, 512, 300)])
def test_split_k_is_bit_exact_and_leaves_its_scratch_clean(splits, m, k, n, monkeypatch):
    """QB200_GEMM_SPLITS forces the split-K kernel; two calls in a row must both be exact (the second one sees the
    scratch the first one left behind), for the int32 and the fused entry points."""
    monkeypatch.setenv("QB200_GEMM_SPLITS", str(splits))
    a, b = random_packed(m, k, 61), random_packed(n, k, 62)
    ad, bd = a.to(DEV), b.to(DEV)
    a_add, a_mul, b_add, b_mul = epilogue_inputs(m, n, 63)
    ref_i = O.matmul_int4_int4t_int32(a, b)
    ref_f = O.fused_matmul_dequantize_int4_int4t_bf16(a, b, a_add, b_add, a_mul, b_mul)
    for _ in range(2):
        assert quest.matmul_int4_int4t_int32(ad, bd).cpu().equal(ref_i)
        got = quest.fused_matmul_dequantize_int4_int4t_bf16(ad, bd, a_add.to(DEV), b_add.to(DEV), a_mul.to(DEV), b_mul.to(DEV))
        assert got.cpu().equal(ref_f)


def test_small_m_gemm_picks_split_k_and_matches_cublas():
    """Decode-like shape (M=16, K=N=4096): whatever the library picks must equal cuBLAS int8 on the unpacked codes."""
    m, k, n = 16, 4096, 4096
    ad, bd = random_packed(m, k, 71).to(DEV), random_packed(n, k, 72).to(DEV)
    ref = torch._int_mm(torch.cat([quest.unpack_int4(ad), torch.zeros(16, k, dtype=torch.int8, device=DEV)]),
                        quest.unpack_int4(bd).t().contiguous())[:m]
    for _ in range(3):
        assert quest.matmul_int4_int4t_int32(ad, bd).equal(ref)


@pytest.mark.parametrize("m", [1, 2, 3, 5, 8, 9, 16])
@pytest.mark.parametrize("k,n", [(4096, 520), (256, 7), (14336, 260), (1024, 4104)])
def test_small_m_cuda_core_kernel_is_bit_exact(m, k, n):
    """M <= 16 with a small enough product takes the dp4a kernel: int32 and fused outputs against the oracle, twice."""
    a, b = random_packed(m, k, 81), random_packed(n, k, 82)
    ad, bd = a.to(DEV), b.to(DEV)
    a_add, a_mul, b_add, b_mul = epilogue_inputs(m, n, 83)
    ref_i = O.matmul_int4_int4t_int32(a, b)
    ref_f = O.fused_matmul_dequantize_int4_int4t_bf16(a, b, a_add, b_add, a_mul, b_mul)
    for _ in range(2):
        assert quest.matmul_int4_int4t_int32(ad, bd).cpu().equal(ref_i)
        got = quest.fused_matmul_dequantize_int4_int4t_bf16(ad, bd, a_add.to(DEV), b_add.to(DEV), a_mul.to(DEV), b_mul.to(DEV))
        assert got.cpu().equal(ref_f)


def test_small_m_kernels_agree_on_extreme_codes(monkeypatch):
    """All codes -8 at the longest K: the dp4a kernel, the split-K kernel and the plain tensor-core kernel."""
    m, k, n = 4, 28672, 136
    a = torch.full((m, k // 2), 0x88, dtype=torch.uint8, device=DEV)
    b = torch.full((n, k // 2), 0x88, dtype=torch.uint8, device=DEV)
    c0 = quest.matmul_int4_int4t_int32(a, b)
    assert int(c0.min()) == 64 * k and int(c0.max()) == 64 * k
    monkeypatch.setenv("QB200_GEMM_GEMV", "0")
    assert quest.matmul_int4_int4t_int32(a, b).equal(c0)
    monkeypatch.setenv("QB200_GEMM_SPLITS", "1")
    assert quest.matmul_int4_int4t_int32(a, b).equal(c0)


def test_fused_into_column_slice():
    m, k, n, n_total = 96, 512, 128, 512
    a, b = random_packed(m, k, 31), random_packed(n, k, 32)
    a_add, a_mul, b_add, b_mul = epilogue_inputs(m, n, 33)
    full = torch.zeros(m, n_total, dtype=torch.bfloat16, device=DEV)
    quest.fused_matmul_dequantize_int4_int4t_bf16_into(a.to(DEV), b.to(DEV), a_add.to(DEV), b_add.to(DEV),
                                                       a_mul.to(DEV), b_mul.to(DEV), full[:, 256:384])
    ref = O.fused_matmul_dequantize_int4_int4t_bf16(a, b, a_add, b_add, a_mul, b_mul)
    assert full[:, 256:384].cpu().equal(ref)
    assert int(full[:, :256].abs().sum()) == 0 and int(full[:, 384:].abs().sum()) == 0


# ------------------------------------------------------------------ layer / module ---------------------
@pytest.mark.parametrize("case", GOLDEN_CASES)
def test_linear_forward_matches_reference_golden(case):
    gd = load_golden(case)
    w = gd["weight"].to(DEV)
    wp, ws, wa, meta = quest.preprocess_weight(w.clone(), use_hadamard=False)
    assert meta is None
    assert wp.cpu().equal(gd["w_int_packed"]) and ws.cpu().equal(gd["w_scale"]) and wa.cpu().equal(gd["w_add"])
    y = quest.linear_forward(gd["activation"].to(DEV), wp, ws, wa, use_hadamard=False)
    assert y.cpu().equal(gd["m"])
    # debug route (int32 GEMM + add_mul_vv) gives the same bits
    c = torch.empty(y.shape, dtype=torch.int32, device=DEV)
    y2 = quest.linear_forward(gd["activation"].to(DEV), wp, ws, wa, use_hadamard=False, _c=c, debug_mode=True)
    assert y2.equal(y) and c.cpu().equal(gd["c_ref"])
    # as in the reference, a caller-provided _c alone does not leave the fused route (and is not written)
    c.fill_(-7)
    y3 = quest.linear_forward(gd["activation"].to(DEV), wp, ws, wa, use_hadamard=False, _c=c)
    assert y3.equal(y) and int((c != -7).sum()) == 0


def test_linear_forward_with_hadamard_config1():
    """CPU-runnable config: x [512,2048] N(0,1) + 0.5 % x20 outliers, W [2048,2048] N(0,0.02), block 128."""
    x = make_activations("outlier", 512, 2048, seed=0)
    w = (0.02 * torch.randn(2048, 2048, generator=torch.Generator().manual_seed(0))).to(torch.bfloat16)
    wp_ref, ws_ref, wa_ref, _ = O.preprocess_weight(w, use_hadamard=True)
    wp, ws, wa, _ = quest.preprocess_weight(w.to(DEV), use_hadamard=True)
    assert ws.cpu().equal(ws_ref)
    nflip, maxd = O.count_code_flips(wp.cpu(), wp_ref)
    assert maxd <= 1 and nflip <= 8
    # with identical weights the layer output may differ only through activation tie flips
    y = quest.linear_forward(x.to(DEV), wp_ref.to(DEV), ws_ref.to(DEV), wa_ref.to(DEV), use_hadamard=True).cpu()
    y_ref = O.linear_forward(x, wp_ref, ws_ref, wa_ref, use_hadamard=True)
    pa, sa, ra = quest.hadamard_quantize_int4(x.to(DEV))
    pa_ref, sa_ref, ra_ref, _ = O.hadamard_quantize_int4(x)
    if pa.cpu().equal(pa_ref) and sa.cpu().equal(sa_ref):
        assert y.equal(y_ref)
    else:
        assert (y != y_ref).float().mean() < 0.02
    rel = ((y.float() - y_ref.float()).norm() / y_ref.float().norm()).item()
    assert rel < 1e-3
    dense = x.float() @ w.float().t()
    assert ((y.float() - dense).norm() / dense.norm()).item() < 0.25


def test_linear4bit_module_and_workspaces():
    torch.manual_seed(0)
    lin = quest.Linear4bit(512, 384, bias=True, device=DEV, dtype=torch.bfloat16, use_hadamard=True)
    assert lin.weight.is_meta and lin.w_int_packed.shape == (384, 256) and lin.w_meta_e is None
    x = make_activations("student", 6 * 20, 512, seed=4).view(6, 20, 512).to(DEV)
    y = lin(x)
    assert y.shape == (6, 20, 384) and y.dtype == torch.bfloat16
    flat = x.flatten(end_dim=-2)
    ws = dict(_a_scale=torch.empty(120, 1, dtype=torch.bfloat16, device=DEV),
              _a_int_packed=torch.empty(120, 256, dtype=torch.uint8, device=DEV),
              _a_int_row_sum=torch.empty(120, 1, dtype=torch.int32, device=DEV))
    out = torch.empty(120, 384, dtype=torch.bfloat16, device=DEV)
    y2 = quest.linear_forward(flat, lin.w_int_packed, lin.w_scale, lin.w_add, out=out, use_hadamard=True, **ws)
    assert y2 is out
    assert (y2 + lin.bias).unflatten(0, (6, 20)).equal(y)
    noop = quest.Linear4bit(512, 384, bias=False, device=DEV, dtype=torch.bfloat16, use_hadamard=True, use_noop=True)
    assert int(noop(x).abs().sum()) == 0


def test_cuda_graph_capture_and_replay():
    """Mirrors the reference's graph test (gemm-quest/benchmarks/utils.py:765-784), for the whole layer."""
    m, k, n = 160, 768, 224
    a, b = random_packed(m, k, 41), random_packed(n, k, 42)
    x = make_activations("randn", m, k, seed=43)
    w = make_activations("randn", n, k, seed=44)
    wp, ws, wa, _ = quest.preprocess_weight(w.to(DEV), use_hadamard=True)
    gt = {
        "a": torch.zeros(m, k // 2, dtype=torch.uint8, device=DEV), "b": torch.zeros(n, k // 2, dtype=torch.uint8, device=DEV),
        "c": torch.zeros(m, n, dtype=torch.int32, device=DEV), "x": torch.zeros(m, k, dtype=torch.bfloat16, device=DEV),
        "y": torch.zeros(m, n, dtype=torch.bfloat16, device=DEV),
        "s": torch.empty(m, 1, dtype=torch.bfloat16, device=DEV), "p": torch.empty(m, k // 2, dtype=torch.uint8, device=DEV),
        "r": torch.empty(m, 1, dtype=torch.int32, device=DEV),
    }

    def step():
        quest.matmul_int4_int4t_int32(gt["a"], gt["b"], out=gt["c"])
        quest.linear_forward(gt["x"], wp, ws, wa, out=gt["y"], _a_scale=gt["s"], _a_int_packed=gt["p"],
                             _a_int_row_sum=gt["r"], use_hadamard=True)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    gt["a"].copy_(a)
    gt["b"].copy_(b)
    gt["x"].copy_(x)
    graph.replay()
    torch.cuda.synchronize()
    assert gt["c"].cpu().equal(O.matmul_int4_int4t_int32(a, b))
    assert gt["y"].equal(quest.linear_forward(x.to(DEV), wp, ws, wa, use_hadamard=True))


# ------------------------------------------------------------------ prefill of a small decoder ---------
def test_prefill_decoder_module_swap_and_graph():
    """Small Llama-style decoder: the swapped model tracks the bf16 one within W4A4 noise, a CUDA-graph replay
    reproduces the eager result bit for bit, and each swapped linear equals the oracle layer on its own input."""
    from quest_b200.prefill import Decoder, DecoderConfig, swap_linears, prefill_time
    torch.manual_seed(0)
    cfg = DecoderConfig(n_embd=256, n_layer=2, n_head=4, ffn=768, vocab_size=512, sequence_length=64)
    ref_model = Decoder(cfg).to(device=DEV, dtype=torch.bfloat16).eval()
    q_model = Decoder(cfg).to(device=DEV, dtype=torch.bfloat16).eval()
    q_model.load_state_dict(ref_model.state_dict())
    first_w = q_model.transformer.h[0].attn.c_attn.weight.data.clone()
    swap_linears(q_model, "int4", use_hadamard=True)
    assert all(isinstance(m, quest.Linear4bit) for m in [q_model.transformer.h[0].attn.c_attn, q_model.transformer.h[1].mlp.c_proj])
    idx = torch.randint(0, cfg.vocab_size, (4, 64), generator=torch.Generator().manual_seed(1)).to(DEV)
    with torch.inference_mode():
        y_ref, y_q = ref_model(idx), q_model(idx)
        # one swapped linear against the oracle layer, same input
        x_in = ref_model.transformer.h[0].ln_1(ref_model.transformer.wte(idx)).flatten(end_dim=-2)
        got = q_model.transformer.h[0].attn.c_attn(x_in)
    wp, ws, wa, _ = O.preprocess_weight(first_w.cpu(), use_hadamard=True)
    want = O.linear_forward(x_in.cpu(), wp, ws, wa, use_hadamard=True)
    assert (got.cpu() != want).float().mean() < 0.02 and ((got.cpu().float() - want.float()).norm() / want.float().norm()) < 2e-3
    rel = ((y_q.float() - y_ref.float()).norm() / y_ref.float().norm()).item()
    assert rel < 0.5, rel
    eager_ms, graph_ms, y_graph = prefill_time(q_model, 4, 64, n_warmup=2, n_iter=3, seed=1)
    assert eager_ms > 0 and graph_ms > 0
    assert y_graph.equal(y_q)
    noop = swap_linears(Decoder(cfg).to(device=DEV, dtype=torch.bfloat16).eval(), "noop")
    with torch.inference_mode():
        assert noop(idx).shape == y_ref.shape


def test_push_entry_point_copies_tiles_to_every_destination():
    """The multi-GPU entry point on ONE GPU: two further local buffers stand in for the peers' outputs.  Every
    destination must receive exactly the column block, and nothing outside it."""
    m, k, n, n_total = 300, 1024, 264, 1056
    a, b = random_packed(m, k, 61).to(DEV), random_packed(n, k, 62).to(DEV)
    a_add, a_mul, b_add, b_mul = [t.to(DEV) for t in epilogue_inputs(m, n, 63)]
    bufs = [torch.zeros(m, n_total, dtype=torch.bfloat16, device=DEV) for _ in range(3)]
    col0 = 528
    ptrs = [t.data_ptr() + col0 * 2 for t in bufs]
    quest.fused_matmul_dequantize_int4_int4t_bf16_push(a, b, a_add, b_add, a_mul, b_mul, ptrs, n_total)
    want = O.fused_matmul_dequantize_int4_int4t_bf16(a.cpu(), b.cpu(), a_add.cpu(), b_add.cpu(), a_mul.cpu(), b_mul.cpu())
    for t in bufs:
        assert t[:, col0:col0 + n].cpu().equal(want)
        assert int(t[:, :col0].abs().sum()) == 0 and int(t[:, col0 + n:].abs().sum()) == 0


# ------------------------------------------------------------------ checkpoint conversion -------------
def test_checkpoint_conversion_matches_oracle_and_module_swap():
    """A synthetic QuEST-style checkpoint (DDP-prefixed keys, block names of the reference's Llama model): every
    quantised linear is packed exactly as the oracle's preprocess_weight does, the rest passes through, and a
    model loaded from the converted entries computes what a model swapped in place computes."""
    from quest_b200 import convert
    g = torch.Generator().manual_seed(3)
    d, ff = 256, 512

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.attn = torch.nn.Module()
            self.attn.c_attn = torch.nn.Linear(d, 3 * d, bias=False)
            self.attn.c_proj = torch.nn.Linear(d, d, bias=False)
            self.mlp = torch.nn.Module()
            self.mlp.w1 = torch.nn.Linear(d, ff, bias=False)
            self.mlp.w2 = torch.nn.Linear(d, ff, bias=False)
            self.mlp.c_proj = torch.nn.Linear(ff, d, bias=True)

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.transformer = torch.nn.ModuleDict({"wte": torch.nn.Embedding(64, d), "h": torch.nn.ModuleList([Block(), Block()])})
            self.lm_head = torch.nn.Linear(d, 64, bias=False)

    src = Tiny()
    for p_ in src.parameters():
        p_.data.copy_(0.05 * torch.randn(p_.shape, generator=g))
    ckpt = {"model": {"module." + k: v for k, v in src.state_dict().items()}, "itr": 7}
    sd = convert.unwrap_checkpoint(ckpt)
    names = convert.quantised_layer_names(sd)
    assert len(names) == 10 and "transformer.h.1.mlp.c_proj" in names and "lm_head" not in names
    conv = convert.convert_state_dict(ckpt, device=DEV)
    assert "transformer.h.0.attn.c_attn.weight" not in conv and conv["lm_head.weight"].dtype == torch.bfloat16
    for name in names:
        w = sd[name + ".weight"].to(torch.bfloat16)
        p_ref, s_ref, a_ref, _ = O.preprocess_weight(w, use_hadamard=True)
        assert conv[name + ".w_scale"].cpu().equal(s_ref)
        nflip, maxd = O.count_code_flips(conv[name + ".w_int_packed"].cpu(), p_ref)
        assert maxd <= 1 and nflip <= 1 + int(5e-6 * w.numel())
    # a model swapped in place vs a model filled from the converted entries
    a = Tiny().to(DEV).to(torch.bfloat16)
    a.load_state_dict({k: v.to(torch.bfloat16) for k, v in sd.items()})
    convert.swap_quantised_linears(a, names)
    b = Tiny().to(DEV).to(torch.bfloat16)
    convert.swap_quantised_linears(b, names)   # same structure, its own (random) weights
    convert.load_converted(b, conv)
    x = torch.randn(5, d, generator=g).to(torch.bfloat16).to(DEV)
    for blk_a, blk_b in zip(a.transformer["h"], b.transformer["h"]):
        assert blk_a.mlp.c_proj(blk_a.mlp.w1(x)).equal(blk_b.mlp.c_proj(blk_b.mlp.w1(x)))
        assert blk_a.attn.c_attn(x).equal(blk_b.attn.c_attn(x))


# ------------------------------------------------------------------ int8-operand route ----------------
@pytest.mark.parametrize("block", [64, 128, 256])
@pytest.mark.parametrize("m,k,n", [(300, 512, 264), (129, 4096, 520), (2048, 4096, 4096), (70, 28672, 256), (1, 128, 8)])
def test_int8_operand_route_matches_the_packed_route(block, m, k, n, monkeypatch):
    """hadamard_quantize_a8 writes 16 x the same codes in the GEMM's operand order (even positions of every 32-group
    first); the GEMM on that operand gives the bits of the packed route and of the oracle epilogue.  Both quantiser
    calls use the tcgen05 kernel (the only one that writes the int8 operand), so their codes must be identical."""
    if k % block != 0:
        pytest.skip("K is not a multiple of the block")
    monkeypatch.setenv("QB200_HQ_KERNEL", "tc")
    x = make_activations("student", m, k, seed=m + k).to(DEV)
    w = (0.02 * torch.randn(n, k, generator=torch.Generator().manual_seed(n))).to(torch.bfloat16).to(DEV)
    wp, ws, wa, _ = quest.preprocess_weight(w, use_hadamard=True, block=block)
    packed, scale, rsum = quest.hadamard_quantize_int4(x, block)
    a8, scale8, rsum8 = quest.hadamard_quantize_a8(x, block)
    assert scale8.equal(scale) and rsum8.equal(rsum)
    codes = quest.unpack_int4(packed).view(m, k // 32, 16, 2)                     # [.., position pair, even/odd]
    expect = torch.cat([codes[..., 0], codes[..., 1]], dim=-1).reshape(m, k)       # evens of a 32-group, then odds
    assert a8.view(torch.int8).equal((expect * 16).to(torch.int8))
    ref = quest.fused_matmul_dequantize_int4_int4t_bf16(packed, wp, rsum, wa, scale, ws)
    got = quest.fused_matmul_dequantize_a8(a8, wp, rsum8, wa, scale8, ws)
    assert got.equal(ref)
    cpu = O.fused_matmul_dequantize_int4_int4t_bf16(packed.cpu(), wp.cpu(), rsum.cpu(), wa.cpu(), scale.cpu(), ws.cpu())
    assert got.cpu().equal(cpu)


def test_linear_forward_takes_the_int8_operand_route_where_preferred(monkeypatch):
    m, k, n = 2048, 4096, 4096
    x = make_activations("student", m, k, seed=1).to(DEV)
    w = (0.02 * torch.randn(n, k, generator=torch.Generator().manual_seed(2))).to(torch.bfloat16).to(DEV)
    wp, ws, wa, _ = quest.preprocess_weight(w, use_hadamard=True)
    monkeypatch.setenv("QB200_HQ_KERNEL", "tc")  # same quantiser arithmetic on both routes
    monkeypatch.setenv("QB200_A8", "0")
    assert not quest.prefers_a8(m, k, n)
    y_packed = quest.linear_forward(x, wp, ws, wa, use_hadamard=True)
    monkeypatch.setenv("QB200_A8", "1")
    assert quest.prefers_a8(m, k, n)
    y_a8 = quest.linear_forward(x, wp, ws, wa, use_hadamard=True)
    assert y_a8.equal(y_packed)
    monkeypatch.delenv("QB200_A8")
    assert not quest.prefers_a8(16, k, n) and not quest.prefers_a8(m, 5632, n)
    # the library's own choice at this shape is the int8-operand route; a caller's packed workspace keeps the packed one
    assert quest.prefers_a8(m, k, n)
    assert quest.linear_forward(x, wp, ws, wa, use_hadamard=True).equal(y_packed)
    pk = torch.empty(m, k // 2, dtype=torch.uint8, device=DEV)
    assert quest.linear_forward(x, wp, ws, wa, use_hadamard=True, _a_int_packed=pk).equal(y_packed)
    assert pk.equal(quest.hadamard_quantize_int4(x)[0])
    # and the module (workspaces from the shared cache) gives the same bits, call after call
    lin = quest.Linear4bit(k, n, bias=False, device=DEV, dtype=torch.bfloat16, use_hadamard=True, weight=w)
    assert lin(x).equal(y_packed) and lin(x).equal(y_packed)
