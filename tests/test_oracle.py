"""CPU tests: the oracle against the golden vectors produced by the reference's own baselines, and
the identities of the reference's unit test (gemm-quest/benchmarks/utils.py:626-688) restated."""
from __future__ import annotations

import pytest
import torch

from oracle import quest_oracle as O
from conftest import make_activations


def test_scale_matches_reference_baseline(golden):
    for tag, key in (("a", "activation"), ("w", "weight")):
        assert O.find_scale_int4(golden[key]).equal(golden[f"{tag}_scale"])


def test_quantize_matches_reference_baseline(golden):
    for tag, key in (("a", "activation"), ("w", "weight")):
        x = golden[key].clone()
        rows, k = x.shape
        x_int = torch.empty(rows, k, dtype=torch.int8)
        packed = torch.empty(rows, k // 2, dtype=torch.uint8)
        row_sum = torch.empty(rows, 1, dtype=torch.int32)
        ret = O.quantize_int4(x, golden[f"{tag}_scale"], x_int, packed, row_sum, True)
        assert ret[0] is x and ret[1] is x_int and ret[2] is packed and ret[3] is row_sum
        assert x.equal(golden[f"{tag}_dq"])
        assert x_int.equal(golden[f"{tag}_int"])
        assert packed.equal(golden[f"{tag}_int_packed"])
        assert row_sum.equal(golden[f"{tag}_int_row_sum"])


def test_none_outputs_are_returned_as_none(golden):
    x = golden["activation"].clone()
    ret = O.quantize_int4(x, golden["a_scale"])
    assert ret[0] is x and ret[1] is None and ret[2] is None and ret[3] is None
    assert x.equal(golden["activation"])  # no dequantize -> untouched


def test_pack_unpack_round_trip(golden):
    assert O.unpack_int4(golden["a_int_packed"]).equal(golden["a_int"])
    assert O.pack_int4(golden["w_int"]).equal(golden["w_int_packed"])
    allbytes = torch.arange(256, dtype=torch.uint8).view(1, 256)
    assert O.pack_int4(O.unpack_int4(allbytes)).equal(allbytes)
    u = O.unpack_int4(torch.tensor([[0x8F, 0x70]], dtype=torch.uint8))
    assert u.tolist() == [[-1, -8, 0, 7]]  # low nibble = even column, two's complement


def test_int_matmul_and_epilogue_match_reference(golden):
    c = O.matmul_int4_int4t_int32(golden["a_int_packed"], golden["w_int_packed"])
    assert c.equal(golden["c_ref"])
    m = O.add_mul_vv(golden["a_int_row_sum"], golden["a_scale"], golden["w_add"], golden["w_scale"], c)
    assert m.equal(golden["m"])
    assert golden["m_equals_fp64_ref"] is True
    m2 = O.fused_matmul_dequantize_int4_int4t_bf16(golden["a_int_packed"], golden["w_int_packed"],
                                                   golden["a_int_row_sum"], golden["w_add"],
                                                   golden["a_scale"], golden["w_scale"])
    assert m2.equal(golden["m"])


def test_fp64_identity(golden):
    """a_s (2 A W^T + sum a + sum w^T + K/2) (w_s/2) == dq(a) dq(w)^T, exactly, in fp64."""
    a_int, w_int = golden["a_int"], golden["w_int"]
    k = a_int.size(1)
    m_ref = O.ideal_quantized_linear_fp64(a_int, golden["a_scale"], w_int, golden["w_scale"])
    a64, w64 = a_int.double(), w_int.double()
    m = golden["a_scale"].double() * (2. * a64 @ w64.t() + a64.sum(-1, keepdim=True)
                                      + w64.sum(-1, keepdim=True).t() + .5 * k) * (.5 * golden["w_scale"].double()).t()
    assert m.equal(m_ref)
    assert golden["m"].equal(m_ref.to(torch.bfloat16))


def test_preprocess_and_linear_forward_compose(golden):
    w_packed, w_scale, w_add, meta = O.preprocess_weight(golden["weight"].clone(), use_hadamard=False)
    assert meta is None
    assert w_packed.equal(golden["w_int_packed"]) and w_scale.equal(golden["w_scale"]) and w_add.equal(golden["w_add"])
    y = O.linear_forward(golden["activation"].clone(), w_packed, w_scale, w_add, use_hadamard=False)
    assert y.equal(golden["m"])


def test_constants():
    assert O.hadamard_constant(128) == 0.08837890625
    assert O.hadamard_constant(64) == 0.125 and O.hadamard_constant(256) == 0.0625
    f = torch.tensor(2.513930578568423, dtype=torch.float32) * 2. / 15.
    assert f.view(torch.int32).item() == 0x3EAB9E1F
    h = O.sylvester_sign_matrix(128)
    assert (h @ h.t()).equal(128 * torch.eye(128, dtype=torch.float64))
    i, j = 37, 101
    assert h[i, j].item() == (-1) ** bin(i & j).count("1")


def test_round_f64_to_bf16_is_single_rounding():
    # 1 + 2^-8 + 2^-40 is above the bf16 tie, but fp64->fp32 rounds it onto the tie (-> even = 1.0)
    v = torch.tensor([1.0 + 2.0 ** -8 + 2.0 ** -40, 1.0 + 2.0 ** -8, 3.0, -0.0, 1e-30], dtype=torch.float64)
    r = O.round_f64_to_bf16(v)
    assert r[0].item() == 1.0078125 and r[1].item() == 1.0 and r[2].item() == 3.0
    assert v.float().to(torch.bfloat16)[0].item() == 1.0  # the double-rounding trap it avoids
    x = torch.randn(4096, dtype=torch.float64)
    assert O.round_f64_to_bf16(x.float().double()).equal(x.float().to(torch.bfloat16))


@pytest.mark.parametrize("block", [64, 128, 256])
def test_block_hadamard_properties(block):
    x = make_activations("randn", 8, 4 * block, seed=3)
    y = O.block_hadamard(x, block)
    # involution up to bf16 rounding and the (slightly off-unit) bf16 constant
    z = O.block_hadamard(y, block)
    c = (O.hadamard_constant(block) ** 2) * block
    assert torch.allclose(z.float(), x.float() * c, atol=0.05, rtol=0.02)
    # energy is preserved (RMS changes by the constant's relative error only)
    assert torch.allclose(y.float().square().sum(-1), x.float().square().sum(-1) * c, rtol=0.01)
    # the reference's own op (library bf16 GEMM on CPU) differs from the canonical one at most by rounding ties
    yr = O.block_hadamard_reference_op(x, block)
    assert O.bf16_ulp_distance(y, yr).max().item() <= 1
    assert (y != yr).float().mean().item() < 1e-2
    # a one-hot row yields the Sylvester signs times the constant
    e = torch.zeros(1, block, dtype=torch.bfloat16)
    e[0, 5] = 1
    signs = O.sylvester_sign_matrix(block)[:, 5]
    assert O.block_hadamard(e, block).double().equal((signs * O.hadamard_constant(block)).view(1, -1))


def test_hadamard_quantize_tie_flip_rate_vs_reference_op():
    """Canonical oracle vs the reference's op run on the CPU: flips are rare and only +-1."""
    x = make_activations("student", 256, 4096, seed=0)
    p0, s0, r0, _ = O.hadamard_quantize_int4(x, 128, reference_op=False)
    p1, s1, r1, _ = O.hadamard_quantize_int4(x, 128, reference_op=True)
    nflip, maxd = O.count_code_flips(p0, p1)
    same_scale_rows = (s0 == s1).view(-1)
    nflip_same, _ = O.count_code_flips(p0[same_scale_rows], p1[same_scale_rows])
    assert maxd <= 1
    assert nflip_same / max(1, int(same_scale_rows.sum()) * 4096) < 1e-5


def test_cpu_config_layer_is_accurate():
    """Config-1 sized layer: x fp32 [512,2048] ~N(0,1) with 0.5 % x20 outliers, W ~N(0,0.02), block 128."""
    g = torch.Generator().manual_seed(0)
    x = make_activations("outlier", 512, 2048, seed=0)
    w = (0.02 * torch.randn(2048, 2048, generator=g)).to(torch.bfloat16)
    wp, ws, wa, _ = O.preprocess_weight(w, use_hadamard=True)
    y = O.linear_forward(x, wp, ws, wa, use_hadamard=True)
    ref = x.float() @ w.float().t()
    rel = ((y.float() - ref).norm() / ref.norm()).item()
    assert rel < 0.25, rel
