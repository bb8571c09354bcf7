"""CPU oracle for the QuEST W4A4 inference linear layer.

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA path is
compared against; only the test-suite, the smoke check and the benchmark's
CPU-baseline leg may import it.  The product (``quest_b200``) never does.

Every function restates, in plain torch on the CPU, one function of the
reference project (paths are relative to the reference repository root):

* ``find_scale_int4``        <- gemm-quest/benchmarks/utils.py:193-209
                                (CUDA twin: gemm-quest/quest/quantize_kernel.cu:38-94)
* ``quantize_int4``          <- gemm-quest/benchmarks/utils.py:334-365
                                (CUDA twin: gemm-quest/quest/quantize_kernel.cu:120-229)
* ``unpack_int4``            <- gemm-quest/benchmarks/utils.py:420-445
* ``add_mul_vv``             <- gemm-quest/benchmarks/utils.py:535-545
                                (CUDA twin: gemm-quest/quest/quantize_kernel.cu:264-306)
* ``matmul_int4_int4t_int32``<- gemm-quest/benchmarks/utils.py:680 (exact matmul of the codes)
* ``fused_matmul_dequantize``<- gemm-quest/benchmarks/utils.py:548-587 (debug_mode=True composition)
* ``block_hadamard*``        <- gemm-quest/benchmarks/utils.py:17, 89-90 (activations) and :38-39 (weights)
* ``preprocess_weight``      <- gemm-quest/benchmarks/utils.py:20-53 (dense branch)
* ``linear_forward``         <- gemm-quest/benchmarks/utils.py:56-111 (dense branch)

Parity status.  The scale / quantize / unpack / epilogue restatements are
pinned: tests/golden/ holds vectors produced by executing the reference's own
``*_baseline`` functions (see tests/golden/make_golden.py) and the oracle must
reproduce them bit for bit.  The Hadamard step is "parity unpinned": the
reference computes it with a cuBLAS bf16 GEMM (activations) or the third-party
``fast_hadamard_transform`` package (weights, unpinned dependency, absent),
whose fp32 summation order is not specified and which no reference test
exercises.  The canonical oracle here is "exact (fp64) sum, one rounding to
bf16"; any fp32 summation order differs from it only at rounding ties.
"""
from __future__ import annotations

import math

import numpy as np
import torch
import torch.nn.functional as F

# gemm-quest/quest/quantize_kernel.cu:85, gemm-quest/benchmarks/utils.py:208,
# src/models/quantization/base_linear.py:43 (OPTIMAL_GAUSSIAN_SCALES[4]).
GAUSSIAN_CLIP_4BIT = 2.513930578568423
SCALE_FACTOR = GAUSSIAN_CLIP_4BIT * 2.0 / ((1 << 4) - 1)
SCALE_EPS = 1e-8
QMIN, QMAX = 16 // -2, 16 // 2 - 1


# ----------------------------------------------------------------------------
# scale / quantize / pack
# ----------------------------------------------------------------------------
def find_scale_int4(x: torch.Tensor, scale: torch.Tensor | None = None) -> torch.Tensor:
    """Per-row Gaussian-MSE-optimal 4-bit step: sqrt(mean(x^2)) * (2.5139*2/15) + 1e-8.

    Follows gemm-quest/benchmarks/utils.py:193-209.  The result is stored in
    ``scale``'s dtype (bf16 on the drop-in path), which is the second of the two
    rounding points that decide the codes.
    """
    if scale is None:
        scale = torch.empty(*x.shape[:-1], 1, dtype=x.dtype)
    xf = x.to(dtype=torch.float32)
    scale_ = (xf * xf).mean(dim=-1, keepdim=True).sqrt() * SCALE_FACTOR + SCALE_EPS
    return scale.copy_(scale_)


def quantize_int4(
        x: torch.Tensor,
        scale: torch.Tensor,
        x_int: torch.Tensor | None = None,
        x_int_packed: torch.Tensor | None = None,
        x_int_row_sum: torch.Tensor | None = None,
        do_dequantize: bool = False,
):
    """q = clamp(floor(x / scale), -8, 7); optional dense / packed / row-sum outputs.

    Follows gemm-quest/benchmarks/utils.py:334-365.  Byte j of a packed row is
    ``(q[2j+1] << 4) | (q[2j] & 0xF)``.  With ``do_dequantize`` x is overwritten
    by (q + 0.5) * scale.  Returns the caller's own objects (None where absent).
    """
    x_q = (x.to(dtype=torch.float32) / scale.to(dtype=torch.float32)).floor().clamp(QMIN, QMAX)
    if do_dequantize:
        x_dq = x_q * scale + (scale * .5)
        x.copy_(x_dq)
    if x_int is not None or x_int_packed is not None or x_int_row_sum is not None:
        x_int_ = x_q.to(dtype=torch.int8)
        if x_int is not None:
            x_int.copy_(x_int_)
        if x_int_packed is not None:
            x_int_packed.copy_(pack_int4(x_int_))
        if x_int_row_sum is not None:
            x_int_row_sum.copy_(x_int_.to(dtype=torch.int32).sum(dim=-1, keepdim=True))
    return x, x_int, x_int_packed, x_int_row_sum


def pack_int4(x_int: torch.Tensor) -> torch.Tensor:
    """int8 codes (..., K) -> uint8 (..., K/2); even column in the low nibble
    (gemm-quest/benchmarks/utils.py:359)."""
    packed = (x_int[..., 1::2] << 4) | (x_int[..., ::2] & 0xF)
    return packed.view(torch.uint8) if packed.dtype == torch.int8 else packed.to(torch.uint8)


def unpack_int4(x_int_packed: torch.Tensor) -> torch.Tensor:
    """uint8 (..., K/2) -> int8 codes (..., K); inverse of ``pack_int4``
    (gemm-quest/benchmarks/utils.py:420-445, dense branch)."""
    x_int = torch.empty(*x_int_packed.shape[:-1], x_int_packed.size(-1) * 2, dtype=torch.int8)
    x_int[..., ::2] = x_int_packed & 0xF
    x_int[..., 1::2] = x_int_packed >> 4
    return torch.where(x_int >= 8, x_int - 16, x_int)


# ----------------------------------------------------------------------------
# int4 x int4 GEMM and the dequantising epilogue
# ----------------------------------------------------------------------------
def matmul_int4_int4t_int32(mat_a: torch.Tensor, mat_b: torch.Tensor) -> torch.Tensor:
    """C[M,N] (int32) = A[M,K] . B[N,K]^T on packed int4 operands.

    The reference checks its CUTLASS kernel against an exact floating-point
    matmul of the codes (gemm-quest/benchmarks/utils.py:680, 707-708).  fp32 is
    exact while 64*K < 2^24, fp64 beyond that.
    """
    a = unpack_int4(mat_a)
    b = unpack_int4(mat_b)
    k = a.size(-1)
    dt = torch.float32 if 64 * k < (1 << 24) else torch.float64
    return (a.to(dt) @ b.to(dt).t()).to(torch.int32)


def add_mul_vv(vec_a_add, vec_a_mul, vec_b_add, vec_b_mul, mat_c, mat_d: torch.Tensor | None = None):
    """D = float(2C + a_add + b_add^T) * (0.5 * a_mul * b_mul^T) -> dtype of a_mul.

    Follows gemm-quest/benchmarks/utils.py:535-545; this *exact* epilogue is the
    parity target for the fused GEMM as well.
    """
    if mat_d is None:
        mat_d = torch.empty(mat_c.shape, dtype=vec_a_mul.dtype)
    acc = torch.float32
    mat_d_ = (mat_c * 2 + vec_a_add + vec_b_add.t()).to(dtype=acc) * (
        .5 * vec_a_mul.to(dtype=acc) * vec_b_mul.t().to(dtype=acc))
    return mat_d.copy_(mat_d_)


def fused_matmul_dequantize_int4_int4t_bf16(mat_a, mat_b, vec_a_add, vec_b_add, vec_a_mul, vec_b_mul,
                                            out: torch.Tensor | None = None):
    """Exact int32 GEMM followed by ``add_mul_vv`` (the reference's debug_mode
    composition, gemm-quest/benchmarks/utils.py:581-584).

    The reference's fused CUTLASS epilogue first casts the accumulator to fp16
    (gemm-quest/include/symmetric/epilogue/thread/linear_combination_dequant.h:133-144),
    which is lossy for |acc| > 2048; that defect is not reproduced.
    """
    c = matmul_int4_int4t_int32(mat_a, mat_b)
    return add_mul_vv(vec_a_add, vec_a_mul, vec_b_add, vec_b_mul, c, out)


# ----------------------------------------------------------------------------
# block Hadamard transform along K
# ----------------------------------------------------------------------------
def sylvester_sign_matrix(block: int) -> torch.Tensor:
    """(+1/-1) Sylvester-ordered Hadamard matrix, H[i][j] = (-1)^popcount(i & j), fp64."""
    assert block & (block - 1) == 0
    h = torch.ones(1, 1, dtype=torch.float64)
    while h.size(0) < block:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return h


def hadamard_constant(block: int, weight_side: bool = False) -> float:
    """Normalisation used by the reference.

    Activations: entries of HADAMARD_MATRIX are bf16(block^-0.5)
    (gemm-quest/benchmarks/utils.py:17) - 0.08837890625 for block 128, exact for
    64 and 256.  Weights: the exact fp32 value of 2^-3.5 for block 128
    (gemm-quest/benchmarks/utils.py:39); generalised here to fp32(block^-0.5).
    """
    if weight_side:
        return float(torch.tensor(block ** -0.5, dtype=torch.float32))
    return float(torch.tensor(block ** -0.5, dtype=torch.bfloat16))


def hadamard_matrix_bf16(block: int) -> torch.Tensor:
    """What ``hadamard_transform(eye(block, bf16), scale=block**-0.5)`` materialises
    (gemm-quest/benchmarks/utils.py:17): Sylvester signs times bf16(block^-0.5)."""
    return (sylvester_sign_matrix(block) * hadamard_constant(block)).to(torch.bfloat16)


def round_f64_to_bf16(v: torch.Tensor) -> torch.Tensor:
    """Round fp64 -> bf16 in ONE step (round-to-nearest-even on the fp64 bits),
    avoiding the double rounding of fp64 -> fp32 -> bf16."""
    a = np.ascontiguousarray(v.detach().numpy().astype(np.float64))
    bits = a.view(np.uint64)
    drop = np.uint64(52 - 7)
    lsb = (bits >> drop) & np.uint64(1)
    rounded = (bits + ((np.uint64(1) << (drop - np.uint64(1))) - np.uint64(1)) + lsb) >> drop << drop
    out = rounded.view(np.float64)
    tiny = np.abs(a) < 2.0 ** -120  # bf16 subnormal territory: defer to the two-step path
    out = np.where(tiny, a.astype(np.float32).astype(np.float64), out)
    return torch.from_numpy(out.astype(np.float32)).to(torch.bfloat16)


def block_hadamard(x: torch.Tensor, block: int = 128, weight_side: bool = False) -> torch.Tensor:
    """Canonical block Hadamard along the last dim: exact sum, one rounding to bf16.

    Each product x*h is exact in fp32/fp64 (8-bit x 8-bit mantissas); only the
    summation order distinguishes implementations, so the exact sum rounded once
    is the order-independent reference point.
    """
    assert x.dtype == torch.bfloat16 and x.size(-1) % block == 0
    h = sylvester_sign_matrix(block) * hadamard_constant(block, weight_side)
    y = x.to(torch.float64).reshape(-1, block) @ h.t()
    return round_f64_to_bf16(y).view_as(x)


def block_hadamard_reference_op(x: torch.Tensor, block: int = 128) -> torch.Tensor:
    """The reference's own activation-side op, executed on the CPU:
    ``F.linear(x.view(-1, 128), HADAMARD_MATRIX)`` (gemm-quest/benchmarks/utils.py:89-90).
    bf16 in, bf16 out, library summation order.  Used as the timed CPU baseline."""
    return F.linear(x.view(-1, block), hadamard_matrix_bf16(block)).view_as(x)


def hadamard_quantize_int4(x: torch.Tensor, block: int = 128, reference_op: bool = False):
    """Hadamard -> scale -> quantize/pack/row-sum: the composition the fused CUDA
    kernel replaces (gemm-quest/benchmarks/utils.py:89-100).
    Returns (packed u8 [M,K/2], scale bf16 [M,1], row_sum i32 [M,1], xh bf16 [M,K])."""
    xh = block_hadamard_reference_op(x, block) if reference_op else block_hadamard(x, block)
    m, k = xh.shape
    scale = find_scale_int4(xh)
    packed = torch.empty(m, k // 2, dtype=torch.uint8)
    row_sum = torch.empty(m, 1, dtype=torch.int32)
    quantize_int4(xh, scale, None, packed, row_sum, False)
    return packed, scale, row_sum, xh


# ----------------------------------------------------------------------------
# layer logic
# ----------------------------------------------------------------------------
def preprocess_weight(weight: torch.Tensor, use_hadamard: bool = False, block: int = 128):
    """gemm-quest/benchmarks/utils.py:20-53, dense branch:
    optional Hadamard -> scale -> quantize -> w_add = row_sum + K // 2."""
    if use_hadamard:
        weight = block_hadamard(weight, block, weight_side=True)
    weight = weight.contiguous()
    n, k = weight.shape
    w_scale = find_scale_int4(weight)
    w_int_packed = torch.empty(n, k // 2, dtype=torch.uint8)
    w_int_row_sum = torch.empty(n, 1, dtype=torch.int32)
    quantize_int4(weight, w_scale, None, w_int_packed, w_int_row_sum, False)
    w_add = w_int_row_sum + k // 2
    return w_int_packed, w_scale, w_add, None


def linear_forward(activation, w_int_packed, w_scale, w_add, use_hadamard: bool = False,
                   block: int = 128, reference_op: bool = False) -> torch.Tensor:
    """gemm-quest/benchmarks/utils.py:56-111, dense branch."""
    if use_hadamard:
        activation = (block_hadamard_reference_op(activation, block) if reference_op
                      else block_hadamard(activation, block))
    m, k = activation.shape
    a_scale = find_scale_int4(activation)
    a_int_packed = torch.empty(m, k // 2, dtype=torch.uint8)
    a_int_row_sum = torch.empty(m, 1, dtype=torch.int32)
    quantize_int4(activation, a_scale, None, a_int_packed, a_int_row_sum, False)
    return fused_matmul_dequantize_int4_int4t_bf16(a_int_packed, w_int_packed, a_int_row_sum, w_add,
                                                   a_scale, w_scale)


# ----------------------------------------------------------------------------
# helpers for tests
# ----------------------------------------------------------------------------
def count_code_flips(packed_a: torch.Tensor, packed_b: torch.Tensor) -> tuple[int, int]:
    """(number of differing codes, max |difference|) between two packed tensors."""
    a = unpack_int4(packed_a).to(torch.int16)
    b = unpack_int4(packed_b).to(torch.int16)
    d = (a - b).abs()
    return int((d != 0).sum()), int(d.max()) if d.numel() else 0


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Distance in bf16 units-in-the-last-place (monotone integer mapping of the bit patterns)."""
    def key(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(a) - key(b)).abs()


def ideal_quantized_linear_fp64(a_int, a_scale, w_int, w_scale):
    """dq(a) . dq(w)^T in fp64 with dq(q) = (q + 0.5) * s
    (gemm-quest/benchmarks/utils.py:667-670)."""
    a_dq = (a_int.to(torch.float64) + .5) * a_scale.to(torch.float64)
    w_dq = (w_int.to(torch.float64) + .5) * w_scale.to(torch.float64)
    return a_dq @ w_dq.t()


assert math.isclose(SCALE_FACTOR, 0.33519074380912307, rel_tol=1e-15)
