"""Layer logic on top of the ops: weight preparation, the W4A4 linear forward and the module.

Mirrors the dense branches of gemm-quest/benchmarks/utils.py (``preprocess_weight`` :20-53,
``linear_forward`` :56-111, ``unpack_int4`` :420-445) and ``Linear4bit`` of
gemm-quest/benchmarks/bench_e2e.py:41-70, without the backend switch (there is one backend) and without
the 4:8-sparse branch.  With ``use_hadamard`` the activation side is ONE fused kernel
(Hadamard + scale + quantise + pack + row sum) followed by the fused GEMM: two launches per layer
instead of the reference's four.
"""
from __future__ import annotations

import torch
from torch import nn

import quest_b200 as quest
from .workspace import default_cache

HADAMARD_BLOCK = 128  # the reference hard-codes block 128 (utils.py:17, 39, 90)


def preprocess_weight(
        weight: torch.Tensor,
        use_sparse: bool = False,
        use_hadamard: bool = False,
        backend: str = 'cuda',
        block: int = HADAMARD_BLOCK,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """weight bf16 (N, K) -> (w_int_packed u8 (N, K//2), w_scale bf16 (N, 1), w_add i32 (N, 1), None).

    ``w_add = row_sum + K // 2`` folds the +0.5 offsets of both operands into the epilogue
    (utils.py:48).  ``backend`` is accepted for signature compatibility and ignored.
    """
    if use_sparse:
        raise NotImplementedError("quest_b200 implements the dense W4A4 path only")
    weight = weight.contiguous()
    if use_hadamard:
        weight = quest.hadamard_transform(weight, block=block, weight_side=True)
    N, K = weight.shape
    w_scale = torch.empty(N, 1, dtype=weight.dtype, device=weight.device)
    w_int_packed = torch.empty(N, K // 2, dtype=torch.uint8, device=weight.device)
    w_int_row_sum = torch.empty(N, 1, dtype=torch.int32, device=weight.device)
    quest.find_scale_int4(x=weight, scale=w_scale)
    quest.quantize_int4(x=weight, scale=w_scale, x_int=None, x_int_packed=w_int_packed,
                        x_int_row_sum=w_int_row_sum, do_dequantize=False)
    w_add = w_int_row_sum + K // 2
    return w_int_packed, w_scale, w_add, None


def fused_matmul_dequantize_int4_bf16(
        mat_a: torch.Tensor,
        mat_b: torch.Tensor,
        vec_a_add: torch.Tensor,
        vec_b_add: torch.Tensor,
        vec_a_mul: torch.Tensor,
        vec_b_mul: torch.Tensor,
        mat_d: torch.Tensor,
        _mat_c: torch.Tensor = None,
        debug_mode: bool = True,
) -> torch.Tensor:
    """mat_d (M, N) bf16 = (2 * mat_a @ mat_b^T + vec_a_add + vec_b_add^T) * (.5 * vec_a_mul * vec_b_mul^T).

    The switch of gemm-quest/benchmarks/utils.py:548-587: ``debug_mode=True`` (the reference's default) takes the
    unfused route - int32 GEMM into ``_mat_c`` (allocated if absent), then ``add_mul_vv`` - and ``debug_mode=False``
    the fused kernel.  Here both routes evaluate the same exact expression, so their results are bit-identical.
    ``mat_d`` may be None (allocated in the dtype of ``vec_a_mul``)."""
    M, N = mat_a.size(0), mat_b.size(0)
    device = mat_a.device
    if mat_d is None:
        mat_d = torch.empty(M, N, dtype=vec_a_mul.dtype, device=device)
    if debug_mode:
        mat_c = torch.empty(M, N, dtype=torch.int32, device=device) if _mat_c is None else _mat_c
        quest.matmul_int4_int4t_int32(mat_a=mat_a, mat_b=mat_b, out=mat_c)
        quest.add_mul_vv(vec_a_add=vec_a_add, vec_a_mul=vec_a_mul, vec_b_add=vec_b_add, vec_b_mul=vec_b_mul,
                         mat_c=mat_c, mat_d=mat_d)
    else:
        quest.fused_matmul_dequantize_int4_int4t_bf16(mat_a=mat_a, mat_b=mat_b, vec_a_add=vec_a_add, vec_b_add=vec_b_add,
                                                      vec_a_mul=vec_a_mul, vec_b_mul=vec_b_mul, out=mat_d)
    return mat_d


def _one_call_ok(*tensors: torch.Tensor) -> bool:
    """The one-call layer entry points take dense row-major buffers only."""
    return all(t.is_contiguous() for t in tensors)


def linear_forward(
        activation: torch.Tensor,
        w_int_packed: torch.Tensor,
        w_scale: torch.Tensor,
        w_add: torch.Tensor,
        w_meta_e: torch.Tensor = None,
        out: torch.Tensor = None,
        _a_scale: torch.Tensor = None,
        _a_int_packed: torch.Tensor = None,
        _a_int_row_sum: torch.Tensor = None,
        _c: torch.Tensor = None,
        use_hadamard: bool = False,
        backend: str = 'cuda',
        block: int = HADAMARD_BLOCK,
        _a_int8: torch.Tensor = None,
        debug_mode: bool = False,
) -> torch.Tensor:
    """out (M, N) bf16 = activation (M, K) @ weight^T in W4A4.  The ``_a_*`` arguments are optional
    caller-owned workspaces (CUDA-graph friendly), as in the reference.  As in the reference (utils.py:100) the
    fused kernel is used whether or not ``_c`` is given; ``debug_mode=True`` (not in the reference's signature)
    takes the unfused int32 GEMM + add_mul_vv route with ``_c`` as its int32 workspace.

    With ``use_hadamard`` and a shape for which the library prefers it, the quantiser writes the GEMM's int8 operand
    directly (``_a_int8`` [M, K] uint8 is its workspace) instead of packed int4: same codes, same result, no unpack
    of A inside the GEMM.  A caller that passes ``_a_int_packed`` but no ``_a_int8`` keeps the packed route.

    With ``use_hadamard`` (and dense buffers) the layer is ONE library call: the quantiser, then the GEMM kernel launched
    with a programmatic dependency on it, so that the GEMM's set-up and first weight copies overlap the quantiser's end."""
    if w_meta_e is not None:
        raise NotImplementedError("quest_b200 implements the dense W4A4 path only")
    M, K, N = activation.size(0), activation.size(1), w_int_packed.size(0)
    dtype, device = activation.dtype, activation.device
    if out is None:
        out = torch.empty(M, N, dtype=dtype, device=device)
    a_scale = torch.empty(M, 1, dtype=dtype, device=device) if _a_scale is None else _a_scale
    a_int_row_sum = torch.empty(M, 1, dtype=torch.int32, device=device) if _a_int_row_sum is None else _a_int_row_sum
    if (use_hadamard and not debug_mode and (_a_int8 is not None or _a_int_packed is None) and K % block == 0
            and quest.prefers_a8(M, K, N)):
        a_int8 = torch.empty(M, K, dtype=torch.uint8, device=device) if _a_int8 is None else _a_int8
        if _one_call_ok(activation, out, a_int8, a_scale, a_int_row_sum, w_int_packed, w_add, w_scale):
            return quest.w4a4_linear_hadamard(activation, w_int_packed, w_add, w_scale, out, a_int8, a_scale, a_int_row_sum,
                                              block=block)
        quest.hadamard_quantize_a8(activation, block=block, x_a8=a_int8, scale=a_scale, x_int_row_sum=a_int_row_sum)
        quest.fused_matmul_dequantize_a8(mat_a8=a_int8, mat_b=w_int_packed, vec_a_add=a_int_row_sum, vec_b_add=w_add,
                                         vec_a_mul=a_scale, vec_b_mul=w_scale, out=out)
        return out
    a_int_packed = torch.empty(M, K // 2, dtype=torch.uint8, device=device) if _a_int_packed is None else _a_int_packed
    if use_hadamard and not debug_mode and _one_call_ok(activation, out, a_int_packed, a_scale, a_int_row_sum, w_int_packed, w_add, w_scale):
        # one library call: the GEMM kernel starts behind the quantiser with a dependent launch
        return quest.w4a4_linear_hadamard(activation, w_int_packed, w_add, w_scale, out, a_int_packed, a_scale, a_int_row_sum,
                                          block=block)
    if use_hadamard:
        quest.hadamard_quantize_int4(activation, block=block, x_int_packed=a_int_packed, scale=a_scale,
                                     x_int_row_sum=a_int_row_sum)
    else:
        quest.find_scale_int4(x=activation, scale=a_scale)
        quest.quantize_int4(x=activation, scale=a_scale, x_int=None, x_int_packed=a_int_packed,
                            x_int_row_sum=a_int_row_sum, do_dequantize=False)
    fused_matmul_dequantize_int4_bf16(mat_a=a_int_packed, mat_b=w_int_packed, vec_a_add=a_int_row_sum, vec_b_add=w_add,
                                      vec_a_mul=a_scale, vec_b_mul=w_scale, mat_d=out, _mat_c=_c, debug_mode=debug_mode)
    return out


def unpack_int4(x_int_packed: torch.Tensor) -> torch.Tensor:
    """uint8 (..., K // 2) -> int8 codes (..., K); test helper, plain torch (utils.py:420-445)."""
    x_int = torch.empty(*x_int_packed.shape[:-1], x_int_packed.size(-1) * 2, dtype=torch.int8,
                        device=x_int_packed.device)
    x_int[..., ::2] = x_int_packed & 0xF
    x_int[..., 1::2] = x_int_packed >> 4
    return torch.where(x_int >= 8, x_int - 16, x_int)


class Linear4bit(nn.Module):
    """nn.Linear whose weight is stored as packed int4 + per-row scale/offset and whose forward runs
    the W4A4 kernels (gemm-quest/benchmarks/bench_e2e.py:41-70).  Needs a CUDA device."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=None,
                 use_sparse: bool = False, use_hadamard: bool = False, use_noop: bool = False,
                 weight: torch.Tensor | None = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.use_hadamard: bool = use_hadamard
        self.use_noop: bool = use_noop
        self.workspaces = default_cache  # a WorkspaceCache; replace it to give a module (or a model) its own
        nn_linear = nn.Linear(in_features, out_features, bias=bias, device=device, dtype=dtype)
        if weight is not None:
            nn_linear.weight.data.copy_(weight)
        self.bias = nn_linear.bias
        w = nn_linear.weight.data
        self.weight = torch.empty_like(w, device=torch.device('meta'))
        w_int_packed, w_scale, w_add, w_meta_e = preprocess_weight(weight=w, use_sparse=use_sparse,
                                                                   use_hadamard=use_hadamard)
        self.register_buffer('w_int_packed', w_int_packed)
        self.register_buffer('w_scale', w_scale)
        self.register_buffer('w_add', w_add)
        self.register_buffer('w_meta_e', w_meta_e)

    def forward_quantized(self, a_int_packed: torch.Tensor, a_scale: torch.Tensor, a_int_row_sum: torch.Tensor,
                          out: torch.Tensor = None) -> torch.Tensor:
        """The layer on activations that are already quantised ([M, K/2] packed codes, [M, 1] scales and row sums, as
        written by ``hadamard_quantize_int4`` or one of its producer-fused variants): only the fused GEMM runs.  Several
        layers that read the same activations (w1 and w2 of a SwiGLU block) can share one quantisation this way."""
        y = quest.fused_matmul_dequantize_int4_int4t_bf16(mat_a=a_int_packed, mat_b=self.w_int_packed, vec_a_add=a_int_row_sum,
                                                          vec_b_add=self.w_add, vec_a_mul=a_scale, vec_b_mul=self.w_scale, out=out)
        if self.bias is not None:
            y += self.bias
        return y

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not self.use_noop:
            a = x.contiguous().flatten(end_dim=-2)
            # activation-side workspaces come from the shared per-stream cache: nothing but the output is allocated
            m, k = a.shape
            a8 = self.use_hadamard and k % HADAMARD_BLOCK == 0 and quest.prefers_a8(m, k, self.out_features)
            ws = self.workspaces.get(m, k, a.device, a.dtype, int8_operand=a8)
            y = linear_forward(activation=a, w_int_packed=self.w_int_packed, w_scale=self.w_scale, w_add=self.w_add,
                               w_meta_e=self.w_meta_e, out=None, use_hadamard=self.use_hadamard, **ws)
            y = y.unflatten(dim=0, sizes=x.shape[:-1])
        else:
            if self.use_hadamard:
                x = quest.hadamard_transform(x.contiguous(), block=HADAMARD_BLOCK, weight_side=True)
            y = torch.zeros(*x.shape[:-1], self.out_features, dtype=x.dtype, device=x.device)
        if self.bias is not None:
            y += self.bias
        return y
