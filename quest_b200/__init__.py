"""quest_b200 - drop-in replacement of the reference's ``quest`` op package on B200 (sm_100a).

The dense ops keep the signatures, dtype/contiguity asserts, output allocation and return conventions
of gemm-quest/quest/__init__.py; each forwards raw device pointers to one ``extern "C"`` entry point
of ``libquest_b200.so`` on the current CUDA stream of the tensors' device.  Two ops are new:
``hadamard_quantize_int4`` (the fused kernel that replaces the Hadamard GEMM + find_scale + quantize
launches of the reference's ``linear_forward``) and ``hadamard_transform``.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import device_status  # noqa: F401


def _call(name: str, device: torch.device, *args) -> None:
    fn = getattr(_lib.load(), name)
    if torch.cuda.current_device() != device.index:
        with torch.cuda.device(device):
            _lib.check(fn(*args), name)
    else:
        _lib.check(fn(*args), name)


def fused_matmul_dequantize_int4_int4t_bf16(
        mat_a: torch.Tensor,
        mat_b: torch.Tensor,
        vec_a_add: torch.Tensor,
        vec_b_add: torch.Tensor,
        vec_a_mul: torch.Tensor,
        vec_b_mul: torch.Tensor,
        out: torch.Tensor = None,
) -> torch.Tensor:
    """out[M,N] bf16 = add_mul_vv(vec_a_add, vec_a_mul, vec_b_add, vec_b_mul, mat_a @ mat_b^T) in one kernel.
    Mirrors gemm-quest/quest/__init__.py:6-20."""
    if out is None:
        out = torch.empty(mat_a.size(0), mat_b.size(0), dtype=torch.bfloat16, device=mat_a.device)
    assert mat_a.dtype == torch.uint8 and mat_b.dtype == torch.uint8 and vec_a_add.dtype == torch.int32 and vec_b_add.dtype == torch.int32 and vec_a_mul.dtype == torch.bfloat16 and vec_b_mul.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert mat_a.is_contiguous() and mat_b.is_contiguous() and vec_a_add.is_contiguous() and vec_b_add.is_contiguous() and vec_a_mul.is_contiguous() and vec_b_mul.is_contiguous() and out.is_contiguous()
    dev = _lib.require_cuda(mat_a, mat_b, vec_a_add, vec_b_add, vec_a_mul, vec_b_mul, out)
    _call("fused_matmul_dequantize_int4_int4t_bf16_cuda", dev, _lib.ptr(out), _lib.ptr(mat_a), _lib.ptr(mat_b),
          _lib.ptr(vec_a_add), _lib.ptr(vec_b_add), _lib.ptr(vec_a_mul), _lib.ptr(vec_b_mul),
          mat_a.size(0), mat_b.size(1) * 2, mat_b.size(0), _lib.stream_of(out))
    return out


def fused_matmul_dequantize_int4_int4t_bf16_into(
        mat_a: torch.Tensor,
        mat_b: torch.Tensor,
        vec_a_add: torch.Tensor,
        vec_b_add: torch.Tensor,
        vec_a_mul: torch.Tensor,
        vec_b_mul: torch.Tensor,
        out_cols: torch.Tensor,
) -> torch.Tensor:
    """Same computation, written into a column slice ``out_cols = full[:, n0:n0+N]`` of a wider
    row-major bf16 matrix (row stride = out_cols.stride(0)).  Used by the column-sharded layer."""
    assert out_cols.dtype == torch.bfloat16 and out_cols.dim() == 2 and out_cols.stride(1) == 1
    assert out_cols.size(0) == mat_a.size(0) and out_cols.size(1) == mat_b.size(0)
    assert mat_a.dtype == torch.uint8 and mat_b.dtype == torch.uint8 and vec_a_add.dtype == torch.int32 and vec_b_add.dtype == torch.int32 and vec_a_mul.dtype == torch.bfloat16 and vec_b_mul.dtype == torch.bfloat16
    assert mat_a.is_contiguous() and mat_b.is_contiguous() and vec_a_add.is_contiguous() and vec_b_add.is_contiguous() and vec_a_mul.is_contiguous() and vec_b_mul.is_contiguous()
    dev = _lib.require_cuda(mat_a, mat_b, vec_a_add, vec_b_add, vec_a_mul, vec_b_mul, out_cols)
    _call("fused_matmul_dequantize_int4_int4t_bf16_strided_cuda", dev, _lib.ptr(out_cols), out_cols.stride(0),
          _lib.ptr(mat_a), _lib.ptr(mat_b), _lib.ptr(vec_a_add), _lib.ptr(vec_b_add), _lib.ptr(vec_a_mul),
          _lib.ptr(vec_b_mul), mat_a.size(0), mat_b.size(1) * 2, mat_b.size(0), _lib.stream_of(out_cols))
    return out_cols


def fused_matmul_dequantize_int4_int4t_bf16_noalloc(
        mat_a: torch.Tensor,
        mat_b: torch.Tensor,
        vec_a_add: torch.Tensor,
        vec_b_add: torch.Tensor,
        vec_a_mul: torch.Tensor,
        vec_b_mul: torch.Tensor,
        out: torch.Tensor,
        splits: int = 0,
) -> torch.Tensor:
    """Same computation through the entry point that allocates nothing: ``out`` is required, and a split-K launch
    takes its scratch from the library's fixed 8 MiB device array (``splits`` = 0: the library's choice of K ranges,
    n >= 2: n ranges).  Raises if the scratch needed exceeds that array."""
    assert mat_a.dtype == torch.uint8 and mat_b.dtype == torch.uint8 and vec_a_add.dtype == torch.int32 and vec_b_add.dtype == torch.int32 and vec_a_mul.dtype == torch.bfloat16 and vec_b_mul.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert mat_a.is_contiguous() and mat_b.is_contiguous() and vec_a_add.is_contiguous() and vec_b_add.is_contiguous() and vec_a_mul.is_contiguous() and vec_b_mul.is_contiguous() and out.is_contiguous()
    assert out.shape == (mat_a.size(0), mat_b.size(0))
    dev = _lib.require_cuda(mat_a, mat_b, vec_a_add, vec_b_add, vec_a_mul, vec_b_mul, out)
    _call("fused_matmul_dequantize_int4_int4t_bf16_noalloc_cuda", dev, _lib.ptr(out), _lib.ptr(mat_a), _lib.ptr(mat_b),
          _lib.ptr(vec_a_add), _lib.ptr(vec_b_add), _lib.ptr(vec_a_mul), _lib.ptr(vec_b_mul), mat_a.size(0),
          mat_b.size(1) * 2, mat_b.size(0), int(splits), _lib.stream_of(mat_a))
    return out


def fused_matmul_dequantize_int4_int4t_bf16_push(
        mat_a: torch.Tensor,
        mat_b: torch.Tensor,
        vec_a_add: torch.Tensor,
        vec_b_add: torch.Tensor,
        vec_a_mul: torch.Tensor,
        vec_b_mul: torch.Tensor,
        dst_ptrs: list[int],
        ld: int,
) -> None:
    """Same computation; every output tile is stored to each address in ``dst_ptrs`` (raw device pointers of
    [M, ld]-strided bf16 matrices, the caller's own first, then buffers of peer GPUs mapped into this process,
    each already offset to the caller's first column).  The caller synchronises the GPUs afterwards."""
    import ctypes
    assert mat_a.dtype == torch.uint8 and mat_b.dtype == torch.uint8 and vec_a_add.dtype == torch.int32 and vec_b_add.dtype == torch.int32 and vec_a_mul.dtype == torch.bfloat16 and vec_b_mul.dtype == torch.bfloat16
    assert mat_a.is_contiguous() and mat_b.is_contiguous() and vec_a_add.is_contiguous() and vec_b_add.is_contiguous() and vec_a_mul.is_contiguous() and vec_b_mul.is_contiguous()
    assert 1 <= len(dst_ptrs) <= 8
    dev = _lib.require_cuda(mat_a, mat_b, vec_a_add, vec_b_add, vec_a_mul, vec_b_mul)
    arr = (ctypes.c_void_p * len(dst_ptrs))(*dst_ptrs)
    _call("fused_matmul_dequantize_int4_int4t_bf16_push_cuda", dev, arr, len(dst_ptrs), int(ld),
          _lib.ptr(mat_a), _lib.ptr(mat_b), _lib.ptr(vec_a_add), _lib.ptr(vec_b_add), _lib.ptr(vec_a_mul),
          _lib.ptr(vec_b_mul), mat_a.size(0), mat_b.size(1) * 2, mat_b.size(0), _lib.stream_of(mat_a))


def matmul_int4_int4t_int32(
        mat_a: torch.Tensor,
        mat_b: torch.Tensor,
        out: torch.Tensor = None,
) -> torch.Tensor:
    """out[M,N] int32 = mat_a[M,K/2] @ mat_b[N,K/2]^T on packed int4 codes, exact.
    Mirrors gemm-quest/quest/__init__.py:23-33."""
    if out is None:
        out = torch.empty(mat_a.size(0), mat_b.size(0), dtype=torch.int32, device=mat_a.device)
    assert mat_a.dtype == torch.uint8 and mat_b.dtype == torch.uint8 and out.dtype == torch.int32
    assert mat_a.is_contiguous() and mat_b.is_contiguous() and out.is_contiguous()
    dev = _lib.require_cuda(mat_a, mat_b, out)
    _call("matmul_int4_int4t_int32_cuda", dev, _lib.ptr(out), _lib.ptr(mat_a), _lib.ptr(mat_b),
          mat_a.size(0), mat_b.size(1) * 2, mat_b.size(0), _lib.stream_of(out))
    return out


def matmul_int4sp_int4t_int32(*args, **kwargs):
    """4:8-sparse GEMM of the reference (gemm-quest/quest/__init__.py:36-47): not part of the dense path."""
    raise NotImplementedError("quest_b200 implements the dense W4A4 path only")


def reorder_meta48_int4(*args, **kwargs):
    raise NotImplementedError("quest_b200 implements the dense W4A4 path only")


def uncompress_meta48_int4(*args, **kwargs):
    raise NotImplementedError("quest_b200 implements the dense W4A4 path only")


def generate_random_meta48_int4(*args, **kwargs):
    raise NotImplementedError("quest_b200 implements the dense W4A4 path only")


def find_scale_int4(
        x: torch.Tensor,
        scale: torch.Tensor = None,
) -> torch.Tensor:
    """scale[M,1] = sqrt(mean(x^2)) * (2.5139 * 2 / 15) + 1e-8 in x's dtype.
    Mirrors gemm-quest/quest/__init__.py:87-96."""
    if scale is None:
        scale = torch.empty(x.size(0), 1, dtype=x.dtype, device=x.device)
    assert x.dtype == torch.bfloat16 and scale.dtype == torch.bfloat16
    assert x.is_contiguous() and scale.is_contiguous()
    dev = _lib.require_cuda(x, scale)
    _call("find_scale_int4_cuda_bf16", dev, _lib.ptr(scale), _lib.ptr(x), x.size(1), x.size(0), _lib.stream_of(x))
    return scale


def quantize_int4(
        x: torch.Tensor,
        scale: torch.Tensor,
        x_int: torch.Tensor = None,
        x_int_packed: torch.Tensor = None,
        x_int_row_sum: torch.Tensor = None,
        do_dequantize: bool = False,
) -> tuple[torch.Tensor, torch.Tensor | None, torch.Tensor | None, torch.Tensor | None]:
    """Floor-quantise x by its per-row scale into any of: dense int8 codes, packed codes, int32 row
    sums; optionally overwrite x with the dequantised values.  Returns the caller's own objects
    (None where not supplied).  Mirrors gemm-quest/quest/__init__.py:99-114."""
    assert x.dtype == torch.bfloat16 and scale.dtype == torch.bfloat16 and (x_int is None or x_int.dtype == torch.int8) and (x_int_packed is None or x_int_packed.dtype == torch.uint8) and (x_int_row_sum is None or x_int_row_sum.dtype == torch.int32)
    assert x.is_contiguous() and scale.is_contiguous() and (x_int is None or x_int.is_contiguous()) and (x_int_packed is None or x_int_packed.is_contiguous()) and (x_int_row_sum is None or x_int_row_sum.is_contiguous())
    dev = _lib.require_cuda(x, scale, x_int, x_int_packed, x_int_row_sum)
    _call("quantize_int4_cuda_bf16", dev, _lib.ptr(x), _lib.ptr(scale), _lib.ptr(x_int), _lib.ptr(x_int_packed),
          _lib.ptr(x_int_row_sum), x.size(1), x.size(0), int(bool(do_dequantize)), _lib.stream_of(x))
    return x, x_int, x_int_packed, x_int_row_sum


def add_mul_vv(
        vec_a_add: torch.Tensor,
        vec_a_mul: torch.Tensor,
        vec_b_add: torch.Tensor,
        vec_b_mul: torch.Tensor,
        mat_c: torch.Tensor,
        mat_d: torch.Tensor = None,
) -> torch.Tensor:
    """mat_d = float(2 * mat_c + vec_a_add + vec_b_add^T) * (0.5 * vec_a_mul * vec_b_mul^T) -> bf16.
    Mirrors gemm-quest/quest/__init__.py:117-130."""
    if mat_d is None:
        mat_d = torch.empty(mat_c.shape, dtype=vec_a_mul.dtype, device=mat_c.device)
    assert vec_a_add.dtype == torch.int32 and vec_a_mul.dtype == torch.bfloat16 and vec_b_add.dtype == torch.int32 and vec_b_mul.dtype == torch.bfloat16 and mat_c.dtype == torch.int32 and mat_d.dtype == torch.bfloat16
    assert vec_a_add.is_contiguous() and vec_a_mul.is_contiguous() and vec_b_add.is_contiguous() and vec_b_mul.is_contiguous() and mat_c.is_contiguous() and mat_d.is_contiguous()
    dev = _lib.require_cuda(vec_a_add, vec_a_mul, vec_b_add, vec_b_mul, mat_c, mat_d)
    _call("add_mul_vv_cuda_bf16", dev, _lib.ptr(mat_d), _lib.ptr(vec_a_add), _lib.ptr(vec_a_mul), _lib.ptr(vec_b_add),
          _lib.ptr(vec_b_mul), _lib.ptr(mat_c), mat_c.size(0), mat_c.size(1), _lib.stream_of(mat_c))
    return mat_d


def hadamard_quantize_int4(
        x: torch.Tensor,
        block: int = 128,
        x_int_packed: torch.Tensor = None,
        scale: torch.Tensor = None,
        x_int_row_sum: torch.Tensor = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Fused block-Hadamard + find_scale_int4 + quantize_int4 (packed codes + row sums) in one pass over x.
    x is not modified.  Equivalent to gemm-quest/benchmarks/utils.py:89-100 with use_hadamard=True.
    Returns (x_int_packed [M,K/2] u8, scale [M,1] bf16, x_int_row_sum [M,1] i32)."""
    assert x.dim() == 2
    m, k = x.shape
    if x_int_packed is None:
        x_int_packed = torch.empty(m, k // 2, dtype=torch.uint8, device=x.device)
    if scale is None:
        scale = torch.empty(m, 1, dtype=x.dtype, device=x.device)
    if x_int_row_sum is None:
        x_int_row_sum = torch.empty(m, 1, dtype=torch.int32, device=x.device)
    assert x.dtype == torch.bfloat16 and scale.dtype == torch.bfloat16 and x_int_packed.dtype == torch.uint8 and x_int_row_sum.dtype == torch.int32
    assert x.is_contiguous() and scale.is_contiguous() and x_int_packed.is_contiguous() and x_int_row_sum.is_contiguous()
    dev = _lib.require_cuda(x, scale, x_int_packed, x_int_row_sum)
    _call("hadamard_quantize_int4_cuda_bf16", dev, _lib.ptr(x_int_packed), _lib.ptr(scale), _lib.ptr(x_int_row_sum),
          _lib.ptr(x), k, m, int(block), _lib.stream_of(x))
    return x_int_packed, scale, x_int_row_sum


def _quant_outputs(m: int, k: int, like: torch.Tensor, x_int_packed, scale, x_int_row_sum):
    if x_int_packed is None:
        x_int_packed = torch.empty(m, k // 2, dtype=torch.uint8, device=like.device)
    if scale is None:
        scale = torch.empty(m, 1, dtype=like.dtype, device=like.device)
    if x_int_row_sum is None:
        x_int_row_sum = torch.empty(m, 1, dtype=torch.int32, device=like.device)
    assert scale.dtype == torch.bfloat16 and x_int_packed.dtype == torch.uint8 and x_int_row_sum.dtype == torch.int32
    assert scale.is_contiguous() and x_int_packed.is_contiguous() and x_int_row_sum.is_contiguous()
    return x_int_packed, scale, x_int_row_sum


def rmsnorm_hadamard_quantize_int4(
        x: torch.Tensor,
        norm_weight: torch.Tensor,
        eps: float,
        block: int = 128,
        x_int_packed: torch.Tensor = None,
        scale: torch.Tensor = None,
        x_int_row_sum: torch.Tensor = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``hadamard_quantize_int4(RMSNorm(x))`` in one kernel: y = ((x.float() * rsqrt(mean(x^2) + eps)).type_as(x)
    * norm_weight) is never written to memory (the RMSNorm of src/models/llama.py:64-76).  x [M, K] bf16,
    norm_weight [K] bf16.  Returns (x_int_packed, scale, x_int_row_sum) of y."""
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and x.is_contiguous()
    assert norm_weight.dtype == torch.bfloat16 and norm_weight.is_contiguous() and norm_weight.numel() == x.size(1)
    m, k = x.shape
    x_int_packed, scale, x_int_row_sum = _quant_outputs(m, k, x, x_int_packed, scale, x_int_row_sum)
    dev = _lib.require_cuda(x, norm_weight, scale, x_int_packed, x_int_row_sum)
    _call("rmsnorm_hadamard_quantize_int4_cuda_bf16", dev, _lib.ptr(x_int_packed), _lib.ptr(scale), _lib.ptr(x_int_row_sum),
          _lib.ptr(x), _lib.ptr(norm_weight), float(eps), k, m, int(block), _lib.stream_of(x))
    return x_int_packed, scale, x_int_row_sum


def silu_mul_hadamard_quantize_int4(
        gate: torch.Tensor,
        up: torch.Tensor,
        block: int = 128,
        x_int_packed: torch.Tensor = None,
        scale: torch.Tensor = None,
        x_int_row_sum: torch.Tensor = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``hadamard_quantize_int4(silu(gate) * up)`` in one kernel (the SwiGLU product of src/models/llama.py:118 is never
    written to memory).  gate, up [M, K] bf16.  Returns (x_int_packed, scale, x_int_row_sum) of the product."""
    assert gate.dim() == 2 and gate.shape == up.shape and gate.dtype == torch.bfloat16 and up.dtype == torch.bfloat16
    assert gate.is_contiguous() and up.is_contiguous()
    m, k = gate.shape
    x_int_packed, scale, x_int_row_sum = _quant_outputs(m, k, gate, x_int_packed, scale, x_int_row_sum)
    dev = _lib.require_cuda(gate, up, scale, x_int_packed, x_int_row_sum)
    _call("silu_mul_hadamard_quantize_int4_cuda_bf16", dev, _lib.ptr(x_int_packed), _lib.ptr(scale), _lib.ptr(x_int_row_sum),
          _lib.ptr(gate), _lib.ptr(up), k, m, int(block), _lib.stream_of(gate))
    return x_int_packed, scale, x_int_row_sum


def w4a4_linear_hadamard(
        x: torch.Tensor,
        w_int_packed: torch.Tensor,
        w_add: torch.Tensor,
        w_scale: torch.Tensor,
        out: torch.Tensor,
        a_int_packed: torch.Tensor,
        a_scale: torch.Tensor,
        a_int_row_sum: torch.Tensor,
        block: int = 128,
) -> torch.Tensor:
    """The layer in one library call: fused Hadamard + quantise of ``x`` into the given workspaces, then the fused GEMM
    into ``out``.  The GEMM kernel is launched with a programmatic dependency on the quantiser (its set-up and first
    weight copies overlap the quantiser's end); results equal the two ops called one after the other.  ``a_int_packed``
    of shape [M, K] instead of [M, K/2] selects the int8-operand route (``hadamard_quantize_a8`` +
    ``fused_matmul_dequantize_a8``)."""
    assert x.dim() == 2 and x.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and w_int_packed.dtype == torch.uint8
    assert a_int_packed.dtype == torch.uint8 and a_scale.dtype == torch.bfloat16 and a_int_row_sum.dtype == torch.int32
    assert w_add.dtype == torch.int32 and w_scale.dtype == torch.bfloat16
    assert all(t.is_contiguous() for t in (x, w_int_packed, w_add, w_scale, out, a_int_packed, a_scale, a_int_row_sum))
    m, k = x.shape
    n = w_int_packed.size(0)
    assert w_int_packed.size(1) * 2 == k and out.shape == (m, n) and a_int_packed.shape in ((m, k // 2), (m, k))
    entry = "w4a4_linear_hadamard_a8_bf16_cuda" if a_int_packed.shape == (m, k) else "w4a4_linear_hadamard_bf16_cuda"
    dev = _lib.require_cuda(x, w_int_packed, w_add, w_scale, out, a_int_packed, a_scale, a_int_row_sum)
    _call(entry, dev, _lib.ptr(out), _lib.ptr(x), _lib.ptr(w_int_packed), _lib.ptr(w_add),
          _lib.ptr(w_scale), _lib.ptr(a_int_packed), _lib.ptr(a_scale), _lib.ptr(a_int_row_sum), m, k, n, int(block),
          _lib.stream_of(x))
    return out


def copy_block_to_peers(src: torch.Tensor, dsts) -> bool:
    """Copies the 2-D bf16 view ``src`` into every view of ``dsts`` (same shape and strides; typically the same column
    block of the peers' output buffers) with one kernel launch.  Returns False, having copied nothing, where the views
    are not made of whole 16-byte pieces (the caller then copies them one by one)."""
    assert src.dim() == 2 and src.dtype == torch.bfloat16 and src.stride(1) == 1 and 1 <= len(dsts) <= 7
    rows, cols = src.shape
    ld = src.stride(0)
    for d in dsts:
        assert d.dtype == torch.bfloat16 and d.shape == src.shape and d.stride() == src.stride() and d.device == src.device
    if rows == 0 or cols == 0:
        return True
    if cols % 8 or ld % 8 or src.data_ptr() % 16 or any(d.data_ptr() % 16 for d in dsts):
        return False
    dev = _lib.require_cuda(src, *dsts)
    ptrs = (ctypes.c_void_p * len(dsts))(*[d.data_ptr() for d in dsts])
    _call("quest_b200_copy_block_to_peers_cuda", dev, _lib.ptr(src), ptrs, len(dsts), rows, cols, ld, _lib.stream_of(src))
    return True


class layer_launches:
    """Context manager: inside it a Hadamard+quantise call followed by a fused GEMM call of this thread are launched as
    one layer, with programmatic dependencies where the library found them faster (what the one-call layer entry points
    do).  Nothing else may be launched into the stream between the two calls."""

    def __enter__(self):
        _lib.load().quest_b200_begin_layer()
        return self

    def __exit__(self, *exc):
        _lib.load().quest_b200_end_layer()
        return False


def prefers_a8(m: int, k: int, n: int) -> bool:
    """Whether the int8-operand route (``hadamard_quantize_a8`` + ``fused_matmul_dequantize_a8``) is the faster one
    for a layer of this shape."""
    return bool(_lib.load().quest_b200_prefers_a8(int(m), int(k), int(n)))


def hadamard_quantize_a8(
        x: torch.Tensor,
        block: int = 128,
        x_a8: torch.Tensor = None,
        scale: torch.Tensor = None,
        x_int_row_sum: torch.Tensor = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``hadamard_quantize_int4`` with the codes written as the GEMM's int8 operand (16 x code, even positions of every
    32-group first) instead of packed int4.  Returns (x_a8 [M,K] u8, scale [M,1] bf16, x_int_row_sum [M,1] i32)."""
    assert x.dim() == 2
    m, k = x.shape
    if x_a8 is None:
        x_a8 = torch.empty(m, k, dtype=torch.uint8, device=x.device)
    if scale is None:
        scale = torch.empty(m, 1, dtype=x.dtype, device=x.device)
    if x_int_row_sum is None:
        x_int_row_sum = torch.empty(m, 1, dtype=torch.int32, device=x.device)
    assert x.dtype == torch.bfloat16 and scale.dtype == torch.bfloat16 and x_a8.dtype == torch.uint8 and x_int_row_sum.dtype == torch.int32
    assert x.is_contiguous() and scale.is_contiguous() and x_a8.is_contiguous() and x_int_row_sum.is_contiguous()
    assert x_a8.shape == (m, k)
    dev = _lib.require_cuda(x, scale, x_a8, x_int_row_sum)
    _call("hadamard_quantize_a8_cuda_bf16", dev, _lib.ptr(x_a8), _lib.ptr(scale), _lib.ptr(x_int_row_sum), _lib.ptr(x), k, m,
          int(block), _lib.stream_of(x))
    return x_a8, scale, x_int_row_sum


def fused_matmul_dequantize_a8(
        mat_a8: torch.Tensor,
        mat_b: torch.Tensor,
        vec_a_add: torch.Tensor,
        vec_b_add: torch.Tensor,
        vec_a_mul: torch.Tensor,
        vec_b_mul: torch.Tensor,
        out: torch.Tensor = None,
) -> torch.Tensor:
    """``fused_matmul_dequantize_int4_int4t_bf16`` with the A operand as written by ``hadamard_quantize_a8``."""
    if out is None:
        out = torch.empty(mat_a8.size(0), mat_b.size(0), dtype=torch.bfloat16, device=mat_a8.device)
    assert mat_a8.dtype == torch.uint8 and mat_b.dtype == torch.uint8 and vec_a_add.dtype == torch.int32 and vec_b_add.dtype == torch.int32 and vec_a_mul.dtype == torch.bfloat16 and vec_b_mul.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
    assert mat_a8.is_contiguous() and mat_b.is_contiguous() and vec_a_add.is_contiguous() and vec_b_add.is_contiguous() and vec_a_mul.is_contiguous() and vec_b_mul.is_contiguous() and out.is_contiguous()
    assert mat_a8.size(1) == mat_b.size(1) * 2 and out.shape == (mat_a8.size(0), mat_b.size(0))
    dev = _lib.require_cuda(mat_a8, mat_b, vec_a_add, vec_b_add, vec_a_mul, vec_b_mul, out)
    _call("fused_matmul_dequantize_a8_int4t_bf16_cuda", dev, _lib.ptr(out), _lib.ptr(mat_a8), _lib.ptr(mat_b),
          _lib.ptr(vec_a_add), _lib.ptr(vec_b_add), _lib.ptr(vec_a_mul), _lib.ptr(vec_b_mul), mat_a8.size(0),
          mat_a8.size(1), mat_b.size(0), _lib.stream_of(mat_a8))
    return out


def hadamard_transform(x: torch.Tensor, block: int = 128, weight_side: bool = False, out: torch.Tensor = None) -> torch.Tensor:
    """bf16(H_block @ x) blockwise along the last dim.  ``weight_side`` selects the exact fp32
    normalisation of gemm-quest/benchmarks/utils.py:39 instead of the bf16 one of utils.py:17."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    if out is None:
        out = torch.empty_like(x)
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == x.shape
    k = x.size(-1)
    m = x.numel() // k if k else 0
    dev = _lib.require_cuda(x, out)
    _call("hadamard_transform_cuda_bf16", dev, _lib.ptr(out), _lib.ptr(x), k, m, int(block), int(bool(weight_side)),
          _lib.stream_of(x))
    return out


from .layer import (Linear4bit, fused_matmul_dequantize_int4_bf16, linear_forward, preprocess_weight,  # noqa: E402,F401
                    unpack_int4)
