"""ctypes binding of ``libquest_b200.so``.  There is no fallback: if the library is missing or a call
fails, the caller gets an exception."""
from __future__ import annotations

import ctypes
import os

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libquest_b200.so")
_lib = None

_P = ctypes.c_void_p
_I = ctypes.c_int
_LL = ctypes.c_longlong

# name -> argtypes, exactly as declared in include/quest_b200.h
SIGNATURES = {
    "find_scale_int4_cuda_bf16": [_P, _P, _I, _I, _P],
    "quantize_int4_cuda_bf16": [_P, _P, _P, _P, _P, _I, _I, _I, _P],
    "add_mul_vv_cuda_bf16": [_P, _P, _P, _P, _P, _P, _I, _I, _P],
    "matmul_int4_int4t_int32_cuda": [_P, _P, _P, _I, _I, _I, _P],
    "fused_matmul_dequantize_int4_int4t_bf16_cuda": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "fused_matmul_dequantize_int4_int4t_bf16_noalloc_cuda": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "fused_matmul_dequantize_int4_int4t_bf16_strided_cuda": [_P, _LL, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "fused_matmul_dequantize_int4_int4t_bf16_push_cuda": [ctypes.POINTER(ctypes.c_void_p), _I, _LL, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "hadamard_quantize_int4_cuda_bf16": [_P, _P, _P, _P, _I, _I, _I, _P],
    "w4a4_linear_hadamard_bf16_cuda": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "w4a4_linear_hadamard_a8_bf16_cuda": [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "hadamard_quantize_a8_cuda_bf16": [_P, _P, _P, _P, _I, _I, _I, _P],
    "rmsnorm_hadamard_quantize_int4_cuda_bf16": [_P, _P, _P, _P, _P, ctypes.c_float, _I, _I, _I, _P],
    "silu_mul_hadamard_quantize_int4_cuda_bf16": [_P, _P, _P, _P, _P, _I, _I, _I, _P],
    "fused_matmul_dequantize_a8_int4t_bf16_cuda": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _P],
    "quest_b200_prefers_a8": [_I, _I, _I],
    "quest_b200_copy_block_to_peers_cuda": [_P, ctypes.POINTER(ctypes.c_void_p), _I, _I, _I, _LL, _P],
    "quest_b200_begin_layer": [],
    "quest_b200_end_layer": [],
    "hadamard_transform_cuda_bf16": [_P, _P, _I, _I, _I, _I, _P],
    "quest_b200_test_bounded_wait_cuda": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _LL, _P],
    "quest_b200_device_status": [ctypes.POINTER(ctypes.c_int)],
    "quest_b200_version": [],
}


def lib_path() -> str:
    return _LIB_PATH


def load() -> ctypes.CDLL:
    """Load the library once.  Raises if it has not been built (``python -m quest_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m quest_b200.build` (needs nvcc). "
                "quest_b200 has no CPU or PyTorch fallback.")
        lib = ctypes.CDLL(_LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = ctypes.c_int
        lib.quest_b200_error_string.argtypes = [ctypes.c_int]
        lib.quest_b200_error_string.restype = ctypes.c_char_p
        _lib = lib
    return _lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().quest_b200_error_string(status).decode()
        raise RuntimeError(f"quest_b200.{what} failed: {msg} (status {status})")


def ptr(t: torch.Tensor | None):
    """Device pointer of a tensor, or NULL for None / 0-element tensors."""
    if t is None or t.numel() == 0:
        return None
    return t.data_ptr()


def stream_of(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("quest_b200 ops need CUDA tensors; there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} vs {t.device}")
    return dev


def device_status() -> int:
    """Read and clear the device status word (synchronises). 0 means no kernel reported a problem."""
    v = ctypes.c_int(0)
    check(load().quest_b200_device_status(ctypes.byref(v)), "device_status")
    return v.value
