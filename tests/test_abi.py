"""CPU checks of the C-ABI boundary: the shared library builds/loads and exports exactly the entry points that
``include/quest_b200.h`` declares; the Python wrappers refuse to run without CUDA tensors (no fallback)."""
from __future__ import annotations

import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT


def declared_functions() -> list[str]:
    text = open(os.path.join(ROOT, "include", "quest_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return re.findall(r"^\s*(?:const\s+char\s*\*|int)\s+(\w+)\s*\(", text, flags=re.M)


def test_header_declares_the_reference_launchers():
    names = declared_functions()
    for ref_name in ("find_scale_int4_cuda_bf16", "quantize_int4_cuda_bf16", "add_mul_vv_cuda_bf16",
                     "matmul_int4_int4t_int32_cuda", "fused_matmul_dequantize_int4_int4t_bf16_cuda",
                     "hadamard_quantize_int4_cuda_bf16"):
        assert ref_name in names


def test_library_exports_every_declared_symbol():
    from quest_b200 import build, _lib
    build.build()
    lib = ctypes.CDLL(_lib.lib_path())
    names = declared_functions()
    assert len(names) >= 10
    for name in names:
        assert hasattr(lib, name), name
    bound = set(_lib.SIGNATURES) | {"quest_b200_error_string"}
    assert bound == set(names), bound ^ set(names)
    assert _lib.load().quest_b200_version() >= 100
    assert b"invalid" in _lib.load().quest_b200_error_string(1)


def test_argument_validation_without_gpu():
    """Validation happens before any CUDA call, so these status codes can be checked on a CPU box."""
    from quest_b200 import _lib
    lib = _lib.load()
    assert lib.find_scale_int4_cuda_bf16(None, None, 128, 4, None) == 1
    assert lib.find_scale_int4_cuda_bf16(None, None, 128, 0, None) == 0          # empty batch is a no-op
    assert lib.hadamard_quantize_int4_cuda_bf16(None, None, None, None, 128, 4, 100, None) == 2  # bad block
    assert lib.hadamard_quantize_int4_cuda_bf16(None, None, None, None, 128, 0, 128, None) == 0
    assert lib.matmul_int4_int4t_int32_cuda(None, None, None, 4, 128, 4, None) == 1
    assert lib.matmul_int4_int4t_int32_cuda(None, None, None, 0, 128, 4, None) == 0
    buf = (ctypes.c_char * 4096)()
    p = ctypes.addressof(buf)
    p += (-p) % 16
    assert lib.matmul_int4_int4t_int32_cuda(p, p, p, 4, 100, 4, None) == 2        # K % 32 != 0
    assert lib.matmul_int4_int4t_int32_cuda(p, p + 1, p, 4, 128, 4, None) == 1    # misaligned operand
    assert lib.quantize_int4_cuda_bf16(p, p, None, p, None, 7, 1, 0, None) == 1   # packed output needs even K
    assert lib.add_mul_vv_cuda_bf16(None, None, None, None, None, None, 0, 8, None) == 0
    # the one-call layer and the block copy validate before they launch, too
    assert lib.w4a4_linear_hadamard_bf16_cuda(p, p, p, p, p, p, p, None, 4, 128, 4, 128, None) == 1     # row sums required
    assert lib.w4a4_linear_hadamard_a8_bf16_cuda(p, p, p, p, p, p, p, None, 4, 128, 4, 128, None) == 1
    dsts = (ctypes.c_void_p * 2)(p + 256, p + 512)
    assert lib.quest_b200_copy_block_to_peers_cuda(p, dsts, 2, 0, 64, 64, None) == 0                      # nothing to copy
    assert lib.quest_b200_copy_block_to_peers_cuda(p, dsts, 8, 4, 64, 64, None) == 1                      # at most 7 destinations
    assert lib.quest_b200_copy_block_to_peers_cuda(p, dsts, 2, 4, 64, 32, None) == 1                      # ld < cols
    assert lib.quest_b200_copy_block_to_peers_cuda(p, dsts, 2, 4, 60, 64, None) == 2                      # not whole 16-byte pieces
    odd = (ctypes.c_void_p * 2)(p + 256, p + 514)
    assert lib.quest_b200_copy_block_to_peers_cuda(p, odd, 2, 4, 64, 64, None) == 2                       # misaligned destination
    # layer mode is host-thread state: begin / end always succeed and leave the ordinary entry points usable
    assert lib.quest_b200_begin_layer() == 0 and lib.quest_b200_end_layer() == 0
    assert lib.matmul_int4_int4t_int32_cuda(None, None, None, 0, 128, 4, None) == 0


def test_no_cpu_fallback():
    import quest_b200 as quest
    x = torch.zeros(2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        quest.find_scale_int4(x)
    with pytest.raises(NotImplementedError):
        quest.matmul_int4sp_int4t_int32()


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "quest_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text, os.path.join(dirpath, f)
