"""Shared fixtures.  GPU tests carry ``@pytest.mark.gpu`` and go through the C-ABI library;
everything else runs on the CPU."""
from __future__ import annotations

import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")
BF16_KEYS = ("activation", "weight", "a_scale", "w_scale", "a_dq", "w_dq", "m")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); runs the kernels through the C-ABI")


def load_golden(name: str) -> dict:
    """Load a golden case; bf16 tensors were stored as uint16 bit patterns."""
    raw = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for k in raw.files:
        v = raw[k]
        if k in BF16_KEYS:
            out[k] = torch.from_numpy(v.view(np.int16).copy()).view(torch.bfloat16)
        elif v.shape == ():
            out[k] = v.item()
        else:
            out[k] = torch.from_numpy(v.copy())
    return out


GOLDEN_CASES = ("unit_randn_m64_k768_n96", "outlier_m32_k512_n40")


@pytest.fixture(params=GOLDEN_CASES)
def golden(request):
    return load_golden(request.param)


def make_activations(kind: str, m: int, k: int, seed: int = 0) -> torch.Tensor:
    """Seeded synthetic activations (CPU generator, so the GPU and the oracle see the same bits).

    randn   : N(0,1)                               (reference unit test distribution)
    outlier : N(0,1) with 0.5 % of entries x20      (CPU-runnable single-layer config)
    student : Student-t(nu=4) scaled to unit RMS    (Llama-7B-shaped sweep)
    laplace : Laplace(0,1), 1 % of columns x50      (Hadamard+quantize bandwidth sweep)
    """
    g = torch.Generator().manual_seed(seed)
    if kind == "randn":
        x = torch.randn(m, k, generator=g)
    elif kind == "outlier":
        x = torch.randn(m, k, generator=g)
        x = torch.where(torch.rand(m, k, generator=g) < 0.005, x * 20, x)
    elif kind == "student":
        z = torch.randn(m, k, generator=g)
        chi = torch.randn(4, m, k, generator=g).square().sum(0)
        x = z / (chi / 4).sqrt()
        x = x / x.square().mean().sqrt()
    elif kind == "laplace":
        u = torch.rand(m, k, generator=g) - 0.5
        x = -u.sign() * torch.log1p(-2 * u.abs())
        cols = torch.randperm(k, generator=g)[: max(1, k // 100)]
        x[:, cols] *= 50
    else:
        raise ValueError(kind)
    return x.to(torch.bfloat16)
