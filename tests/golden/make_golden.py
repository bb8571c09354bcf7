"""Generate golden vectors by EXECUTING the reference's own CPU baselines.

The reference module gemm-quest/benchmarks/utils.py cannot be imported as a
whole (its top level imports triton, fast_hadamard_transform and the compiled
``quest`` extension and creates a CUDA tensor).  Its four ``*_baseline`` /
helper functions are pure torch, so this script parses the file, compiles only
those function definitions (unmodified source, taken from the reference tree at
run time) and runs them on seeded CPU inputs.  The outputs are written to
``tests/golden/*.npz`` and committed; the tests never need the reference tree.

Usage (in a container that has the reference checked out):
    python tests/golden/make_golden.py /path/to/reference

bf16 tensors are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import ast
import os
import sys

import numpy as np
import torch

WANTED = ("find_scale_int4_baseline", "quantize_int4_baseline", "unpack_int4", "add_mul_vv_baseline")
HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference_functions(ref_root: str) -> dict:
    path = os.path.join(ref_root, "gemm-quest", "benchmarks", "utils.py")
    src = open(path).read()
    tree = ast.parse(src)
    keep = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in WANTED]
    assert sorted(n.name for n in keep) == sorted(WANTED), [n.name for n in keep]
    module = ast.Module(body=keep, type_ignores=[])
    ns = {"torch": torch}
    exec(compile(module, path, "exec"), ns)
    return {k: ns[k] for k in WANTED}


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def make_case(fn: dict, name: str, activation: torch.Tensor, weight: torch.Tensor) -> None:
    """Mirror of the dense part of the reference's _unit_test
    (gemm-quest/benchmarks/utils.py:626-688) with backend='pytorch'."""
    out = {"activation": bits(activation), "weight": bits(weight)}
    res = {}
    for tag, x in (("a", activation), ("w", weight)):
        rows, k = x.shape
        scale = torch.empty(rows, 1, dtype=x.dtype)
        fn["find_scale_int4_baseline"](x, scale)
        x_int = torch.empty(rows, k, dtype=torch.int8)
        x_packed = torch.empty(rows, k // 2, dtype=torch.uint8)
        x_row_sum = torch.empty(rows, 1, dtype=torch.int32)
        x_dq = x.clone()
        fn["quantize_int4_baseline"](x_dq, scale, x_int, x_packed, x_row_sum, True)
        assert fn["unpack_int4"](x_packed).equal(x_int)
        res[tag] = (scale, x_int, x_packed, x_row_sum, x_dq)
        out[f"{tag}_scale"] = bits(scale)
        out[f"{tag}_int"] = bits(x_int)
        out[f"{tag}_int_packed"] = bits(x_packed)
        out[f"{tag}_int_row_sum"] = bits(x_row_sum)
        out[f"{tag}_dq"] = bits(x_dq)
    a_scale, a_int, a_packed, a_row_sum, _ = res["a"]
    w_scale, w_int, w_packed, w_row_sum, _ = res["w"]
    k = activation.size(1)
    c_ref = (a_int.to(torch.float64) @ w_int.to(torch.float64).t()).to(torch.int32)  # utils.py:680
    w_add = w_int.to(torch.int32).sum(dim=-1, keepdim=True).to(torch.int32) + k // 2  # utils.py:682
    m = torch.empty(c_ref.shape, dtype=a_scale.dtype)
    fn["add_mul_vv_baseline"](a_row_sum, a_scale, w_add, w_scale, c_ref, m)
    # the fp64 identity of utils.py:667-678, 684
    a_dq64 = (a_int.to(torch.float64) + .5) * a_scale.to(torch.float64)
    w_dq64 = (w_int.to(torch.float64) + .5) * w_scale.to(torch.float64)
    m_ref = a_dq64 @ w_dq64.t()
    out["c_ref"] = bits(c_ref)
    out["w_add"] = bits(w_add)
    out["m"] = bits(m)
    out["m_equals_fp64_ref"] = np.array(bool(m.equal(m_ref.to(torch.bfloat16))))
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **out)
    print(name, {k: v.shape for k, v in out.items()}, "m==fp64 ref:", bool(out["m_equals_fp64_ref"]))


def main() -> None:
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("QUEST_REFERENCE_ROOT")
    if not ref_root:
        sys.exit("usage: make_golden.py <path of the reference checkout>  (or set QUEST_REFERENCE_ROOT)")
    fn = load_reference_functions(ref_root)

    g = torch.Generator().manual_seed(0)
    # same distribution as the reference's _get_random_inputs (randn, bf16), CPU generator
    weight = torch.randn(96, 768, generator=g).to(torch.bfloat16)
    activation = torch.randn(64, 768, generator=g).to(torch.bfloat16)
    make_case(fn, "unit_randn_m64_k768_n96", activation, weight)

    # outliers, clipping rows, an all-zero row, a constant row
    g = torch.Generator().manual_seed(1)
    activation = torch.randn(32, 512, generator=g)
    mask = torch.rand(32, 512, generator=g) < 0.005
    activation = torch.where(mask, activation * 20, activation)
    activation[3] = 0
    activation[4] = 1.0
    activation[5, ::7] *= 1e3
    activation = activation.to(torch.bfloat16)
    weight = (0.02 * torch.randn(40, 512, generator=g)).to(torch.bfloat16)
    make_case(fn, "outlier_m32_k512_n40", activation, weight)


if __name__ == "__main__":
    main()
