"""State dict of a QuEST-trained model -> packed W4A4 weights for ``Linear4bit``.

A QuEST checkpoint is ``{"model": state_dict, "optimizer": ..., "scheduler": ..., "itr": ...}`` written by
``save_checkpoint`` (src/optim/utils.py:245-257).  The quantised layers are the ``QuantizedLinear`` modules inside the
transformer blocks - ``attn.c_attn``, ``attn.c_proj``, ``mlp.c_fc`` / ``mlp.w1`` / ``mlp.w2``, ``mlp.c_proj``
(src/models/base.py:37-55, 120-131; src/models/llama.py:89-115) - which hold an ordinary ``weight`` (and optional
``bias``); embeddings, norms and ``lm_head`` stay in bf16.  Training applies the Hadamard transform and the 4-bit
quantiser to weights and activations on the fly (``HalfHadamardTrustQuantizer``, src/models/quantization/
base_linear.py:187-215), so serving such a layer is ``Linear4bit(use_hadamard=True)``: the weight goes through
``preprocess_weight`` (Hadamard, scale, int4 codes, packing, row sums) once, here.
"""
from __future__ import annotations

import re
from typing import Iterable, Mapping

import torch
from torch import nn

from .layer import Linear4bit, preprocess_weight

# names of the quantised linears inside a transformer block, as the reference's model classes call them
DEFAULT_PATTERN = r"(^|\.)h\.\d+\.(attn\.(c_attn|c_proj)|mlp\.(c_fc|c_proj|w1|w2))$"
_WRAPPER_PREFIXES = ("module.", "_orig_mod.")


def unwrap_checkpoint(obj: Mapping) -> dict:
    """The model's state dict out of a checkpoint object (or the state dict itself), with the prefixes that
    DistributedDataParallel and torch.compile put in front of every key removed."""
    sd = obj["model"] if "model" in obj and isinstance(obj["model"], Mapping) else obj
    out = {}
    for key, value in sd.items():
        changed = True
        while changed:
            changed = False
            for prefix in _WRAPPER_PREFIXES:
                if key.startswith(prefix):
                    key, changed = key[len(prefix):], True
        out[key] = value
    return out


def quantised_layer_names(state_dict: Mapping, pattern: str = DEFAULT_PATTERN) -> list[str]:
    rx = re.compile(pattern)
    names = []
    for key, value in state_dict.items():
        if key.endswith(".weight") and getattr(value, "dim", lambda: 0)() == 2 and rx.search(key[: -len(".weight")]):
            names.append(key[: -len(".weight")])
    return names


def convert_state_dict(state_dict: Mapping, pattern: str = DEFAULT_PATTERN, device: torch.device | str = "cuda",
                       use_hadamard: bool = True) -> dict:
    """Replaces ``<layer>.weight`` of every quantised linear by ``<layer>.w_int_packed`` (uint8 [N, K/2]),
    ``<layer>.w_scale`` (bf16 [N, 1]) and ``<layer>.w_add`` (int32 [N, 1]); all other entries are passed through
    (cast to bf16 where floating point).  The packing runs on ``device`` with the library's kernels."""
    sd = unwrap_checkpoint(state_dict)
    layers = set(quantised_layer_names(sd, pattern))
    out = {}
    for key, value in sd.items():
        base = key[: -len(".weight")] if key.endswith(".weight") else None
        if base in layers:
            w = value.to(device=device, dtype=torch.bfloat16).contiguous()
            packed, scale, add, _ = preprocess_weight(w, use_hadamard=use_hadamard)
            out[base + ".w_int_packed"], out[base + ".w_scale"], out[base + ".w_add"] = packed, scale, add
        else:
            out[key] = value.to(torch.bfloat16) if torch.is_floating_point(value) else value
    return out


def swap_quantised_linears(model: nn.Module, names: Iterable[str], use_hadamard: bool = True) -> nn.Module:
    """Replaces the named ``nn.Linear``-like submodules of ``model`` (already on a CUDA device) by ``Linear4bit`` built
    from their current weights - the in-place counterpart of ``convert_state_dict`` for a model that has been loaded."""
    for name in names:
        parent_name, _, leaf = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        old = getattr(parent, leaf)
        new = Linear4bit(old.in_features, old.out_features, bias=old.bias is not None, device=old.weight.device,
                         dtype=torch.bfloat16, use_hadamard=use_hadamard, weight=old.weight.data.to(torch.bfloat16))
        if old.bias is not None:
            new.bias.data.copy_(old.bias.data)
        setattr(parent, leaf, new)
    return model


def load_converted(model: nn.Module, converted: Mapping) -> None:
    """Fills the buffers of the ``Linear4bit`` modules of ``model`` (and every other parameter / buffer that has an
    entry) from the output of ``convert_state_dict``."""
    own = dict(model.named_parameters())
    own.update(dict(model.named_buffers()))
    missing = []
    for key, value in converted.items():
        if key in own:
            own[key].data.copy_(value.to(own[key].device))
        else:
            missing.append(key)
    if missing:
        raise KeyError(f"entries without a destination in the model: {missing[:5]}{' ...' if len(missing) > 5 else ''}")
