"""Host-side logic of the checkpoint converter (no GPU): key handling and layer selection."""
from __future__ import annotations

import torch

from quest_b200 import convert


def _state_dict():
    return {
        "module._orig_mod.transformer.wte.weight": torch.zeros(8, 4),
        "module._orig_mod.transformer.h.0.ln_1.weight": torch.zeros(4),
        "module._orig_mod.transformer.h.0.attn.c_attn.weight": torch.zeros(12, 4),
        "module._orig_mod.transformer.h.0.attn.c_proj.weight": torch.zeros(4, 4),
        "module._orig_mod.transformer.h.0.mlp.w1.weight": torch.zeros(6, 4),
        "module._orig_mod.transformer.h.0.mlp.w2.weight": torch.zeros(6, 4),
        "module._orig_mod.transformer.h.0.mlp.c_proj.weight": torch.zeros(4, 6),
        "module._orig_mod.transformer.h.0.mlp.c_proj.bias": torch.zeros(4),
        "module._orig_mod.transformer.h.11.mlp.c_fc.weight": torch.zeros(16, 4),
        "module._orig_mod.lm_head.weight": torch.zeros(8, 4),
    }


def test_unwrap_checkpoint_strips_wrapper_prefixes():
    sd = convert.unwrap_checkpoint({"model": _state_dict(), "optimizer": {}, "itr": 3})
    assert "transformer.wte.weight" in sd and all(not k.startswith(("module.", "_orig_mod.")) for k in sd)
    assert convert.unwrap_checkpoint(_state_dict()).keys() == sd.keys()


def test_only_the_block_linears_are_selected():
    names = convert.quantised_layer_names(convert.unwrap_checkpoint(_state_dict()))
    assert names == ["transformer.h.0.attn.c_attn", "transformer.h.0.attn.c_proj", "transformer.h.0.mlp.w1",
                     "transformer.h.0.mlp.w2", "transformer.h.0.mlp.c_proj", "transformer.h.11.mlp.c_fc"]
    # a custom pattern, e.g. to include the output head
    assert "lm_head" in convert.quantised_layer_names(convert.unwrap_checkpoint(_state_dict()), r"lm_head$")
