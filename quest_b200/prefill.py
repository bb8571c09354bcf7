"""End-to-end prefill of a Llama-style decoder whose linears run the W4A4 kernels.

The caller of the hot path in the reference: gemm-quest/benchmarks/bench_e2e.py:73-121 builds the model of
src/models/llama.py (RMSNorm -> c_attn -> RoPE -> causal SDPA -> c_proj; RMSNorm -> SiLU(w1 x) * w2 x -> c_proj),
swaps every linear under ``model.transformer`` for ``Linear4bit`` and times one forward pass, eagerly and as a
CUDA graph.  This module provides the same three pieces: a shape-donor decoder with random-init weights (attention
stays bf16 torch SDPA, the lm_head is outside ``transformer`` and is not executed, as in the reference call
``model(idx)`` without logits), the module swap, and the timing harness.
"""
from __future__ import annotations

import dataclasses
import math

import torch
import torch.nn.functional as F
from torch import nn

import quest_b200 as quest
from .layer import HADAMARD_BLOCK, Linear4bit
from .workspace import default_cache

FUSED_MODES = ("int4_fused",)  # modes in which the quantiser is fused into the producer of each linear's input


@dataclasses.dataclass
class DecoderConfig:
    n_embd: int = 2048
    n_layer: int = 16
    n_head: int = 16
    ffn: int = 5632
    vocab_size: int = 32000
    sequence_length: int = 1024
    rmsnorm_eps: float = 1e-5


def rope_table(head_dim: int, length: int, theta: float = 10000.0) -> torch.Tensor:
    """(length, head_dim/2, 2) cos/sin table (src/models/llama.py:17-24)."""
    freqs = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    ang = torch.outer(torch.arange(length).float(), freqs)
    return torch.stack((ang.cos(), ang.sin()), dim=-1)


def apply_rope(q: torch.Tensor, k: torch.Tensor, table: torch.Tensor):
    """Rotate interleaved pairs of q, k (B, T, nh, hs) by the table rows 0..T-1 (src/models/llama.py:43-62)."""
    def rot(x):
        xf = x.float().unflatten(-1, (-1, 2))
        c, s = table[None, : x.size(1), None, :, 0], table[None, : x.size(1), None, :, 1]
        out = torch.stack((xf[..., 0] * c - xf[..., 1] * s, xf[..., 0] * s + xf[..., 1] * c), dim=-1)
        return out.flatten(-2).to(x.dtype)
    return rot(q), rot(k)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).type_as(x) * self.weight


class Attention(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.n_head, self.n_embd = cfg.n_head, cfg.n_embd
        self.c_attn = nn.Linear(cfg.n_embd, 3 * cfg.n_embd, bias=False)
        self.c_proj = nn.Linear(cfg.n_embd, cfg.n_embd, bias=False)

    def forward(self, x, table):
        B, T, C = x.shape
        q, k, v = self.c_attn(x).split(self.n_embd, dim=2)
        q, k = apply_rope(q.view(B, T, self.n_head, -1), k.view(B, T, self.n_head, -1), table)
        v = v.view(B, T, self.n_head, -1)
        y = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        return self.c_proj(y.transpose(1, 2).contiguous().view(B, T, C))


class MLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.w1 = nn.Linear(cfg.n_embd, cfg.ffn, bias=False)
        self.w2 = nn.Linear(cfg.n_embd, cfg.ffn, bias=False)
        self.c_proj = nn.Linear(cfg.ffn, cfg.n_embd, bias=False)

    def forward(self, x):
        return self.c_proj(F.silu(self.w1(x)) * self.w2(x))


class Block(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.ln_1, self.attn = RMSNorm(cfg.n_embd, cfg.rmsnorm_eps), Attention(cfg)
        self.ln_2, self.mlp = RMSNorm(cfg.n_embd, cfg.rmsnorm_eps), MLP(cfg)

    def forward(self, x, table):
        if getattr(self, "fused", False):
            return self.forward_fused(x, table)
        x = x + self.attn(self.ln_1(x), table)
        return x + self.mlp(self.ln_2(x))

    def forward_fused(self, x, table):
        """The same block with every quantiser fused into the producer of its input: RMSNorm -> quantise is one kernel
        (its result feeds c_attn, and w1 and w2 share one quantisation), SiLU(w1 x) * w2 x -> quantise is one kernel.
        Needs W4A4 linears with the Hadamard transform (swap_linears(..., 'int4_fused'))."""
        B, T, C = x.shape

        def ws(m, k):
            w = default_cache.get(m, k, x.device, x.dtype)
            return dict(x_int_packed=w["_a_int_packed"], scale=w["_a_scale"], x_int_row_sum=w["_a_int_row_sum"])

        flat = x.reshape(-1, C)
        q = quest.rmsnorm_hadamard_quantize_int4(flat, self.ln_1.weight, self.ln_1.eps, HADAMARD_BLOCK, **ws(flat.size(0), C))
        att = self.attn
        qkv = att.c_attn.forward_quantized(*q).view(B, T, 3 * C)
        qh, kh, vh = qkv.split(C, dim=2)
        qh, kh = apply_rope(qh.view(B, T, att.n_head, -1), kh.view(B, T, att.n_head, -1), table)
        vh = vh.view(B, T, att.n_head, -1)
        y = F.scaled_dot_product_attention(qh.transpose(1, 2), kh.transpose(1, 2), vh.transpose(1, 2), is_causal=True)
        x = x + att.c_proj(y.transpose(1, 2).contiguous().view(B, T, C))
        flat = x.reshape(-1, C)
        q = quest.rmsnorm_hadamard_quantize_int4(flat, self.ln_2.weight, self.ln_2.eps, HADAMARD_BLOCK, **ws(flat.size(0), C))
        gate = self.mlp.w1.forward_quantized(*q)
        up = self.mlp.w2.forward_quantized(*q)
        q = quest.silu_mul_hadamard_quantize_int4(gate, up, HADAMARD_BLOCK, **ws(gate.size(0), gate.size(1)))
        return x + self.mlp.c_proj.forward_quantized(*q).view(B, T, C)


class Decoder(nn.Module):
    """``transformer`` holds everything that is executed; ``lm_head`` exists but prefill timing stops at ln_f."""

    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.transformer = nn.ModuleDict(dict(
            wte=nn.Embedding(cfg.vocab_size, cfg.n_embd),
            h=nn.ModuleList([Block(cfg) for _ in range(cfg.n_layer)]),
            ln_f=RMSNorm(cfg.n_embd, cfg.rmsnorm_eps)))
        self.lm_head = nn.Linear(cfg.n_embd, cfg.vocab_size, bias=False)
        self.register_buffer("rope", rope_table(cfg.n_embd // cfg.n_head, cfg.sequence_length), persistent=False)
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, mean=0.0, std=0.02)

    def forward(self, idx: torch.Tensor) -> torch.Tensor:
        x = self.transformer.wte(idx)
        for blk in self.transformer.h:
            x = blk(x, self.rope)
        return self.transformer.ln_f(x)


def swap_linears(model: Decoder, mode: str = "int4", use_hadamard: bool = True) -> Decoder:
    """Replace every nn.Linear under ``model.transformer`` (gemm-quest/benchmarks/bench_e2e.py:79-96).
    mode: 'bf16' (leave as is), 'int4' (W4A4 kernels, weights quantised from the current ones), 'int4_fused' (the same
    linears, with every activation quantiser fused into the kernel that produces the linear's input), 'noop'."""
    if mode == "bf16":
        return model
    if mode not in ("int4", "noop") + FUSED_MODES:
        raise NotImplementedError(mode)
    if mode in FUSED_MODES and not use_hadamard:
        raise ValueError("the producer-fused quantisers include the Hadamard transform")
    targets = [(name, m) for name, m in model.transformer.named_modules() if isinstance(m, nn.Linear)]
    for name, m in targets:
        new = Linear4bit(m.in_features, m.out_features, bias=m.bias is not None, device=m.weight.device,
                         dtype=m.weight.dtype, use_hadamard=use_hadamard, use_noop=(mode == "noop"), weight=m.weight.data)
        model.transformer.set_submodule(name, new)
    for blk in model.transformer.h:
        blk.fused = mode in FUSED_MODES
    return model


@torch.inference_mode()
def prefill_time(model: Decoder, batch_size: int, seq_len: int, n_warmup: int = 5, n_iter: int = 10, seed: int = 0):
    """(eager_ms, graph_ms) of one forward over uniform random token ids, CUDA-event timed
    (gemm-quest/benchmarks/bench_e2e.py:98-121 takes the minimum of the two)."""
    dev = next(model.parameters()).device
    g = torch.Generator(device="cpu").manual_seed(seed)
    idx = torch.randint(0, model.cfg.vocab_size, (batch_size, seq_len), generator=g).to(dev)

    def run_timed(fn):
        for _ in range(n_warmup):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(n_iter):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record(); fn(); e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2]

    eager_ms = run_timed(lambda: model(idx))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            model(idx)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = model(idx)
    graph_ms = run_timed(graph.replay)
    return eager_ms, graph_ms, out
