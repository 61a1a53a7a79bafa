"""Seeded synthetic workloads with the shapes, sizes and value distributions of the benchmark
configurations (no external dataset is involved): parameter shapes of the model families, and
gradients N(0, sigma) times a per-row log-normal scale that is fixed across steps, which is what
gives the gradients the block structure the period search detects.
"""
from __future__ import annotations

from typing import List, Tuple

import torch

Shape = Tuple[int, ...]


def gpt2_125m() -> List[Tuple[str, Shape]]:
    """GPT-2 125M parameter set: 148 tensors, 124 439 808 parameters."""
    out = [("wte", (50257, 768)), ("wpe", (1024, 768))]
    for i in range(12):
        out += [
            ("h{}.ln_1.weight".format(i), (768,)), ("h{}.ln_1.bias".format(i), (768,)),
            ("h{}.attn.c_attn.weight".format(i), (768, 2304)), ("h{}.attn.c_attn.bias".format(i), (2304,)),
            ("h{}.attn.c_proj.weight".format(i), (768, 768)), ("h{}.attn.c_proj.bias".format(i), (768,)),
            ("h{}.ln_2.weight".format(i), (768,)), ("h{}.ln_2.bias".format(i), (768,)),
            ("h{}.mlp.c_fc.weight".format(i), (768, 3072)), ("h{}.mlp.c_fc.bias".format(i), (3072,)),
            ("h{}.mlp.c_proj.weight".format(i), (3072, 768)), ("h{}.mlp.c_proj.bias".format(i), (768,)),
        ]
    out += [("ln_f.weight", (768,)), ("ln_f.bias", (768,))]
    return out


def llama(hidden: int, layers: int, q_out: int, kv_out: int, ffn: int, vocab: int) -> List[Tuple[str, Shape]]:
    out = [("embed_tokens", (vocab, hidden))]
    for i in range(layers):
        out += [
            ("l{}.input_norm".format(i), (hidden,)),
            ("l{}.q_proj".format(i), (q_out, hidden)), ("l{}.k_proj".format(i), (kv_out, hidden)),
            ("l{}.v_proj".format(i), (kv_out, hidden)), ("l{}.o_proj".format(i), (hidden, q_out)),
            ("l{}.post_norm".format(i), (hidden,)),
            ("l{}.gate_proj".format(i), (ffn, hidden)), ("l{}.up_proj".format(i), (ffn, hidden)),
            ("l{}.down_proj".format(i), (hidden, ffn)),
        ]
    out += [("lm_head", (vocab, hidden))]
    return out


def llama_1_5b() -> List[Tuple[str, Shape]]:
    """Llama-style 1.5B: 146 tensors, 1 498 480 640 parameters. Stored shapes follow the
    configuration text ("q/o 2048x2048, k/v 2048x512, gate/up 2048x8192, down 8192x2048"): dim 0 is
    the row that carries the gradient scale."""
    out = [("embed_tokens", (128256, 2048))]
    for i in range(16):
        out += [
            ("l{}.input_norm".format(i), (2048,)),
            ("l{}.q_proj".format(i), (2048, 2048)), ("l{}.k_proj".format(i), (2048, 512)),
            ("l{}.v_proj".format(i), (2048, 512)), ("l{}.o_proj".format(i), (2048, 2048)),
            ("l{}.post_norm".format(i), (2048,)),
            ("l{}.gate_proj".format(i), (2048, 8192)), ("l{}.up_proj".format(i), (2048, 8192)),
            ("l{}.down_proj".format(i), (8192, 2048)),
        ]
    out += [("lm_head", (128256, 2048))]
    return out


def llama_32b() -> List[Tuple[str, Shape]]:
    """Llama-style 32B: 542 tensors, 32 528 936 960 parameters."""
    out = [("embed_tokens", (32000, 6656))]
    for i in range(60):
        out += [
            ("l{}.input_norm".format(i), (6656,)),
            ("l{}.q_proj".format(i), (6656, 6656)), ("l{}.k_proj".format(i), (6656, 6656)),
            ("l{}.v_proj".format(i), (6656, 6656)), ("l{}.o_proj".format(i), (6656, 6656)),
            ("l{}.post_norm".format(i), (6656,)),
            ("l{}.gate_proj".format(i), (6656, 17920)), ("l{}.up_proj".format(i), (6656, 17920)),
            ("l{}.down_proj".format(i), (17920, 6656)),
        ]
    out += [("lm_head", (32000, 6656))]
    return out


def qwen3_1_7b_matrices() -> List[Tuple[str, Shape]]:
    """The 2-D matrices of a Qwen3-1.7B-shaped model: 196 matrices, 1 409 286 144 elements."""
    out = []
    for i in range(28):
        out += [
            ("l{}.q_proj".format(i), (2048, 2048)), ("l{}.k_proj".format(i), (2048, 1024)),
            ("l{}.v_proj".format(i), (2048, 1024)), ("l{}.o_proj".format(i), (2048, 2048)),
            ("l{}.gate_proj".format(i), (2048, 6144)), ("l{}.up_proj".format(i), (2048, 6144)),
            ("l{}.down_proj".format(i), (6144, 2048)),
        ]
    return out


def numel(shape: Shape) -> int:
    n = 1
    for s in shape:
        n *= s
    return n


def _gen(device, seed: int, index: int, step: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1_000_000 + 1000 * index + step)
    return g


def init_param(name: str, shape: Shape, index: int, dtype, device, seed: int = 0) -> torch.Tensor:
    """N(0, 0.02); norm weights 1; biases 0."""
    if len(shape) == 1:
        if "norm" in name or ("ln_" in name and name.endswith("weight")):
            return torch.ones(shape, dtype=dtype, device=device)
        if name.endswith("bias"):
            return torch.zeros(shape, dtype=dtype, device=device)
    return (torch.randn(shape, generator=_gen(device, seed, index, 998), device=device) * 0.02).to(dtype)


def row_scale(shape: Shape, index: int, device, tau: float, seed: int = 0) -> torch.Tensor:
    rows = shape[0] if len(shape) == 2 else 1
    return torch.exp(torch.randn(rows, 1, generator=_gen(device, seed, index, 999), device=device) * tau)


def make_grad(shape: Shape, index: int, step: int, dtype, device, sigma: float = 1e-3, tau: float = 1.0,
              seed: int = 0) -> torch.Tensor:
    base = torch.randn(shape, generator=_gen(device, seed, index, step), device=device)
    scale = row_scale(shape, index, device, tau, seed) * sigma
    if len(shape) == 2:
        base.mul_(scale)
    else:
        base.mul_(scale.reshape(()))
    return base.to(dtype)


def step_bytes(shapes, periods, param_bytes: int, state_bytes: int) -> int:
    """Algorithmic HBM bytes of one fused step: gradient read once, parameter read and written,
    code read and written (3s + 2 bytes per element), plus magnitude and second moment read and
    written once per block; period-1 tensors carry a per-element second moment."""
    total = 0
    for (_, shape), period in zip(shapes, periods):
        n = numel(shape)
        total += n * (3 * param_bytes + 2)
        if period == 1:
            total += n * 2 * state_bytes + 2 * state_bytes
        else:
            total += (n // period) * 4 * state_bytes
    return total
