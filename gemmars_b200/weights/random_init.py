"""Random weights for an architecture, from a configuration and a seed, and the model folder
(config.json, model.safetensors) that holds them.

Every tensor has a generator of its own, seeded from the seed and the tensor's name, so a
tensor's values do not depend on which other tensors exist.  Matrices, the embedding and biases
are N(0, 0.02); norm weights are 1 + N(0, 0.1).  Values are drawn in float32 and stored in
bfloat16 (or kept in float32 when asked, which gives weights that bfloat16 cannot hold).

Reference: the reference has no random-weights mode for models (only LCG data in its kernel
tests, src/kernels.rs:1568-1571).
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..config.registry import resolve_architecture
from .safetensors_io import write_safetensors

_STD = {"matrix": (0.0, 0.02), "bias": (0.0, 0.02), "norm": (1.0, 0.1)}


def _fnv1a(text: str) -> int:
    h = 0xCBF29CE484222325
    for b in text.encode():
        h = ((h ^ b) * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return h


def random_tensor(name: str, shape, kind: str, seed: int, device="cpu", dtype=torch.bfloat16) -> torch.Tensor:
    mean, std = _STD[kind]
    g = torch.Generator(device=device)
    g.manual_seed((_fnv1a(name) ^ (seed * 0x9E3779B97F4A7C15)) & 0x7FFFFFFFFFFFFFFF)
    n = 1
    for s in shape:
        n *= s
    if n > (1 << 28) and torch.device(device).type != "cpu":
        # large tables are drawn in row blocks to bound the float32 staging memory
        out = torch.empty(shape, dtype=dtype, device=device)
        rows = max(1, (1 << 27) // max(1, n // shape[0]))
        for r in range(0, shape[0], rows):
            blk = out[r:r + rows]
            blk.copy_(torch.randn(blk.shape, generator=g, device=device, dtype=torch.float32) * std + mean)
        return out
    t = torch.randn(tuple(shape), generator=g, device=device, dtype=torch.float32) * std + mean
    return t.to(dtype)


def random_weights(raw_config: dict, seed: int, device="cpu", dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """{tensor name: tensor} of a complete random checkpoint of the architecture that
    ``raw_config`` (a config.json object) names."""
    arch = resolve_architecture(raw_config)
    if arch.checkpoint_layout is None:
        raise ValueError(f"architecture {arch.name} does not describe its checkpoint layout")
    cfg = arch.config_class.from_dict(raw_config)
    return {name: random_tensor(name, shape, kind, seed, device, dtype)
            for name, (shape, kind) in arch.checkpoint_layout(cfg).items()}


def write_random_model(folder: str, raw_config: dict, seed: int, dtype=torch.bfloat16) -> str:
    """Writes ``folder/config.json`` and ``folder/model.safetensors`` with random weights."""
    os.makedirs(folder, exist_ok=True)
    tensors = random_weights(raw_config, seed, "cpu", dtype)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(raw_config, f, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed, "generator": "gemmars_b200.random_init"})
    return folder
