"""Random weights: write a model folder from a configuration and a seed, or fill a
model on the device directly (for measurements at sizes one would not write to disk).

Distribution: matrices and embeddings N(0, 0.02), norm weights 1 + U(-0.1, 0.1),
"zeros" parameters 0.  tinyserve has no such mode; it always loads a checkpoint
(serve.py:1289-1404)."""
from __future__ import annotations

import json
import os

import torch
from safetensors.torch import save_file

from .loader import expected_tensors

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def _draw(init: str, shape, generator, device="cpu"):
    if init == "normal":
        return torch.empty(shape, dtype=torch.float32, device=device).normal_(0.0, 0.02, generator=generator)
    if init == "norm_weight":
        return 1.0 + torch.empty(shape, dtype=torch.float32, device=device).uniform_(-0.1, 0.1, generator=generator)
    if init == "zeros":
        return torch.zeros(shape, dtype=torch.float32, device=device)
    raise ValueError(f"unknown init {init!r}")


def write_random_model(config, out_dir: str, seed: int = 0, store_dtype: str = "bfloat16",
                       vector_dtype: str | None = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (a ModelConfig).

    Tensors are drawn on the CPU from one generator seeded with ``seed``, in the model's
    fixed tensor order, in 32-bit, then stored as ``store_dtype``; ``vector_dtype`` (default:
    the same) is the storage type of norm weights and other vectors."""
    from ..parts.model import build_model
    model = build_model(config)
    gen = torch.Generator(device="cpu")
    gen.manual_seed(int(seed))
    mat_dtype = _STORE[store_dtype]
    vec_dtype = _STORE[vector_dtype or store_dtype]
    tensors = {}
    for e in expected_tensors(model):
        value = _draw(e.spec.init, e.shape, gen)
        if e.spec.role == "int_table":
            value = value.to(torch.int32)
        else:
            value = value.to(vec_dtype if e.spec.role == "vector" else mat_dtype)
        tensors[e.name] = value.contiguous()
    os.makedirs(out_dir, exist_ok=True)
    raw = config.to_dict()
    raw["torch_dtype"] = store_dtype
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(raw, fh, indent=1)
    save_file(tensors, os.path.join(out_dir, "model.safetensors"), metadata={"format": "pt"})
    return out_dir


def fill_random_on_device(model, dtype: torch.dtype, device, seed: int = 0) -> int:
    """Give every part of ``model`` random tensors made on ``device``; returns bytes."""
    gen = torch.Generator(device=device)
    gen.manual_seed(int(seed))
    total = 0
    for part in model.named_parts():
        bound = {}
        for local, spec in part.param_specs().items():
            if spec.role == "int_table":
                value = torch.zeros(spec.shape, dtype=torch.int32, device=device)
            else:
                value = _draw(spec.init, spec.shape, gen, device).to(dtype)
            bound[local] = value
            total += value.numel() * value.element_size()
        part.bind(bound)
    return total
