"""Random weights for a configuration.

``write_random_model`` writes a model folder (``config.json`` and
``model.safetensors``) from a configuration and a seed; the folder loads like
any checkpoint.  ``random_fetch`` produces the same kind of tensors directly
on a device, for sizes that are not worth a round trip through a file.

Matrices are N(0, std) and vectors (norm weights) 1 + N(0, vector_std), unless a
tensor's spec names another rule (``TensorSpec.init``), each
tensor from a generator seeded by (seed, tensor name) so that a tensor's values
do not depend on which other tensors exist.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Callable, Dict, Optional

import torch

from ..config.base import ModelConfig, get_architecture
from ..models.model import Model
from .safetensors_io import write_safetensors


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def _make(name: str, ts, seed: int, device, dtype: torch.dtype, std: float, vector_std: float) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    shape = tuple(ts.init_arg if d == -1 else d for d in ts.shape)      # (a size the checkpoint decides: the part's choice for random weights)
    if ts.role == "table":
        if ts.init != "distinct_below" or len(ts.shape) != 2 or ts.shape[1] > ts.init_arg:
            raise ValueError(f"{name}: no random rule for this integer table")
        # every row: the first entries of a random order of 0 .. init_arg - 1
        keys = torch.rand((ts.shape[0], ts.init_arg), generator=g, device=device)
        return keys.argsort(dim=1)[:, :ts.shape[1]].to(torch.int32).contiguous()
    if ts.init == "unit_interval":
        return (0.2 + 0.6 * torch.rand(ts.shape, generator=g, device=device, dtype=torch.float32)).to(dtype)
    t = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
    if ts.init == "conv_taps":                         # a short filter: taps that add up to something of the input's size
        t = t / float(ts.shape[-1]) ** 0.5
    elif ts.init == "router":                          # scores that differ from token to token
        t = t / float(ts.shape[-1]) ** 0.5 * 4.0
    elif ts.init == "mix_pair":                        # [x; x0] -> x: near the sum of the two halves' identities
        half = ts.shape[1] // 2
        t = std * t
        eye = torch.eye(ts.shape[0], half, device=device, dtype=torch.float32)
        t[:, :half] += 0.7 * eye
        t[:, half:2 * half] += 0.7 * eye
    elif ts.init == "decay_out":                       # the second step of a decay's projection: logits that differ from token to token
        t = 4.0 * t
    elif ts.init == "decay_bias":                      # logits whose sigmoid lies mostly above one half
        t = 1.0 + t
    elif ts.init == "around_zero":
        t = vector_std * t
    elif ts.role == "vector":
        t = 1.0 + vector_std * t
    else:
        t = std * t
    return t.to(dtype)


def random_fetch(model: Model, seed: int, *, std: float = 0.02, vector_std: float = 0.1,
                 tied: Optional[bool] = None) -> Callable[[str], Optional[torch.Tensor]]:
    """A ``get(name)`` for :meth:`Model.load` that draws each tensor on the
    model's device.  Optional tensors (an untied head) are drawn unless the
    model's spec ties them."""
    table = model.tensor_table()
    dev = model.ctx.device
    store_dtype = model.ctx.dtype

    def get(name: str):
        ts = table.get(name)
        if ts is None:
            return None
        if ts.optional and (ts.init == "absent" or getattr(model.head, "tied", False)):
            return None
        return _make(name, ts, seed, dev, torch.float32 if ts.role == "vector" else store_dtype, std, vector_std)

    return get


def write_random_model(config: ModelConfig, seed: int, out_dir: str, *, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02, vector_std: float = 0.1) -> str:
    """Write ``config.json`` and ``model.safetensors`` under ``out_dir``."""
    arch = get_architecture(config.architecture)
    model = Model(arch.build_spec(config), torch.float32, "cpu")
    tensors: Dict[str, torch.Tensor] = {}
    for name, ts in model.tensor_table().items():
        if ts.optional and (ts.init == "absent" or getattr(model.head, "tied", False)):
            continue
        tensors[name] = _make(name, ts, seed, "cpu", dtype, std, vector_std)
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_json(), f, indent=2)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors)
    return out_dir
