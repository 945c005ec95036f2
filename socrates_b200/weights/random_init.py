"""Random weights: a model folder (config.json, model.safetensors) from a
configuration and a seed.

Matrices and the embedding are drawn from N(0, 0.02), gains from 1 + N(0, 0.1) (the
reference's own test fixture draws matrices from 0.5*N(0,1) and vectors from
1 + 0.2*N(0,1), tests/tiny.py:24-32).  Matrices are stored as bfloat16, so the
bfloat16 and the float32 engine read exactly the same values; gains are stored as
float32.  Each tensor has a generator of its own, seeded from (seed, name), so the
values do not depend on the order of creation.
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from ..parts.base import ParamSpec


def _generator(seed: int, name: str) -> torch.Generator:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    g = torch.Generator(device="cpu")
    g.manual_seed(int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF)
    return g


def random_tensors(expected: Mapping[str, ParamSpec], seed: int,
                   matrix_dtype: torch.dtype = torch.bfloat16) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    for name, spec in expected.items():
        g = _generator(seed, name)
        if spec.init == "gain":
            out[name] = (1.0 + 0.1 * torch.randn(spec.shape, generator=g)).to(torch.float32)
        elif spec.init == "normal":
            out[name] = (0.02 * torch.randn(spec.shape, generator=g)).to(matrix_dtype)
        else:
            raise ValueError(f"{name}: unknown init {spec.init!r}")
    return out


def write_model_folder(config, seed: int, out_dir, matrix_dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write `<out_dir>/config.json` and `<out_dir>/model.safetensors` with random weights."""
    from safetensors.torch import save_file

    from ..engine.model import Model

    out_dir = Path(out_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    model = Model(config.plan())
    tensors = random_tensors(model.parameters(), seed, matrix_dtype)
    (out_dir / "config.json").write_text(json.dumps(config.to_dict(), indent=1))
    save_file(tensors, str(out_dir / "model.safetensors"))
    return out_dir


def random_tensors_on_device(expected: Mapping[str, ParamSpec], seed: int, dtype: torch.dtype,
                             device) -> Dict[str, torch.Tensor]:
    """The same distributions drawn on the device, for models too large to draw on the
    host in reasonable time (benchmarks).  Values differ from `random_tensors`."""
    g = torch.Generator(device=device)
    out: Dict[str, torch.Tensor] = {}
    for i, (name, spec) in enumerate(expected.items()):
        g.manual_seed(seed * 1000003 + i)
        if spec.init == "gain":
            out[name] = 1.0 + 0.1 * torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32)
        else:
            t = torch.empty(spec.shape, device=device, dtype=dtype)
            t.normal_(0.0, 0.02, generator=g)
            out[name] = t
    return out
