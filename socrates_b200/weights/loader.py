"""Read a model folder's tensors by checkpoint name.

The reference downloads an index and every shard from the hub, strips a leading
"model." and loads strictly (model/qwen/qwen_kv_cont.py:35-42,
model/inference_paged.py:72-76).  Here the folder is local (`model.safetensors`, or
`model.safetensors.index.json` with its shards), the names are used as they are in the
file, and every problem with the file is reported in ONE error that lists missing
tensors, unexpected tensors and wrong shapes.

Dtypes: a matrix stored as bfloat16 stays bfloat16 in the bfloat16 engine and is
widened (exactly) in the float32 engine; a tensor stored in 32-bit stays 32-bit;
gains are always held as float32 (widening bfloat16 is exact); integer tables become
int32.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Mapping

import torch

from ..parts.base import ParamSpec


class WeightsError(RuntimeError):
    """The tensors in a model folder do not match what the model needs."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)


def _open_files(model_dir: Path):
    from safetensors import safe_open
    index = model_dir / "model.safetensors.index.json"
    single = model_dir / "model.safetensors"
    if index.exists():
        weight_map = json.loads(index.read_text())["weight_map"]
        files = sorted(set(weight_map.values()))
    elif single.exists():
        files = [single.name]
    else:
        raise WeightsError(f"{model_dir} holds neither model.safetensors nor model.safetensors.index.json")
    return [safe_open(str(model_dir / f), framework="pt") for f in files]


def _short(names, limit=12):
    names = list(names)
    more = f" ... and {len(names) - limit} more" if len(names) > limit else ""
    return ", ".join(names[:limit]) + more


def load_weights(model_dir, expected: Mapping[str, ParamSpec], dtype: torch.dtype,
                 device="cuda", duplicates: Mapping[str, str] = {}) -> Dict[str, torch.Tensor]:
    """Tensors named by `expected`, checked and moved to `device`.

    `dtype` is the engine's dtype (bfloat16 or float32).  Raises WeightsError naming
    every missing tensor, every tensor no part asked for, and every shape that differs.

    `duplicates` names tensors a file may hold beside the one the model reads: {name in the
    file: the expected tensor it must repeat}, e.g. `lm_head.weight` beside a tied
    embedding.  Such a tensor is accepted only if it equals the other bit for bit; a copy
    that differs is reported with the unexpected tensors, because the file then says
    something else than config.json about what the model is.
    """
    model_dir = Path(model_dir)
    handles = _open_files(model_dir)
    where = {}
    for h in handles:
        for k in h.keys():
            where[k] = h
    missing = [n for n in expected if n not in where]
    unexpected = []
    for n in where:
        if n in expected:
            continue
        same_as = duplicates.get(n)
        if same_as in where and same_as in expected:
            a, b = where[n].get_tensor(n), where[same_as].get_tensor(same_as)
            if a.shape == b.shape and a.dtype == b.dtype and torch.equal(a, b):
                continue                                    # a faithful copy: nothing to read from it
            unexpected.append(f"{n} (differs from {same_as}, which it should repeat)")
        else:
            unexpected.append(n)
    wrong_shape, wrong_dtype = [], []
    for n, spec in expected.items():
        if n in where:
            sl = where[n].get_slice(n)
            shape = tuple(sl.get_shape())
            if shape != tuple(spec.shape):
                wrong_shape.append(f"{n}: file has {shape}, model needs {tuple(spec.shape)}")
            st_dtype = sl.get_dtype()
            if spec.role in ("matrix", "gain") and st_dtype not in ("BF16", "F32", "F16"):
                wrong_dtype.append(f"{n}: stored as {st_dtype}, a floating-point tensor is needed")
    if missing or unexpected or wrong_shape or wrong_dtype:
        parts = []
        if missing:
            parts.append(f"{len(missing)} missing: {_short(missing)}")
        if unexpected:
            parts.append(f"{len(unexpected)} unexpected: {_short(unexpected)}")
        if wrong_shape:
            parts.append(f"{len(wrong_shape)} with wrong shape: {_short(wrong_shape)}")
        if wrong_dtype:
            parts.append(f"{len(wrong_dtype)} with wrong dtype: {_short(wrong_dtype)}")
        raise WeightsError(f"{model_dir}: tensors do not match the model; " + "; ".join(parts),
                           missing, unexpected, wrong_shape, wrong_dtype)

    out: Dict[str, torch.Tensor] = {}
    for n, spec in expected.items():
        t = where[n].get_tensor(n)
        out[n] = place(t, spec, dtype, device)
    return out


def place(t: torch.Tensor, spec: ParamSpec, dtype: torch.dtype, device) -> torch.Tensor:
    """One tensor in the dtype the engine holds it in, on the device."""
    if spec.role == "gain":
        target = torch.float32
    elif spec.role == "int":
        target = torch.int32
    elif t.dtype == torch.float32:
        target = torch.float32          # stored in 32-bit: stays so
    else:
        target = dtype                  # bfloat16 stays; float32 engine widens it exactly
    return t.to(device=device, dtype=target).contiguous()
