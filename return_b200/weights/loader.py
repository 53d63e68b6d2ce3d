"""Fills a model's parameters from checkpoint tensors by name, or with seeded random numbers.

The reference never touches weight files: it lets Hugging Face load a bfloat16 model and keeps
its modules as containers (rollout/engine_actor.py:14-21), concatenating gate and up
projections afterwards (rollout/monkey_patch/qwen3.py:99-105).  Here the loader reads the
safetensors itself.  A model parameter is filled from one or several checkpoint tensors
(``Source``), concatenated along dim 0.

Dtype rule.  On the bfloat16 path, operands of matrix products are kept in bfloat16, tables of
integers in int32, and a "vector" parameter (a norm weight) that the file stores in 32-bit
stays in 32-bit.  On the float32 path everything is float32.

Errors.  All faults of a checkpoint are gathered and raised as one ``WeightError`` that lists
the missing tensors, the unexpected ones and those of the wrong shape.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from dataclasses import dataclass
from typing import Dict, List, Set, Tuple

import torch

from .safetensors_io import ModelFiles, write_safetensors


@dataclass(frozen=True)
class Source:
    """Checkpoint tensors that make up one parameter: concatenated along dim 0, or, with
    ``interleave`` = b, woven in blocks of b rows (b rows of the first, b of the second, ...)."""
    names: Tuple[str, ...]
    interleave: int = 0


class WeightError(ValueError):
    def __init__(self, missing: List[str], unexpected: List[str], wrong_shape: List[str], other: List[str] = ()):
        self.missing, self.unexpected, self.wrong_shape, self.other = missing, unexpected, wrong_shape, list(other)
        parts = []
        if missing:
            parts.append(f"missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            parts.append(f"unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            parts.append(f"wrong shapes ({len(wrong_shape)}): " + "; ".join(wrong_shape))
        if self.other:
            parts.append("; ".join(self.other))
        super().__init__("checkpoint does not fit the model: " + " | ".join(parts))


def _target_dtype(stored: torch.dtype, role: str, act_dtype: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if act_dtype == torch.float32:
        return torch.float32
    if role == "vector" and stored in (torch.float32, torch.float64):
        return torch.float32
    return act_dtype


def check_checkpoint(expected: Dict[str, Tuple[int, ...]], files, ignorable=frozenset()) -> None:
    """Raises one WeightError unless ``files`` holds exactly the tensors of ``expected`` (checkpoint
    name -> shape), each with its shape.  ``ignorable``: names that may be present without being used;
    given as a map name -> twin, such a tensor must equal its twin (a tied output head saved beside the
    embedding: the reference ties unconditionally, rollout/engine_actor.py:46, so a head that differs
    would be silently lost)."""
    missing = sorted(n for n in expected if n not in files)
    unexpected = sorted(n for n in files.names() if n not in expected and n not in ignorable)
    wrong = [f"{n} is {list(files.shape(n))}, the model wants {list(shape)}"
             for n, shape in expected.items() if n in files and tuple(files.shape(n)) != tuple(shape)]
    other = []
    if isinstance(ignorable, dict):
        for n, twin in ignorable.items():
            if n not in files or twin not in files:
                continue
            if tuple(files.shape(n)) != tuple(files.shape(twin)):
                wrong.append(f"{n} is {list(files.shape(n))}, its twin {twin} is {list(files.shape(twin))}")
            elif files.dtype(n) != files.dtype(twin) or not torch.equal(files.tensor(n), files.tensor(twin)):
                other.append(f"{n} differs from {twin} although the configuration ties them")
    if missing or unexpected or wrong or other:
        raise WeightError(missing, unexpected, wrong, other)


def load_parameters(params: Dict[str, "ParamSpec"], sources: Dict[str, Source],
                    expected: Dict[str, Tuple[int, ...]], model_dir: str, act_dtype: torch.dtype, device,
                    ignorable=frozenset()) -> Dict[str, torch.Tensor]:
    """Every parameter as a device tensor, filled from the model folder's safetensors.

    ``expected``: checkpoint name -> shape, as ``checkpoint_shapes`` derives it."""
    absent = [p for p in params if p not in sources]
    if absent:
        raise WeightError([], [], [], [f"the architecture names no checkpoint tensor for parameters {absent}"])
    files = ModelFiles(model_dir)
    try:
        check_checkpoint(expected, files, ignorable)
        out: Dict[str, torch.Tensor] = {}
        for pname, spec in params.items():
            names = sources[pname].names
            stored = files.dtype(names[0])
            dt = _target_dtype(stored, spec.role, act_dtype)
            dst = torch.empty(spec.shape, dtype=dt, device=device)
            b = sources[pname].interleave
            if b:
                woven = dst.view(-1, len(names), b, *dst.shape[1:])       # [blocks, source, b rows, ...]
                for i, n in enumerate(names):
                    woven[:, i].copy_(files.tensor(n).view(-1, b, *dst.shape[1:]))
            else:
                row = 0
                for n in names:
                    t = files.tensor(n)
                    k = t.shape[0] if t.dim() else 1
                    view = dst[row:row + k] if t.dim() else dst
                    view.copy_(t)
                    row += k
            out[pname] = dst
        return out
    finally:
        files.close()


# ------------------------------------------------------------------------------- random weights

def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(seed: int, name: str, shape, init: str, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """The random value of one named tensor: matrices N(0, 0.02), norm weights 1 + N(0, 0.1).

    Drawn in float32 from a generator seeded by (seed, name), so a tensor's value does not
    depend on which other tensors exist.  CPU and CUDA generators give different streams."""
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    x = torch.randn(tuple(shape), generator=g, dtype=torch.float32, device=device)
    if init == "ones_normal":
        x.mul_(0.1).add_(1.0)
    else:
        x.mul_(0.02)
    return x.to(dtype)


def write_random_model(model_dir: str, config, seed: int, dtype: torch.dtype = torch.float32) -> str:
    """Writes config.json and model.safetensors of a randomly initialised model; returns the folder.

    Every matrix is N(0, 0.02), every norm weight 1 + N(0, 0.1), each drawn from (seed, tensor name).
    A tied output head is not written: it is the embedding."""
    from ..config import registry
    arch = registry.resolve(config.to_dict())
    shapes = checkpoint_shapes(arch, config)
    os.makedirs(model_dir, exist_ok=True)
    cfg = config.to_dict()
    cfg["torch_dtype"] = {torch.float32: "float32", torch.bfloat16: "bfloat16"}[dtype]
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    tensors = [(n, random_tensor(seed, n, shp, init, dtype)) for n, (shp, init) in shapes.items()]
    write_safetensors(os.path.join(model_dir, "model.safetensors"), tensors,
                      metadata={"format": "pt", "seed": seed})
    return model_dir


def checkpoint_shapes(arch, config) -> Dict[str, Tuple[Tuple[int, ...], str]]:
    """Checkpoint tensor name -> (shape, init law), derived from the model's parameters and the
    architecture's sources.  Fused parameters are split by the architecture's ``split_rows``."""
    from ..models.decoder import DecoderModel
    from ..parts.base import BuildEnv
    model = DecoderModel(arch.decoder_spec(config, 8), BuildEnv(torch.float32, torch.device("cpu")))
    params, sources = model.params(), arch.weight_sources(config)
    split = getattr(arch, "split_rows", None)
    out: Dict[str, Tuple[Tuple[int, ...], str]] = {}
    for pname, spec in params.items():
        names = sources[pname].names
        if len(names) == 1:
            out[names[0]] = (tuple(spec.shape), spec.init)
            continue
        rows = split(config, pname) if split else None
        if rows is None:
            if spec.shape[0] % len(names):
                raise ValueError(f"cannot split parameter {pname} evenly over {names}")
            rows = [spec.shape[0] // len(names)] * len(names)
        for n, r in zip(names, rows):
            out[n] = ((r,) + tuple(spec.shape[1:]), spec.init)
    return out


def random_parameters(params: Dict[str, "ParamSpec"], sources: Dict[str, Source],
                      shapes: Dict[str, Tuple[Tuple[int, ...], str]], seed: int, act_dtype: torch.dtype,
                      device) -> Dict[str, torch.Tensor]:
    """Random parameters made on the device, without a model folder: for benchmarks of models too
    large to write out first.  Same laws as ``write_random_model``, but the numbers come from the
    device's generator, so they differ from those of a folder written with the same seed."""
    out: Dict[str, torch.Tensor] = {}
    for pname, spec in params.items():
        dt = act_dtype
        dst = torch.empty(spec.shape, dtype=dt, device=device)
        row = 0                       # random numbers have no order to keep: an interleaved layout is filled the same way
        for n in sources[pname].names:
            shp, init = shapes[n]
            k = shp[0]
            # large matrices are drawn in slabs so that the float32 temporary stays small
            step = max(1, (1 << 26) // max(1, math.prod(shp[1:])))
            for r0 in range(0, k, step):
                r1 = min(k, r0 + step)
                dst[row + r0:row + r1].copy_(random_tensor(seed, f"{n}:{r0}", (r1 - r0,) + tuple(shp[1:]), init, dt, device))
            row += k
        out[pname] = dst
    return out
