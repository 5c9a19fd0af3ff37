"""Weights of a model folder, taken by tensor name and checked against what the model expects.

The reference looks names up in a manifest and exits on the first missing one,
without checking shapes or dtypes (src/include/qwen_loader.h:61-65, :52).  Here
every problem of a folder is gathered into one `WeightError`: missing tensors,
unexpected tensors and wrong shapes together.  Tensors that a checkpoint may carry
without the model using them - names the architecture declares as such (a buffer
of rotation frequencies; the copy of the embedding that the reference's exporter
stores as `lm_head.weight` beside a tied head, tools/dump_weights.py:24-26) - are
left alone and reported as a warning; with `strict=False` so is every other
tensor the model does not use.

Storage policy: 16-bit floating tensors are kept in bfloat16; a tensor stored
in 32-bit floating point stays 32-bit; integer tables become int32.  What a
part makes of its tensors afterwards (a matrix cast to the compute type, a norm
weight widened to float32) is the part's business.
"""
from __future__ import annotations

import fnmatch
import json
import os
import sys
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile

FLOAT = "float"
INTEGER = "int"


class WeightError(ValueError):
    """A model folder whose tensors do not fit the model; the message lists every fault."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_kind=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_kind = list(wrong_kind)


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one checkpoint tensor."""
    shape: Tuple[int, ...]
    kind: str = FLOAT          # FLOAT or INTEGER
    optional: bool = False     # an absent optional tensor is not an error (a tied output matrix)


def _normalise(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.to(torch.bfloat16)
    if t.dtype in (torch.float32, torch.float64):
        return t.to(torch.float32)
    return t.to(torch.int32)


def _open_files(folder: str) -> List[SafetensorsFile]:
    index = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    try:
        if os.path.isfile(single):
            return [SafetensorsFile(single)]
        if os.path.isfile(index):
            with open(index, "r", encoding="utf-8") as fh:
                names = sorted(set(json.load(fh)["weight_map"].values()))
            absent = [n for n in names if not os.path.isfile(os.path.join(folder, n))]
            if absent:
                raise WeightError(f"{folder}: model.safetensors.index.json names files that are not there: " + ", ".join(absent))
            return [SafetensorsFile(os.path.join(folder, n)) for n in names]
    except SafetensorsError as exc:
        raise WeightError(str(exc)) from None
    raise WeightError(f"{folder}: neither model.safetensors nor model.safetensors.index.json found")


def load_tensors(folder: str, specs: Mapping[str, TensorSpec], *, strict: bool = True, ignorable: Sequence[str] = (),
                 ignored: Optional[List[str]] = None) -> Dict[str, torch.Tensor]:
    """Returns `{name: CPU tensor}` for every expected tensor that the folder holds.

    Raises one `WeightError` naming all missing tensors, all unexpected tensors,
    all tensors of wrong shape and all tensors of the wrong kind.  A tensor the model does
    not use is unexpected unless its name matches one of the `ignorable` patterns (shell
    style) or `strict` is off; those are skipped, named on standard error and appended to
    `ignored` if a list is given.
    """
    files = _open_files(folder)
    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.names():
            where[name] = f
    missing = [n for n, s in specs.items() if n not in where and not s.optional]
    extra = sorted(n for n in where if n not in specs)
    skipped = [n for n in extra if not strict or any(fnmatch.fnmatchcase(n, pattern) for pattern in ignorable)]
    unexpected = [n for n in extra if n not in skipped]
    wrong_shape, wrong_kind = [], []
    for name, spec in specs.items():
        if name not in where:
            continue
        f = where[name]
        if tuple(f.shape(name)) != tuple(spec.shape):
            wrong_shape.append((name, tuple(spec.shape), tuple(f.shape(name))))
        is_float = f.dtype(name).is_floating_point
        if is_float != (spec.kind == FLOAT):
            wrong_kind.append((name, spec.kind, str(f.dtype(name))))
    if missing or unexpected or wrong_shape or wrong_kind:
        lines = [f"{folder}: the checkpoint does not fit the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} found {list(g)}" for n, e, g in wrong_shape))
        if wrong_kind:
            lines.append(f"  wrong kinds ({len(wrong_kind)}): " + ", ".join(
                f"{n} expected {k} found {d}" for n, k, d in wrong_kind))
        raise WeightError("\n".join(lines), missing, unexpected, wrong_shape, wrong_kind)
    if skipped:
        print(f"[kvcache_b200] {folder}: {len(skipped)} tensors the model does not use are left alone: "
              + ", ".join(skipped[:8]) + (" ..." if len(skipped) > 8 else ""), file=sys.stderr)
        if ignored is not None:
            ignored.extend(skipped)
    out = {name: _normalise(where[name].tensor(name)) for name in specs if name in where}
    for f in files:
        f.close()
    return out
