"""Binding a checkpoint's tensors to what a model's parts ask for, by tensor name.

The parts of a plan say which tensors they want and with which shapes; ``load_checkpoint``
checks the whole checkpoint against that list before it copies anything and raises ONE error
that lists every missing tensor, every unexpected tensor and every wrong shape.

Reference: the reference checks tensor by tensor and stops at the first problem
(``missing tensor X`` src/qwen.rs:364, ``tensor X has shape …, expected …`` src/qwen.rs:365-367,
src/model.rs:282-285); the messages here keep those words.
"""
from __future__ import annotations

import fnmatch
from typing import Dict, Iterable, Optional, Tuple

import torch

from .safetensors_io import ModelFiles, kept_dtype


class WeightError(ValueError):
    """A checkpoint that does not fit the model.  ``missing``, ``unexpected`` and ``wrong_shape``
    hold the details the message lists."""

    def __init__(self, missing, unexpected, wrong_shape, where=""):
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)
        lines = [f"checkpoint {where} does not fit the model:".replace("  ", " ")]
        for n in self.missing:
            lines.append(f"  missing tensor {n}")
        for n, got, want in self.wrong_shape:
            lines.append(f"  tensor {n} has shape {list(got)}, expected {list(want)}")
        for n in self.unexpected:
            lines.append(f"  unexpected tensor {n}")
        super().__init__("\n".join(lines))


def check_checkpoint(available: Dict[str, Tuple[int, ...]], expected: Dict[str, Tuple[int, ...]],
                     ignored: Iterable[str] = (), where: str = "") -> None:
    """Raises ``WeightError`` unless ``available`` ({name: shape}) holds exactly the expected
    tensors with the expected shapes, apart from names matching an ``ignored`` pattern."""
    ignored = list(ignored)
    missing = sorted(n for n in expected if n not in available)
    wrong = sorted((n, available[n], tuple(expected[n])) for n in expected
                   if n in available and tuple(available[n]) != tuple(expected[n]))
    unexpected = sorted(n for n in available if n not in expected
                        and not any(fnmatch.fnmatchcase(n, pat) for pat in ignored))
    if missing or wrong or unexpected:
        raise WeightError(missing, unexpected, wrong, where)


def load_checkpoint(files: ModelFiles, expected: Dict[str, Tuple[int, ...]], ignored: Iterable[str] = (),
                    device: Optional[torch.device] = None) -> Dict[str, torch.Tensor]:
    """{name: tensor on ``device``} for every expected tensor, each in the precision it is kept
    in (bfloat16 stays bfloat16, 32-bit stays 32-bit, float16 widens, integers become int32)."""
    available = {n: files.info(n)[1] for n in files.names()}
    check_checkpoint(available, expected, ignored, where=files.folder)
    out = {}
    for n in expected:
        t = files.tensor(n)
        keep = kept_dtype(t.dtype)
        if device is not None and torch.device(device).type != "cpu":
            t = t.to(device, non_blocking=False)
        t = t.to(keep) if t.dtype != keep else t
        out[n] = t.clone() if t.device.type == "cpu" else t
    return out
