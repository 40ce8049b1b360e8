"""Binding checkpoint tensors to the parameters a model declares.

The reference binds GGUF tensors by name with ``tensorEntries.get("blk.N.attn_q.weight")`` and
fails late with a null pointer when one is absent (model/loader/ModelLoader.java:265-303 of the
reference project).  Here every parameter the model's parts declare is looked up by its
checkpoint name before anything is copied, and one ``WeightError`` lists every missing tensor,
every unexpected tensor and every wrong shape together.

Storage policy.  Floating tensors stored in 16 bits are kept in bfloat16; a tensor stored in
32-bit floats stays in 32 bits; integer tables become int32.  The float32 run converts every
floating tensor to float32 (exact for 16-bit inputs), which makes the whole model a true 32-bit
computation."""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import WeightError, open_model_files


@dataclass(frozen=True)
class ParamSpec:
    """One parameter of a part: its shape and how the random-weights mode fills it
    (``matrix``: N(0, std); ``norm``: 1 + N(0, norm_std); ``zeros``; ``int_table``)."""
    shape: tuple[int, ...]
    init: str = "matrix"


def storage_dtype(stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_names_and_shapes(expected: dict[str, tuple[int, ...]], found: dict[str, tuple[int, ...]],
                           where: str, optional: set[str] = frozenset()) -> None:
    """Raise one WeightError that lists everything wrong; ``optional`` names may be present or not."""
    missing = sorted(n for n in expected if n not in found)
    unexpected = sorted(n for n in found if n not in expected and n not in optional)
    wrong = sorted((n, found[n], expected[n]) for n in expected if n in found and tuple(found[n]) != tuple(expected[n]))
    if not (missing or unexpected or wrong):
        return
    lines = [f"weights in {where} do not match the model:"]
    if missing:
        lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shape ({len(wrong)}): " +
                     ", ".join(f"{n} is {list(f)}, expected {list(e)}" for n, f, e in wrong))
    raise WeightError("\n".join(lines))


def load_checkpoint_tensors(model_dir: str | Path, expected: dict[str, tuple[int, ...]], run_dtype: torch.dtype,
                            optional: set[str] = frozenset()) -> dict[str, torch.Tensor]:
    """CPU tensors by checkpoint name, checked against ``expected`` and converted by the storage
    policy.  ``optional`` names (a stored output head of a tied model, rotary tables) are ignored."""
    files = open_model_files(model_dir)
    found = {name: f.shape(name) for name, f in files.items()}
    check_names_and_shapes(expected, found, str(model_dir), optional)
    out: dict[str, torch.Tensor] = {}
    for name in expected:
        f = files[name]
        stored = f.dtype(name)
        if not (stored.is_floating_point or stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8)):
            raise WeightError(f"{name}: stored dtype {stored} is not supported")
        out[name] = f.tensor(name).to(storage_dtype(stored, run_dtype))
    return out
