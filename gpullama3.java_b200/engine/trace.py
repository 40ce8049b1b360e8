"""Trace replay: feed given token ids through a model step by step and write logits.

Nothing is sampled.  The replay drives the same model, step function, cache and kernels that
generation uses; it has no forward pass, cache or loader of its own.  One JSON object per input
line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which logits are wanted, ``<out>/<step>.f32`` receives them as little-endian
float32 [wanted, vocab], in the order of the entries and of each entry's ``want``.  After every
step a line ``done <step>`` is printed and flushed."""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

from ..cache.pages import PAGE_TOKENS
from ..config.registry import architecture_of
from ..config.base import read_config_json
from .step import SequenceInput, StepFunction

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class TraceError(ValueError):
    pass


def load_model(model_dir: str | Path, dtype: torch.dtype, device="cuda"):
    """Build the model class that ``config.json`` names and load its weights from the folder."""
    d = read_config_json(model_dir)
    arch = architecture_of(d)
    config = arch.config_class.from_dict(d)
    model = arch.model_factory(config, dtype, device)
    model.load_folder(model_dir)
    return model


class TraceRunner:
    def __init__(self, model, max_tokens: int, out_dir: str | Path):
        max_tokens = max(PAGE_TOKENS, -(-max_tokens // PAGE_TOKENS) * PAGE_TOKENS)
        self.model = model
        self.cache = model.new_cache(max_tokens)
        self.step_fn = StepFunction(model, self.cache)
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.slot_of: dict[str, int] = {}

    def run_step(self, record: dict) -> None:
        if "step" not in record:
            raise TraceError(f"trace line without 'step': {record!r}")
        step = record["step"]
        inputs = []
        for e in record.get("entries", []):
            rid = str(e["id"])
            if rid not in self.slot_of:
                self.slot_of[rid] = self.cache.acquire()
            inputs.append(SequenceInput(self.slot_of[rid], list(e["tokens"]), list(e.get("want", []))))
        if inputs:
            logits = self.step_fn(inputs)
            if logits is not None:
                arr = logits.to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
                arr.tofile(self.out_dir / f"{step}.f32")
        for rid in record.get("end", []):
            rid = str(rid)
            if rid not in self.slot_of:
                raise TraceError(f"step {step} ends request {rid!r}, which is not live")
            self.cache.release(self.slot_of.pop(rid))


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=sorted(DTYPES))
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 3
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    model = load_model(args.model, DTYPES[args.dtype], "cuda")
    runner = TraceRunner(model, args.max_tokens, args.out)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        runner.run_step(record)
        torch.cuda.synchronize()
        print(f"done {record['step']}", flush=True)
    return 0
