"""Builders of replay traces (the JSON steps ``bin/trace_run`` reads) for the ways of cutting the
same requests: whole, with the last tokens decoded one by one, and in batches of unequal
lengths.  Each builder returns the steps and, per step, which (request, position) each written
row belongs to."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import torch


def trace_whole(requests: dict[str, list[int]]):
    steps, rows = [], {}
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
        rows[i] = [(rid, p) for p in range(len(toks))]
    return steps, rows


def trace_tail_one_by_one(requests: dict[str, list[int]], tail: int = 32):
    """Each request alone: all but the last ``tail`` tokens in one step, then one token a step."""
    steps, rows, n = [], {}, 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": [head - 1]}],
                      "end": [rid] if head == len(toks) else []})
        rows[n] = [(rid, head - 1)]
        n += 1
        for p in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
            rows[n] = [(rid, p)]
            n += 1
    return steps, rows


def trace_batches(requests: dict[str, list[int]], batch_size: int, prompt_fraction: float = 0.5):
    """Batches of ``batch_size`` requests that start together: a prompt of unequal length each in
    one step, then one token each per step; shorter requests end earlier; one batch after another."""
    ids = list(requests)
    steps, rows, n = [], {}, 0
    for b in range(0, len(ids), batch_size):
        batch = ids[b:b + batch_size]
        plen = {r: max(1, int(len(requests[r]) * prompt_fraction)) for r in batch}
        entries = [{"id": r, "tokens": requests[r][:plen[r]], "want": [plen[r] - 1]} for r in batch]
        ended = [r for r in batch if plen[r] == len(requests[r])]
        steps.append({"step": n, "entries": entries, "end": ended})
        rows[n] = [(r, plen[r] - 1) for r in batch]
        n += 1
        live = [r for r in batch if r not in ended]
        pos = dict(plen)
        while live:
            entries = [{"id": r, "tokens": [requests[r][pos[r]]], "want": [0]} for r in live]
            ended = [r for r in live if pos[r] == len(requests[r]) - 1]
            steps.append({"step": n, "entries": entries, "end": ended})
            rows[n] = [(r, pos[r]) for r in live]
            n += 1
            for r in live:
                pos[r] += 1
            live = [r for r in live if r not in ended]
    return steps, rows


def max_live_tokens(steps) -> int:
    """The most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held: dict[str, int] = {}
    best = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        best = max(best, sum(-(-v // 64) * 64 for v in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return best


def run_in_process(model, steps, out_dir: Path, max_tokens: int) -> None:
    from gpullama3.java_b200.engine.trace import TraceRunner

    runner = TraceRunner(model, max_tokens, out_dir)
    for s in steps:
        runner.run_step(s)
    torch.cuda.synchronize()
    runner.cache.check_invariants()
    assert not runner.cache.live_slots(), "requests were left live at the end of the trace"


def read_rows(out_dir: Path, rows: dict, vocab: int) -> dict:
    """(request, position) -> logits row, from the files a replay wrote."""
    got = {}
    for step, keys in rows.items():
        a = np.fromfile(Path(out_dir) / f"{step}.f32", dtype="<f4").reshape(len(keys), vocab)
        for k, row in zip(keys, a):
            got[k] = torch.from_numpy(row.copy())
    return got


def write_trace(path: Path, steps) -> None:
    path.write_text("".join(json.dumps(s) + "\n" for s in steps))
