"""Benchmark of the serving step on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 4096] [--layers L]

Default run: the Llama-3.2-1B shape (BASELINE.json configs[2]) with random bfloat16 weights, a
batch of 8 sequences at context length 4096.  A "step" is one decode step.  ``value`` is decoded
tokens per second timed on the device with CUDA events; ``e2e`` is the same through the Python
entry point (``Engine.generate``), host token ids in and out, timed on the host between the
callbacks of two decode steps.  The same line carries the 2,048-token prefill, the decode-step
roofline (bytes the step has to read over its time, against the measured copy bandwidth) and
decode at batch 1 and 64.  One JSON line on stdout; everything else goes to stderr.

The library runs on one GPU: for --gpus N > 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
PUBLISHED_BEST_1B_TOKS = 96.65  # reference README.md:55, Llama-3.2-1B FP16 on an RTX 5090, batch 1


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            flat = {}
            def walk(x):
                if isinstance(x, dict):
                    for k, v in x.items():
                        if isinstance(v, (int, float)) and k in FALLBACK_PEAKS:
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(d)
            if "hbm_gbs" in flat and "bf16_tflops" in flat:
                flat.setdefault("bf16_tflops_sustained", flat["bf16_tflops"])
                return flat, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ["clocks.sm", "clocks.max.sm", "clocks_event_reasons.hw_slowdown",
              "clocks_event_reasons.hw_thermal_slowdown", "clocks_event_reasons.sw_thermal_slowdown",
              "clocks_event_reasons.sw_power_cap"]

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", "--query-gpu=" + ",".join(self.FIELDS),
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [x.strip() for x in line.split(",")]))

    def mark(self):
        return time.time()

    def stop(self):
        if self.proc:
            self.proc.terminate()

    def summary(self, t0, t1):
        rows = [r for t, r in self.samples if t0 <= t <= t1 + 0.15] or [r for _, r in self.samples[-3:]]
        mhz, max_mhz, reasons = [], 0, set()
        for r in rows:
            try:
                mhz.append(int(r[0]))
                max_mhz = max(max_mhz, int(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[2:]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max_mhz or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def model_config(args):
    base = json.loads((ROOT / "BASELINE.json").read_text())["configs"][2]  # read for the record; sizes below restate it
    cfg = {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": 16, "hidden_size": 2048,
        "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64, "intermediate_size": 8192,
        "vocab_size": 128256, "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
        "max_position_embeddings": 131072,
        "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 8192},
    }
    assert "16 layers, hidden 2048, 32 heads, 8 kv heads, head_dim 64, intermediate 8192, vocab 128256" in base
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    return cfg, full_layers


def weight_bytes(c, el=2):
    q_dim, kv_dim = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    per_layer = (c["hidden_size"] * (q_dim + 2 * kv_dim) + q_dim * c["hidden_size"]
                 + 3 * c["hidden_size"] * c["intermediate_size"] + 2 * c["hidden_size"])
    head = c["vocab_size"] * c["hidden_size"]  # the tied table is read once, as the output head
    return el * (c["num_hidden_layers"] * per_layer + head + c["hidden_size"])


def kv_bytes_per_token(c, el=2):
    return 2 * c["num_hidden_layers"] * c["num_key_value_heads"] * c["head_dim"] * el


def prefill_flops(c, T, wanted_rows=1):
    q_dim, kv_dim = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    per_token = 2 * (c["hidden_size"] * (q_dim + 2 * kv_dim) + q_dim * c["hidden_size"]
                     + 3 * c["hidden_size"] * c["intermediate_size"])
    attn = 2 * T * T * q_dim  # causal: QK^T and PV over half the square
    return c["num_hidden_layers"] * (T * per_token + attn) + 2 * wanted_rows * c["vocab_size"] * c["hidden_size"]


def time_decode(engine, batch, context, steps, warmup, sampler=None):
    """Prefill ``batch`` sequences so that the timed steps end at ``context``; returns per-step ms."""
    import torch
    from gpullama3.java_b200.engine.step import SequenceInput
    from gpullama3.java_b200.kernels import ops

    V = engine.config.vocab_size
    g = torch.Generator().manual_seed(1)
    start_len = context - (steps + warmup)
    cache, step = engine.cache, engine.step_fn
    slots = [cache.acquire() for _ in range(batch)]
    try:
        group = max(1, 16384 // start_len)
        for i in range(0, batch, group):
            part = slots[i:i + group]
            prompts = [torch.randint(0, V, (start_len,), generator=g).tolist() for _ in part]
            step([SequenceInput(s, p, []) for s, p in zip(part, prompts)])
        torch.cuda.synchronize()
        toks = torch.randint(0, V, (batch,), generator=g).tolist()
        times, launches0 = [], None
        # a step's clock starts when its host side (token and page-table staging) is done, right before the launch;
        # the host side is part of the end-to-end number
        started = []
        step.before_launch = lambda: started.append(True) or started[0].record()
        for it in range(warmup + steps):
            if it == warmup:
                torch.cuda.synchronize()
                launches0 = ops.launch_count() + step.graph_launches
                t_begin = time.time()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            started[:] = [e0]
            logits = step([SequenceInput(s, [t], [0]) for s, t in zip(slots, toks)], reuse_output=True)
            if len(started) == 1:
                raise RuntimeError("the decode step did not go through the recorded path; bench.py times that path")
            out = torch.empty(batch, dtype=torch.int32, device=logits.device)
            ops.argmax_rows(logits, out)
            e1.record()
            torch.cuda.synchronize()
            toks = [int(t) % V for t in out.tolist()]
            if it >= warmup:
                times.append(e0.elapsed_time(e1))
        t_end = time.time()
        launches = ops.launch_count() + step.graph_launches - launches0
        return times, launches, (t_begin, t_end)
    finally:
        step.before_launch = None
        for s in slots:
            cache.release(s)


def time_prefill(engine, T, repeats=3):
    import torch
    from gpullama3.java_b200.engine.step import SequenceInput

    g = torch.Generator().manual_seed(2)
    best = None
    for _ in range(repeats + 1):
        slot = engine.cache.acquire()
        prompt = torch.randint(0, engine.config.vocab_size, (T,), generator=g).tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step_fn([SequenceInput(slot, prompt, [T - 1])])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        engine.cache.release(slot)
        best = ms if best is None else min(best, ms)  # the first pass is the warm-up
    return best


def time_e2e(engine, batch, context, steps, warmup):
    """Decode tokens per second through Engine.generate: host token ids in, host token ids out.
    Timed on the host between the callbacks that deliver decode step `warmup` and `warmup+steps`."""
    import torch

    V = engine.config.vocab_size
    g = torch.Generator().manual_seed(3)
    n_new = warmup + steps + 1
    prompts = [torch.randint(0, V, (context - n_new,), generator=g).tolist() for _ in range(batch)]
    stamps = {}
    count = [0]

    def on_token(i, tok):
        count[0] += 1
        if count[0] % batch == 0:
            stamps[count[0] // batch] = time.perf_counter()

    engine.generate(prompts, max_new_tokens=n_new, stop_ids=(), on_token=on_token)
    dt = stamps[warmup + 1 + steps] - stamps[warmup + 1] if (warmup + 1 + steps) in stamps else None
    if dt is None:
        dt = stamps[max(stamps)] - stamps[warmup + 1]
        steps = max(stamps) - (warmup + 1)
    gaps = sorted((stamps[k + 1] - stamps[k]) * 1e3 for k in range(warmup + 1, warmup + 1 + steps) if k + 1 in stamps)
    if gaps:
        log(f"e2e steps: median {gaps[len(gaps) // 2]:.3f} ms, longest {gaps[-1]:.3f} ms, shortest {gaps[0]:.3f} ms")
    return batch * steps / dt, dt / steps * 1e3


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (both are recorded)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "AskMyu/GPULlama3.java is a Java 21 + TornadoVM application (no Python package, no JDK, Maven or "
                          "TornadoVM SDK on this image, no network); pip install of the reference checkout finds no Python project to build"}))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from gpullama3.java_b200.engine.api import Engine
    from gpullama3.java_b200.kernels import ops

    peaks, peak_source = load_peaks()
    cfg, full_layers = model_config(args)
    t0 = time.time()
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    engine = Engine.from_random(cfg, seed=0, dtype="bfloat16", max_tokens=max_batch * args.context + 4096, max_batch=max_batch)
    torch.cuda.synchronize()
    log(f"model ready in {time.time() - t0:.1f} s ({cfg['num_hidden_layers']} of {full_layers} layers)")

    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)
    times, launches, (tb, te) = time_decode(engine, args.batch, args.context, args.steps, args.warmup)
    clock_summary = clocks.summary(tb, te)
    total_ms = sum(times)
    ms_per_step = total_ms / len(times)
    value = args.batch * len(times) / (total_ms / 1e3)
    log(f"decode b{args.batch}: {ms_per_step:.3f} ms/step, {value:.0f} tok/s, {launches} launches")

    mean_ctx = args.context - args.steps / 2
    step_bytes = weight_bytes(cfg) + kv_bytes_per_token(cfg) * args.batch * mean_ctx
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peak_source}

    T = 2048
    pre_ms = time_prefill(engine, T)
    pre_flops = prefill_flops(cfg, T)
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(pre_flops / (pre_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4)}
    log(f"prefill {T}: {pre_ms:.2f} ms, {prefill['value']:.0f} tok/s, frac {prefill['frac']}")

    points = {}
    if not args.no_points:
        for b in (1, 64):
            ts, _, _ = time_decode(engine, b, args.context, max(8, args.steps // 2), args.warmup)
            points[f"decode_b{b}"] = round(b * len(ts) / (sum(ts) / 1e3), 1)
            log(f"decode b{b}: {sum(ts) / len(ts):.3f} ms/step, {points[f'decode_b{b}']:.0f} tok/s")

    e2e = None
    if not args.no_e2e:
        e_val, e_ms = time_e2e(engine, args.batch, args.context, args.steps, args.warmup)
        e2e = {"value": round(e_val, 1), "unit": "tokens/s", "ms_per_step": round(e_ms, 3),
               "h2d_bytes_per_step": int(engine.step_fn.last_h2d_bytes) if hasattr(engine.step_fn, "last_h2d_bytes") else None,
               "d2h_bytes_per_step": int(getattr(engine.step_fn, "last_d2h_bytes", 0)) or 4 * args.batch}
        log(f"e2e b{args.batch}: {e_ms:.3f} ms/step, {e_val:.0f} tok/s")
    clocks.stop()

    b1 = points.get("decode_b1")
    line = {
        "metric": f"decode tokens/s (Llama-3.2-1B shape, batch {args.batch}, context {args.context})", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": len(times), "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": round(b1 / PUBLISHED_BEST_1B_TOKS, 2) if b1 else None,
        "vs_baseline_note": "decode_b1 over the reference's best published 1B figure (96.65 tok/s, RTX 5090, batch 1, prompt included)",
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": "Llama-3.2-1B shape", "layers": cfg["num_hidden_layers"], "layers_full": full_layers,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "tied": True, "global_batch": args.batch, "seq_len": args.context, "context_len": args.context,
                   "prefill_tokens": T, "parallelism": "single GPU", "l2": "step reads more than L2 (126 MB)",
                   "sampling": "greedy on device"},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e, "gpu_launches": launches,
        "clocks": clock_summary, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
