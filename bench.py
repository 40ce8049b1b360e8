"""Benchmark of the serving step on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model 1b|3b|8b] [--dtype bfloat16|float32]
                    [--batch 8] [--context 4096] [--layers L] [--sizes all|none]

Default run: the Llama-3.2-1B shape (BASELINE.json configs[2]) with random bfloat16 weights, a
batch of 8 sequences at context length 4096.  A "step" is one decode step.  ``value`` is decoded
tokens per second timed on the device with CUDA events; ``e2e`` is the same through the Python
entry point (``Engine.generate``), host token ids in and out, timed on the host between the
callbacks of two decode steps.  The same line carries the 2,048-token prefill, the decode-step
roofline (bytes the step has to read over its time, against the measured copy bandwidth), decode
at batch 1 and 64, and, unless ``--sizes none``, the other sizes BASELINE.json names: the 3B shape
with an unequal batch of 8 prompts of 64 to 2,048 tokens and 256 decode steps (configs[3]), the 8B
shape with 64 prompts of 512 tokens in one prompt step and 512 decode steps (configs[4]), and the
1B shape in true float32.  ``--model 3b`` / ``--model 8b`` / ``--dtype float32`` make one of those
the headline of the line instead.  One JSON line on stdout; everything else goes to stderr.

The reference counts prompt and generated tokens over the whole loop's wall time, load excluded
(auxiliary/LastRunMetrics.java:20-32, inference/InferenceEngine.java:281,358-363 of the reference
project); here the prompt step and the decode steps are timed apart, on the device.

The library runs on one GPU: for --gpus N > 1 it says so and exits with 2.
"""
from __future__ import annotations

import argparse
import gc
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

# The three shapes of BASELINE.json (configs[2], [3], [4]); ``check`` is the wording each is checked against.
SHAPES = {
    "1b": dict(name="Llama-3.2-1B shape", baseline=2, layers=16, hidden=2048, heads=32, kv_heads=8, head_dim=64,
               intermediate=8192, vocab=128256, tied=True, rope_factor=32.0,
               check="16 layers, hidden 2048, 32 heads, 8 kv heads, head_dim 64, intermediate 8192, vocab 128256"),
    "3b": dict(name="Llama-3.2-3B shape", baseline=3, layers=28, hidden=3072, heads=24, kv_heads=8, head_dim=128,
               intermediate=8192, vocab=128256, tied=True, rope_factor=32.0,
               check="28 layers, hidden 3072, 24 heads, 8 kv heads, head_dim 128, intermediate 8192, vocab 128256"),
    "8b": dict(name="Llama-3.1-8B shape", baseline=4, layers=32, hidden=4096, heads=32, kv_heads=8, head_dim=128,
               intermediate=14336, vocab=128256, tied=False, rope_factor=8.0,
               check="32 layers, hidden 4096, 32 heads, 8 kv heads, head_dim 128, intermediate 14336, vocab 128256"),
}


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


def model_config(shape: str, layers: int = 0):
    """config.json of one of BASELINE.json's shapes (checked against its wording) and its full layer count."""
    s = SHAPES[shape]
    base = json.loads((ROOT / "BASELINE.json").read_text())["configs"][s["baseline"]]
    assert s["check"] in base, f"bench.py's {shape} sizes no longer restate BASELINE.json configs[{s['baseline']}]"
    cfg = {
        "architectures": ["LlamaForCausalLM"], "num_hidden_layers": layers or s["layers"], "hidden_size": s["hidden"],
        "num_attention_heads": s["heads"], "num_key_value_heads": s["kv_heads"], "head_dim": s["head_dim"],
        "intermediate_size": s["intermediate"], "vocab_size": s["vocab"], "rope_theta": 500000.0, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": s["tied"], "max_position_embeddings": 131072,
        "rope_scaling": {"rope_type": "llama3", "factor": s["rope_factor"], "low_freq_factor": 1.0,
                         "high_freq_factor": 4.0, "original_max_position_embeddings": 8192},
    }
    return cfg, s["layers"]


def weight_bytes(c, el=2):
    """Bytes of every weight a decode step uses once: the layers, the final norm and the output head (the
    embedding table is only gathered from; when tied it is read once, as the head)."""
    q_dim, kv_dim = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    per_layer = (c["hidden_size"] * (q_dim + 2 * kv_dim) + q_dim * c["hidden_size"]
                 + 3 * c["hidden_size"] * c["intermediate_size"] + 2 * c["hidden_size"])
    head = c["vocab_size"] * c["hidden_size"]
    return el * (c["num_hidden_layers"] * per_layer + head + c["hidden_size"])


def kv_bytes_per_token(c, el=2):
    return 2 * c["num_hidden_layers"] * c["num_key_value_heads"] * c["head_dim"] * el


def prefill_flops(c, lengths, wanted_rows=None):
    q_dim, kv_dim = c["num_attention_heads"] * c["head_dim"], c["num_key_value_heads"] * c["head_dim"]
    per_token = 2 * (c["hidden_size"] * (q_dim + 2 * kv_dim) + q_dim * c["hidden_size"]
                     + 3 * c["hidden_size"] * c["intermediate_size"])
    attn = sum(2 * T * T * q_dim for T in lengths)  # causal: QK^T and PV over half the square
    rows = len(lengths) if wanted_rows is None else wanted_rows
    return c["num_hidden_layers"] * (sum(lengths) * per_token + attn) + 2 * rows * c["vocab_size"] * c["hidden_size"]


REST_AFTER_PROMPT_S = 3.0


def time_decode(engine, lengths, steps, warmup):
    """Put sequences of ``lengths`` tokens into the cache, then run ``warmup + steps`` decode steps of all of them
    together; returns the timed steps' device times (ms), the kernels launched in them and the wall-clock span."""
    import torch
    from gpullama3.java_b200.engine.step import SequenceInput
    from gpullama3.java_b200.kernels import ops

    V = engine.config.vocab_size
    g = torch.Generator().manual_seed(1)
    cache, step = engine.cache, engine.step_fn
    batch = len(lengths)
    slots = [cache.acquire() for _ in range(batch)]
    try:
        i = 0
        while i < batch:   # prompts go in a pass-full at a time
            j, total = i, 0
            while j < batch and (j == i or total + lengths[j] <= 16384):
                total += lengths[j]
                j += 1
            prompts = [torch.randint(0, V, (lengths[k],), generator=g).tolist() for k in range(i, j)]
            step([SequenceInput(s, p, []) for s, p in zip(slots[i:j], prompts)])
            i = j
        torch.cuda.synchronize()
        # Every decode measurement of this file follows the same protocol: prompt step, a rest, warm-up steps, timed
        # steps.  Without the rest, decode steps that follow a prompt burst on a GPU that has been busy for seconds run
        # at a lower SM clock (about 12 % slower), and how much depends on what was measured before.
        time.sleep(REST_AFTER_PROMPT_S)
        toks = torch.randint(0, V, (batch,), generator=g).tolist()
        times, launches0 = [], None
        # a step's clock starts when its host side (token and page-table staging) is done, right before the launch;
        # the host side is part of the end-to-end number
        started = []
        step.before_launch = lambda: started.append(True) or started[0].record()
        t_begin = time.time()
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


def time_prefill(engine, lengths, repeats=2):
    """All prompts of ``lengths`` in one step (logits at each last token); the best device time of ``repeats``
    runs after one warm-up run, in ms."""
    import torch
    from gpullama3.java_b200.engine.step import SequenceInput

    g = torch.Generator().manual_seed(2)
    best = None
    for _ in range(repeats + 1):
        slots = [engine.cache.acquire() for _ in lengths]
        prompts = [torch.randint(0, engine.config.vocab_size, (T,), generator=g).tolist() for T in lengths]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        engine.step_fn([SequenceInput(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        for s in slots:
            engine.cache.release(s)
        best = ms if best is None else min(best, ms)  # the first pass is the warm-up
    return best


def time_e2e(engine, batch, context, steps, warmup, idle_after_prompt=0.0):
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
        if count[0] == batch and idle_after_prompt > 0:
            time.sleep(idle_after_prompt)   # (see the caller: the prompt step's burst is over, the GPU rests once)
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


def make_engine(cfg, dtype, max_tokens, max_batch):
    import torch
    from gpullama3.java_b200.engine.api import Engine

    t0 = time.time()
    engine = Engine.from_random(cfg, seed=0, dtype=dtype, max_tokens=max_tokens, max_batch=max_batch)
    torch.cuda.synchronize()
    log(f"model ready in {time.time() - t0:.1f} s ({cfg['num_hidden_layers']} layers, hidden {cfg['hidden_size']}, {dtype})")
    return engine


def drop(engine):
    import torch

    del engine
    gc.collect()
    torch.cuda.empty_cache()


def decode_record(cfg, el, lengths, times, peaks, launches=None):
    """tokens/s, ms/step and the roofline of the timed decode steps, the first of which found ``lengths`` tokens
    cached."""
    batch, n = len(lengths), len(times)
    ms = sum(times) / n
    mean_tokens = sum(lengths) + batch * (n / 2)          # tokens in the cache, averaged over the timed steps
    step_bytes = weight_bytes(cfg, el) + kv_bytes_per_token(cfg, el) * mean_tokens
    achieved = step_bytes / (ms / 1e3) / 1e9
    return {"tokens_per_s": round(batch * n / (sum(times) / 1e3), 1), "ms_per_step": round(ms, 4), "steps": n,
            "bytes_per_step": int(step_bytes), "gbs": round(achieved, 1), "frac": round(achieved / peaks["hbm_gbs"], 4),
            "launches": launches}


def prefill_record(cfg, lengths, ms, peak_tflops):
    if ms != ms:  # not timed
        return {"tokens_per_s": None, "tokens": sum(lengths), "ms": None, "tflops": None, "frac": None}
    flops = prefill_flops(cfg, lengths)
    tf = flops / (ms / 1e3) / 1e12
    return {"tokens_per_s": round(sum(lengths) / (ms / 1e3), 1), "tokens": sum(lengths), "ms": round(ms, 3),
            "tflops": round(tf, 1), "frac": round(tf / peak_tflops, 4) if peak_tflops else None}


def unequal_lengths(n=8, lo=64, hi=2048, seed=0):
    import torch

    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (n,), generator=g).tolist()


def run_3b(peaks, layers, warmup, steps=256, prefill=True):
    """BASELINE.json configs[3]: unequal batch of 8 prompts of 64 to 2,048 tokens in one prompt step, 256 decode steps."""
    cfg, full = model_config("3b", layers)
    lengths = unequal_lengths()
    engine = make_engine(cfg, "bfloat16", sum(-(-(n + steps + warmup + 8) // 64) * 64 for n in lengths) + 64, 8)
    try:
        pre = prefill_record(cfg, lengths, time_prefill(engine, lengths) if prefill else float("nan"), peaks["bf16_tflops"])
        times, launches, _ = time_decode(engine, lengths, steps, warmup)
        dec = decode_record(cfg, 2, [n + warmup for n in lengths], times, peaks, launches)
    finally:
        drop(engine)
    log(f"3B unequal b8 (prompts {lengths}): prefill {pre['ms']} ms ({pre['tokens_per_s']} tok/s, frac {pre['frac']}); "
        f"decode {dec['ms_per_step']} ms/step ({dec['tokens_per_s']:.0f} tok/s, frac {dec['frac']})")
    return {"layers": cfg["num_hidden_layers"], "layers_full": full, "prompt_lengths": lengths, "prefill": pre, "decode": dec}


def run_8b(peaks, layers, warmup, steps=512, prefill=True):
    """BASELINE.json configs[4]: 64 prompts of 512 tokens in one prompt step, 512 decode steps."""
    cfg, full = model_config("8b", layers)
    lengths = [512] * 64
    engine = make_engine(cfg, "bfloat16", 64 * (-(-(512 + steps + warmup + 8) // 64) * 64) + 64, 64)
    try:
        pre = prefill_record(cfg, lengths, time_prefill(engine, lengths, repeats=1) if prefill else float("nan"),
                             peaks["bf16_tflops_sustained"])
        times, launches, _ = time_decode(engine, lengths, steps, warmup)
        dec = decode_record(cfg, 2, [n + warmup for n in lengths], times, peaks, launches)
    finally:
        drop(engine)
    log(f"8B 64 x 512: prefill {pre['ms']} ms ({pre['tokens_per_s']} tok/s, frac {pre['frac']} of the sustained peak); "
        f"decode {dec['ms_per_step']} ms/step ({dec['tokens_per_s']:.0f} tok/s, frac {dec['frac']})")
    return {"layers": cfg["num_hidden_layers"], "layers_full": full, "prefill": pre, "decode": dec}


def run_1b_f32(peaks, layers, warmup, context, batch):
    """The 1B shape in true float32 (plain FMA kernels, float32 weights and cache): prefill 2,048, decode at ``batch``."""
    cfg, full = model_config("1b", layers)
    engine = make_engine(cfg, "float32", batch * context + 4096, batch)
    try:
        pre = prefill_record(cfg, [2048], time_prefill(engine, [2048], repeats=1), None)
        steps = 8
        lengths = [context - steps - warmup] * batch
        times, launches, _ = time_decode(engine, lengths, steps, warmup)
        dec = decode_record(cfg, 4, [n + warmup for n in lengths], times, peaks, launches)
    finally:
        drop(engine)
    log(f"1B float32: prefill 2048 {pre['ms']} ms ({pre['tflops']} TFLOP/s of FMA); decode b{batch} {dec['ms_per_step']} ms/step "
        f"({dec['tokens_per_s']:.0f} tok/s, frac {dec['frac']})")
    return {"layers": cfg["num_hidden_layers"], "layers_full": full, "prefill": pre, "decode": dec}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed decode steps (default: 32 for the 1B headline, 256 for --model 3b, 512 for --model 8b)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="1b", choices=sorted(SHAPES), help="whose workload is the line's headline")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (both are recorded)")
    ap.add_argument("--sizes", default="all", choices=["all", "none"],
                    help="all: also time the other sizes of BASELINE.json (3B unequal batch, 8B 64 x 512, 1B float32)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-prefill", action="store_true", help="--model 3b/8b: skip the timed prompt step (launch lists of decode steps)")
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
    headline_steps = args.steps
    if args.steps is None:
        args.steps = 32

    import torch  # noqa: F401
    from gpullama3.java_b200.kernels import ops  # noqa: F401

    peaks, peak_source = load_peaks()
    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)
    if args.model != "1b" or args.dtype != "bfloat16":
        return other_headline(args, peaks, peak_source, clocks, headline_steps)

    cfg, full_layers = model_config("1b", args.layers)
    max_batch = args.batch if args.no_points else max(args.batch, 64)
    engine = make_engine(cfg, "bfloat16", max_batch * args.context + 4096, max_batch)

    lengths = [args.context - (args.steps + args.warmup)] * args.batch
    times, launches, (tb, te) = time_decode(engine, lengths, args.steps, args.warmup)
    clock_summary = clocks.summary(tb, te)
    total_ms = sum(times)
    ms_per_step = total_ms / len(times)
    value = args.batch * len(times) / (total_ms / 1e3)
    log(f"decode b{args.batch}: {ms_per_step:.3f} ms/step, {value:.0f} tok/s, {launches} launches")
    dec = decode_record(cfg, 2, [n + args.warmup for n in lengths], times, peaks)
    roofline = {"bound": "hbm", "achieved": dec["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": dec["frac"],
                "peak_source": peak_source}

    T = 2048
    pre = prefill_record(cfg, [T], time_prefill(engine, [T], repeats=3), peaks["bf16_tflops"])
    prefill = {"value": pre["tokens_per_s"], "tokens": T, "ms": pre["ms"], "frac": pre["frac"]}
    log(f"prefill {T}: {pre['ms']:.2f} ms, {pre['tokens_per_s']:.0f} tok/s, frac {pre['frac']}")

    points = {}
    if not args.no_points:
        for b in (1, 64):
            n = max(8, args.steps // 2)
            ts, _, _ = time_decode(engine, [args.context - n - args.warmup] * b, n, args.warmup)
            rec = decode_record(cfg, 2, [args.context - n] * b, ts, peaks)
            points[f"decode_b{b}"] = rec["tokens_per_s"]
            points[f"decode_b{b}_hbm_frac"] = rec["frac"]
            log(f"decode b{b}: {rec['ms_per_step']:.3f} ms/step, {rec['tokens_per_s']:.0f} tok/s, frac {rec['frac']}")

    e2e = None
    if not args.no_e2e:
        # The same conditions as the device-timed run above, whose prompt step was the process's first work on a cold
        # GPU: decode steps that follow a prompt burst on a GPU that has been busy for seconds run at a lower SM clock
        # (about 12 % slower) until it has rested, so the run pauses once, after its prompt step and before the
        # warm-up steps.  The pause is outside the timed steps.
        e_val, e_ms = time_e2e(engine, args.batch, args.context, args.steps, args.warmup, idle_after_prompt=REST_AFTER_PROMPT_S)
        e2e = {"value": round(e_val, 1), "unit": "tokens/s", "ms_per_step": round(e_ms, 3),
               "h2d_bytes_per_step": int(engine.step_fn.last_h2d_bytes) if hasattr(engine.step_fn, "last_h2d_bytes") else None,
               "d2h_bytes_per_step": int(getattr(engine.step_fn, "last_d2h_bytes", 0)) or 4 * args.batch}
        log(f"e2e b{args.batch}: {e_ms:.3f} ms/step, {e_val:.0f} tok/s")
    drop(engine)
    engine = None

    sizes = {}
    if args.sizes == "all":
        sizes["3b_unequal_b8"] = r = run_3b(peaks, 0, args.warmup)
        points.update({"decode_3b_unequal_b8": r["decode"]["tokens_per_s"], "decode_3b_hbm_frac": r["decode"]["frac"],
                       "prefill_3b_unequal_b8": r["prefill"]["tokens_per_s"], "prefill_3b_frac": r["prefill"]["frac"]})
        sizes["8b_64x512"] = r = run_8b(peaks, 0, args.warmup)
        points.update({"decode_8b_b64": r["decode"]["tokens_per_s"], "decode_8b_hbm_frac": r["decode"]["frac"],
                       "prefill_8b_64x512": r["prefill"]["tokens_per_s"], "prefill_8b_frac_of_sustained": r["prefill"]["frac"]})
        sizes["1b_float32"] = r = run_1b_f32(peaks, 0, args.warmup, args.context, args.batch)
        points.update({"decode_1b_float32_b8": r["decode"]["tokens_per_s"], "decode_1b_float32_hbm_frac": r["decode"]["frac"],
                       "prefill_1b_float32_2048": r["prefill"]["tokens_per_s"]})
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
                   "sampling": "greedy on device", "rest_after_prompt_s": 3},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e, "gpu_launches": launches,
        "clocks": clock_summary, "impl": "ours",
    }
    if sizes:
        line["other_sizes"] = sizes
    print(json.dumps(line))
    return 0


def other_headline(args, peaks, peak_source, clocks, headline_steps=None) -> int:
    """``--model 3b``, ``--model 8b`` or ``--dtype float32``: that workload as the line's headline."""
    t0 = time.time()
    if args.dtype == "float32":
        if args.model != "1b":
            print("bench.py: --dtype float32 is timed for --model 1b")
            return 2
        r, what = run_1b_f32(peaks, args.layers, args.warmup, args.context, args.batch), \
            f"Llama-3.2-1B shape in float32, batch {args.batch}, context {args.context}"
        batch, seq = args.batch, args.context
    elif args.model == "3b":
        steps = headline_steps or 256
        r, what, batch, seq = run_3b(peaks, args.layers, args.warmup, steps, not args.no_prefill), \
            f"Llama-3.2-3B shape, unequal batch of 8 prompts of 64..2048 tokens, {steps} decode steps", 8, 2048 + steps
    else:
        steps = headline_steps or 512
        r, what, batch, seq = run_8b(peaks, args.layers, args.warmup, steps, not args.no_prefill), \
            f"Llama-3.1-8B shape, 64 prompts of 512 tokens, {steps} decode steps", 64, 512 + steps
    clock_summary = clocks.summary(t0, time.time())
    clocks.stop()
    s = SHAPES[args.model]
    dec, pre = r["decode"], r["prefill"]
    line = {
        "metric": f"decode tokens/s ({what})", "value": dec["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1,
        "steps": dec["steps"], "warmup": args.warmup, "ms_per_step": dec["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "config": {"model": s["name"], "layers": r["layers"], "layers_full": r["layers_full"], "hidden": s["hidden"],
                   "heads": s["heads"], "kv_heads": s["kv_heads"], "head_dim": s["head_dim"], "intermediate": s["intermediate"],
                   "vocab": s["vocab"], "tied": s["tied"], "global_batch": batch, "seq_len": seq, "prefill_tokens": pre["tokens"],
                   "parallelism": "single GPU", "l2": "step reads more than L2 (126 MB)", "sampling": "greedy on device"},
        "prefill": {"value": pre["tokens_per_s"], "tokens": pre["tokens"], "ms": pre["ms"], "frac": pre["frac"]},
        "roofline": {"bound": "hbm", "achieved": dec["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": dec["frac"],
                     "peak_source": peak_source},
        "points": {}, "e2e": None, "gpu_launches": dec["launches"], "clocks": clock_summary, "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
