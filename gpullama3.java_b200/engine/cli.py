"""Command line in the manner of the reference's ``llama-tornado`` launcher: the same option
names and meanings where the reference has them (llama-tornado:330-492 and Options.java:31-48,
103-114 of the reference project), for an engine that takes and gives token ids.

    llama-b200 --model DIR --prompt "128000 9906 1917" -n 32 --temperature 0 --stream true

Differences that follow from the engine's scope: ``--model`` is a folder (config.json +
model.safetensors) instead of a GGUF file; ``--prompt`` holds token ids (the tokenizer and the chat
template are outside this library) and may be given several times, which makes a batch; the
chat mode, the fill-in-the-middle suffix and the TornadoVM/JVM switches do not exist."""
from __future__ import annotations

import argparse
import json
import sys
import time


def _bool(v: str) -> bool:
    if v.lower() in ("true", "1", "yes"):
        return True
    if v.lower() in ("false", "0", "no"):
        return False
    raise argparse.ArgumentTypeError(f"expected true or false, got {v!r}")


def parse_token_ids(text: str) -> list[int]:
    parts = text.replace(",", " ").split()
    try:
        ids = [int(p) for p in parts]
    except ValueError:
        raise argparse.ArgumentTypeError(
            f"--prompt takes token ids separated by spaces or commas (this library has no tokenizer), got {text!r}")
    if not ids:
        raise argparse.ArgumentTypeError("--prompt must hold at least one token id")
    return ids


def create_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="llama-b200", description="Llama 3 generation on one NVIDIA B200",
                                formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    p.add_argument("--model", "-m", dest="model_path", help="model folder (config.json + model.safetensors)")
    p.add_argument("--config", help="config.json of a model to fill with random weights (with --random-weights)")
    p.add_argument("--random-weights", type=int, metavar="SEED", help="use seeded random weights instead of a checkpoint")
    p.add_argument("--norm-std", type=float, default=0.0,
                   help="with --random-weights: norm weights are 1 + N(0, this) instead of 1")

    g = p.add_argument_group("Prompt and sampling")
    g.add_argument("--prompt", "-p", action="append", type=parse_token_ids, help="prompt as token ids; repeat for a batch")
    g.add_argument("--prompt-file", help="file with one prompt (token ids) per line")
    g.add_argument("-sp", "--system-prompt", type=parse_token_ids, help="token ids put before every prompt")
    g.add_argument("--temperature", "--temp", type=float, default=0.1, help="softmax temperature of the draw; 0 takes the arg-max")
    g.add_argument("--top-p", type=float, default=0.95, help="probability mass of the nucleus a token is drawn from; 0 or 1: all tokens")
    g.add_argument("--seed", "-s", type=int, default=None, help="seed of the draws (when absent: the clock, printed with --verbose-init)")
    g.add_argument("-n", "--max-tokens", type=int, default=512, help="most new tokens per request")
    g.add_argument("--max-len", type=int, default=None,
                   help="most positions (prompt and new tokens together) a request may reach; "
                        "default: the model's context length, or the cache if that is smaller")
    g.add_argument("--stream", type=_bool, default=True, help="print each token when it is drawn (single prompt)")
    g.add_argument("--echo", type=_bool, default=False, help="copy every token, the prompt's too, to stderr")
    g.add_argument("--suffix", help="(fill-in-the-middle is not part of this library)")
    g.add_argument("--stop", type=parse_token_ids,
                   help="stop token ids (default: eos_token_id of generation_config.json, else of config.json)")

    m = p.add_argument_group("Mode")
    m.add_argument("-i", "--interactive", "--chat", action="store_true", help="(chat mode is not part of this library)")
    m.add_argument("--instruct", action="store_true", default=True, help="run once on the given prompts (default)")

    h = p.add_argument_group("Device and memory")
    h.add_argument("--gpu", dest="use_gpu", action="store_true", default=True, help="run on the GPU (always on)")
    h.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="precision of the run")
    h.add_argument("--cache-tokens", type=int, default=None, help="tokens the cache holds (default: what the prompts need)")
    h.add_argument("--max-batch", type=int, default=64, help="most sequences decoded together")

    d = p.add_argument_group("Diagnostics")
    d.add_argument("--verbose-init", action="store_true", help="print load, build and cache set-up times")
    d.add_argument("--show-config", action="store_true", help="print the model's typed configuration and derived sizes, then stop")
    d.add_argument("--show-command", action="store_true", help="print the resolved run (prompts, sampling, cache) and stop")
    d.add_argument("--execute-after-show", action="store_true", help="run after --show-command")
    d.add_argument("--profile", action="store_true",
                   help="time every kernel launch with CUDA events (steps are then launched one by one, not replayed) "
                        "and print a table per kernel to stderr")
    d.add_argument("--bench", action="store_true",
                   help="print prompt and decode tokens per second of the run as one JSON line to stderr")
    return p


def describe_config(config) -> dict:
    """The typed configuration as config.json would hold it, and the sizes that follow from it."""
    from .model import parameter_specs_by_checkpoint_name
    import math

    specs = parameter_specs_by_checkpoint_name(config)
    d = {"config": config.to_dict(), "parameters": sum(math.prod(s.shape) for s in specs.values()), "tensors": len(specs),
         "layers": len(config.layer_specs()), "schedule": [(e.layer, e.cache, e.writes_cache) for e in config.schedule()],
         "max_sequence_length": config.max_sequence_length(), "stop_token_ids": list(config.stop_token_ids)}
    for name in ("q_dim", "kv_dim"):
        if hasattr(config, name):
            d[name] = getattr(config, name)
    return d


def format_profile(rows: dict) -> str:
    """``{kernel: (launches, total ms)}`` as a table, the longest first."""
    total = sum(ms for _, ms in rows.values()) or 1.0
    lines = [f"{'kernel':34s} {'launches':>9s} {'total ms':>10s} {'mean us':>9s} {'share':>6s}"]
    for name, (n, ms) in sorted(rows.items(), key=lambda kv: -kv[1][1]):
        lines.append(f"{name:34s} {n:9d} {ms:10.3f} {1e3 * ms / max(n, 1):9.2f} {100 * ms / total:5.1f}%")
    return "\n".join(lines)


def main(argv=None) -> int:
    parser = create_parser()
    args = parser.parse_args(argv)
    if args.interactive:
        parser.error("--interactive: the chat mode needs a tokenizer and is not part of this library")
    if args.suffix:
        parser.error("--suffix: fill-in-the-middle is not part of this library")
    if args.temperature < 0:
        parser.error("--temperature must be non-negative")
    if not (0 <= args.top_p <= 1):
        parser.error("--top-p must be within [0, 1]")
    if (args.model_path is None) == (args.random_weights is None):
        parser.error("give either --model DIR or --config FILE --random-weights SEED")
    if args.random_weights is not None and not args.config:
        parser.error("--random-weights needs --config")
    prompts = list(args.prompt or [])
    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts += [parse_token_ids(line) for line in f if line.strip()]
    if not prompts:
        parser.error("Missing argument: --prompt is required (token ids)")
    if args.system_prompt:
        prompts = [args.system_prompt + p for p in prompts]
    seed = args.seed if args.seed is not None else int(time.time())
    need = sum(-(-(len(p) + args.max_tokens) // 64) * 64 for p in prompts[:args.max_batch])
    cache_tokens = args.cache_tokens or max(need, 64)

    if args.show_config:
        from ..config.base import read_config_json
        from ..config.registry import config_from_dict

        if args.model_path:
            raw = read_config_json(args.model_path)
        else:
            with open(args.config) as f:
                raw = json.load(f)
        print(json.dumps(describe_config(config_from_dict(raw)), indent=2))
        return 0

    if args.show_command:
        print(json.dumps({"model": args.model_path, "config": args.config, "random_weights": args.random_weights,
                          "dtype": args.dtype, "prompts": len(prompts), "temperature": args.temperature,
                          "top_p": args.top_p, "seed": seed, "max_tokens": args.max_tokens,
                          "max_len": args.max_len, "cache_tokens": cache_tokens, "max_batch": args.max_batch}, indent=2))
        if not args.execute_after_show:
            return 0

    from .api import Engine

    t0 = time.perf_counter()
    if args.model_path:
        engine = Engine.from_folder(args.model_path, dtype=args.dtype, max_tokens=cache_tokens, max_batch=args.max_batch,
                                    max_length=args.max_len)
    else:
        with open(args.config) as f:
            engine = Engine.from_random(json.load(f), args.random_weights, dtype=args.dtype, norm_std=args.norm_std,
                                        max_tokens=cache_tokens, max_batch=args.max_batch, max_length=args.max_len)
    if args.verbose_init:
        print(f"model and cache ready in {time.perf_counter() - t0:.2f} s "
              f"(cache: {engine.cache.n_pages} pages of 64 tokens; longest sequence {engine.max_length}; seed {seed})",
              file=sys.stderr)
    if args.profile:
        from ..kernels import ops
        engine.step_fn.use_graphs = False     # a replayed step has no launches to put events around
        ops.profile_start()
    if args.echo:
        for p in prompts:
            print(" ".join(map(str, p)), file=sys.stderr)

    single = len(prompts) == 1

    def on_token(i, tok):
        if args.echo:
            print(tok, end=" ", file=sys.stderr, flush=True)
        if args.stream and single:
            print(tok, end=" ", flush=True)

    outs = engine.generate(prompts, max_new_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                           seed=seed, stop_ids=args.stop, on_token=on_token)
    if args.stream and single:
        print()
    else:
        for o in outs:
            print(" ".join(map(str, o)))
    if args.profile:
        print(format_profile(ops.profile_stop()), file=sys.stderr)
    m = engine.last_metrics
    if args.bench:
        print(json.dumps({"prompt_tokens": m.prompt_tokens, "generated_tokens": m.generated_tokens,
                          "prefill_seconds": round(m.prefill_seconds, 6), "decode_seconds": round(m.decode_seconds, 6),
                          "decode_steps": m.decode_steps,
                          "prefill_tokens_per_s": round(m.prompt_tokens / m.prefill_seconds, 1) if m.prefill_seconds else None,
                          "decode_tokens_per_s": round((m.generated_tokens - len(prompts)) / m.decode_seconds, 1)
                          if m.decode_seconds and m.generated_tokens > len(prompts) else None}), file=sys.stderr)
    total = m.prompt_tokens + m.generated_tokens
    print(f"\n\nachieved tok/s: {m.tokens_per_second:.2f}. Tokens: {total}, seconds: {m.seconds:.2f}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
