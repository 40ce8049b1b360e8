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

    g = p.add_argument_group("LLaMA Configuration")
    g.add_argument("--prompt", "-p", action="append", type=parse_token_ids, help="prompt as token ids; repeat for a batch")
    g.add_argument("--prompt-file", help="file with one prompt (token ids) per line")
    g.add_argument("-sp", "--system-prompt", type=parse_token_ids, help="token ids put before every prompt")
    g.add_argument("--temperature", "--temp", type=float, default=0.1, help="sampling temperature, 0 = greedy")
    g.add_argument("--top-p", type=float, default=0.95, help="top-p (nucleus) sampling parameter; 0 or 1 = off")
    g.add_argument("--seed", "-s", type=int, default=None, help="random seed (default: current timestamp)")
    g.add_argument("-n", "--max-tokens", type=int, default=512, help="maximum number of tokens to generate")
    g.add_argument("--stream", type=_bool, default=True, help="print tokens as they are generated")
    g.add_argument("--echo", type=_bool, default=False, help="print all tokens, prompt included, to stderr")
    g.add_argument("--suffix", help="(fill-in-the-middle is not part of this library)")
    g.add_argument("--stop", type=parse_token_ids, help="stop token ids (default: eos_token_id of config.json)")

    m = p.add_argument_group("Mode Selection")
    m.add_argument("-i", "--interactive", "--chat", action="store_true", help="(chat mode is not part of this library)")
    m.add_argument("--instruct", action="store_true", default=True, help="run once on the given prompts (default)")

    h = p.add_argument_group("Hardware Configuration")
    h.add_argument("--gpu", dest="use_gpu", action="store_true", default=True, help="run on the GPU (always on)")
    h.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="precision of the run")
    h.add_argument("--cache-tokens", type=int, default=None, help="tokens the cache holds (default: what the prompts need)")
    h.add_argument("--max-batch", type=int, default=64, help="most sequences decoded together")

    d = p.add_argument_group("Debug and Profiling")
    d.add_argument("--verbose-init", action="store_true", help="print load, build and cache set-up times")
    d.add_argument("--show-command", action="store_true", help="print the resolved configuration and stop")
    d.add_argument("--execute-after-show", action="store_true", help="run after --show-command")
    return p


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

    if args.show_command:
        print(json.dumps({"model": args.model_path, "config": args.config, "random_weights": args.random_weights,
                          "dtype": args.dtype, "prompts": len(prompts), "temperature": args.temperature,
                          "top_p": args.top_p, "seed": seed, "max_tokens": args.max_tokens,
                          "cache_tokens": cache_tokens, "max_batch": args.max_batch}, indent=2))
        if not args.execute_after_show:
            return 0

    from .api import Engine

    t0 = time.perf_counter()
    if args.model_path:
        engine = Engine.from_folder(args.model_path, dtype=args.dtype, max_tokens=cache_tokens, max_batch=args.max_batch)
    else:
        with open(args.config) as f:
            engine = Engine.from_random(json.load(f), args.random_weights, dtype=args.dtype, max_tokens=cache_tokens,
                                        max_batch=args.max_batch)
    if args.verbose_init:
        print(f"model and cache ready in {time.perf_counter() - t0:.2f} s "
              f"(cache: {engine.cache.n_pages} pages of 64 tokens)", file=sys.stderr)
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
    m = engine.last_metrics
    total = m.prompt_tokens + m.generated_tokens
    print(f"\n\nachieved tok/s: {m.tokens_per_second:.2f}. Tokens: {total}, seconds: {m.seconds:.2f}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
