"""``tileinfer`` command line, in the manner of AntoineBut/TileInfer.jl's (src/cli.jl): commands
with ``--name value`` options, unknown options refused, exit code 0 or 1, a statistics line on
stderr. Prompts are token ids (the library has no tokenizer), so ``run`` takes the ids where the
reference takes text. ``pull/ls/rm/chat`` have no counterpart: a model is a local folder.
"""
from __future__ import annotations

import json
import random
import sys
import time
from typing import Dict, List, Sequence, Tuple

USAGE = """usage: tileinfer <command> [arguments]

commands:
  run <model> <prompt> [options]       generate a continuation of `prompt`: token ids separated by
                                       spaces or commas; <model> is a folder with config.json and
                                       safetensors
  generate <model> <file> [options]    the same for a batch: one prompt a line in <file>
                                       ("-" reads standard input); prints one line of ids per prompt
  random <config.json> <out> [--seed S] [--dtype D]
                                       write a model folder with random weights for a configuration

run and generate options:
  --max-tokens N        tokens to generate per prompt at most (default 512)
  --max-context N       longest sequence in tokens; sizes the KV cache (default 4096)
  --temperature T       0 for greedy (defaults come from the model's generation_config.json)
  --top-k K, --top-p P  sampling filters
  --seed S              random seed
  --backend fast|plain  tensor-core kernels (default) or the plain reference kernels
  --dtype bfloat16|float32
                        element type of weights, activations and cache (default bfloat16)
  --max-seqs N          sequences per batch at most (default 8)
  --stop-ids IDS        stop tokens instead of the configuration's EOS ids ("" for none)
"""

GENERATION_OPTIONS = ("max-tokens", "max-context", "temperature", "top-k", "top-p", "seed", "backend", "dtype",
                      "max-seqs", "stop-ids")
FLAGS: Tuple[str, ...] = ()


class ArgumentError(ValueError):
    pass


def parse_args(args: Sequence[str], flags: Sequence[str] = FLAGS):
    """Positionals and ``--name value`` options; names in ``flags`` take no value (src/cli.jl:40-58)."""
    positional: List[str] = []
    options: Dict[str, str] = {}
    i = 0
    while i < len(args):
        a = args[i]
        if a.startswith("--") and a[2:] in flags:
            options[a[2:]] = "true"
            i += 1
        elif a.startswith("--"):
            if i + 1 >= len(args):
                raise ArgumentError(f"option {a} needs a value")
            options[a[2:]] = args[i + 1]
            i += 2
        else:
            positional.append(a)
            i += 1
    return positional, options


def check_options(options, allowed):
    for name in options:
        if name not in allowed:
            raise ArgumentError(f"unknown option --{name}")


def parse_option(kind, options, name, default):
    if name not in options:
        return default
    try:
        return kind(options[name])
    except ValueError:
        raise ArgumentError(f"--{name} expects {'an integer' if kind is int else 'a number'}, got {options[name]}") from None


def parse_ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise ArgumentError(f"a prompt is a list of token ids, got \"{text}\"") from None


def load_for_generation(model_dir: str, options):
    from .api import generation_defaults, load_model
    from .sampling import SamplingParams
    backend = options.get("backend", "fast")
    if backend not in ("fast", "plain"):
        raise ArgumentError("--backend expects fast or plain")
    dtype = options.get("dtype", "bfloat16")
    if dtype not in ("bfloat16", "float32"):
        raise ArgumentError("--dtype expects bfloat16 or float32")
    max_seqs = parse_option(int, options, "max-seqs", 8)
    engine = load_model(model_dir, dtype=dtype, backend=backend, max_seqs=max_seqs,
                        max_context=parse_option(int, options, "max-context", 4096))
    defaults, stop = generation_defaults(model_dir, engine)
    sampling = SamplingParams(temperature=parse_option(float, options, "temperature", defaults.temperature),
                              top_k=parse_option(int, options, "top-k", defaults.top_k),
                              top_p=parse_option(float, options, "top-p", defaults.top_p))
    if "stop-ids" in options:
        stop = parse_ids(options["stop-ids"])
    seed = parse_option(int, options, "seed", random.getrandbits(32))
    return engine, sampling, stop, seed


class TimedStream:
    """Records when the first two tokens arrived (src/cli.jl:158-187): decode speed is measured
    from the second token on, so that it excludes warm-up."""

    def __init__(self, out=None):
        self.out, self.start, self.first, self.second, self.count = out, time.time(), 0.0, 0.0, 0

    def __call__(self, request: int, token: int):
        now = time.time()
        if self.first == 0:
            self.first = now
        elif self.second == 0:
            self.second = now
        self.count += 1
        if self.out is not None:
            self.out.write(f"{token} ")
            self.out.flush()

    def summary(self, generated: int) -> str:
        stop = time.time()
        rate = (generated - 2) / (stop - self.second) if generated > 2 and stop > self.second else float("nan")
        ttft = (self.first or stop) - self.start
        return f"first token after {ttft:.2f} s, then {rate:.1f} tok/s"


def cmd_run(positional, options) -> None:
    check_options(options, GENERATION_OPTIONS)
    if len(positional) != 2:
        raise ArgumentError("run takes a model and a prompt")
    from .api import generate
    model_dir, prompt = positional
    ids = parse_ids(prompt)
    if not ids:
        raise ArgumentError("the prompt has no token ids")
    engine, sampling, stop, seed = load_for_generation(model_dir, options)
    stream = TimedStream(sys.stdout)
    out = generate(engine, ids, max_new_tokens=parse_option(int, options, "max-tokens", 512), sampling=sampling,
                   stop_ids=stop, seed=seed, on_token=stream)
    print(flush=True)
    print(f"[{len(ids)} prompt tokens, {len(out)} generated; {stream.summary(len(out))}]", file=sys.stderr)


def cmd_generate(positional, options) -> None:
    check_options(options, GENERATION_OPTIONS)
    if len(positional) != 2:
        raise ArgumentError("generate takes a model and a file of prompts")
    from .api import generate
    model_dir, path = positional
    lines = (sys.stdin if path == "-" else open(path)).read().splitlines()
    prompts = [parse_ids(l) for l in lines if l.strip()]
    if not prompts:
        raise ArgumentError("no prompts")
    engine, sampling, stop, seed = load_for_generation(model_dir, options)
    stream = TimedStream()
    outs = generate(engine, prompts, max_new_tokens=parse_option(int, options, "max-tokens", 512), sampling=sampling,
                    stop_ids=stop, seed=seed, on_token=stream)
    for o in outs:
        print(" ".join(str(t) for t in o))
    total = sum(len(o) for o in outs)
    print(f"[{sum(len(p) for p in prompts)} prompt tokens in {len(prompts)} prompts, {total} generated; "
          f"{stream.summary(total)}]", file=sys.stderr)


def cmd_random(positional, options) -> None:
    check_options(options, ("seed", "dtype"))
    if len(positional) != 2:
        raise ArgumentError("random takes a config.json and an output folder")
    import torch
    from .config import config_from_dict
    from .weights import write_model_folder
    with open(positional[0]) as f:
        config = config_from_dict(json.load(f))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}.get(options.get("dtype", "bfloat16"))
    if dtype is None:
        raise ArgumentError("--dtype expects bfloat16 or float32")
    print("wrote", write_model_folder(config, parse_option(int, options, "seed", 0), positional[1], dtype=dtype))


COMMANDS = {"run": cmd_run, "generate": cmd_generate, "random": cmd_random}


def cli(args: Sequence[str]) -> int:
    """Run the command line on ``args``; returns the process exit code (src/cli.jl:258-277)."""
    args = list(args)
    if not args or args[0] in ("-h", "--help", "help"):
        print(USAGE, end="")
        return 1 if not args else 0
    command = COMMANDS.get(args[0])
    if command is None:
        print(f"unknown command: {args[0]}\n", file=sys.stderr)
        print(USAGE, end="", file=sys.stderr)
        return 1
    try:
        command(*parse_args(args[1:]))
    except (ArgumentError, ValueError, FileNotFoundError, RuntimeError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


def main() -> None:
    sys.exit(cli(sys.argv[1:]))
