"""``tileinfer`` command line, in the manner of AntoineBut/TileInfer.jl's (src/cli.jl:4-34, 253-277):
``tileinfer <command> <arguments> [--name value ...]``, unknown options refused, exit code 0 or 1, a
statistics line on stderr whose decode rate counts from the second token (src/cli.jl:177-187). Its
option names and meanings are kept where it has them (``--max-tokens``, ``--max-context``,
``--temperature``, ``--top-k``, ``--top-p``, ``--seed``, ``--backend``). Prompts are token ids (the
library has no tokenizer), so ``run`` takes ids where the reference takes text; ``pull/ls/rm/chat``
have no counterpart: a model is a local folder.

Everything the parser knows is in two tables: ``OPTIONS`` (name, type or choices, default, help)
and ``COMMANDS`` (positional arguments, the options a command takes, its function). The usage text
is printed from them.
"""
from __future__ import annotations

import json
import random
import sys
import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple


class ArgumentError(ValueError):
    pass


def token_ids(text: str) -> List[int]:
    """Token ids separated by spaces or commas."""
    try:
        return [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise ArgumentError(f"a prompt is a list of token ids, got \"{text}\"") from None


@dataclass(frozen=True)
class Option:
    name: str
    kind: object                    # int, float, token_ids, or a tuple of allowed words
    default: object                 # None: decided later (the model's generation defaults, a random seed)
    help: str

    def read(self, text: str):
        if isinstance(self.kind, tuple):
            if text not in self.kind:
                raise ArgumentError(f"--{self.name} expects {' or '.join(self.kind)}")
            return text
        if self.kind is token_ids:
            return token_ids(text)
        try:
            return self.kind(text)
        except ValueError:
            what = "an integer" if self.kind is int else "a number"
            raise ArgumentError(f"--{self.name} expects {what}, got {text}") from None

    def usage(self) -> str:
        value = "|".join(self.kind) if isinstance(self.kind, tuple) else {int: "N", float: "X", token_ids: "IDS"}[self.kind]
        default = f" (default {self.default})" if self.default is not None else ""
        return f"  --{self.name} {value}".ljust(34) + self.help + default


OPTIONS: Dict[str, Option] = {o.name: o for o in (
    Option("max-tokens", int, 512, "tokens to generate per prompt at most"),
    Option("max-context", int, 4096, "longest sequence in tokens; sizes the KV cache"),
    Option("temperature", float, None, "0 for greedy (default: the model's generation_config.json, else 0)"),
    Option("top-k", int, None, "keep the K most likely tokens (0: all)"),
    Option("top-p", float, None, "keep the smallest set of tokens with this much probability (1: all)"),
    Option("seed", int, None, "random seed (default: drawn at random)"),
    Option("backend", ("fast", "plain"), "fast", "tensor-core kernels or the plain reference kernels"),
    Option("dtype", ("bfloat16", "float32"), "bfloat16", "element type of weights, activations and cache"),
    Option("max-seqs", int, 8, "sequences per batch at most"),
    Option("stop-ids", token_ids, None, "stop tokens instead of the configuration's EOS ids (\"\" for none)"),
)}
GENERATION = ("max-tokens", "max-context", "temperature", "top-k", "top-p", "seed", "backend", "dtype", "max-seqs", "stop-ids")


@dataclass(frozen=True)
class Command:
    name: str
    positionals: Tuple[str, ...]
    takes: str                      # "run takes a model and a prompt"
    options: Tuple[str, ...]
    help: str
    run: Callable

    def read(self, args: Sequence[str]):
        """Positionals and typed option values of ``args``; options not given have their defaults."""
        positional: List[str] = []
        values = {name: OPTIONS[name].default for name in self.options}
        words = iter(args)
        for word in words:
            if not word.startswith("--"):
                positional.append(word)
                continue
            name = word[2:]
            if name not in self.options:
                raise ArgumentError(f"unknown option --{name}")
            text = next(words, None)
            if text is None:
                raise ArgumentError(f"option --{name} needs a value")
            values[name] = OPTIONS[name].read(text)
        if len(positional) != len(self.positionals):
            raise ArgumentError(self.takes)
        return positional, values


class GenerationStats:
    """An ``on_token`` callback that notes when the first two tokens arrived: the decode rate is counted from
    the second token on, so that it leaves out the prompt's step and warm-up (src/cli.jl:158-187)."""

    def __init__(self, out=None):
        self.out, self.count = out, 0
        self.started = time.time()
        self.arrivals: List[float] = []             # of the first two tokens

    def __call__(self, request: int, token: int):
        if len(self.arrivals) < 2:
            self.arrivals.append(time.time())
        self.count += 1
        if self.out is not None:
            self.out.write(f"{token} ")
            self.out.flush()

    def summary(self, generated: int) -> str:
        now = time.time()
        first = self.arrivals[0] if self.arrivals else now
        rate = float("nan")
        if generated > 2 and len(self.arrivals) == 2 and now > self.arrivals[1]:
            rate = (generated - 2) / (now - self.arrivals[1])
        return f"first token after {first - self.started:.2f} s, then {rate:.1f} tok/s"


def load_for_generation(model_dir: str, values):
    """The engine and the sampling settings of a ``run`` or ``generate`` call: options given on the command
    line win over the model's generation_config.json."""
    from .api import generation_defaults, load_model
    from .sampling import SamplingParams
    engine = load_model(model_dir, dtype=values["dtype"], backend=values["backend"], max_seqs=values["max-seqs"],
                        max_context=values["max-context"])
    defaults, stop = generation_defaults(model_dir, engine)
    pick = lambda name, fallback: fallback if values[name] is None else values[name]
    sampling = SamplingParams(temperature=pick("temperature", defaults.temperature), top_k=pick("top-k", defaults.top_k),
                              top_p=pick("top-p", defaults.top_p))
    return engine, sampling, pick("stop-ids", stop), pick("seed", random.getrandbits(32))


def cmd_run(positional, values) -> None:
    from .api import generate
    model_dir, prompt = positional
    ids = token_ids(prompt)
    if not ids:
        raise ArgumentError("the prompt has no token ids")
    engine, sampling, stop, seed = load_for_generation(model_dir, values)
    stats = GenerationStats(sys.stdout)
    out = generate(engine, ids, max_new_tokens=values["max-tokens"], sampling=sampling, stop_ids=stop, seed=seed, on_token=stats)
    print(flush=True)
    print(f"[{len(ids)} prompt tokens, {len(out)} generated; {stats.summary(len(out))}]", file=sys.stderr)


def cmd_generate(positional, values) -> None:
    from .api import generate
    model_dir, path = positional
    lines = (sys.stdin if path == "-" else open(path)).read().splitlines()
    prompts = [token_ids(l) for l in lines if l.strip()]
    if not prompts:
        raise ArgumentError("no prompts")
    engine, sampling, stop, seed = load_for_generation(model_dir, values)
    stats = GenerationStats()
    outs = generate(engine, prompts, max_new_tokens=values["max-tokens"], sampling=sampling, stop_ids=stop, seed=seed,
                    on_token=stats)
    for o in outs:
        print(" ".join(str(t) for t in o))
    total = sum(len(o) for o in outs)
    print(f"[{sum(len(p) for p in prompts)} prompt tokens in {len(prompts)} prompts, {total} generated; "
          f"{stats.summary(total)}]", file=sys.stderr)


def cmd_random(positional, values) -> None:
    import torch
    from .config import config_from_dict
    from .weights import write_model_folder
    with open(positional[0]) as f:
        config = config_from_dict(json.load(f))
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[values["dtype"]]
    print("wrote", write_model_folder(config, values["seed"] or 0, positional[1], dtype=dtype))


COMMANDS: Dict[str, Command] = {c.name: c for c in (
    Command("run", ("model", "prompt"), "run takes a model and a prompt", GENERATION,
            "generate a continuation of <prompt>: token ids separated by spaces or commas; <model> is a folder with "
            "config.json and safetensors", cmd_run),
    Command("generate", ("model", "file"), "generate takes a model and a file of prompts", GENERATION,
            "the same for a batch: one prompt a line in <file> (\"-\" reads standard input); prints one line of ids per prompt",
            cmd_generate),
    Command("random", ("config.json", "out"), "random takes a config.json and an output folder", ("seed", "dtype"),
            "write a model folder with random weights for a configuration", cmd_random),
)}


def usage() -> str:
    lines = ["usage: tileinfer <command> [arguments]", "", "commands:"]
    for c in COMMANDS.values():
        head = f"  {c.name} " + " ".join(f"<{p}>" for p in c.positionals) + " [options]"
        lines += [head, f"      {c.help}"]
    lines += ["", "options of run and generate:"] + [OPTIONS[n].usage() for n in GENERATION]
    lines += ["", "options of random: --seed N (default 0), --dtype bfloat16|float32"]
    return "\n".join(lines) + "\n"


def cli(args: Sequence[str]) -> int:
    """Run the command line on ``args``; returns the process exit code: 0, or 1 after an error message on
    stderr (src/cli.jl:258-277)."""
    args = list(args)
    if not args or args[0] in ("-h", "--help", "help"):
        print(usage(), end="")
        return 0 if args else 1
    command = COMMANDS.get(args[0])
    if command is None:
        print(f"unknown command: {args[0]}\n", file=sys.stderr)
        print(usage(), end="", file=sys.stderr)
        return 1
    try:
        command.run(*command.read(args[1:]))
    except (ArgumentError, ValueError, FileNotFoundError, RuntimeError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    return 0


def main() -> None:
    sys.exit(cli(sys.argv[1:]))
