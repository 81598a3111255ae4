"""The command line's parsing and exit codes, as far as they need no device (the reference's
test/cli.jl:11-36 is the model: ``--name value`` options, flags, unknown options refused, exit code 0 or 1),
and the ``random`` command, which writes a model folder on the CPU."""
import json
import os

import pytest

import helpers
from tileinfer_b200.cli import COMMANDS, OPTIONS, ArgumentError, GenerationStats, cli, token_ids, usage


def test_options_and_positionals():
    run = COMMANDS["run"]
    pos, values = run.read(["model", "1 2 3", "--max-tokens", "7", "--temperature", "0.5"])
    assert pos == ["model", "1 2 3"] and values["max-tokens"] == 7 and values["temperature"] == 0.5
    assert values["max-context"] == 4096 and values["backend"] == "fast" and values["seed"] is None      # defaults
    pos, values = run.read(["--seed", "3", "m", "4,5", "--stop-ids", ""])
    assert pos == ["m", "4,5"] and values["seed"] == 3 and values["stop-ids"] == []
    with pytest.raises(ArgumentError, match="option --seed needs a value"):
        run.read(["m", "1", "--seed"])
    with pytest.raises(ArgumentError, match="unknown option --sed"):
        run.read(["m", "1", "--sed", "1"])
    with pytest.raises(ArgumentError, match="unknown option --max-tokens"):
        COMMANDS["random"].read(["c.json", "out", "--max-tokens", "3"])
    with pytest.raises(ArgumentError, match="--seed expects an integer, got x"):
        run.read(["m", "1", "--seed", "x"])
    with pytest.raises(ArgumentError, match="--top-p expects a number"):
        run.read(["m", "1", "--top-p", "much"])
    with pytest.raises(ArgumentError, match="run takes a model and a prompt"):
        run.read(["m"])
    # The reference's option names, where it has them (src/cli.jl:14-33).
    assert {"max-tokens", "max-context", "temperature", "top-k", "top-p", "seed", "backend"} <= set(OPTIONS)
    text = usage()
    assert all(f"--{name}" in text for name in OPTIONS) and all(name in text for name in COMMANDS)


def test_prompts_are_token_ids():
    assert token_ids("5 17 3") == [5, 17, 3] and token_ids("5,17, 3") == [5, 17, 3] and token_ids("") == []
    with pytest.raises(ArgumentError, match="token ids"):
        token_ids("hello world")


def test_exit_codes_and_messages(capsys, tmp_path):
    assert cli([]) == 1 and "usage: tileinfer" in capsys.readouterr().out
    assert cli(["help"]) == 0 and "run <model> <prompt>" in capsys.readouterr().out
    assert cli(["frobnicate"]) == 1 and "unknown command: frobnicate" in capsys.readouterr().err
    assert cli(["run", "folder"]) == 1 and "run takes a model and a prompt" in capsys.readouterr().err
    assert cli(["run", "folder", "1 2", "--bogus", "1"]) == 1 and "unknown option --bogus" in capsys.readouterr().err
    assert cli(["run", "folder", "one two"]) == 1 and "token ids" in capsys.readouterr().err
    assert cli(["run", "folder", " "]) == 1 and "no token ids" in capsys.readouterr().err
    assert cli(["run", "folder", "1", "--backend", "cpu"]) == 1 and "--backend expects fast or plain" in capsys.readouterr().err
    assert cli(["run", "folder", "1", "--dtype", "float16"]) == 1 and "--dtype expects" in capsys.readouterr().err
    empty = tmp_path / "prompts.txt"
    empty.write_text("\n\n")
    assert cli(["generate", "folder", str(empty)]) == 1 and "no prompts" in capsys.readouterr().err
    assert cli(["generate", "folder"]) == 1 and "a file of prompts" in capsys.readouterr().err
    assert cli(["random", "nowhere.json"]) == 1 and "random takes" in capsys.readouterr().err


def test_random_writes_a_model_folder(tmp_path, capsys):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(helpers.TINY_A))
    out = tmp_path / "model"
    assert cli(["random", str(cfg), str(out), "--seed", "4"]) == 0
    assert "wrote" in capsys.readouterr().out
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    assert json.loads((out / "config.json").read_text())["hidden_size"] == helpers.TINY_A["hidden_size"]
    assert cli(["random", str(cfg), str(out), "--dtype", "int8"]) == 1 and "--dtype expects" in capsys.readouterr().err
    assert cli(["random", str(tmp_path / "missing.json"), str(out)]) == 1


def test_the_statistics_line_counts_from_the_second_token():
    s = GenerationStats()
    for t in range(5):
        s(0, t)
    assert s.count == 5 and len(s.arrivals) == 2 and s.started <= s.arrivals[0] <= s.arrivals[1]
    text = s.summary(5)
    assert text.startswith("first token after ") and text.endswith(" tok/s") and "nan" not in text
    assert "nan" in GenerationStats().summary(1)                 # no rate from fewer than three tokens
