"""The command line's parsing and exit codes, as far as they need no device (the reference's
test/cli.jl:11-36 is the model: ``--name value`` options, flags, unknown options refused, exit code 0 or 1),
and the ``random`` command, which writes a model folder on the CPU."""
import json
import os

import pytest

import helpers
from tileinfer_b200.cli import ArgumentError, TimedStream, check_options, cli, parse_args, parse_ids, parse_option


def test_options_and_positionals():
    pos, opt = parse_args(["model", "1 2 3", "--max-tokens", "7", "--temperature", "0.5"])
    assert pos == ["model", "1 2 3"] and opt == {"max-tokens": "7", "temperature": "0.5"}
    pos, opt = parse_args(["--raw", "m", "--seed", "3"], flags=("raw",))
    assert pos == ["m"] and opt == {"raw": "true", "seed": "3"}
    with pytest.raises(ArgumentError, match="needs a value"):
        parse_args(["m", "--seed"])
    check_options({"seed": "1"}, ("seed", "dtype"))
    with pytest.raises(ArgumentError, match="unknown option --sed"):
        check_options({"sed": "1"}, ("seed", "dtype"))
    assert parse_option(int, {"seed": "12"}, "seed", 0) == 12 and parse_option(float, {}, "temperature", 0.25) == 0.25
    with pytest.raises(ArgumentError, match="--seed expects an integer, got x"):
        parse_option(int, {"seed": "x"}, "seed", 0)
    with pytest.raises(ArgumentError, match="--top-p expects a number"):
        parse_option(float, {"top-p": "much"}, "top-p", 1.0)


def test_prompts_are_token_ids():
    assert parse_ids("5 17 3") == [5, 17, 3] and parse_ids("5,17, 3") == [5, 17, 3] and parse_ids("") == []
    with pytest.raises(ArgumentError, match="token ids"):
        parse_ids("hello world")


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
    s = TimedStream()
    for t in range(5):
        s(0, t)
    assert s.count == 5 and 0 < s.first <= s.second
    text = s.summary(5)
    assert text.startswith("first token after ") and text.endswith(" tok/s")
    assert "nan" in TimedStream().summary(1)                     # no rate from fewer than three tokens
