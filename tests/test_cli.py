"""The command line's forms that need no GPU: help, a random model folder from a configuration
file and a seed, and `inspect` of that folder (geometry, tensor check, kernel choice)."""
import json

import pytest

from llm_b200 import cli
from tiny import TINY_B


def test_help_names_every_form(capsys):
    assert cli.main(["--help"]) == 0
    text = capsys.readouterr().out
    for word in ("bench", "inspect", "random", "--max-tokens", "--temperature"):
        assert word in text
    assert cli.main([]) == 2                      # nothing to do: the same text, a failing status


def test_random_folder_and_inspect(tmp_path, capsys):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(TINY_B))
    out = tmp_path / "model"
    assert cli.main(["random", "--config", str(config), "--out", str(out), "--seed", "5"]) == 0
    assert (out / "config.json").is_file() and (out / "model.safetensors").is_file()
    capsys.readouterr()
    assert cli.main(["inspect", str(out)]) == 0
    text = capsys.readouterr().out
    assert "kernel plan" in text and "attention_generic" not in text.split("kernel plan")[1]
    assert "runnable" in text
    # the same seed writes the same bytes, another seed other bytes
    again = tmp_path / "again"
    cli.main(["random", "--config", str(config), "--out", str(again), "--seed", "5"])
    other = tmp_path / "other"
    cli.main(["random", "--config", str(config), "--out", str(other), "--seed", "6"])
    first = (out / "model.safetensors").read_bytes()
    assert first == (again / "model.safetensors").read_bytes()
    assert first != (other / "model.safetensors").read_bytes()


def test_a_prompt_that_is_no_list_of_ids_is_refused():
    with pytest.raises(SystemExit, match="bad list"):
        cli.main(["--model", "nowhere", "hello"])
    with pytest.raises(SystemExit, match="usage"):
        cli.main(["--model", "nowhere"])
