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


@pytest.mark.gpu
def test_completion_prints_the_tokens_of_the_plain_implementation(tmp_path, capsys):
    """`python -m llm_b200 --model DIR --temperature 0 --dtype float32 ID ...`: the generated ids on
    standard output are the plain implementation's greedy ids, the statistics go to standard error."""
    import torch

    import plain_llama
    from tiny import make_folder, random_tokens
    folder = make_folder(tmp_path, "B", torch.bfloat16)
    config, weights = plain_llama.read_model_folder(folder)
    prompt = random_tokens(9, config["vocab_size"], 3)
    want, _ = plain_llama.generate(config, weights, prompt, 7, temperature=0.0, stop_tokens=(1, 5))
    code = cli.main(["--model", str(folder), "--dtype", "float32", "--context", "64", "--max-tokens", "7",
                     "--temperature", "0", ",".join(str(t) for t in prompt[:4])] + [str(t) for t in prompt[4:]])
    captured = capsys.readouterr()
    assert code == 0
    assert [int(t) for t in captured.out.split()] == want
    assert "prompt tokens" in captured.err and "stop:" in captured.err


@pytest.mark.gpu
def test_bench_runs_both_tests_on_a_folder_and_on_a_random_shape(tmp_path, capsys):
    """`bench -m DIR -p 40,8 -n 6 -b 1,3 -r 2 -o json`: one row per (test, batch) with a positive mean,
    pp and tg named as in MythEclipse/llm's bench; the table form ends with the identities."""
    import torch

    from tiny import make_folder
    folder = make_folder(tmp_path, "D", torch.bfloat16)
    assert cli.main(["bench", "-m", str(folder), "-c", "128", "-p", "40,8", "-n", "6", "-b", "1,3", "-r", "2",
                     "-o", "json"]) == 0
    rows = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert [(r["test"], r["batch"]) for r in rows] == [("pp40", 1), ("pp8", 1), ("tg6", 1),
                                                       ("pp40", 3), ("pp8", 3), ("tg6", 3)]
    assert all(r["avg_ts"] > 0 and r["stddev_ts"] >= 0 for r in rows)
    assert cli.main(["bench", "--random", "llama-3.2-1b", "--layers", "1", "-c", "256", "-p", "32", "-n", "4",
                     "-r", "1"]) == 0
    text = capsys.readouterr().out
    assert "| pp32 |" in text and "| tg4 |" in text and "kernel plan" in text and "scratch plan" in text
    with pytest.raises(SystemExit, match="one of them"):
        cli.main(["bench"])
