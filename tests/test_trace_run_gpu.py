"""bin/trace_run as a user runs it: a child process, steps through standard
input, logits from files; whole requests, the last 32 tokens one by one, and
batches of unequal lengths on a cache too small to hold both batches at once."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama
from tiny import make_folder, random_tokens

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


class Replay:
    def __init__(self, model, dtype, out, max_tokens):
        self.out = Path(out)
        self.process = subprocess.Popen(
            [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype,
             "--out", str(out), "--max-tokens", str(max_tokens)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        self.step_id = 0

    def step(self, entries, end=()):
        line = json.dumps({"step": self.step_id, "entries": entries, "end": list(end)})
        self.process.stdin.write(line + "\n")
        self.process.stdin.flush()
        answer = self.process.stdout.readline().strip()
        assert answer == f"done {self.step_id}", answer
        path = self.out / f"{self.step_id}.f32"
        self.step_id += 1
        return np.fromfile(path, dtype="<f4") if path.exists() else None

    def close(self):
        self.process.stdin.close()
        assert self.process.wait(timeout=60) == 0


def check(got, want, dtype):
    want = want.numpy()
    got = got.reshape(want.shape)
    scale = max(float(np.abs(want).max()), 1.0)
    error = np.abs(got - want)
    if dtype == "float32":
        assert error.max() <= 5e-5 * scale
    else:
        assert error.max() <= 0.04 * scale and error.mean() <= 0.008 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["A", "B"])
def test_replay(tmp_path, dtype, which):
    folder = make_folder(tmp_path, which, torch.bfloat16)
    config, weights = plain_llama.read_model_folder(folder)
    vocab = config["vocab_size"]
    requests = {name: random_tokens(n, vocab, 40 + n) for name, n in
                (("a", 70), ("b", 33), ("c", 100), ("d", 41), ("e", 64))}
    expected = {name: plain_llama.forward(config, weights, t) for name, t in requests.items()}
    replay = Replay(folder, dtype, tmp_path / f"out_{dtype}", max_tokens=64 * 5)
    try:
        # whole, each alone
        for name in ("a", "b"):
            t = requests[name]
            got = replay.step([{"id": name + "-whole", "tokens": t, "want": list(range(len(t)))}],
                              end=[name + "-whole"])
            check(got, expected[name], dtype)
        # the last 32 tokens one by one
        t = requests["c"]
        head = len(t) - 32
        got = replay.step([{"id": "c", "tokens": t[:head], "want": list(range(head))}])
        check(got, expected["c"][:head], dtype)
        for k in range(head, len(t)):
            got = replay.step([{"id": "c", "tokens": [t[k]], "want": [0]}],
                              end=["c"] if k == len(t) - 1 else [])
            check(got, expected["c"][k:k + 1], dtype)
        # two batches of unequal lengths, one after the other; nothing wanted in some steps
        for batch in (("a", "b", "d"), ("e", "c", "b")):
            starts = {name: max(1, len(requests[name]) - 6 - 2 * i) for i, name in enumerate(batch)}
            got = replay.step([{"id": n, "tokens": requests[n][:starts[n]], "want": [starts[n] - 1]}
                               for n in batch])
            want = torch.stack([expected[n][starts[n] - 1] for n in batch])
            check(got, want, dtype)
            live, k = list(batch), 0
            while live:
                entries, rows, ending = [], [], []
                for n in live:
                    at = starts[n] + k
                    wanted = [0] if k % 2 == 0 else []
                    entries.append({"id": n, "tokens": [requests[n][at]], "want": wanted})
                    if wanted:
                        rows.append(expected[n][at])
                    if at == len(requests[n]) - 1:
                        ending.append(n)
                got = replay.step(entries, end=ending)
                if rows:
                    check(got, torch.stack(rows), dtype)
                else:
                    assert got is None
                live = [n for n in live if n not in ending]
                k += 1
    finally:
        replay.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_three_modes_of_a_trace_file(tmp_path, dtype):
    """--trace FILE --mode whole|tail32|batches: the program makes the steps itself and writes
    one logits file and one sidecar per request; all three modes agree with the plain
    implementation at every position, on a cache that holds one batch but not both."""
    folder = make_folder(tmp_path, "D", torch.bfloat16)
    config, weights = plain_llama.read_model_folder(folder)
    vocab = config["vocab_size"]
    requests = {name: random_tokens(n, vocab, 60 + n) for name, n in
                (("a", 70), ("b", 33), ("c", 100), ("d", 1), ("e", 64))}
    trace = tmp_path / "trace.json"
    trace.write_text(json.dumps({"requests": [{"id": k, "tokens": t} for k, t in requests.items()],
                                 "batches": [["a", "b", "c"], ["d", "e", "b"]]}))
    expected = {name: plain_llama.forward(config, weights, t) for name, t in requests.items()}
    for mode in ("whole", "tail32", "batches"):
        out = tmp_path / f"out_{dtype}_{mode}"
        done = subprocess.run(
            [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
             "--out", str(out), "--max-tokens", str(64 * 5), "--trace", str(trace), "--mode", mode],
            stdin=subprocess.DEVNULL, stdout=subprocess.PIPE, text=True, timeout=600)
        assert done.returncode == 0
        assert done.stdout.strip().splitlines()[-1].startswith("done ")
        for name, tokens in requests.items():
            side = json.loads((out / f"logits_{name}.json").read_text())
            assert side["id"] == name and side["vocab"] == vocab and side["mode"] == mode
            assert side["positions"] == list(range(len(tokens)))
            check(np.fromfile(out / f"logits_{name}.f32", dtype="<f4"), expected[name], dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_of_continued_prompts_and_a_mixed_step(tmp_path, dtype):
    """Through the program: a prompt that arrives in three pieces (the later pieces attend to the
    cache of the earlier ones), and a step in which two requests bring one token while a third
    brings 70 tokens onto a slot that already holds 50."""
    folder = make_folder(tmp_path, "F", torch.bfloat16)
    config, weights = plain_llama.read_model_folder(folder)
    vocab = config["vocab_size"]
    a, b, c = (random_tokens(n, vocab, 70 + n) for n in (300, 90, 130))
    want = {k: plain_llama.forward(config, weights, t) for k, t in (("a", a), ("b", b), ("c", c))}
    replay = Replay(folder, dtype, tmp_path / f"out_{dtype}", max_tokens=64 * 10)
    try:
        at = 0
        for piece in (48, 152, 100):
            got = replay.step([{"id": "a", "tokens": a[at:at + piece], "want": list(range(piece))}],
                              end=["a"] if at + piece == len(a) else [])
            check(got, want["a"][at:at + piece], dtype)
            at += piece
        got = replay.step([{"id": "b", "tokens": b[:80], "want": [79]}, {"id": "c", "tokens": c[:50], "want": [49]}])
        check(got, torch.stack([want["b"][79], want["c"][49]]), dtype)
        got = replay.step([{"id": "b", "tokens": [b[80]], "want": [0]},
                           {"id": "c", "tokens": c[50:120], "want": [0, 69]}])
        check(got, torch.stack([want["b"][80], want["c"][50], want["c"][119]]), dtype)
        got = replay.step([{"id": "b", "tokens": [b[81]], "want": [0]}, {"id": "c", "tokens": [c[120]], "want": [0]}],
                          end=["b", "c"])
        check(got, torch.stack([want["b"][81], want["c"][120]]), dtype)
    finally:
        replay.close()
