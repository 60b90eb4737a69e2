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
        assert error.max() <= 2e-4 * scale
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
