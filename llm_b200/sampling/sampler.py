"""The device sampler: per-sequence parameters, recent-token windows and
generator states, and one kernel launch per step for all live sequences."""
from __future__ import annotations

import torch

from .. import ops
from ..errors import KernelError

MASK64 = (1 << 64) - 1


def _as_signed(value: int) -> int:
    value &= MASK64
    return value - (1 << 64) if value >= (1 << 63) else value


class BatchSampler:
    """State for one batch: row i belongs to the batch's i-th sequence for its
    whole life, whichever rows of logits it later appears in.

    The generator of a sequence starts at `seed | 1` and advances once per
    drawn token, as one `Sampler` per request does in MythEclipse/llm
    (apps/engine/src/sampler.rs:43-48); the window holds generated tokens only
    (apps/engine/src/generate.rs:84-89)."""

    def __init__(self, params: list, vocab: int, device):
        for p in params:
            p.check(vocab)
        self.n = len(params)
        self.vocab = vocab
        self.device = torch.device(device)
        self.params = params
        self.all_greedy = all(p.temperature <= 0.0 and
                              (p.repeat_penalty == 1.0 or p.repeat_last_n == 0) for p in params)
        cap = max([p.repeat_last_n for p in params] + [1])
        f = torch.tensor([[p.temperature, p.top_p, p.min_p, p.repeat_penalty] for p in params],
                         dtype=torch.float32)
        i = torch.tensor([[p.top_k, p.repeat_last_n] for p in params], dtype=torch.int32)
        rng = torch.tensor([_as_signed(p.seed | 1) for p in params], dtype=torch.int64)
        self.fparams = f.to(self.device)
        self.iparams = i.to(self.device)
        self.rng = rng.to(self.device)
        self.recent = torch.zeros((self.n, cap), dtype=torch.int32, device=self.device)
        self.recent_len = torch.zeros((self.n,), dtype=torch.int32, device=self.device)
        self.status = torch.zeros((self.n,), dtype=torch.int32, device=self.device)

    def sample(self, logits: torch.Tensor, rows: list) -> torch.Tensor:
        """One token for every row of `logits` (float32 [len(rows), vocab],
        overwritten); rows[i] is the batch index of the sequence in row i.
        Returns int32 [len(rows)] on the device and records the tokens in the
        sequences' windows."""
        if logits.shape[0] != len(rows):
            raise KernelError("sample: one logits row per live sequence is needed")
        if self.all_greedy:
            return ops.argmax_rows(logits)
        state_rows = None
        if len(rows) != self.n or rows != list(range(self.n)):
            state_rows = torch.tensor(rows, dtype=torch.int32, device=self.device)
        out = torch.empty((len(rows),), dtype=torch.int32, device=self.device)
        # one launch: the kernel finds each row's sequence state through state_rows and also
        # records the drawn tokens in the windows (a ring over the generated tokens)
        ops.sample_rows(logits, self.fparams, self.iparams, self.recent, self.recent_len, self.rng, out,
                        self.status, record=True, state_rows=state_rows)
        return out

    def check_status(self, status=None) -> None:
        """Raise if the kernel refused a row since the last check. The kernel only ever sets
        the flags; they are cleared here, after they were read. `status`: a host copy that the
        caller fetched together with the ids (else the device array is read)."""
        if self.all_greedy:
            return
        flags = self.status if status is None else status
        if bool((flags != 0).any()):
            self.status.zero_()
            raise KernelError("the device sampler refused a row (top_k beyond its limit, or too many "
                              "equal logits at the top-k cut); token 0 was emitted in its place")
