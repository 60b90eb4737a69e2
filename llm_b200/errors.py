"""Error types of the library.

The kinds follow the engine error enum of MythEclipse/llm
(apps/engine/src/error.rs:9-17): a bad file or value (Format), a missing
configuration key (MissingKey), missing or mismatched tensors (WeightError),
a feature that is not built (Unsupported), a full cache (ContextFull,
CacheFull) and a missing or failing native extension (KernelError).
"""
from __future__ import annotations


class LlmError(Exception):
    """Base of every error the library raises on purpose."""


class FormatError(LlmError):
    """A file or a value that cannot be read as what it claims to be."""


class MissingKey(LlmError):
    """A required configuration key is absent."""

    def __init__(self, key: str, where: str = "config.json"):
        super().__init__(f"{where}: required key '{key}' is missing")
        self.key = key


class Unsupported(LlmError):
    """The configuration asks for something the library does not build."""


class WeightError(LlmError):
    """Tensors of a checkpoint do not match what the model declares.

    One error lists everything: `missing` names, `unexpected` names and
    `mismatched` entries (name, found shape/dtype, expected shape).
    """

    def __init__(self, missing=(), unexpected=(), mismatched=(), where: str = ""):
        self.missing = sorted(missing)
        self.unexpected = sorted(unexpected)
        self.mismatched = sorted(mismatched)
        lines = [f"weights of {where or 'model'} do not match the configuration:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, found, expected in self.mismatched:
            lines.append(f"  wrong shape: {name} has {found}, expected {expected}")
        super().__init__("\n".join(lines))


class ContextFull(LlmError):
    """A sequence would grow past the positions its model or cache allows."""

    def __init__(self, used: int, capacity: int):
        super().__init__(f"context full: {used} positions used of {capacity}")
        self.used = used
        self.capacity = capacity


class CacheFull(LlmError):
    """No free slot or page is left in the cache."""


class KernelError(LlmError):
    """The native extension is missing, failed to build, or refused a size."""
