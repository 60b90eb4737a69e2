"""Interfaces and registries of the parts a decoder is put together from.

A part is built from its spec alone (`Part(spec)`), declares the tensors it
binds (`parameters()`), receives them once (`bind`) and then runs on the
tokens of a step (`forward`). No part knows which model it is in: sizes,
constants and tensor names all come with the spec, and what a step is
(which token belongs to which sequence at which position, where the cache
pages are) comes with the `StepContext`.

Registries map a spec's `kind` to the class that runs it:

    register_mixer("attention", AttentionMixer)
    build_mixer(spec)          # -> AttentionMixer(spec)

The same holds for feed-forwards, norms, position encodings and blocks.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..errors import Unsupported


@dataclass
class StepContext:
    """One step's batch as the parts see it. Device tensors are int32."""
    n_tokens: int                  # T: tokens of this step, packed sequence after sequence
    n_seqs: int                    # B
    dtype: torch.dtype             # activation dtype of the run (bfloat16 or float32)
    device: torch.device
    tok_pos: torch.Tensor          # [T] absolute position of each token
    tok_seq: torch.Tensor          # [T] index in the batch of each token's sequence
    cu_seqlens: torch.Tensor       # [B + 1] first packed token of each sequence
    seq_lens: torch.Tensor         # [B] length of each sequence after this step
    slot_ids: torch.Tensor         # [B] cache slot of each sequence
    block_tables: list             # per cache group: [B, width] physical pages
    cache: object                  # the PagedCache
    decode: bool                   # every sequence brings exactly one token
    new_counts: list               # host: tokens each sequence brings
    starts: list                   # host: position of each sequence's first new token
    max_len: int                   # host: longest sequence after this step
    workspace: object = None       # engine.workspace.Views of this step, or None
    seq_order: torch.Tensor = None # [B] the sequences by falling length (work lists start the longest first)
    extras: dict = field(default_factory=dict)

    def scratch(self, name: str, shape=None, dtype=None):
        """The planned buffer `name` of the part that is running, or None. With `shape` the
        front of the buffer in that form (blocks of different sizes share one plan)."""
        return self.workspace.get(name, shape, dtype) if self.workspace is not None else None


class Part:
    """Common to every part."""

    #: names of the csrc files whose kernels this part launches
    libraries: tuple = ()
    #: True if `forward` only launches work on the current stream and reads every
    #: per-step value from the context's device tensors, so that a decode step
    #: can be captured in a CUDA graph and replayed
    graph_safe: bool = False

    #: True if `forward` takes `emit=` (an ops.Emit, or None) and then leaves, together with its
    #: update of the residual stream, the next norm's input there (bfloat16 rows and their sums of
    #: squares); a block runs ops.cast_sumsq behind parts that do not
    emits: bool = False

    def parameters(self) -> dict:
        """tensor name -> ParamSpec of everything this part binds."""
        return {}

    def replay_key(self, step):
        """None (the default): a recorded pass must not stand in for a later pass of this part.
        Else a tuple that holds every host-side value of the step (`step` has the host fields of a
        StepContext: n_tokens, n_seqs, decode, new_counts, starts, max_len) that the arguments of
        this part's launches depend on, beyond n_tokens and n_seqs; everything else the part's
        kernels read from the context's device arrays. Two passes with equal keys then make the
        same launches with the same arguments, and the engine may run the second from the record
        of the first, walked by the native host library."""
        return None

    def fold_input_norm(self, gain) -> bool:
        """Offered by the block after `bind`, where the norm in front of this part is an RMS norm
        (y = x / sqrt(mean(x^2) + eps) * gain): take `gain` (float32 [hidden]) into the weights
        that read the part's input and answer True. `forward` then receives an ops.FoldedNorm (the
        un-normalised rows as bfloat16, their sums of squares, eps) instead of normalised rows, and
        scales by the norm's factor itself: y . W^T = rstd(x) * (x . (gain * W)^T). The default
        keeps the norm as a kernel of its own."""
        return False

    def kernel_shapes(self, dtype, token_counts) -> list:
        """(label, family, chooser arguments) of the kernel choices this part's forward pass makes
        for steps of `token_counts` tokens: what `inspect` prints and the plan identity hashes."""
        return []

    def bind(self, tensors: dict, dtype: torch.dtype, device) -> None:
        """Take the declared tensors (CPU or device, storage dtype) and keep
        what `forward` needs on `device` for a run in `dtype`."""

    def prepare(self, max_positions: int, device) -> None:
        """Build tables that depend on the longest sequence the engine allows."""

    def scratch_requests(self, n_tokens: int, dtype) -> list:
        """engine.workspace.BufferRequest for every activation `forward` writes for
        n_tokens tokens, with phases counted from 0 inside this part. A part that
        declares nothing lets its kernels allocate."""
        return []

    def weights(self) -> list:
        """The tensors a step reads in full (for the byte count of a decode step)."""
        return [v for v in vars(self).values() if isinstance(v, torch.Tensor)]


class Mixer(Part):
    """Mixes information between the positions of a sequence."""

    def kv_request(self):
        """A cache.KvRequest if the mixer keeps keys and values, else None."""
        return None

    def state_request(self):
        """A cache.StateRequest if the mixer keeps fixed-size state, else None."""
        return None

    def forward(self, h, ctx: StepContext, entry: int, cache_entry: int, residual) -> None:
        """Add the mixer's output for normed input h [T, hidden] to `residual`
        (float32 [T, hidden]) in place. `entry` is this run's place in the
        schedule (its own state and cache storage); `cache_entry` is the place
        whose keys and values it reads (== entry unless it shares a cache)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h, ctx: StepContext, residual) -> None:
        """Add the feed-forward output for normed input h to `residual` in place."""
        raise NotImplementedError


class Norm(Part):
    def forward(self, x, out_dtype, rows=None, out=None):
        """Normalise float32 rows x [T, hidden] (or the gathered `rows`) -> out_dtype
        (into `out` if given)."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Owned by the mixers that use it; shared between layers with equal specs."""


class Block(Part):
    def forward(self, x, ctx: StepContext, entry: int, cache_entry: int) -> None:
        """Run one layer on the residual stream x (float32 [T, hidden]) in place."""
        raise NotImplementedError


_REGISTRIES = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def _register(family, kind, cls):
    _REGISTRIES[family][kind] = cls


def _build(family, spec, *args):
    kind = getattr(spec, "kind", None)
    try:
        cls = _REGISTRIES[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES[family])) or "none"
        raise Unsupported(f"no {family} of kind '{kind}' is registered (known: {known})") from None
    return cls(spec, *args)


def register_mixer(kind, cls): _register("mixer", kind, cls)
def register_feed_forward(kind, cls): _register("feed_forward", kind, cls)
def register_norm(kind, cls): _register("norm", kind, cls)
def register_position(kind, cls): _register("position", kind, cls)
def register_block(kind, cls): _register("block", kind, cls)


def build_mixer(spec): return _build("mixer", spec)
def build_feed_forward(spec): return _build("feed_forward", spec)
def build_norm(spec): return _build("norm", spec)
def build_block(spec): return _build("block", spec)


_position_cache: dict = {}


def build_position(spec):
    """Position encodings with equal specs are one object (one table)."""
    if spec is None:
        return None
    try:
        key = (getattr(spec, "kind", None), spec)
        hash(key)
    except TypeError:
        return _build("position", spec)
    if key not in _position_cache:
        _position_cache[key] = _build("position", spec)
    return _position_cache[key]


def to_run_dtype(t: torch.Tensor, dtype, device) -> torch.Tensor:
    return t.to(device=device, dtype=dtype).contiguous()


def to_float32(t: torch.Tensor, device) -> torch.Tensor:
    return t.to(device=device, dtype=torch.float32).contiguous()
