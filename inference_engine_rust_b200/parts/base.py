"""Interfaces of the parts a layer is assembled from, the registry that maps a part's
`kind` to its class, and the objects every part shares during a step.

A part is built from its own `PartSpec` (sizes and constants) and a `Runtime`; it never
learns which model it belongs to.  Adding a part means registering a class under a new
kind; the configuration then names that kind for the layers that use it.

    norm      Norm(spec, hidden_size, rt)        .forward(x_f32, out, ctx, rows_idx=None, rows=None)
    position  PositionEncoding(spec, head_dim, rt)   .encode(qkv, ctx, heads, kv_heads)   [.rotary_constants()]
    mixer     Mixer(spec, rt)                    .forward(xn, residual, ctx, cache_view, writes_cache)
    ffn       FeedForward(spec, rt)              .forward(xn, residual, ctx)
    block     Block(layer_spec, norm1, mixer, norm2, ffn, rt[, extra_norms={role: norm}])   .forward(x, ctx, cache_view, writes_cache)
    head      Head(spec, hidden_size, vocab_size, rt)   .forward(hn, logits_f32, n_rows, ctx)
    input     StepInput(spec, hidden_size, vocab_size, rt)   .prepare(tokens, x_f32, ctx)

Optional, for one-token steps (see `NormRequest`, `LazyInput`): a norm may let the kernel that writes
its input rows do its element-wise half and the projection that reads its output its row-wise half.

Mixers and feed-forwards ADD their result into `residual` (fp32, [tokens, hidden]): the
residual sum stays in 32-bit and the last projection can fuse the addition.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, Mapping, Optional, Tuple, Type

import torch

from ..cache import CacheRequest
from ..config.specs import LayerSpec, PartSpec
from ..weights.loader import TensorSpec

_REGISTRY: Dict[Tuple[str, str], type] = {}
CATEGORIES = ("norm", "position", "mixer", "ffn", "block", "head", "input")


def register_part(category: str, kind: str, cls: type, *, replace: bool = False) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; categories: {CATEGORIES}")
    if (category, kind) in _REGISTRY and not replace:
        raise ValueError(f"{category} kind {kind!r} is already registered")
    _REGISTRY[(category, kind)] = cls


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.pop((category, kind), None)


def part_class(category: str, kind: str) -> type:
    try:
        return _REGISTRY[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _REGISTRY if c == category)
        raise KeyError(f"no {category} of kind {kind!r} is registered; registered: {known}") from None


class Workspace:
    """Named scratch tensors that live as long as the workspace: a part that asks twice
    under one name with sizes that fit gets the same memory, so steps allocate nothing once
    warm (and captured graphs keep valid addresses)."""

    def __init__(self, device):
        self.device = device
        self._bufs: Dict[str, torch.Tensor] = {}

    def take(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = max(n * torch.empty((), dtype=dtype).element_size(), 16)
        buf = self._bufs.get(name)
        if buf is None or buf.numel() < nbytes:
            buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            self._bufs[name] = buf
        return buf[:n * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)

    def bytes(self) -> int:
        return sum(b.numel() for b in self._bufs.values())


@dataclass
class Runtime:
    """What all parts of one model share: the activation dtype, the device, whether only
    the plain kernels may run, the device error word, and the workspace."""

    dtype: torch.dtype                    # torch.bfloat16 or torch.float32
    device: torch.device
    plain_only: bool = False              # float32 always runs the plain (true 32-bit) kernels
    err: Optional[torch.Tensor] = None    # int32[1] on the device, bits in csrc/common.cuh
    workspace: Optional[Workspace] = None

    def __post_init__(self):
        self.device = torch.device(self.device)
        if self.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"run dtype must be bfloat16 or float32, got {self.dtype}")
        if self.dtype == torch.float32:
            self.plain_only = True
        if self.err is None:
            self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        if self.workspace is None:
            self.workspace = Workspace(self.device)

    @property
    def fast(self) -> bool:
        return not self.plain_only


class LazyInput:
    """The input of a part's first projection, not in memory in its final form: the projection's
    kernel may finish it on the way (one-token steps, where a kernel boundary costs more than the
    work), and `materialize(n_rows)` computes it into memory with the kernel of its own, for
    whoever cannot.  A part says with `takes_lazy_input = True` that it hands its input to
    `Linear.apply` (or calls `materialize`) and never reads it as a tensor."""

    def materialize(self, n_rows: int) -> torch.Tensor:
        raise NotImplementedError


@dataclass
class NormRequest:
    """What a norm asks of whoever writes the rows it will be applied to next (one-token steps): to
    write, beside the new rows x, bf16(x * weight) and partial sums of squares of each row.  The
    row factor 1 / sqrt(mean(x^2) + eps) is applied later, by the projection that reads the scaled
    rows.  Whoever cannot do that ignores the request and the norm runs as a kernel of its own."""
    norm: object                  # the Norm that asks
    weight: torch.Tensor
    eps: float


@dataclass
class StepContext:
    """The sequences of the running step as parts see them.

    kind          "prompt": every sequence starts at position 0 with all its tokens;
                  "decode": every sequence brings exactly one token
    batch         csrc.bindings.BatchView (device arrays cu_q, slot_ids, tok_seq, pos0)
    n_tokens      packed tokens, padding included;  n_seqs likewise
    q_lens, pos0, slots   host copies (lists) for sizing launches and for host-side checks; in a step that
                  is being captured into a CUDA graph, `slots` (and, for one-token steps, `pos0`) are
                  `HostCopyUnavailable`: reading them raises
    unequal_lengths       one-token steps: a mixer asked for its work to be cut by the sequences'
                          lengths rather than evenly (`Mixer.cut_by_length`)
    """
    kind: str
    batch: object
    n_tokens: int
    n_seqs: int
    q_lens: list
    pos0: list
    slots: list
    stream: int
    rt: Runtime
    unequal_lengths: bool = False                  # one-token step whose mixers want a cut by length
    norm_ahead: Optional[NormRequest] = None      # set before a part (or the embedding) runs: the norm that will be
                                                   # applied next to the residual rows it writes
    rows_ahead: Optional[LazyInput] = None         # set by whoever honoured `norm_ahead`: that norm's lazy result
    next_block: object = None                      # the block that runs after the current one (None: the last)
    shared: dict = field(default_factory=dict)     # what the model's step inputs published for the blocks, by name
    slot_ids_dev: Optional[torch.Tensor] = None   # int32 [n_seqs] view, for parts written in Python
    pos0_dev: Optional[torch.Tensor] = None
    cu_q_dev: Optional[torch.Tensor] = None

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @property
    def max_kv_len(self) -> int:
        return max((p + q for p, q in zip(self.pos0, self.q_lens)), default=0)


class HostCopyUnavailable:
    """Stands in for `StepContext.slots` or `StepContext.pos0` while a step is being captured into a
    CUDA graph.  The captured launches are replayed later for other sequences, so what a part reads
    from the host lists at capture time would be frozen into them: any read raises instead.  A part
    that declares `graph_safe` takes the sequences from device memory (`ctx.batch`,
    `ctx.slot_ids_dev`, `ctx.pos0_dev`)."""

    def __init__(self, what: str):
        self.what = what

    def _refuse(self, *args, **kwargs):
        raise RuntimeError(
            f"StepContext.{self.what} was read while the step was being captured into a CUDA graph; "
            f"a part that declares graph_safe must read the step's sequences from device memory "
            f"(ctx.batch, ctx.slot_ids_dev, ctx.pos0_dev), or declare graph_safe = False")

    __getitem__ = __iter__ = __len__ = __bool__ = __contains__ = _refuse

    def __repr__(self):
        return f"<{self.what}: unavailable in a captured step>"


def first_norm_request_of(block, ctx) -> Optional["NormRequest"]:
    """What `block` (any registered block class, or None) asks of whoever writes the rows it receives."""
    ask = getattr(block, "first_norm_request", None)
    return ask(ctx) if ask is not None else None


class Part:
    """Common to all parts: which tensors it expects (local names) and how it takes them."""

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        if tensors:
            raise ValueError(f"{type(self).__name__} takes no tensors, got {sorted(tensors)}")


class Norm(Part):
    def forward(self, x, out, ctx, rows_idx=None, rows=None) -> None:
        raise NotImplementedError

    def request_ahead(self) -> Optional[NormRequest]:
        """A request to whoever writes the rows this norm is applied to next (see `NormRequest`), or
        None (the default) if this norm cannot be split that way."""
        return None


class PositionEncoding(Part):
    """Gives queries and keys their positions.  It does not touch the cache: storing keys and
    values is the mixer's business."""

    def encode(self, qkv, ctx: StepContext, heads: int, kv_heads: int) -> None:
        """Give the step's queries and keys their positions, in place in `qkv`
        ([tokens, (heads + 2 kv_heads) * head_dim]: queries, keys, values; a token's absolute
        position is ctx.batch.pos0[sequence] + its index in the sequence)."""
        raise NotImplementedError

    def rotary_constants(self):
        """(inv_freq fp32 device tensor, rotary_dim, pairing code) if the encoding is a plain
        rotation that a mixer's kernel may apply itself (fused with its cache write or with its
        attention), else None (the default): the mixer then calls `encode`."""
        return None


class Mixer(Part):
    def cache_request(self) -> CacheRequest:
        return None

    def cut_by_length(self, pos0, cache_view) -> bool:
        """Asked once per one-token step with the positions of the live sequences and the view of
        the cache that this mixer's layer reads: would this
        mixer rather cut its work by the sequences' lengths than evenly?  The engine replays a
        captured step of its own for either answer and passes the answer on as
        `StepContext.unequal_lengths`.  The default is no.  Mixers whose answers are always the
        same (layers of one shape) may say so with an equal `cut_by_length_key()`; one of them
        is asked then."""
        return False

    def forward(self, xn, residual, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, xn, residual, ctx: StepContext) -> None:
        raise NotImplementedError


class Block(Part):
    def forward(self, x, ctx: StepContext, cache_view, writes_cache: bool) -> None:
        raise NotImplementedError

    def first_norm_request(self, ctx: StepContext) -> Optional[NormRequest]:
        """What this block's first norm asks of whoever writes the rows the block will receive (the
        block before it, or the embedding); None (the default): nothing."""
        return None


class Head(Part):
    """Logits from the rows that the final norm produced.  Its one tensor, "weight"
    [vocab, hidden], is the output matrix; the model hands it the embedding table instead when the
    output is tied.  `forward` writes float32 logits for `n_rows` rows."""

    def forward(self, hn, logits, n_rows: int, ctx: StepContext) -> None:
        raise NotImplementedError

    def nbytes(self) -> int:
        """Bytes of weights a step reads through this head."""
        raise NotImplementedError


class StepInput(Part):
    """Runs once per step, after the embedding and before the first block, on the step's token ids
    (int32 on the device, padding included) and the embedded rows `x` (fp32 [tokens, hidden]).  It may
    change `x` in place (a norm or a bias on the embedding) and may publish tensors for the blocks in
    `ctx.shared[name]` (an input that every layer reads, computed from the ids once).  Its tensors are
    found under the prefix that `ModelSpec.inputs` names beside its spec."""

    def prepare(self, tokens, x, ctx: StepContext) -> None:
        raise NotImplementedError

