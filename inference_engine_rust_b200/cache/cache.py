"""The cache of a running model: a slot per live sequence; per layer group, paged keys and
values (all of them, or a ring that holds a window); and beside them per-sequence state of
fixed size for mixers that keep one.

Reference: `KVCache` holds `[max_seq, kv_heads, head_dim]` keys and values per layer for one
sequence and appends at `current_pos` (src/layers/attention.rs:16-74); a window is only a
mask over that full-length buffer (:610-613).  Here memory is counted in pages of
`page_tokens` positions shared by all live sequences, each sequence has its own length, and
a windowed group keeps only `ceil(window / page_tokens)` pages per sequence, written round
and round.  Because keys are rotated before they are stored, where a key lies in the ring
does not matter to the result.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .allocators import CacheError, CacheFull, IndexPool

PAGE_TOKENS = 64


@dataclass(frozen=True)
class KVRequest:
    """What an attention-like mixer asks of the cache for its layer."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every earlier key stays visible


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size state per sequence (zeroed when a sequence starts)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


CacheRequest = Union[KVRequest, StateRequest, None]


class KVGroup:
    """Layers with the same key/value geometry and the same visibility share page tables."""

    def __init__(self, req: KVRequest, layers: Sequence[int], n_pages: int, n_slots: int,
                 max_seq_len: int, dtype: torch.dtype, device, page_tokens: int, poison: bool):
        self.req = req
        self.layers = tuple(layers)
        self.page_tokens = page_tokens
        self.n_pages = n_pages
        self.n_slots = n_slots
        self.dtype = dtype
        self.device = device
        self.table_width = max(1, math.ceil(max_seq_len / page_tokens))
        if req.window is None:
            self.ring_pages = self.table_width
        else:
            self.ring_pages = min(self.table_width, max(1, math.ceil(req.window / page_tokens)))
        shape = (len(self.layers), n_pages, req.kv_heads, page_tokens, req.head_dim)
        self.k = torch.empty(shape, dtype=dtype, device=device)
        self.v = torch.empty(shape, dtype=dtype, device=device)
        self.poison = poison
        if poison:
            self.k.fill_(float("nan"))
            self.v.fill_(float("nan"))
        self.pages = IndexPool(n_pages, "page")
        self.table_host = np.full((n_slots, self.table_width), -1, dtype=np.int32)
        self.table = torch.full((n_slots, self.table_width), -1, dtype=torch.int32, device=device)
        self._pages_of: Dict[int, List[int]] = {}
        self._dirty: set = set()

    @property
    def ring_capacity(self) -> int:
        return self.ring_pages * self.page_tokens

    def pages_needed(self, length: int) -> int:
        return min(self.ring_pages, math.ceil(length / self.page_tokens))

    def open_slot(self, slot: int) -> None:
        self._pages_of[slot] = []

    def ensure(self, slot: int, length: int) -> None:
        """Pages for positions [0, length) of `slot` (or for the ring, if shorter)."""
        have = self._pages_of[slot]
        if length <= len(have) * self.page_tokens or len(have) >= self.ring_pages > 0:
            return                      # the usual case of a one-token step: the last page has room
        need = self.pages_needed(length)
        if need > self.table_width:
            raise CacheFull(f"sequence of {length} tokens exceeds the cache's longest sequence "
                            f"({self.table_width * self.page_tokens})")
        if need > len(have):
            new = self.pages.alloc_many(need - len(have))
            for p in new:
                self.table_host[slot, len(have)] = p
                have.append(p)
            self._dirty.add(slot)

    def close_slot(self, slot: int) -> None:
        pages = self._pages_of.pop(slot)
        self.pages.free_many(pages)
        if self.poison and pages:
            idx = torch.tensor(pages, dtype=torch.long, device=self.device)
            self.k[:, idx] = float("nan")
            self.v[:, idx] = float("nan")
        self.table_host[slot, :] = -1
        self._dirty.add(slot)

    def upload(self) -> None:
        """Bring the device page tables up to date (rows of slots that changed)."""
        if not self._dirty:
            return
        rows = sorted(self._dirty)
        self._dirty.clear()
        if self.table.device.type == "cpu":
            self.table[rows] = torch.from_numpy(self.table_host[rows])
            return
        # one copy of the whole table when it is small or many rows changed (each copy from
        # pageable memory synchronises), else row by row
        if self.table_host.nbytes <= (1 << 20) or len(rows) * 4 >= self.n_slots:
            self.table.copy_(torch.from_numpy(self.table_host), non_blocking=False)
        else:
            for r in rows:
                self.table[r].copy_(torch.from_numpy(self.table_host[r]), non_blocking=False)

    def pages_of(self, slot: int) -> List[int]:
        return list(self._pages_of[slot])

    def bytes_per_token(self) -> int:
        return 2 * len(self.layers) * self.req.kv_heads * self.req.head_dim * self.k.element_size()


class StateGroup:
    def __init__(self, req: StateRequest, layers: Sequence[int], n_slots: int, device):
        self.req = req
        self.layers = tuple(layers)
        self.state = torch.zeros((len(self.layers), n_slots) + tuple(req.shape), dtype=req.dtype, device=device)

    def open_slot(self, slot: int) -> None:
        self.state[:, slot].zero_()

    def close_slot(self, slot: int) -> None:
        pass


@dataclass
class KVLayerView:
    """What an attention-like mixer is handed for its layer."""
    group: KVGroup
    index: int                     # position of the layer inside the group
    struct: object                 # csrc.bindings.KvView, or None on a CPU-only cache

    @property
    def k(self) -> torch.Tensor:
        return self.group.k[self.index]

    @property
    def v(self) -> torch.Tensor:
        return self.group.v[self.index]


@dataclass
class StateLayerView:
    group: StateGroup
    index: int

    @property
    def state(self) -> torch.Tensor:      # [n_slots, *shape]
        return self.group.state[self.index]


class Cache:
    """Slots, page pools and state for one model.

    max_tokens     positions the page pools hold in total, every live sequence's length
                   rounded up to `page_tokens`
    max_seq_len    the longest single sequence (width of a page table)
    max_sequences  number of slots
    """

    def __init__(self, requests: Mapping[int, CacheRequest], *, max_tokens: int, max_seq_len: int,
                 max_sequences: int, dtype: torch.dtype, device, page_tokens: int = PAGE_TOKENS,
                 poison: bool = False):
        if max_tokens <= 0 or max_seq_len <= 0 or max_sequences <= 0:
            raise ValueError("cache sizes must be positive")
        self.page_tokens = page_tokens
        self.n_pages = math.ceil(max_tokens / page_tokens)
        self.max_seq_len = min(max_seq_len, self.n_pages * page_tokens)
        self.n_slots = max_sequences
        self.dtype = dtype
        self.device = torch.device(device)
        self.slots = IndexPool(self.n_slots, "slot")
        self.seq_lens = np.zeros(self.n_slots, dtype=np.int64)

        kv_by_key: Dict[KVRequest, List[int]] = {}
        st_by_key: Dict[StateRequest, List[int]] = {}
        for layer in sorted(requests):
            req = requests[layer]
            if req is None:
                continue
            if isinstance(req, KVRequest):
                kv_by_key.setdefault(req, []).append(layer)
            elif isinstance(req, StateRequest):
                st_by_key.setdefault(req, []).append(layer)
            else:
                raise TypeError(f"layer {layer}: unknown cache request {req!r}")
        self.kv_groups: List[KVGroup] = [
            KVGroup(req, layers, self.n_pages, self.n_slots, self.max_seq_len, dtype, self.device,
                    page_tokens, poison) for req, layers in kv_by_key.items()]
        self.state_groups: List[StateGroup] = [
            StateGroup(req, layers, self.n_slots, self.device) for req, layers in st_by_key.items()]
        self._views: Dict[int, object] = {}
        for g in self.kv_groups:
            for i, layer in enumerate(g.layers):
                self._views[layer] = KVLayerView(g, i, self._kv_struct(g, i))
        for g in self.state_groups:
            for i, layer in enumerate(g.layers):
                self._views[layer] = StateLayerView(g, i)

    def _kv_struct(self, g: KVGroup, i: int):
        if self.device.type != "cuda":
            return None
        from ..csrc import bindings as B
        return B.KvView(k=g.k[i].data_ptr(), v=g.v[i].data_ptr(), page_table=g.table.data_ptr(),
                        table_width=g.table_width, ring_pages=g.ring_pages, page_tokens=g.page_tokens,
                        n_pages=g.n_pages, kv_heads=g.req.kv_heads, head_dim=g.req.head_dim,
                        dtype=B.dtype_code(g.dtype), window=g.req.window or 0)

    # ---- slots ------------------------------------------------------------------------
    def open_sequence(self) -> int:
        slot = self.slots.alloc()
        self.seq_lens[slot] = 0
        for g in self.kv_groups:
            g.open_slot(slot)
        for g in self.state_groups:
            g.open_slot(slot)
        return slot

    def close_sequence(self, slot: int) -> None:
        self.slots.free(slot)           # raises if not held, before anything is touched
        for g in self.kv_groups:
            g.close_slot(slot)
        for g in self.state_groups:
            g.close_slot(slot)
        self.seq_lens[slot] = 0

    def length(self, slot: int) -> int:
        if slot not in self.slots._held:
            raise CacheError(f"slot {slot} is not held")
        return int(self.seq_lens[slot])

    def reserve(self, slot: int, new_length: int) -> None:
        """Make room for the sequence to grow to `new_length` positions."""
        if slot not in self.slots._held:
            raise CacheError(f"slot {slot} is not held")
        if new_length > self.max_seq_len:
            raise CacheFull(f"sequence would reach {new_length} tokens; the cache's longest "
                            f"sequence is {self.max_seq_len}")
        for g in self.kv_groups:
            g.ensure(slot, new_length)

    def advance(self, slot: int, n_tokens: int) -> None:
        self.seq_lens[slot] += n_tokens

    def upload(self) -> None:
        for g in self.kv_groups:
            g.upload()

    def layer_view(self, layer: int):
        return self._views.get(layer)

    # ---- accounting ---------------------------------------------------------------------
    def tokens_held(self) -> int:
        """Positions held by live sequences, each rounded up to a page."""
        pt = self.page_tokens
        return sum(math.ceil(int(self.seq_lens[s]) / pt) * pt for s in self.slots.held())

    def kv_bytes_read(self, slots: Sequence[int]) -> int:
        """Bytes of keys and values a one-token step over `slots` has to read."""
        total = 0
        for g in self.kv_groups:
            for s in slots:
                n = int(self.seq_lens[s])
                if g.req.window is not None:
                    n = min(n, g.req.window)
                total += n * g.bytes_per_token()
        return total

    def check(self) -> None:
        """Invariants: nothing lost, nothing held twice."""
        self.slots.check()
        for g in self.kv_groups:
            g.pages.check()
            owned: List[int] = []
            for slot, pages in g._pages_of.items():
                if slot not in self.slots._held:
                    raise CacheError(f"pages are recorded for slot {slot}, which is not held")
                owned.extend(pages)
            if len(owned) != len(set(owned)):
                raise CacheError("a page belongs to two sequences")
            if set(owned) != g.pages.held():
                raise CacheError("held pages and the sequences' page lists disagree")
