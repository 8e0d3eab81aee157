"""Storage of the cache: what mixers ask for, grouped, allocated once.

A mixer asks for cache through a request object; the model hands the requests
of all its cache entries to ``Cache``, which groups equal requests and gives
each group storage of its own:

* ``KVRequest(n_kv_heads, head_dim, window)``: keys and values per token, in
  pages ``[n_entries, n_pages, n_kv_heads, PAGE_TOKENS, head_dim]`` for K and
  for V.  Groups that keep all keys and groups that keep a window of them have
  separate page pools, and a windowed group gives pages back while the
  sequence is still running.
  ``v_head_dim`` gives values a size of their own (``None``: the keys' size).
  ``chunk`` says that a query sees only keys of its own chunk of that many
  positions (chunks counted from position 0): such a group gives a page back
  once every key in it lies before the chunk the sequence has reached.
  ``keys_only`` says that the mixer reads its values out of the key rows (a
  latent from which keys and values are both made): no storage for V.
* ``StateRequest(shape, dtype)``: state of fixed size per sequence,
  ``[max_seqs + 1, *shape]`` per entry, zeroed when a slot is opened.  The last
  row belongs to no sequence (``Cache.spare_slot``): rows that pad a step up to
  a captured graph's size carry that slot number, so a mixer that updates
  ``state[ctx.seq_slots]`` on the device never touches a live sequence's state
  from a padding row (as page 0 of every K/V group takes their cache writes).
  The Qwen3 dense decoder has no such state; it exists for mixers that carry a
  running state (the reference's GatedDeltaNetState, model.rs:377-492, is such
  a thing).
* ``BundleRequest(items)``: several of the above for ONE cache entry (a layer
  whose mixer holds keys and a running state, with the last inputs of a short
  convolution beside them); the entry's view is the tuple of the items' views.

The reference's equivalent is ``KvCache``/``LayerCache``
(crates/synaptix-models/llm/common/src/model.rs:349-368,1021-1046).
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Sequence, Tuple, Union

import torch

from .pages import PAGE_TOKENS, PagePool, SequenceSlots, pages_for


@dataclasses.dataclass(frozen=True)
class KVRequest:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    v_head_dim: Optional[int] = None
    chunk: Optional[int] = None
    keys_only: bool = False

    @property
    def value_dim(self) -> int:
        if self.keys_only:
            return 0
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclasses.dataclass(frozen=True)
class StateRequest:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclasses.dataclass(frozen=True)
class BundleRequest:
    items: tuple          # of KVRequest, StateRequest, BundleRequest or None


CacheRequest = Union[KVRequest, StateRequest, BundleRequest, None]


class KVView:
    """What an attention-like mixer sees of its cache entry."""
    __slots__ = ("k", "v", "group", "window")

    def __init__(self, k: torch.Tensor, v: torch.Tensor, group: int, window: Optional[int]):
        self.k = k          # [n_pages, n_kv_heads, PAGE_TOKENS, head_dim]
        self.v = v          # [n_pages, n_kv_heads, PAGE_TOKENS, value_dim]
        self.group = group  # index of the block table to use (StepContext.block_tables[group])
        self.window = window


class Cache:
    """All cache storage of one model on one device, with its slot bookkeeping."""

    def __init__(self, requests: Sequence[CacheRequest], *, max_tokens: int,
                 max_seqs: Optional[int], dtype: torch.dtype, device):
        self.device = torch.device(device)
        self.dtype = dtype
        # page 0 of every group is never handed out: rows that pad a batch up to a captured
        # graph's size write there, and released or unused block-table entries point there
        self.n_pages = max(1, pages_for(max_tokens)) + 1
        self.max_tokens = (self.n_pages - 1) * PAGE_TOKENS
        self.max_seqs = int(max_seqs) if max_seqs is not None else self.n_pages
        if self.max_seqs <= 0:
            raise ValueError("max_seqs must be > 0")

        # group equal requests
        self._entry: List = []   # per entry: None, (kind, group, index in group), or a list of those for a bundle
        kv_keys: List[KVRequest] = []
        kv_counts: List[int] = []
        st_keys: List[StateRequest] = []
        st_counts: List[int] = []

        def place(r):
            if r is None:
                return None
            if isinstance(r, KVRequest):
                if r not in kv_keys:
                    kv_keys.append(r)
                    kv_counts.append(0)
                g = kv_keys.index(r)
                kv_counts[g] += 1
                return ("kv", g, kv_counts[g] - 1)
            if isinstance(r, StateRequest):
                if r not in st_keys:
                    st_keys.append(r)
                    st_counts.append(0)
                g = st_keys.index(r)
                st_counts[g] += 1
                return ("state", g, st_counts[g] - 1)
            if isinstance(r, BundleRequest):        # bundles may hold bundles (a block's, with its mixer's inside)
                return [place(i) for i in r.items]
            raise TypeError(f"not a cache request: {r!r}")

        for r in requests:
            self._entry.append(place(r))
        self.kv_groups = kv_keys
        self.state_groups = st_keys

        self._k: List[torch.Tensor] = []
        self._v: List[torch.Tensor] = []
        for r, n in zip(kv_keys, kv_counts):
            shape = (n, self.n_pages, r.n_kv_heads, PAGE_TOKENS)
            self._k.append(torch.zeros(shape + (r.head_dim,), dtype=dtype, device=self.device))
            self._v.append(torch.zeros(shape + (r.value_dim,), dtype=dtype, device=self.device))
        self._state: List[torch.Tensor] = []
        for r, n in zip(st_keys, st_counts):
            self._state.append(torch.zeros((n, self.max_seqs + 1) + tuple(r.shape),
                                           dtype=r.dtype, device=self.device))

        pools = [PagePool(self.n_pages - 1, first=1) for _ in kv_keys]
        if not pools:                       # a model without keys still has lengths to keep
            pools = [PagePool(self.n_pages - 1, first=1)]
            windows: List[Optional[int]] = [None]
        else:
            windows = [r.window for r in kv_keys]
        chunks = [r.chunk for r in kv_keys] if kv_keys else [None]
        self.slots = SequenceSlots(self.max_seqs, pools, windows, chunks)

    @property
    def kv_bytes_per_token(self) -> int:
        """Bytes of keys and values one cached token takes over all layers (the reference's figure of that name,
        crates/synaptix-models/llm/common/src/model.rs:932-954): 147,456 for the Qwen3-4B shape in bfloat16."""
        return sum(t.shape[0] * t.shape[2] * t.shape[4] * t.element_size() for t in self._k + self._v)

    # -- views ------------------------------------------------------------
    @property
    def n_block_tables(self) -> int:
        return len(self.slots.pools)

    @property
    def spare_slot(self) -> int:
        """The slot number of rows that belong to no sequence (padding of a captured step)."""
        return self.max_seqs

    def view(self, entry: int):
        return self._view_of(self._entry[entry])

    def _view_of(self, e):
        if e is None:
            return None
        if isinstance(e, list):
            return tuple(self._view_of(i) for i in e)
        kind, g, i = e
        if kind == "kv":
            return KVView(self._k[g][i], self._v[g][i], g, self.kv_groups[g].window)
        return self._state[g][i]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._k + self._v + self._state)

    # -- slots --------------------------------------------------------------
    def open(self) -> int:
        s = self.slots.open()
        for st in self._state:
            st[:, s].zero_()
        return s

    def close(self, slot: int) -> None:
        self.slots.close(slot)
