"""Paged KV pool and page tables for the B200 decode engine.

Layout contract (unchanged from the reference, cacheir/runtime/cuda.py:266-290
and cacheir/backends/triton_kernels.py:199-206): per layer one K and one V pool
`[slots, kv_heads, page_size, head_dim]`; a page table row holds the slot of
every logical page of a sequence; row t of a sequence lives in
`page_table[t // page_size]` at offset `t % page_size`.

What is different from `TorchKVPageAllocator` / `TorchPagedKVCache`
(cuda.py:121-427), on purpose:
  * no contiguous per-session copy of the history and no `torch.cat` per
    token: the kernels write new rows straight into their page;
  * one page id names the same slot in every layer's pool, so a session has a
    single page list (the reference allocates a page id per layer and ends up
    with identical slot tables layer by layer);
  * slots are reference counted and reused: releasing a session returns its
    pages, and `share_prefix` lets sessions alias the full pages of a common
    prefix (prefix-shared pages) instead of copying snapshots;
  * page boundaries follow `_extend_pages` (cuda.py:395-406; CPU twin
    cacheir/runtime/kv_cache.py:111-123) exactly: a page is opened when
    `cursor % page_size == 0`, otherwise the last page's length grows.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Any

import numpy as np


@dataclass
class KVPage:
    """cacheir/runtime/kv_cache.py:9-16. `page_id` doubles as the pool slot."""

    page_id: int
    start: int
    length: int

    def to_dict(self) -> dict[str, int]:
        return {"page_id": self.page_id, "start": self.start, "length": self.length}


class KVPoolExhausted(RuntimeError):
    """No free slot is left and the pool is not allowed to grow."""


class B200KVPageAllocator:
    """Slot allocator plus the per-layer K/V page pools (torch tensors on one GPU).

    Host-only bookkeeping (ids, refcounts, free list) works without CUDA, which
    is what the CPU tests exercise; the pools are created on first use."""

    _owner_counter = itertools.count(1)

    def __init__(self, *, page_size: int = 16, initial_slots: int = 64, max_slots: int | None = None,
                 max_resident_pages: int | None = None):
        self.page_size = max(1, int(page_size))
        self.capacity = max(1, int(initial_slots))
        self.max_slots = max_slots
        self.max_resident_pages = max_resident_pages
        self._next_slot = 0
        self._free: list[int] = []
        self._refcount: dict[int, int] = {}
        self._owners: dict[str, list[int]] = {}
        self.allocated_pages_total = 0
        self.released_pages = 0
        self.shared_page_refs = 0
        self.pool_writes = 0
        self.pool_grows = 0
        self.generation = 0          # bumps whenever pool storage is (re)allocated
        self.version = 0             # bumps whenever a page changes hands (allocate, retain, release)
        self.page_bytes: int | None = None
        self._pools: dict[int, dict[str, Any]] = {}
        self._pool_spec: tuple[Any, Any, int, int] | None = None  # device, dtype, kv_heads, head_dim

    # ---- ids / refcounts ---------------------------------------------------------
    def new_owner(self) -> str:
        return f"b200-session-{next(self._owner_counter)}"

    def allocate(self, *, owner: str, start: int, length: int) -> KVPage:
        if self._free:
            slot = self._free.pop()
        else:
            slot = self._next_slot
            if self.max_slots is not None and slot >= self.max_slots:
                raise KVPoolExhausted(f"KV page pool exhausted ({self.max_slots} slots)")
            self._next_slot += 1
            if self._next_slot > self.capacity:
                self._grow(self._next_slot)
        self._refcount[slot] = 1
        self._owners.setdefault(owner, []).append(slot)
        self.allocated_pages_total += 1
        self.version += 1
        return KVPage(page_id=slot, start=start, length=length)

    def retain(self, *, owner: str, page: KVPage) -> KVPage:
        """Another session aliases `page` (a full page of a shared prefix)."""
        self._refcount[page.page_id] += 1
        self._owners.setdefault(owner, []).append(page.page_id)
        self.shared_page_refs += 1
        self.version += 1
        return KVPage(page_id=page.page_id, start=page.start, length=page.length)

    def refcount(self, slot: int) -> int:
        return self._refcount.get(int(slot), 0)

    def release_owner(self, owner: str) -> None:
        self.version += 1
        for slot in self._owners.pop(owner, []):
            self._refcount[slot] -= 1
            if self._refcount[slot] == 0:
                del self._refcount[slot]
                self._free.append(slot)
                self.released_pages += 1

    @property
    def slots_in_use(self) -> int:
        return len(self._refcount)

    # ---- pools ---------------------------------------------------------------------
    def configure(self, *, torch: Any, device: Any, dtype: Any, num_layers: int, kv_heads: int, head_dim: int,
                  kv_dtype: str = "same") -> None:
        """`kv_dtype` "int8": pools of unsigned bytes with one fp16 scale per cached row (pool["scales"],
        [slots, kv_heads, 2, page]); "same": pools of the activation type, the reference's layout."""
        if kv_dtype not in {"same", "int8"}:
            raise ValueError(f"unsupported kv_dtype {kv_dtype!r}")
        self.kv_dtype = kv_dtype
        if kv_dtype == "int8":
            dtype = torch.uint8
        spec = (str(device), str(dtype), int(kv_heads), int(head_dim))
        if self._pool_spec is not None:
            if self._pool_spec[:4] != spec or len(self._pools) != num_layers:
                raise ValueError("a KV page allocator serves one model shape, dtype and device")
            return
        self._pool_spec = spec
        self._torch, self._device, self._dtype = torch, device, dtype
        self._kv_heads, self._head_dim = int(kv_heads), int(head_dim)
        for layer in range(num_layers):
            self._pools[layer] = self._new_pool(self.capacity)
        self.pool_grows += 1
        self.generation += 1
        elem = torch.empty((), dtype=dtype).element_size()
        self.page_bytes = 2 * self._kv_heads * self.page_size * self._head_dim * elem
        if kv_dtype == "int8":
            self.page_bytes += 2 * self._kv_heads * self.page_size * 2

    def _new_pool(self, slots: int) -> dict[str, Any]:
        shape = (slots, self._kv_heads, self.page_size, self._head_dim)
        pool = {"keys": self._torch.zeros(shape, device=self._device, dtype=self._dtype),
                "values": self._torch.zeros(shape, device=self._device, dtype=self._dtype)}
        if getattr(self, "kv_dtype", "same") == "int8":
            pool["scales"] = self._torch.zeros((slots, self._kv_heads, 2, self.page_size), device=self._device,
                                               dtype=self._torch.float16)
        return pool

    def reserve_slots(self, slots: int) -> None:
        """Pre-size the pools so that no growth (and no pointer change) happens later."""
        if slots > self.capacity:
            self._grow(slots, exact=True)

    def _grow(self, needed: int, exact: bool = False) -> None:
        new_capacity = needed if exact else max(needed, self.capacity * 2)
        if self.max_slots is not None:
            new_capacity = max(needed, min(new_capacity, self.max_slots))
        old = self.capacity
        self.capacity = new_capacity
        if not self._pools:
            return
        for layer, pool in self._pools.items():
            grown = self._new_pool(new_capacity)
            for name in pool:
                grown[name][:old] = pool[name]
            self._pools[layer] = grown
        self.pool_grows += 1
        self.generation += 1

    def pool_for_layer(self, layer: int) -> dict[str, Any] | None:
        return self._pools.get(int(layer))

    def stats(self) -> dict[str, object]:
        pools = []
        for layer, pool in sorted(self._pools.items()):
            keys = pool["keys"]
            pools.append({
                "layer": layer, "device": str(keys.device), "dtype": str(keys.dtype),
                "kv_heads": int(keys.shape[1]), "head_dim": int(keys.shape[3]),
                "slots": self._next_slot, "capacity": int(keys.shape[0]),
                "bytes": int(2 * keys.numel() * keys.element_size()),
            })
        return {
            "page_size": self.page_size,
            "page_bytes": self.page_bytes,
            "allocated_pages_total": self.allocated_pages_total,
            "resident_pages": self.slots_in_use,
            "released_pages": self.released_pages,
            "shared_page_refs": self.shared_page_refs,
            "max_resident_pages": self.max_resident_pages,
            "spilled_pages": [],
            "pool_writes": self.pool_writes,
            "pool_grows": self.pool_grows,
            "persistent_pools": pools,
        }


@dataclass
class B200PagedKVCache:
    """Page list and length of one session (all layers advance together)."""

    allocator: B200KVPageAllocator
    num_layers: int = 1
    pages: list[KVPage] = field(default_factory=list)
    tokens: int = 0
    owner_id: str = ""
    epoch: int = 0          # bumps when the page list is replaced rather than extended

    def __post_init__(self) -> None:
        self.page_size = self.allocator.page_size
        if not self.owner_id:
            self.owner_id = self.allocator.new_owner()

    def clear(self) -> None:
        self.allocator.release_owner(self.owner_id)
        self.pages = []
        self.tokens = 0
        self.epoch += 1

    def __contains__(self, layer: int) -> bool:
        return 0 <= int(layer) < self.num_layers and self.tokens > 0

    def length(self, layer: int = 0) -> int:
        return self.tokens

    def extend(self, length: int) -> bool:
        """Account for `length` more tokens; same walk as `_extend_pages`
        (cacheir/runtime/cuda.py:395-406). Returns True if a page was opened."""
        if length == 1 and self.tokens % self.page_size != 0:
            # the per-step case: one more token in the open page (the walk below does the same, slower)
            last = self.pages[-1]
            if self.allocator.refcount(last.page_id) > 1:
                raise RuntimeError("cannot append into a page that other sessions alias")
            last.length += 1
            self.tokens += 1
            self.allocator.pool_writes += self.num_layers
            return False
        opened = False
        remaining = int(length)
        cursor = self.tokens
        while remaining > 0:
            page_offset = cursor % self.page_size
            take = min(remaining, self.page_size - page_offset)
            if page_offset == 0:
                self.pages.append(self.allocator.allocate(owner=self.owner_id, start=cursor, length=take))
                opened = True
            else:
                if self.allocator.refcount(self.pages[-1].page_id) > 1:
                    raise RuntimeError("cannot append into a page that other sessions alias")
                self.pages[-1].length += take
            cursor += take
            remaining -= take
        self.tokens = cursor
        self.allocator.pool_writes += int(length) * self.num_layers
        return opened

    def share_prefix(self, other: "B200PagedKVCache", tokens: int) -> int:
        """Alias the full pages covering the first `tokens` tokens of `other`
        (rounded down to whole pages). Returns the number of tokens shared."""
        if self.tokens != 0:
            raise RuntimeError("share_prefix needs an empty session")
        n_pages = min(int(tokens), other.tokens) // self.page_size
        for page in other.pages[:n_pages]:
            self.pages.append(self.allocator.retain(owner=self.owner_id, page=page))
        self.tokens = n_pages * self.page_size
        self.epoch += 1
        return self.tokens

    def page_ids(self) -> list[int]:
        return [page.page_id for page in self.pages]

    def page_table_row(self, width: int) -> np.ndarray:
        row = np.zeros((width,), dtype=np.int32)  # padding aliases slot 0 like the reference (cuda.py:1230-1234)
        ids = self.page_ids()
        row[: len(ids)] = ids
        return row

    def stats(self) -> dict[str, object]:
        pages = [page.to_dict() for page in self.pages]
        return {
            "page_size": self.page_size,
            "layers": {str(layer): {"tokens": self.tokens, "pages": pages} for layer in range(self.num_layers)} if self.tokens else {},
            "page_bytes": self.allocator.page_bytes,
            "allocator": self.allocator.stats(),
        }
