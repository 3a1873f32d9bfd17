"""The cache of a running engine: device arenas plus the host bookkeeping that owns them.

Cache entries (one per layer call that writes keys and values) with the same key/value
shape and window form a *group*. A group has one arena
``[entries, 2 (K|V), pages + 1, kv_heads, page_size, head_dim]`` and one pool of page ids
shared by its entries, as the reference gives each group its own pool and tables
(python/instinct/paged_kv.py:156-202; python/instinct/backends/dense.py:57-70). Inside a
page the layout is head-major, so one (page, kv head) tile is ``page_size * head_dim``
contiguous elements. The extra last page is never handed out: padded batch rows write
there. Everything is allocated once, up front (the reference's CUDA engine does the same,
cuda/qwen_model.cu:26-43).

Entries that keep fixed-size per-request state instead get slot arrays
``[slots, *shape]``; a request's slot is zeroed when it is handed out
(python/instinct/paged_kv.py:189-198,296-313).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from ..csrc.host_module import host
from ..parts.base import KVCacheSpec, StateSpec
from ..parts.context import CacheView


@dataclass
class CacheGroup:
    index: int
    name: str
    spec: KVCacheSpec
    entries: list[int]  # cache entry ids, in arena order
    capacity_pages: int = 0
    arena: torch.Tensor | None = None

    def bytes_per_token(self, element_size: int) -> int:
        return 2 * len(self.entries) * self.spec.kv_heads * self.spec.head_dim * element_size


def plan_groups(cache_specs: dict[int, KVCacheSpec | StateSpec]) -> tuple[list[CacheGroup], dict[int, StateSpec]]:
    groups: dict[KVCacheSpec, CacheGroup] = {}
    states: dict[int, StateSpec] = {}
    for cache_id in sorted(cache_specs):
        spec = cache_specs[cache_id]
        if isinstance(spec, StateSpec):
            states[cache_id] = spec
            continue
        if spec not in groups:
            name = f"window{spec.window}" if spec.window else "full"
            if any(g.name == name for g in groups.values()):
                name = f"{name}_h{spec.kv_heads}d{spec.head_dim}"
            groups[spec] = CacheGroup(len(groups), name, spec, [])
        groups[spec].entries.append(cache_id)
    return list(groups.values()), states


def window_pages(window: int, step_tokens: int, page_size: int) -> int:
    return math.ceil((window + step_tokens) / page_size) + 1


def split_budget(
    groups: list[CacheGroup], budget_bytes: int, page_size: int, element_size: int, max_num_sequences: int, step_tokens: int
) -> None:
    """Pages per group from a byte budget: a windowed group gets every sequence's window
    (capped at half the budget), the others share the rest by bytes per token
    (python/instinct/mlx_engine.py:149-171)."""
    remaining = budget_bytes
    for group in groups:
        if group.spec.window:
            page_bytes = group.bytes_per_token(element_size) * page_size
            pages = max_num_sequences * window_pages(group.spec.window, step_tokens, page_size)
            pages = min(pages, max(1, budget_bytes // 2 // page_bytes))
            group.capacity_pages = pages
            remaining -= pages * page_bytes
    full = [g for g in groups if not g.spec.window]
    per_token = sum(g.bytes_per_token(element_size) for g in full)
    for group in full:
        page_bytes = group.bytes_per_token(element_size) * page_size
        share = remaining * group.bytes_per_token(element_size) / per_token
        group.capacity_pages = max(1, int(share // page_bytes))


class PagedCache:
    def __init__(
        self,
        cache_specs: dict[int, KVCacheSpec | StateSpec],
        *,
        dtype: torch.dtype,
        device: torch.device | str,
        page_size: int,
        max_num_sequences: int,
        max_model_length: int,
        step_tokens: int,
        kv_cache_bytes: int | None = None,
        num_pages: int | None = None,
    ) -> None:
        if page_size <= 0 or max_num_sequences <= 0:
            raise ValueError("sequences and page size must be positive")
        self.dtype, self.device = dtype, torch.device(device)
        self.page_size = page_size
        self.max_num_sequences = max_num_sequences
        self.max_pages_per_request = math.ceil(max_model_length / page_size)
        self.groups, self.state_specs = plan_groups(cache_specs)
        element = torch.empty((), dtype=dtype).element_size()
        if num_pages is not None:
            for group in self.groups:
                group.capacity_pages = num_pages
        elif kv_cache_bytes is not None:
            if kv_cache_bytes <= 0:
                raise ValueError("kv_cache_bytes must be positive")
            if self.groups:
                split_budget(self.groups, kv_cache_bytes, page_size, element, max_num_sequences, step_tokens)
        else:
            raise ValueError("give the cache a byte budget or a page count")
        self.entry_group: dict[int, tuple[CacheGroup, int]] = {}
        self._entry_arenas: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
        for group in self.groups:
            spec = group.spec
            group.arena = torch.zeros(
                (len(group.entries), 2, group.capacity_pages + 1, spec.kv_heads, page_size, spec.head_dim),
                dtype=dtype,
                device=self.device,
            )
            for slot, cache_id in enumerate(group.entries):
                self.entry_group[cache_id] = (group, slot)
        self.state_slots = max_num_sequences if self.state_specs else 0
        self.states: dict[int, list[torch.Tensor]] = {
            cache_id: [
                # One slot more than requests: the target of the padding rows of a captured step.
                torch.zeros((self.state_slots + 1, *shape), dtype=dt, device=self.device)
                for shape, dt in zip(spec.shapes, spec.dtypes)
            ]
            for cache_id, spec in self.state_specs.items()
        }
        h = host()
        self.manager = h.CacheManager(
            page_size,
            [h.GroupSpec(g.name, g.capacity_pages, g.spec.window) for g in self.groups],
            self.state_slots,
            step_tokens,
        )

    # -- bookkeeping passthroughs -------------------------------------------------------------

    def open(self, request_id: int) -> None:
        self.manager.open(request_id)
        self._clear_new_slots()

    def admit(self, request_id: int, total_tokens: int) -> bool:
        ok = self.manager.admit(request_id, total_tokens)
        self._clear_new_slots()
        return ok

    def _clear_new_slots(self) -> None:
        for slot in self.manager.take_slots_to_clear():
            for arrays in self.states.values():
                for array in arrays:
                    array[slot].zero_()

    def clear_new_slots(self) -> None:
        """Zero the slots handed out since the last call (admission may happen in C++)."""
        self._clear_new_slots()

    def null_page(self, group: CacheGroup) -> int:
        return group.capacity_pages

    def null_slot(self) -> int:
        """The state slot no request holds (padding rows write there); -1 without state."""
        return self.state_slots if self.state_specs else -1

    # -- what a step needs ----------------------------------------------------------------------

    def fill_tables(self, request_ids: list[int], out: list[np.ndarray]) -> None:
        """Write the requests' block tables into ``out[g]`` (``[rows, max_pages]`` int32)."""
        for group in self.groups:
            self.manager.fill_tables(request_ids, group.index, out[group.index], self.null_page(group))

    def view(self, cache_id: int, writes: bool, block_tables: list[torch.Tensor]) -> CacheView:
        if cache_id in self.states:
            return CacheView(cache_id=cache_id, writes=writes, state=self.states[cache_id])
        group, slot = self.entry_group[cache_id]
        arenas = self._entry_arenas.get(cache_id)
        if arenas is None:  # the arena never moves: slice it once per entry, not once per layer and step
            arenas = self._entry_arenas[cache_id] = (group.arena[slot, 0], group.arena[slot, 1])
        return CacheView(
            cache_id=cache_id,
            writes=writes,
            keys=arenas[0],
            values=arenas[1],
            block_table=block_tables[group.index],
            num_pages=group.capacity_pages + 1,
            max_pages=self.max_pages_per_request,
            page_size=self.page_size,
            window=group.spec.window,
        )

    def device_bytes(self) -> int:
        total = sum(g.arena.numel() * g.arena.element_size() for g in self.groups)
        return total + sum(a.numel() * a.element_size() for arrays in self.states.values() for a in arrays)

    def stats(self) -> dict:
        out = dict(self.manager.stats())
        element = torch.empty((), dtype=self.dtype).element_size()
        for group in self.groups:
            out["kv_pools"][group.name]["page_bytes"] = group.bytes_per_token(element) * self.page_size
        out["kv_device_bytes"] = self.device_bytes()
        return out
