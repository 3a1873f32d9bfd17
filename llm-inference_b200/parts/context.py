"""What a part sees of one step: the batch's metadata, the cache and scratch buffers."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from ctypes import c_void_p

import numpy as np
import torch

# The raw handle of the current stream without building a Stream object for it (several
# microseconds per launch otherwise); older builds of the library lack the shortcut.
_CURRENT_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _raw_stream(device: torch.device) -> int:
    if _CURRENT_RAW_STREAM is not None:
        index = device.index if device.index is not None else torch.cuda.current_device()
        return _CURRENT_RAW_STREAM(index)
    return torch.cuda.current_stream(device).cuda_stream


@dataclass
class HostBatch:
    """The step's metadata as NumPy arrays on the host (the device holds the same)."""

    token_ids: np.ndarray  # [T] int32
    positions: np.ndarray  # [T] absolute position of each new token in its request
    token_seq: np.ndarray  # [T] index of the token's request within this batch
    seq_q_start: np.ndarray  # [S] first row of each request's run of new tokens
    seq_q_len: np.ndarray  # [S] length of the run (1 = a decoded token)
    seq_kv_len: np.ndarray  # [S] keys the request holds after this step
    seq_slot: np.ndarray  # [S] state slot of each request, -1 if the cache has none
    logit_rows: np.ndarray  # [W] rows whose logits are wanted


@dataclass
class CacheView:
    """One layer call's access to the cache.

    For paged keys and values: ``keys`` / ``values`` are the layer's arenas
    ``[pages, kv_heads, page_size, head_dim]`` and ``block_table`` is ``[S, max_pages]``
    (int32, on the device). For per-request state: ``state`` is the list of slot arrays
    ``[slots, *shape]``. ``writes`` is false when the call only reads a cache that another
    layer call fills.
    """

    cache_id: int
    writes: bool = True
    keys: torch.Tensor | None = None
    values: torch.Tensor | None = None
    block_table: torch.Tensor | None = None
    num_pages: int = 0
    max_pages: int = 0
    page_size: int = 0
    window: int = 0
    state: list[torch.Tensor] | None = None


class Workspace:
    """Named scratch buffers that grow to the largest size asked for and are then reused."""

    def __init__(self, device: torch.device, min_rows: int = 0) -> None:
        self.device = device
        self._flat: dict[str, torch.Tensor] = {}
        # (name, dtype, shape) -> the view handed out last time; valid until a buffer moves.
        self._views: dict[tuple, torch.Tensor] = {}
        # Buffers whose first dimension counts tokens are sized for at least this many rows,
        # so that a later, larger step does not move them.
        self.min_rows = min_rows
        # Bumped whenever a buffer is (re)allocated: addresses captured in a CUDA graph before
        # that are stale afterwards.
        self.generation = 0

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype, *, per_token: bool = True) -> torch.Tensor:
        # A step asks for the same few dozen buffers in every layer: the view itself is kept.
        view_key = (name, dtype, tuple(shape))
        view = self._views.get(view_key)
        if view is not None:
            return view
        count = 1
        for s in shape:
            count *= int(s)
        key = f"{name}:{dtype}"
        flat = self._flat.get(key)
        if flat is None or flat.numel() < count:
            capacity = count
            if per_token and len(shape) >= 1 and shape[0] < self.min_rows:
                capacity = count // max(int(shape[0]), 1) * self.min_rows if shape[0] else self.min_rows
            flat = torch.empty(max(capacity, count, 1), dtype=dtype, device=self.device)
            self._flat[key] = flat
            self.generation += 1
            self._views.clear()
        view = flat[:count].view(shape)
        if len(self._views) > 4096:
            self._views.clear()
        self._views[view_key] = view
        return view

    def zeros(self, name: str, count: int, dtype: torch.dtype) -> torch.Tensor:
        """A buffer that starts zeroed and whose users leave it zeroed (arrival counters)."""
        key = f"{name}:{dtype}:zeros"
        flat = self._flat.get(key)
        if flat is None or flat.numel() < count:
            flat = torch.zeros(count, dtype=dtype, device=self.device)
            self._flat[key] = flat
            self.generation += 1
        return flat

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._flat.values())


@dataclass
class StepContext:
    """Everything a part may use while the step runs."""

    lib: Any  # csrc.library.KernelLibrary
    dtype: torch.dtype
    device: torch.device
    num_tokens: int
    num_seqs: int
    host: HostBatch
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_seq: torch.Tensor
    seq_q_start: torch.Tensor
    seq_q_len: torch.Tensor
    seq_kv_len: torch.Tensor
    seq_slot: torch.Tensor
    logit_rows: torch.Tensor
    err: torch.Tensor  # one int32 the kernels OR error bits into
    workspace: Workspace
    num_decode_seqs: int = 0  # the first this-many requests of the batch feed a single token
    max_kv_len: int = 0
    max_q_len: int = 0
    captured: bool = False  # the step is (or will be) replayed from a CUDA graph
    options: dict[str, Any] = field(default_factory=dict)

    def buffer(
        self, name: str, shape: tuple[int, ...], dtype: torch.dtype | None = None, *, per_token: bool = True
    ) -> torch.Tensor:
        """Scratch for this step. ``per_token=False`` marks buffers whose row count is not
        the step's token count (logits of the wanted rows), which are sized as asked."""
        return self.workspace.get(name, shape, dtype or self.dtype, per_token=per_token)

    @property
    def stream(self):
        """The current CUDA stream's handle (looked up at every launch: it changes while a
        graph is being captured)."""
        return _raw_stream(self.device)
