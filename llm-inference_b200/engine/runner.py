"""The step function: one batch of (request, its next tokens) through the model.

:class:`ModelRunner.step` is the only way tokens reach the model. Generation, the replay
tool and the benchmark all call it. A step takes any mix of prompt portions and single
decoded tokens, cut anywhere; it runs exactly the tokens it is given against the cache
that earlier steps left, writes their keys and values, and returns 32-bit logits at the
wanted places. The reference runs decode and prefill as separate passes per step
(python/instinct/mlx_engine.py:404-425) over ``DecodeBatch`` / ``PrefillBatch``
(python/instinct/batches.py:27-253); here both are rows of one flattened batch.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

import time

import numpy as np
import torch

from ..cache.paged_cache import PagedCache
from ..csrc.library import check_error_word, kernels
from ..parts.context import HostBatch, StepContext, Workspace
from ..parts.model import LayerCall, Model


@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""

    request_id: int
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


@dataclass
class AheadStep:
    """A decode step launched before the step before it had been read back (see
    :meth:`ModelRunner.step_ahead`): who was in it, where each request stood, and its logits."""

    request_ids: list[int]
    starts: list[int]
    logits: torch.Tensor
    issue: int
    tokens: list[int] | None = None  # what it was fed, once the host knows


class _Staging:
    """Host (pinned) and device int32 buffers the step's metadata travels in, as one copy."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.capacity = 0
        self.host: torch.Tensor | None = None
        self.dev: torch.Tensor | None = None
        self.frozen = False
        # Recorded after each host-to-device copy; the host side is not rewritten before it.
        self.copied = torch.cuda.Event()
        self.copy_pending = False

    def wait_for_copy(self) -> None:
        if self.copy_pending:
            self.copied.synchronize()
            self.copy_pending = False

    def reserve(self, count: int) -> None:
        self.wait_for_copy()
        if count <= self.capacity:
            return
        if self.frozen:
            raise RuntimeError("step metadata outgrew its buffer while a CUDA graph holds it")
        self.capacity = max(count, 2 * self.capacity, 4096)
        self.host = torch.empty(self.capacity, dtype=torch.int32, pin_memory=True)
        self.dev = torch.empty(self.capacity, dtype=torch.int32, device=self.device)
        self.host_np = self.host.numpy()


@dataclass
class _Layout:
    """Offsets (in int32 words) of each metadata array inside the staging buffer."""

    tokens: int
    seqs: int
    wanted: int
    max_pages: int
    groups: int

    def __post_init__(self) -> None:
        t, s, w = self.tokens, self.seqs, self.wanted
        offset = 0

        def take(n: int) -> int:
            nonlocal offset
            start = offset
            offset += (n + 3) // 4 * 4  # keep every array 16-byte aligned
            return start

        self.token_ids = take(t)
        self.positions = take(t)
        self.token_seq = take(t)
        self.seq_q_start = take(s)
        self.seq_q_len = take(s)
        self.seq_kv_len = take(s)
        self.seq_slot = take(s)
        self.logit_rows = take(w)
        self.tables = [take(s * self.max_pages) for _ in range(self.groups)]
        self.total = offset


class ModelRunner:
    def __init__(self, model: Model, cache: PagedCache, *, max_batch_tokens: int, options: dict | None = None) -> None:
        if model.device is None:
            raise RuntimeError("load the model's weights before building a runner")
        self.model, self.cache = model, cache
        self.device, self.dtype = model.device, model.dtype
        self.lib = kernels()
        self.max_batch_tokens = max_batch_tokens
        self.options = dict(options or {})
        self.workspace = Workspace(self.device, min_rows=min(max_batch_tokens, int(self.options.get("workspace_rows", 0))))
        self.staging = _Staging(self.device)
        # The metadata buffers never move after this: CUDA graphs hold their addresses.
        groups = len(cache.groups)
        seqs = max_batch_tokens  # a step never holds more requests than tokens
        self.staging.reserve(_Layout(max_batch_tokens, seqs, max_batch_tokens, cache.max_pages_per_request, groups).total)
        self.staging.frozen = True
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.steps = 0
        self.tokens_run = 0
        # Decode-only steps replay a CUDA graph per batch-size bucket (see _decode_graph).
        self.use_graphs = bool(self.options.get("cuda_graphs", True)) and bool(getattr(model, "graph_safe", False))
        # With options["decode_kernel"] = "resident", steps of up to 16 single tokens run as one
        # resident kernel when the model is made of the parts that kernel was written for. The
        # default is the chain of kernels, which is the faster of the two (see parts/resident.py).
        self.options["resident"] = None
        if self.options.get("decode_kernel", "chain") == "resident":
            from ..parts.resident import ResidentDecoder

            self.options["resident"] = ResidentDecoder.for_model(model, cache, self.lib)
        self._graphs: dict[tuple[int, int], tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}
        self._graph_generation = -1
        self.graph_replays = 0
        self.launches_per_graph: dict[int, int] = {}
        self.issue = 0  # batches launched so far; an AheadStep is only good while nothing followed it
        # With options["step_timing"]: the host's wall time inside `step` and, from two events per
        # step that are read only when asked for, the device's time for the same steps.
        self.step_timing = bool(self.options.get("step_timing"))
        self.host_seconds = 0.0
        self._device_ms = 0.0
        self._timed_steps = 0
        self._open_events: list[tuple[torch.cuda.Event, torch.cuda.Event]] = []

    # ------------------------------------------------------------------------------------------

    def step(self, entries: Sequence[StepEntry], *, check: bool = False) -> torch.Tensor:
        """Run one batch; returns ``[wanted, vocab]`` float32 logits on the device, in the
        order of ``entries`` and of each entry's ``want``. They live in scratch memory that the
        next step reuses: copy what must outlast it."""
        entries = [e for e in entries if len(e.tokens) > 0]
        manager = self.cache.manager
        if not entries:
            return torch.empty((0, self.model.head.vocab_size), dtype=torch.float32, device=self.device)
        if self.step_timing:
            began = time.perf_counter()
            events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            events[0].record()
            try:
                return self._step(entries, check)
            finally:
                events[1].record()
                self._open_events.append(events)
                self._timed_steps += 1
                self.host_seconds += time.perf_counter() - began
        return self._step(entries, check)

    def timing(self) -> dict[str, float]:
        """Totals over the steps run with ``step_timing``: the host's time inside `step`
        (building metadata and launching) and the device's time between each step's first
        and last launch. Reading the device's time waits for the steps to finish."""
        for first, last in self._open_events:
            last.synchronize()
            self._device_ms += first.elapsed_time(last)
        self._open_events.clear()
        return {"timed_steps": self._timed_steps, "host_ms": self.host_seconds * 1e3, "device_ms": self._device_ms}

    def _step(self, entries: Sequence[StepEntry], check: bool) -> torch.Tensor:
        manager = self.cache.manager
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id} appears twice in one step")
            seen.add(e.request_id)
        total = sum(len(e.tokens) for e in entries)
        if total > self.max_batch_tokens:
            raise ValueError(f"the step holds {total} tokens, more than max_batch_tokens={self.max_batch_tokens}")

        # Single decoded tokens first, then prompt portions: kernels specialised for one
        # query per request take the front of the batch.
        order = sorted(range(len(entries)), key=lambda i: (len(entries[i].tokens) != 1, i))
        starts = [manager.length(e.request_id) for e in entries]
        longest = self.cache.max_pages_per_request * self.cache.page_size
        for e, start in zip(entries, starts):
            if start + len(e.tokens) > longest:
                raise ValueError(
                    f"request {e.request_id} would hold {start + len(e.tokens)} tokens; the cache was built for "
                    f"requests of at most {longest} (the model's position limit or the pool's size)"
                )
        for e, start in zip(entries, starts):
            manager.ensure(e.request_id, start + len(e.tokens))
        self.cache.clear_new_slots()

        row_of_entry = [0] * len(entries)
        cursor = 0
        for i in order:
            row_of_entry[i] = cursor
            cursor += len(entries[i].tokens)
        wanted_rows: list[int] = []
        for i, e in enumerate(entries):
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.request_id}: wanted place {w} is outside its {len(e.tokens)} tokens")
                wanted_rows.append(row_of_entry[i] + int(w))

        ordered = [entries[i] for i in order]
        ordered_starts = [starts[i] for i in order]
        nvtx = bool(self.options.get("nvtx"))
        if nvtx:  # one range per step, named for what it holds (cuda/engine.cu:53,75 in the reference)
            torch.cuda.nvtx.range_push(f"step {self.steps}: {len(entries)} requests, {total} tokens")
        try:
            if self.use_graphs and total == len(entries) and len(entries) <= self.cache.max_num_sequences:
                logits = self._decode_graph(ordered, ordered_starts, wanted_rows)
            else:
                ctx = self._build_context(ordered, ordered_starts, wanted_rows)
                tables = self._tables
                logits = self.model.forward(ctx, lambda call: self._view(call, tables))
        finally:
            if nvtx:
                torch.cuda.nvtx.range_pop()
        for e, start in zip(entries, starts):
            manager.advance(e.request_id, start + len(e.tokens))
        self.steps += 1
        self.issue += 1
        self.tokens_run += total
        if check:
            self.check()
        return logits

    # -- a decode step launched ahead of its tokens -------------------------------------------------
    #
    # Between two decode steps the device would wait for the host: the sampled tokens travel to
    # the host, the scheduler decides, the next step's metadata travels back. When the next step
    # is known to feed the same requests one token each, everything about it except the token
    # ids is known already, and the ids are on the device. `step_ahead` launches that step with
    # the ids copied device to device, behind the sampling kernels, so it runs while the host
    # catches up. Nothing is committed: the cache lengths stay where they are until
    # `accept_ahead`; a step that turns out not to be wanted (a request ended, another was
    # admitted) is simply never accepted. What it wrote are keys and values at positions that
    # either will be rewritten with the same numbers or belong to a request that is gone.

    def step_ahead(self, request_ids: Sequence[int], tokens_dev: torch.Tensor) -> AheadStep | None:
        """Launch one token per request, the tokens being ``tokens_dev[:len(request_ids)]`` on
        the device. Returns None, launching nothing, unless the step can replay a captured
        graph."""
        count = len(request_ids)
        if not self.use_graphs or count == 0 or count > self.cache.max_num_sequences:
            return None
        bucket = self._bucket(count)
        manager = self.cache.manager
        starts = [manager.length(r) for r in request_ids]
        if any(start + 1 > self.cache.max_pages_per_request * self.cache.page_size for start in starts):
            return None
        reach = self._reach(max(starts) + 1)
        cached = self._graphs.get((bucket, reach))
        if cached is None or self._graph_generation != self.workspace.generation:
            return None
        for r, start in zip(request_ids, starts):
            manager.ensure(r, start + 1)
        self._build_context([StepEntry(r, (0,)) for r in request_ids], starts, list(range(bucket)), pad_to=bucket, reach=reach)
        self.staging.dev[:count].copy_(tokens_dev[:count], non_blocking=True)  # the token ids lead the buffer
        graph, logits, _ = cached
        graph.replay()
        self.graph_replays += 1
        self.issue += 1
        return AheadStep(list(request_ids), starts, logits[:count], self.issue)

    def accept_ahead(self, ahead: AheadStep) -> torch.Tensor:
        """The step launched ahead is the step wanted now: count it and return its logits."""
        if ahead.issue != self.issue:
            raise RuntimeError("another batch ran after the step launched ahead")
        manager = self.cache.manager
        for r, start in zip(ahead.request_ids, ahead.starts):
            manager.advance(r, start + 1)
        self.steps += 1
        self.tokens_run += len(ahead.request_ids)
        return ahead.logits

    def check(self) -> None:
        """Raise if any kernel flagged an error since the last check (synchronises)."""
        check_error_word(self.err, "step")

    # ------------------------------------------------------------------------------------------

    def _view(self, call: LayerCall, tables):
        return self.cache.view(call.cache_id, call.writes, tables)

    # -- decode steps as CUDA graphs ---------------------------------------------------------------
    #
    # A step in which every request feeds one token launches the same kernels with the same
    # arguments every time, once its batch is padded to a fixed size: all that changes lives
    # in the metadata buffer (tokens, positions, lengths, block tables), which the kernels
    # read on the device. So such a step is captured once per batch-size bucket and
    # replayed. Padding rows are requests of length one whose table points at the arena's
    # spare page. The first step of a bucket runs eagerly (that run's results are used) and
    # is then captured for the following ones.

    def _bucket(self, count: int) -> int:
        bucket = 1
        while bucket < count:
            bucket *= 2
        return min(bucket, max(self.cache.max_num_sequences, count))

    def _reach(self, longest: int) -> int:
        """The key count a captured step is launched for: the next power of two (from 1,024 on) at
        or above the longest request of the step, at most the engine's limit. The kernels walk
        each request's own keys whatever this is; it only decides how many blocks cut the keys, so
        that an engine built for long requests does not launch its short ones in 64 pieces."""
        limit = self.cache.max_pages_per_request * self.cache.page_size
        reach = 1024
        while reach < longest:
            reach *= 2
        return min(reach, limit)

    def _decode_graph(self, entries: list[StepEntry], starts: list[int], wanted_rows: list[int]) -> torch.Tensor:
        count = len(entries)
        bucket = self._bucket(count)
        reach = self._reach(max(starts) + 1)
        if self._graph_generation != self.workspace.generation:
            self._graphs.clear()  # a scratch buffer moved: captured addresses are stale
        ctx = self._build_context(entries, starts, list(range(bucket)), pad_to=bucket, reach=reach)
        tables = self._tables
        cached = self._graphs.get((bucket, reach))
        if cached is None:
            calls_before = self.lib.calls
            logits = self.model.forward(ctx, lambda call: self._view(call, tables))
            self.launches_per_graph[bucket] = self.lib.calls - calls_before
            if self._graph_generation != self.workspace.generation:
                # The eager run allocated scratch; capture on the next step, when nothing moves.
                self._graph_generation = self.workspace.generation
                self._graphs.clear()
            else:
                graph = torch.cuda.CUDAGraph()
                torch.cuda.current_stream(self.device).synchronize()
                with torch.cuda.graph(graph):
                    captured = self.model.forward(ctx, lambda call: self._view(call, tables))
                self._graphs[(bucket, reach)] = (graph, captured, self.workspace.generation)
        else:
            graph, logits, _ = cached
            graph.replay()
            self.graph_replays += 1
        if wanted_rows == list(range(count)):
            return logits[:count]
        return logits[torch.tensor(wanted_rows, dtype=torch.long, device=self.device)]

    def _build_context(
        self, entries: list[StepEntry], starts: list[int], wanted_rows: list[int], pad_to: int | None = None,
        reach: int | None = None,
    ) -> StepContext:
        """Lay the step's metadata out in the pinned buffer, copy it to the device and wrap it.
        With ``pad_to`` (single-token steps only) the batch is filled up to that many requests
        with rows that write to the arenas' spare page."""
        real = len(entries)
        t = sum(len(e.tokens) for e in entries)
        s = len(entries)
        if pad_to is not None:
            t = s = pad_to
        w = len(wanted_rows)
        groups = len(self.cache.groups)
        layout = _Layout(t, s, w, self.cache.max_pages_per_request, groups)
        self.staging.reserve(layout.total)
        buf = self.staging.host_np

        def host_view(offset: int, n: int) -> np.ndarray:
            return buf[offset : offset + n]

        token_ids = host_view(layout.token_ids, t)
        positions = host_view(layout.positions, t)
        token_seq = host_view(layout.token_seq, t)
        q_start = host_view(layout.seq_q_start, s)
        q_len = host_view(layout.seq_q_len, s)
        kv_len = host_view(layout.seq_kv_len, s)
        slot = host_view(layout.seq_slot, s)
        rows = host_view(layout.logit_rows, w)
        cursor = 0
        decode = 0
        for i, (e, start) in enumerate(zip(entries, starts)):
            n = len(e.tokens)
            token_ids[cursor : cursor + n] = np.asarray(e.tokens, dtype=np.int32)
            positions[cursor : cursor + n] = np.arange(start, start + n, dtype=np.int32)
            token_seq[cursor : cursor + n] = i
            q_start[i], q_len[i], kv_len[i] = cursor, n, start + n
            slot[i] = self.cache.manager.slot(e.request_id)
            if n == 1 and decode == i:
                decode += 1
            cursor += n
        rows[:] = np.asarray(wanted_rows, dtype=np.int32)
        ids = [e.request_id for e in entries]
        table_views = [
            host_view(layout.tables[g], s * layout.max_pages).reshape(s, layout.max_pages) for g in range(groups)
        ]
        self.cache.fill_tables(ids, table_views)
        if s > real:
            token_ids[real:] = 0
            positions[real:] = 0
            token_seq[real:] = np.arange(real, s, dtype=np.int32)
            q_start[real:] = np.arange(real, s, dtype=np.int32)
            q_len[real:] = 1
            kv_len[real:] = 1
            slot[real:] = self.cache.null_slot()
            for group in self.cache.groups:
                table_views[group.index][real:] = self.cache.null_page(group)
            decode = s
        dev = self.staging.dev
        dev[: layout.total].copy_(self.staging.host[: layout.total], non_blocking=True)
        self.staging.copied.record()
        self.staging.copy_pending = True

        def dev_view(offset: int, n: int) -> torch.Tensor:
            return dev[offset : offset + n]

        self._tables = [dev_view(layout.tables[g], s * layout.max_pages).view(s, layout.max_pages) for g in range(groups)]
        host = HostBatch(
            token_ids=token_ids, positions=positions, token_seq=token_seq, seq_q_start=q_start,
            seq_q_len=q_len, seq_kv_len=kv_len, seq_slot=slot, logit_rows=rows,
        )
        return StepContext(
            lib=self.lib,
            dtype=self.dtype,
            device=self.device,
            num_tokens=t,
            num_seqs=s,
            host=host,
            token_ids=dev_view(layout.token_ids, t),
            positions=dev_view(layout.positions, t),
            token_seq=dev_view(layout.token_seq, t),
            seq_q_start=dev_view(layout.seq_q_start, s),
            seq_q_len=dev_view(layout.seq_q_len, s),
            seq_kv_len=dev_view(layout.seq_kv_len, s),
            seq_slot=dev_view(layout.seq_slot, s),
            logit_rows=dev_view(layout.logit_rows, w),
            err=self.err,
            workspace=self.workspace,
            num_decode_seqs=decode,
            # A captured step is launched for a bucket of key counts (see _reach), not for this
            # step's own longest request.
            max_kv_len=int(kv_len.max()) if pad_to is None else (reach or self.cache.max_pages_per_request * self.cache.page_size),
            max_q_len=int(q_len.max()),
            captured=pad_to is not None,
            options=self.options,
        )
