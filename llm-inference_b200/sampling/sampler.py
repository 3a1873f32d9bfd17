"""Turns a step's logits into tokens on the device.

Greedy rows go through the arg-max kernel, the others through the sampling kernel
(csrc/kernels/sampling.cu); one device-to-host copy brings back every row's token.
"""

from __future__ import annotations

from ctypes import c_int, c_int64
from typing import Sequence

import numpy as np
import torch

from ..csrc.library import kernels, ptr


class Sampler:
    def __init__(self, device: torch.device, max_rows: int) -> None:
        self.device = device
        self.lib = kernels()
        self.max_rows = max_rows = (max_rows + 3) // 4 * 4
        # One packed parameter block per step: [temperature | top_p | min_p | top_k | rows | keys].
        self._host = torch.empty(max_rows * 8, dtype=torch.int32, pin_memory=True)
        self._dev = torch.empty(max_rows * 8, dtype=torch.int32, device=device)
        self._tokens = torch.zeros(max_rows + 1, dtype=torch.int32, device=device)
        self._tokens_host = torch.zeros(max_rows + 1, dtype=torch.int32, pin_memory=True)
        # Scratch of the arg-max over many blocks per row: zero now, left zero by every launch.
        self._best = torch.zeros(max_rows, dtype=torch.int64, device=device)
        self._arrived = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.lib.lib.b200_sample_scratch_bytes.restype = c_int64
        self._sample_scratch = torch.zeros(int(self.lib.lib.b200_sample_scratch_bytes(max_rows)), dtype=torch.uint8, device=device)
        self._done = torch.cuda.Event()  # recorded after the copy of a step's tokens to the host

    @property
    def tokens_device(self) -> torch.Tensor:
        """The last launch's tokens on the device, row by row (valid in stream order)."""
        return self._tokens

    def sample(
        self,
        logits: torch.Tensor,
        params: Sequence,  # objects with temperature, top_p, top_k, min_p, greedy
        keys: Sequence[int],
        err: torch.Tensor | None = None,
    ) -> tuple[list[int], int]:
        """One token per row of ``logits`` (``[rows, vocab]`` float32). ``keys[i]`` seeds
        row i's draw. Returns the tokens and the kernels' error word (0 = none)."""
        return self.result(self.launch(logits, params, keys, err))

    def launch(self, logits: torch.Tensor, params: Sequence, keys: Sequence[int], err: torch.Tensor | None = None) -> int:
        """Enqueue the kernels of :meth:`sample` and the copy of their tokens to the host;
        returns the number of rows for :meth:`result`. Work enqueued after this call does not
        delay the result."""
        rows, vocab = logits.shape
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows to sample, the sampler was sized for {self.max_rows}")
        if rows == 0:
            return 0
        stream = torch.cuda.current_stream(self.device).cuda_stream
        from ctypes import c_void_p

        s = c_void_p(stream)
        greedy = [i for i, p in enumerate(params) if p.greedy]
        sampled = [i for i, p in enumerate(params) if not p.greedy]
        tokens = self._tokens
        if not sampled:
            self.lib.call(
                "b200_argmax_rows", ptr(logits), c_int(rows), c_int(vocab), c_int64(logits.stride(0)),
                c_void_p(0), ptr(tokens), ptr(self._best), ptr(self._arrived), s,
            )
        else:
            n, g = len(sampled), len(greedy)
            host = self._host.numpy()
            m = self.max_rows
            host[0:n].view(np.float32)[:] = [params[i].temperature for i in sampled]
            host[m : m + n].view(np.float32)[:] = [params[i].top_p for i in sampled]
            host[2 * m : 2 * m + n].view(np.float32)[:] = [params[i].min_p for i in sampled]
            host[3 * m : 3 * m + n] = [params[i].top_k for i in sampled]
            host[4 * m : 4 * m + n] = sampled
            host[5 * m : 5 * m + g] = greedy
            host[6 * m : 6 * m + 2 * n].view(np.uint64)[:] = [keys[i] for i in sampled]
            self._dev.copy_(self._host, non_blocking=True)
            dev = self._dev
            if g:
                self.lib.call(
                    "b200_argmax_rows", ptr(logits), c_int(g), c_int(vocab), c_int64(logits.stride(0)),
                    ptr(dev[5 * m :]), ptr(tokens), ptr(self._best), ptr(self._arrived), s,
                )
            self.lib.call(
                "b200_sample_rows", ptr(logits), c_int(n), c_int(vocab), c_int64(logits.stride(0)),
                ptr(dev[0:]), ptr(dev[m:]), ptr(dev[2 * m :]), ptr(dev[3 * m :]), ptr(dev[6 * m :]),
                ptr(dev[4 * m :]), ptr(tokens), ptr(self._sample_scratch), c_int64(self._sample_scratch.numel()), s,
            )
        if err is not None:
            tokens[rows : rows + 1].copy_(err)
        else:
            tokens[rows : rows + 1].zero_()
        self._tokens_host[: rows + 1].copy_(tokens[: rows + 1], non_blocking=True)
        self._done.record()
        return rows

    def result(self, rows: int) -> tuple[list[int], int]:
        """Wait for the tokens of the last :meth:`launch` (and only for them)."""
        if rows == 0:
            return [], 0
        self._done.synchronize()
        out = self._tokens_host[: rows + 1].tolist()
        return out[:rows], out[rows]
