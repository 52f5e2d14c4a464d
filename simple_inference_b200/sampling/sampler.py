"""Draws one token per row of logits with the sampling kernel.

The per-row parameters travel in one pinned buffer and one device buffer with
fixed addresses; the chosen tokens come back in one small copy, which is the
step's only device-to-host read (the reference's ``.tolist()`` after sampling,
``serving/engine.py:444``).
"""

from __future__ import annotations

import numpy as np
import torch

from .. import ops
from .params import SamplingParams

_FIELDS = 6  # temperature, top_k, top_p, seed, stream, counter


class Sampler:
    def __init__(self, device: torch.device, max_rows: int):
        self.device = device
        self.max_rows = max_rows
        pin = device.type == "cuda"
        self._host = torch.zeros(_FIELDS * max_rows, dtype=torch.int32, pin_memory=pin)
        self._np = self._host.numpy()
        self._dev = torch.zeros(_FIELDS * max_rows, dtype=torch.int32, device=device)
        self._out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.zeros(max_rows, dtype=torch.int32, pin_memory=pin)
        self._status_host = torch.zeros(1, dtype=torch.int32, pin_memory=pin)
        self._done = torch.cuda.Event() if pin else None
        # what the rows held at the last call: while the same requests keep drawing (steady
        # decoding) only their counters change, and one slice assignment writes those
        self._last_rows: list[tuple[SamplingParams, int]] | None = None
        # views of the buffers per number of rows, made once (slicing costs more than sampling's
        # other host work)
        self._views: dict[int, tuple] = {}

    @property
    def host_bytes(self) -> int:
        """Bytes of options copied to the device per call of ``sample``."""
        return self._host.numel() * 4

    def _field(self, buf, i: int, n: int):
        return buf[i * self.max_rows: i * self.max_rows + n]

    def sample(self, logits: torch.Tensor,
               rows: list[tuple[SamplingParams, int, int]]) -> list[int]:
        """``rows[i]`` = (options, stream id of the request, index of the token to draw)."""
        n = len(rows)
        if n != logits.shape[0]:
            raise ValueError(f"{logits.shape[0]} rows of logits for {n} sets of options")
        if n > self.max_rows:
            raise ValueError(f"{n} rows exceed the sampler's capacity {self.max_rows}")
        if n == 0:
            return []
        m = self.max_rows
        who = [(p, stream) for p, stream, _ in rows]
        if who == self._last_rows:
            self._np.view(np.uint32)[5 * m:5 * m + n] = [c & 0xFFFFFFFF for _, _, c in rows]
        else:
            f32 = self._np.view(np.float32)
            u32 = self._np.view(np.uint32)
            for i, (p, stream, counter) in enumerate(rows):
                f32[0 * m + i] = p.temperature
                self._np[1 * m + i] = p.top_k
                f32[2 * m + i] = p.top_p
                u32[3 * m + i] = p.seed & 0xFFFFFFFF
                u32[4 * m + i] = stream & 0xFFFFFFFF
                u32[5 * m + i] = counter & 0xFFFFFFFF
            self._last_rows = who
        self._dev.copy_(self._host, non_blocking=True)
        self.sample_on_device(logits)
        self._out_host[:n].copy_(self._out[:n], non_blocking=True)
        if self.device.type == "cuda":
            # the kernels' status word rides home with the tokens: one synchronisation for both
            status = ops.status_tensor(self.device)
            self._status_host.copy_(status, non_blocking=True)
            self._done.record()
            self._done.synchronize()
            if int(self._status_host[0]) != 0:
                ops.check_status(self.device)
        tokens = self._out_host[:n].tolist()
        if min(tokens) < 0:
            bad = [i for i, t in enumerate(tokens) if t < 0]
            raise ops.KernelError(f"sampling: rows {bad} of the logits hold no comparable value "
                                  f"(NaN): a kernel of this step failed")
        return tokens

    def sample_on_device(self, logits: torch.Tensor) -> torch.Tensor:
        """Draw for the rows of ``logits`` with the options of the last ``sample`` call already
        on the device; the tokens stay on the device (no copy, no synchronisation)."""
        n = logits.shape[0]
        v = self._views.get(n)
        if v is None:
            d = self._dev
            v = self._views[n] = (self._field(d, 0, n).view(torch.float32), self._field(d, 1, n),
                                  self._field(d, 2, n).view(torch.float32), self._field(d, 3, n),
                                  self._field(d, 4, n), self._field(d, 5, n), self._out[:n])
        ops.sample(logits, *v)
        return v[6]
