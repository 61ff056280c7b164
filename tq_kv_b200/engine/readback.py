"""Where the sampler's token ids live on the device, and their way back to
the host.

The ids of a step's rows are written into a fixed device buffer, so that the
next decode step can take its tokens from there (`StepRow.source`) while the
host has not read them yet.  `fetch()` starts a copy of the ids, together with
the kernels' status word that sits in front of them, into pinned host memory
and returns a ticket; `wait(ticket)` blocks until that copy has arrived,
raises if a kernel reported a wait that ran out, and returns the ids.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..kernels._lib import REPORT_ROWS, raise_on_status, report_buffer


class SampledIds:
    RING = 8

    def __init__(self, device):
        self.device = torch.device(device)
        self.report = report_buffer(self.device)          # word 0: status; words 1..: ids
        self.ids = self.report[1:]
        self.rows = REPORT_ROWS
        self._host = [torch.zeros(1 + REPORT_ROWS, dtype=torch.int32).pin_memory() for _ in range(self.RING)]
        self._events = [None] * self.RING
        self._turn = 0
        self.d2h_bytes = 0

    def fetch(self, n_rows: int):
        """Starts the copy of ids[0:n_rows] (and the status word) to the host."""
        i = self._turn % self.RING
        self._turn += 1
        self._host[i][:1 + n_rows].copy_(self.report[:1 + n_rows], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._events[i] = ev
        self.d2h_bytes += 4 * (1 + n_rows)
        return (i, n_rows)

    def wait(self, ticket) -> list[int]:
        i, n_rows = ticket
        self._events[i].synchronize()
        got = self._host[i][:1 + n_rows].tolist()
        kernels._lib._tc_launched[0] = 0                  # the status word has just been read
        raise_on_status(got[0], self.device)
        return got[1:]
