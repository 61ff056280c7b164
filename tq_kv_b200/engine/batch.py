"""Packing the rows of a step into one int32 buffer that goes to the device
in a single copy."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..cache import SequenceCache
from ..parts import StepBatch


@dataclass
class StepRow:
    """One sequence's share of a step: its cache slot, the tokens it brings
    and the places among them whose logits are wanted.  A row of one token
    may name `source` instead of the token's value: the row of the ids the
    sampler wrote last (on the device) that holds it; `tokens` is then [0]."""
    slot: int
    tokens: list[int]
    want: list[int]
    source: Optional[int] = None


def _pad4(n: int) -> int:
    return (n + 3) // 4 * 4


class FlatRows:
    """The rows of a step as the host runtime takes them: flat int32 arrays."""
    __slots__ = ("slots", "lens", "tokens", "want_counts", "want", "sources", "any_source")

    def __init__(self, rows: list[StepRow]):
        self.slots = np.fromiter((r.slot for r in rows), dtype=np.int32, count=len(rows))
        self.lens = np.fromiter((len(r.tokens) for r in rows), dtype=np.int32, count=len(rows))
        self.want_counts = np.fromiter((len(r.want) for r in rows), dtype=np.int32, count=len(rows))
        if len(rows) == 1:
            self.tokens = np.asarray(rows[0].tokens, dtype=np.int64)
            self.want = np.asarray(rows[0].want, dtype=np.int64)
        else:
            self.tokens = np.concatenate([np.asarray(r.tokens, dtype=np.int64) for r in rows])
            self.want = np.concatenate([np.asarray(r.want, dtype=np.int64) for r in rows])
        # ids and places that do not fit 32 bits are out of every range: they become -1, which every check refuses
        self.tokens = np.where((self.tokens >= 0) & (self.tokens < 2 ** 31), self.tokens, -1).astype(np.int32)
        self.want = np.where((self.want >= 0) & (self.want < 2 ** 31), self.want, -1).astype(np.int32)
        self.any_source = any(r.source is not None for r in rows)
        self.sources = np.fromiter((-1 if r.source is None else r.source for r in rows), dtype=np.int32,
                                   count=len(rows))


def build_step_batch(rows: list[StepRow], cache: SequenceCache, device, flat: Optional[FlatRows] = None) -> StepBatch:
    """Packs `rows` (already reserved in the cache) into one pinned int32
    buffer and copies it to the device.  The host runtime lays the buffer out
    (csrc/host_runtime.cpp): tokens | tok_seq | tok_pos | cu_seqlens | slots |
    start_pos | new_lens | logit_rows | tok_src | one block table per cache
    group; every segment starts on a 16-byte boundary."""
    flat = flat or FlatRows(rows)
    book = cache.book
    B = len(rows)
    T, R = int(flat.lens.sum()), int(flat.want_counts.sum())
    starts = book.lengths(flat.slots)
    layout = book.step_layout(flat.slots, flat.lens, flat.want_counts)
    dev = torch.device(device)
    host = torch.empty(layout.total, dtype=torch.int32, pin_memory=dev.type == "cuda")
    book.pack_step(flat.slots, flat.lens, flat.tokens, flat.want_counts, flat.want, flat.sources, layout, host.numpy())
    d = host.to(dev, non_blocking=True)
    offs = layout.offs.tolist()
    widths = layout.widths.tolist()

    def seg(i: int, n: int) -> torch.Tensor:
        return d[offs[i]: offs[i] + n]

    return StepBatch(
        n_tokens=T, n_seqs=B, tokens=seg(0, T), tok_seq=seg(1, T), tok_pos=seg(2, T), cu_seqlens=seg(3, B + 1),
        slots=seg(4, B), start_pos=seg(5, B), new_lens=seg(6, B), logit_rows=seg(7, R), n_logit_rows=R,
        block_tables=[(seg(9 + gi, B * widths[gi]), widths[gi]) for gi in range(len(cache.groups))],
        host_slots=flat.slots.tolist(), host_start=starts, host_lens=flat.lens.tolist(),
        packed_bytes=layout.total * 4, tok_src=seg(8, T), any_source=flat.any_source)
