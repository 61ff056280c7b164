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


def build_step_batch(rows: list[StepRow], cache: SequenceCache, device) -> StepBatch:
    """Packs `rows` (already reserved in the cache).  Layout of the buffer:
    tokens | tok_seq | tok_pos | cu_seqlens | slots | start_pos | new_lens |
    logit_rows | tok_src | one block table per cache group; every segment
    starts on a 16-byte boundary."""
    B = len(rows)
    lens = [len(r.tokens) for r in rows]
    T = sum(lens)
    starts = [cache.length(r.slot) for r in rows]
    slots = [r.slot for r in rows]
    R = sum(len(r.want) for r in rows)
    tables = [cache.block_table_rows(gi, slots) for gi in range(len(cache.groups))]

    seg_sizes = [T, T, T, B + 1, B, B, B, R, T] + [B * max(w, 1) for _, w in tables]
    offs, total = [], 0
    for s in seg_sizes:
        offs.append(total)
        total += _pad4(max(s, 1))
    buf = np.zeros(total, dtype=np.int32)

    cu = np.zeros(B + 1, dtype=np.int64)
    cu[1:] = np.cumsum(lens)
    for b, r in enumerate(rows):
        a, e = int(cu[b]), int(cu[b + 1])
        buf[offs[0] + a: offs[0] + e] = r.tokens
        buf[offs[1] + a: offs[1] + e] = b
        buf[offs[2] + a: offs[2] + e] = np.arange(starts[b], starts[b] + lens[b])
    buf[offs[3]: offs[3] + B + 1] = cu
    buf[offs[4]: offs[4] + B] = slots
    buf[offs[5]: offs[5] + B] = starts
    buf[offs[6]: offs[6] + B] = [s + n for s, n in zip(starts, lens)]
    o = offs[7]
    for b, r in enumerate(rows):
        for w in r.want:
            buf[o] = int(cu[b]) + w
            o += 1
    buf[offs[8]: offs[8] + T] = -1
    for b, r in enumerate(rows):
        if r.source is not None:
            buf[offs[8] + int(cu[b])] = r.source
    for gi, (trows, width) in enumerate(tables):
        w = max(width, 1)
        base = offs[9 + gi]
        for b, pages in enumerate(trows):
            buf[base + b * w: base + b * w + len(pages)] = pages

    host = torch.from_numpy(buf)
    dev = torch.device(device)
    if dev.type == "cuda":
        host = host.pin_memory()
    d = host.to(dev, non_blocking=True)

    def seg(i: int, n: int) -> torch.Tensor:
        return d[offs[i]: offs[i] + n]

    return StepBatch(
        n_tokens=T, n_seqs=B, tokens=seg(0, T), tok_seq=seg(1, T), tok_pos=seg(2, T), cu_seqlens=seg(3, B + 1),
        slots=seg(4, B), start_pos=seg(5, B), new_lens=seg(6, B), logit_rows=seg(7, R), n_logit_rows=R,
        block_tables=[(seg(9 + gi, B * max(w, 1)), max(w, 1)) for gi, (_, w) in enumerate(tables)],
        host_slots=slots, host_start=starts, host_lens=lens, packed_bytes=int(buf.nbytes), tok_src=seg(8, T),
        any_source=any(r.source is not None for r in rows))
