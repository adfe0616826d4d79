"""Host-side planning for packed ragged batches and their data-parallel sharding.

The recurrent cells need no exchange between documents, so a multi-GPU run splits DOCUMENTS over ranks and
uses no collective on the data path (the continuous-batching workload: 512 documents, log-normal lengths, rows of
32768 tokens).  Everything here is plain Python on the host; the kernels only ever see `cu_seqlens`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence


@dataclass
class PackedRows:
    """Documents packed into fixed-length rows.  `cu_seqlens` indexes the flattened (rows * row_len) token axis
    and includes the padding tail of each row as a document of its own (so that offsets stay contiguous);
    `doc_ids[i]` is the caller's document index of interval i, or -1 for padding."""
    row_len: int
    rows: int
    cu_seqlens: List[int]
    doc_ids: List[int]


def pack_documents(lengths: Sequence[int], row_len: int) -> PackedRows:
    """First-fit-decreasing packing of documents into rows of `row_len` tokens; no document straddles a row."""
    if any(l <= 0 or l > row_len for l in lengths):
        raise ValueError("document lengths must be in [1, row_len]")
    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    free: List[int] = []          # free tokens per row
    content: List[List[int]] = []  # document ids per row
    for i in order:
        for r, f in enumerate(free):
            if f >= lengths[i]:
                free[r] -= lengths[i]
                content[r].append(i)
                break
        else:
            free.append(row_len - lengths[i])
            content.append([i])
    cu, ids = [0], []
    for r, docs in enumerate(content):
        pos = r * row_len
        for d in docs:
            pos += lengths[d]
            cu.append(pos)
            ids.append(d)
        if pos < (r + 1) * row_len:   # padding tail
            cu.append((r + 1) * row_len)
            ids.append(-1)
    return PackedRows(row_len=row_len, rows=len(content), cu_seqlens=cu, doc_ids=ids)


def shard_documents(lengths: Sequence[int], world_size: int) -> List[List[int]]:
    """Longest-processing-time assignment of documents to ranks (cost = length): every document goes to exactly
    one rank and the token counts are balanced to within one document."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    load = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i in sorted(range(len(lengths)), key=lambda i: -lengths[i]):
        r = min(range(world_size), key=lambda r: load[r])
        out[r].append(i)
        load[r] += lengths[i]
    return out


class SlotPool:
    """State-slot bookkeeping for continuous-batch decoding: finished streams free their slot, queued documents
    take it over; the step kernel addresses states through the slot index, so no state is moved."""

    def __init__(self, num_slots: int):
        self.free = list(range(num_slots - 1, -1, -1))
        self.owner = {}

    def acquire(self, stream_id) -> int:
        if not self.free:
            raise RuntimeError("no free state slot")
        s = self.free.pop()
        self.owner[s] = stream_id
        return s

    def release(self, slot: int) -> None:
        if slot not in self.owner:
            raise KeyError(f"slot {slot} is not in use")
        del self.owner[slot]
        self.free.append(slot)
