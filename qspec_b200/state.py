"""Sequence-state manager shared by the models that the scheduler serves: slots, positions, and the per-step token
table the kernels read.

A live request owns one slot. What a slot holds is the model's business (key/value rows, convolution tails, ...); this
module owns the bookkeeping that is the same for every model: which slots are free, how many tokens each sequence has
consumed, and the flat description of a step (`BatchMeta`) -- for every token its slot, its position, where its
sequence's tokens begin and end in the batch, and which of the two tail buffers holds the state from before the step.
State that a slot held is never cleared on release: the kernels decide from positions alone what is valid, so a reused
slot cannot leak rows of its previous owner.

The reference leaves all of this to vLLM's block manager and scheduler (vllm/core/scheduler.py, block_manager.py), which
are outside the int4 path this framework rebuilds; this is the minimal equivalent the decode loop needs.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Sequence, Tuple

import torch

META_ROWS = 5          # slot, pos, seg_begin, seg_end, phase (include/qspec_b200_seq.h)


class SlotPool:
    """Free list of state slots. The most recently released slot is handed out first."""

    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise ValueError("SlotPool: at least one slot")
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))

    def alloc(self) -> int:
        if not self._free:
            raise RuntimeError(f"all {self.n_slots} sequence slots are in use")
        return self._free.pop()

    def release(self, slot: int) -> None:
        if slot in self._free or not 0 <= slot < self.n_slots:
            raise ValueError(f"slot {slot} is not in use")
        self._free.append(slot)

    @property
    def free(self) -> int:
        return len(self._free)


@dataclass
class BatchMeta:
    """One step's token table. `table` is the device int32 [5, ntok] the kernels read; the rest is host bookkeeping."""
    table: torch.Tensor
    ids: torch.Tensor                                  # device int32 [ntok]: the step's token ids (zeros if none were given)
    rows: torch.Tensor                                 # device int32 [n]: batch rows the caller asked to have gathered
    seg_starts: torch.Tensor                           # device int32 [segments]: batch row of every segment's first token
    ntok: int
    segments: List[Tuple[Hashable, int, int, int]]     # (request id, slot, first position, token count)

    @property
    def max_length(self) -> int:
        """Length of the longest sequence once the step has run: no token of the step sees more keys than this."""
        return max((first + n for _, _, first, n in self.segments), default=0)

    @property
    def slot(self) -> torch.Tensor:
        return self.table[0]

    @property
    def pos(self) -> torch.Tensor:
        return self.table[1]


class SequenceTable:
    """Slots, positions and tail phases of the live sequences."""

    def __init__(self, n_slots: int, device, max_step_tokens: int):
        self.pool = SlotPool(n_slots)
        self.device = torch.device(device)
        self.slot_of: Dict[Hashable, int] = {}
        self.pos = [0] * n_slots            # tokens consumed so far
        self.phase = [0] * n_slots          # tail buffer that holds the current state
        self.max_step_tokens = max_step_tokens

    def open(self, rid: Hashable) -> int:
        if rid in self.slot_of:
            raise ValueError(f"request {rid!r} is already live")
        slot = self.pool.alloc()
        self.slot_of[rid] = slot
        self.pos[slot] = 0
        return slot

    def close(self, rid: Hashable) -> None:
        self.pool.release(self.slot_of.pop(rid))

    def held_tokens(self) -> int:
        return sum(self.pos[s] for s in self.slot_of.values())

    def plan(self, segments: Sequence[Tuple[Hashable, int]], token_ids: Sequence[int] = None,
             rows: Sequence[int] = None) -> BatchMeta:
        """segments: (request id, number of new tokens), each request at most once; unknown requests get a slot.
        token_ids: the step's tokens in batch order; rows: batch rows a caller wants to gather afterwards (at most one
        per token). Both travel to the device in the same copy as the table. Every step stages its table in a fresh
        pinned block: the copy is asynchronous, and the host may plan the next step before the device has fetched this
        one."""
        import numpy as np
        counts = np.fromiter((n for _, n in segments), dtype=np.int64, count=len(segments))
        if len(counts) and counts.min() < 1:
            raise ValueError("a segment needs at least one token")
        ntok = int(counts.sum())
        if ntok > self.max_step_tokens:
            raise ValueError(f"a step of {ntok} tokens exceeds max_step_tokens = {self.max_step_tokens}")
        if token_ids is not None and len(token_ids) != ntok:
            raise ValueError(f"{len(token_ids)} token ids for a step of {ntok} tokens")
        if rows is not None and len(rows) > ntok:
            raise ValueError("more rows to gather than tokens in the step")
        slots, firsts, segs = [], [], []
        for rid, n in segments:
            slot = self.slot_of[rid] if rid in self.slot_of else self.open(rid)
            slots.append(slot)
            firsts.append(self.pos[slot])
            segs.append((rid, slot, self.pos[slot], int(n)))
        if len(set(slots)) != len(slots):
            raise ValueError("a request appears twice in one step")
        begin = np.cumsum(counts) - counts
        h = np.zeros((META_ROWS + 3, ntok), dtype=np.int32)
        h[0] = np.repeat(np.asarray(slots, dtype=np.int64), counts)
        h[2] = np.repeat(begin, counts)
        h[1] = np.repeat(np.asarray(firsts, dtype=np.int64), counts) + (np.arange(ntok) - h[2])
        h[3] = np.repeat(begin + counts, counts)
        h[4] = np.repeat(np.asarray([self.phase[s] for s in slots], dtype=np.int64), counts)
        if token_ids is not None:
            h[META_ROWS] = np.asarray(token_ids, dtype=np.int64)
        nrows = 0
        if rows is not None and len(rows):
            nrows = len(rows)
            h[META_ROWS + 1, :nrows] = np.asarray(rows, dtype=np.int64)
        h[META_ROWS + 2, :len(counts)] = begin         # one entry per segment (a segment has at least one token)
        t = torch.from_numpy(h)
        if self.device.type == "cuda":
            t = t.pin_memory()
        dev = t.to(self.device, non_blocking=True)
        return BatchMeta(table=dev[:META_ROWS], ids=dev[META_ROWS], rows=dev[META_ROWS + 1, :nrows],
                         seg_starts=dev[META_ROWS + 2, :len(segs)], ntok=ntok, segments=segs)

    def commit(self, meta: BatchMeta) -> None:
        """The step described by `meta` has been queued: its tokens now count as consumed."""
        for _, slot, _, n in meta.segments:
            self.pos[slot] += n
            self.phase[slot] ^= 1
