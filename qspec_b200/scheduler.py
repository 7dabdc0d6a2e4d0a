"""Continuous-batching scheduler and step function for the models of this framework.

One step = one flat token batch through `model.forward_batch`: any mix of prompt portions (several tokens of one
request) and decode tokens (one token of a request), each request at most once per step. `Scheduler.feed` is the step
function proper -- given token ids per request it advances their state and returns the logits that were asked for;
`Scheduler.step` is the generation loop built on it (pick work, feed, sample greedily, retire finished requests), and
`bin/trace_run` replays recorded steps through the same `feed`.

A model plugs in with: `n_slots`, `max_step_tokens`, `vocab_size`, `device`, `forward_batch(input_ids, meta) -> hidden`,
`logits(hidden_rows) -> [n, vocab]`, and optionally `max_seq_len` (models whose cache bounds the sequence length).
Sampling is the framework's greedy arg max (`ops.argmax_rows`), as in the speculative engine (`engine.QSpecEngine`).

The reference delegates this layer to vLLM's scheduler (vllm/core/scheduler.py) and LLMEngine.step
(vllm/engine/llm_engine.py); only its behaviour -- chunked prompts mixed with decodes, slots returned on finish -- is
restated here.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from . import ops
from .state import SequenceTable


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    max_new_tokens: int
    eos: Optional[int] = None
    fed: int = 0                                   # prompt tokens already consumed
    output: List[int] = field(default_factory=list)
    done: bool = False


class Scheduler:
    def __init__(self, model, prefill_portion: Optional[int] = None):
        self.model = model
        self.table = SequenceTable(model.n_slots, model.device, model.max_step_tokens)
        self.prefill_portion = min(prefill_portion or model.max_step_tokens, model.max_step_tokens)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: Dict[Hashable, Request] = {}
        self.steps = 0

    # ---- the step function ----------------------------------------------------------------------------------------
    @torch.no_grad()
    def feed(self, entries: Sequence[Tuple[Hashable, Sequence[int], Sequence[int]]]) -> torch.Tensor:
        """entries: (request id, its next tokens, indices among these tokens whose logits are wanted). Runs the tokens
        from the state earlier calls left and returns float32-or-model-typed logits [total wanted, vocab] in the order of
        the entries and of their wanted lists. Entries longer than the model's step size are cut into several passes."""
        model, cap = self.model, self.model.max_step_tokens
        limit = getattr(model, "max_seq_len", None)
        seen = set()
        for rid, toks, want in entries:
            if rid in seen:
                raise ValueError(f"request {rid!r} appears twice in one step")
            seen.add(rid)
            if any(not 0 <= w < len(toks) for w in want):
                raise ValueError(f"request {rid!r}: wanted index outside its {len(toks)} tokens")
            if limit is not None:
                held = self.table.pos[self.table.slot_of[rid]] if rid in self.table.slot_of else 0
                if held + len(toks) > limit:
                    raise RuntimeError(f"request {rid!r} would hold {held + len(toks)} tokens; the cache takes {limit}")
        base, offsets = 0, []
        for _, _, want in entries:
            offsets.append(base)
            base += len(want)
        n_want = base
        parts, order = [], []                           # logits per pass; the output row of every gathered row
        work = [(e, 0) for e in range(len(entries)) if len(entries[e][1])]
        while work:
            segs, rows, at, nxt, ids = [], [], 0, [], []
            for e, done in work:
                rid, toks, want = entries[e]
                n = min(len(toks) - done, cap - at)
                if n <= 0:
                    nxt.append((e, done))
                    continue
                ids.extend(toks[done:done + n])
                segs.append((rid, n))
                for k, w in enumerate(want):
                    if done <= w < done + n:
                        rows.append((offsets[e] + k, at + w - done))
                at += n
                if done + n < len(toks):
                    nxt.append((e, done + n))
            rows.sort()
            split = len(rows) > at                      # a token wanted more than once: gather through a tensor of its own
            meta = self.table.plan(segs, ids, None if split else [r for _, r in rows])
            hidden = model.forward_batch(meta.ids, meta)
            self.table.commit(meta)
            if rows:
                sel = torch.tensor([r for _, r in rows], dtype=torch.int32, device=model.device) if split else meta.rows
                parts.append(model.logits(hidden.index_select(0, sel)))
                order.extend(o for o, _ in rows)
            work = nxt
        if not parts:
            return torch.empty(0, model.vocab_size, dtype=torch.float32, device=model.device)
        out = parts[0] if len(parts) == 1 else torch.cat(parts, 0)
        if order != sorted(order):                      # wanted lists out of order across passes: put the rows in place
            inv = sorted(range(len(order)), key=order.__getitem__)
            out = out.index_select(0, torch.tensor(inv, dtype=torch.int64, device=out.device))
        assert out.shape[0] == n_want
        return out

    def release(self, rid: Hashable) -> None:
        """The request is finished: its slot returns to the pool."""
        if rid in self.table.slot_of:
            self.table.close(rid)

    # ---- generation -------------------------------------------------------------------------------------------------
    def add(self, rid: Hashable, prompt: Sequence[int], max_new_tokens: int, eos: Optional[int] = None) -> None:
        if not len(prompt):
            raise ValueError("empty prompt")
        if rid in self.finished or any(r.rid == rid for r in list(self.waiting) + self.running):
            raise ValueError(f"request id {rid!r} is already known")
        self.waiting.append(Request(rid, list(prompt), max_new_tokens, eos))

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def step(self) -> List[Tuple[Hashable, int]]:
        """One scheduling step: every running request that is decoding gets its last token, then prompts are advanced
        while token budget and slots remain. Returns the (request id, token) pairs sampled in this step."""
        budget = self.model.max_step_tokens
        entries, owners = [], []
        for r in self.running:
            if r.fed == len(r.prompt) and budget > 0:
                entries.append((r.rid, [r.output[-1]], [0]))
                owners.append(r)
                budget -= 1
        while self.waiting and self.table.pool.free > 0 and budget > 0:
            r = self.waiting.popleft()
            self.table.open(r.rid)
            self.running.append(r)
        for r in self.running:
            if r.fed < len(r.prompt) and budget > 0:
                n = min(len(r.prompt) - r.fed, self.prefill_portion, budget)
                last = r.fed + n == len(r.prompt)
                entries.append((r.rid, r.prompt[r.fed:r.fed + n], [n - 1] if last else []))
                r.fed += n
                budget -= n
                if last:
                    owners.append(r)
        if not entries:
            return []
        logits = self.feed(entries)
        self.steps += 1
        toks = ops.argmax_rows(logits).tolist() if logits.shape[0] else []
        sampled = []
        for r, t in zip(owners, toks):
            r.output.append(int(t))
            sampled.append((r.rid, int(t)))
            if len(r.output) >= r.max_new_tokens or (r.eos is not None and t == r.eos):
                r.done = True
        for r in [r for r in self.running if r.done]:
            self.running.remove(r)
            self.release(r.rid)
            self.finished[r.rid] = r
        return sampled

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, eos: Optional[int] = None) -> List[List[int]]:
        """Greedy continuation of every prompt; more prompts than slots queue up and run as slots come free."""
        ids = [("gen", self.steps, k) for k in range(len(prompts))]
        for rid, p in zip(ids, prompts):
            self.add(rid, p, max_new_tokens, eos)
        while self.has_work():
            self.step()
        return [self.finished.pop(rid).output for rid in ids]
