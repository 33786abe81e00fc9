"""Continuous-batching scheduler for models that expose the ragged step interface (admit / release / step / sample, as
sglang.srt.models.karusun.KarusunForCausalLM does): every step runs the single next tokens of the sequences that are decoding together
with portions of the prompts that are still being read, under one token budget.  Slots and cache pages are reserved at admission and
handed back when a request finishes, so later requests run in pages and slots that earlier ones used.

`execute` is the one place where a list of (slot, tokens) entries becomes engine steps; the trace replay of the command line calls it with
entries taken from its input instead of from the policy here."""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

import numpy as np


@dataclass
class SamplingParams:
    temperature: float = 0.0      # <= 0: greedy
    top_k: int = 0                # 0: no limit
    top_p: float = 1.0
    seed: int = 0

    def key(self):
        return (self.temperature, self.top_k, self.top_p)


@dataclass
class Request:
    rid: str
    prompt: List[int]
    max_new_tokens: int = 16
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Tuple[int, ...] = ()
    # filled by the scheduler
    slot: int = -1
    fed: int = 0                          # prompt tokens already run
    output: List[int] = field(default_factory=list)
    reserved_pages: int = 0
    finished: bool = False
    _rng: Optional[np.random.Generator] = None

    def rng(self) -> np.random.Generator:
        if self._rng is None:
            self._rng = np.random.default_rng(self.sampling.seed)
        return self._rng


def execute(model, entries: Sequence[Tuple[int, Sequence[int]]], want: Sequence[Tuple[int, int]], fetch: bool = True):
    """Run entries [(slot, tokens)] as ONE batch, or as consecutive batches when they exceed the model's step size (an entry is then cut
    where the step is full and goes on in the next).  want: (entry index, token index inside the entry).  Returns float32
    [len(want), vocab] in the order of `want` when fetch is on; with fetch off the rows of the LAST batch stay on the device for
    model.sample and the number of rows is returned."""
    limit = int(model.max_step_tokens)
    total = sum(len(t) for _, t in entries)
    want_at = {}
    for k, (ei, ti) in enumerate(want):
        want_at.setdefault(ei, []).append((ti, k))
    rows = np.empty((len(want), model.vocab), dtype=np.float32) if fetch and want else None
    cursor = [0] * len(entries)
    done, last_rows = 0, 0
    while done < total:
        slots, counts, toks, w_local, w_global, room = [], [], [], [], [], limit
        for ei, (slot, t) in enumerate(entries):
            if room == 0:
                break
            lo = cursor[ei]
            if lo >= len(t):
                continue
            hi = min(len(t), lo + room)
            base = len(toks)
            slots.append(slot)
            counts.append(hi - lo)
            toks.extend(int(x) for x in t[lo:hi])
            for ti, k in want_at.get(ei, ()):
                if lo <= ti < hi:
                    w_local.append(base + ti - lo)
                    w_global.append(k)
            cursor[ei] = hi
            room -= hi - lo
        out = model.step(slots, counts, toks, w_local, fetch)
        if rows is not None and w_global:
            rows[w_global] = out
        done += len(toks)
        last_rows = len(w_local)
    return rows if fetch else last_rows


class Scheduler:
    def __init__(self, model, max_step_tokens: Optional[int] = None, max_prefill_chunk: Optional[int] = None):
        self.model = model
        self.budget = min(int(max_step_tokens or model.max_step_tokens), int(model.max_step_tokens))
        self.chunk = int(max_prefill_chunk or self.budget)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.reserved = 0
        self.steps = 0

    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("empty prompt")
        self.waiting.append(req)

    def _admit(self) -> None:
        while self.waiting:
            r = self.waiting[0]
            need = self.model.pages_for(len(r.prompt) + r.max_new_tokens)
            if self.model.free_slots() == 0 or self.model.free_pages() - self.reserved_unused() < need:
                break
            slot = self.model.admit()
            if slot < 0:
                break
            r.slot, r.reserved_pages = slot, need
            self.reserved += need
            self.running.append(self.waiting.popleft())

    def reserved_unused(self) -> int:
        """pages promised to running requests that they do not hold yet"""
        held = sum(self.model.pages_for(r.fed + max(0, len(r.output) - 1)) for r in self.running)
        return self.reserved - held

    def step(self) -> List[Request]:
        """One engine batch.  Returns the requests that finished in it."""
        self._admit()
        entries, want, owners, room = [], [], [], self.budget
        for r in self.running:                                   # decoding sequences first: one token each
            if r.fed == len(r.prompt) and room > 0:
                entries.append((r.slot, [r.output[-1]]))
                want.append((len(entries) - 1, 0))
                owners.append(r)
                room -= 1
        for r in self.running:                                   # then portions of prompts
            if r.fed < len(r.prompt) and room > 0:
                n = min(room, self.chunk, len(r.prompt) - r.fed)
                entries.append((r.slot, r.prompt[r.fed:r.fed + n]))
                if r.fed + n == len(r.prompt):
                    want.append((len(entries) - 1, n - 1))
                    owners.append(r)
                r.fed += n
                room -= n
        if not entries:
            return []
        # rows of equal sampling parameters are drawn together
        order = sorted(range(len(want)), key=lambda k: owners[k].sampling.key())
        want = [want[k] for k in order]
        owners = [owners[k] for k in order]
        logits = execute(self.model, entries, want, fetch=True)       # also when nothing is wanted: the portions must run
        self.steps += 1
        finished = []
        if want:
            nxt = self._draw(logits, owners)
            for r, t in zip(owners, nxt):
                r.output.append(int(t))
                if len(r.output) >= r.max_new_tokens or int(t) in r.stop_ids:
                    r.finished = True
        for r in [r for r in self.running if r.finished]:
            self.model.release(r.slot)
            self.reserved -= r.reserved_pages
            self.running.remove(r)
            finished.append(r)
        return finished

    def _draw(self, logits: np.ndarray, owners: List[Request]) -> np.ndarray:
        """The model's sampling kernel works on the rows the last batch left on the device, in order; groups of equal parameters are
        contiguous (sorted above)."""
        n = len(owners)
        out = np.empty(n, dtype=np.int32)
        if all(r.sampling.temperature <= 0 for r in owners):
            return self.model.sample(n, 0.0)
        k = 0
        while k < n:
            j = k
            while j < n and owners[j].sampling.key() == owners[k].sampling.key():
                j += 1
            sp = owners[k].sampling
            u = np.array([r.rng().random() for r in owners[:j]], dtype=np.float32)
            out[k:j] = self.model.sample(j, sp.temperature, sp.top_k, sp.top_p, u)[k:j]
            k = j
        return out

    def run(self) -> List[Request]:
        done: List[Request] = []
        while self.waiting or self.running:
            before = len(done)
            done.extend(self.step())
            if not self.running and self.waiting and len(done) == before:
                raise RuntimeError("a waiting request does not fit the cache pool even when it is empty")
        return done
