"""Serving-side host logic on top of `Engine`: KV pages handed out on demand and a continuous batcher.

The reference reserves every page of every sequence up front (engine/cache.py:154-159, engine/paging.py:131-153,
engine/runner.py:719-723: "continuous batching is where on-demand growth pays") and has no scheduler.  This module is
that next step, kept to what the CUDA path needs from the host:

* `PageAllocator`  - a free list of physical pages plus the device page table `[max_batch, max_pages]` int32 that the
  kernels read.  `ensure(slot, tokens)` adds pages only when a sequence crosses a page boundary; rows of idle slots
  point at one reserved "spare" page, so a decode step over all slots can never touch a page somebody owns.
* `ContinuousBatcher` - a fixed number of decode slots.  Requests wait in a queue, are admitted into free slots by a
  packed prefill of the newcomers only, decode one token per step together with everybody else (one CUDA-graph replay:
  table, positions, tokens and the active mask are device tensors the host updates between replays), and leave when
  they produce a stop id or reach their token budget; their pages go back to the pool at once.  If the pool runs dry
  while a sequence grows, the youngest request is evicted and re-queued with what it has generated so far
  (preemption by recomputation), so a step never fails for lack of pages as long as one sequence fits.

Nothing here runs on the GPU by itself; the engine it drives does.  The scheduling logic is plain Python and is tested
on the CPU against a stand-in engine.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import torch

PAGE_SIZE = 16


class PoolExhausted(RuntimeError):
    """No free page is left and nothing can be evicted."""


class PageAllocator:
    """Physical KV pages handed out on demand (host free list) and the device page table the kernels read.

    The last physical page is the spare page: never handed out, every table entry that no sequence owns points at it.
    Pages are taken from the END of the free list and returned to it (as engine/paging.py:88-97 does), so repeated
    runs of the same schedule use the same pages."""

    def __init__(self, num_pages: int, max_batch: int, max_pages_per_seq: int, device="cpu"):
        assert num_pages >= 2 and max_batch >= 1 and max_pages_per_seq >= 1
        self.num_pages, self.max_batch, self.max_pages = num_pages, max_batch, max_pages_per_seq
        self.spare = num_pages - 1
        self._free: list[int] = list(range(num_pages - 1))
        self.owned: list[list[int]] = [[] for _ in range(max_batch)]
        self.block_table = torch.full((max_batch, max_pages_per_seq), self.spare, dtype=torch.int32, device=device)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def pages_for(self, tokens: int) -> int:
        return (tokens + PAGE_SIZE - 1) // PAGE_SIZE

    def can_hold(self, slot: int, tokens: int) -> bool:
        need = self.pages_for(tokens)
        return need <= self.max_pages and need - len(self.owned[slot]) <= len(self._free)

    def ensure(self, slot: int, tokens: int) -> int:
        """Make room for `tokens` tokens in `slot`; returns how many pages were added.  Raises `PoolExhausted` when
        the free list is too short and AssertionError when the sequence would outgrow its table row."""
        need = self.pages_for(tokens)
        assert need <= self.max_pages, (
            f"{tokens} tokens need {need} pages, the page table holds {self.max_pages} per sequence")
        held = self.owned[slot]
        missing = need - len(held)
        if missing <= 0:
            return 0
        if missing > len(self._free):
            raise PoolExhausted(f"{missing} pages wanted for slot {slot}, {len(self._free)} free of {self.num_pages - 1}")
        new = self._free[-missing:]
        del self._free[-missing:]
        self.block_table[slot, len(held): need] = torch.tensor(new, dtype=torch.int32, device=self.block_table.device)
        held.extend(new)
        return missing

    def release(self, slot: int) -> None:
        """Give the slot's pages back and point its table row at the spare page again."""
        self._free.extend(self.owned[slot])
        self.owned[slot] = []
        self.block_table[slot].fill_(self.spare)

    def check(self) -> None:
        """Invariants: every page is free or owned by exactly one slot, the spare page by nobody."""
        seen = list(self._free)
        for pages in self.owned:
            seen += pages
        assert len(seen) == len(set(seen)) == self.num_pages - 1, "a page is owned twice or lost"
        assert self.spare not in seen


@dataclass
class Request:
    rid: int
    prompt: list[int]
    max_new_tokens: int
    generated: list[int] = field(default_factory=list)
    arrival: int = 0          # admission order, for "evict the youngest"
    evictions: int = 0

    @property
    def tokens_so_far(self) -> list[int]:
        return self.prompt + self.generated


class ContinuousBatcher:
    """Continuous batching over one engine with `engine.batch` decode slots.

    The engine must offer: `batch`, `max_context`, `pages` (a PageAllocator), `prefill_slots(slots, prompts) -> first
    tokens`, `step() -> tokens of all slots` (advances every ACTIVE slot by one token), `set_active(mask)`,
    `set_tokens(slot_tokens)`.  `b200attn.engine.Engine(on_demand_pages=True)` does."""

    def __init__(self, engine, stop_ids=(), check_invariants: bool = False):
        self.engine = engine
        self.stop_ids = set(stop_ids)
        self.check_invariants = check_invariants
        self.queue: deque[Request] = deque()
        self.slots: list[Request | None] = [None] * engine.batch
        self.context: list[int] = [0] * engine.batch     # tokens cached per slot (host shadow of the device `pos`)
        self.finished: dict[int, list[int]] = {}
        self.steps = 0
        self._next_rid = 0
        self._admissions = 0
        self.stats = {"prefills": 0, "prefill_tokens": 0, "decode_steps": 0, "evictions": 0, "peak_pages": 0}

    # ------------------------------------------------------------------------------------------------ public
    def submit(self, prompt: list[int], max_new_tokens: int) -> int:
        assert len(prompt) >= 1 and max_new_tokens >= 1
        assert len(prompt) + max_new_tokens <= self.engine.max_context, "request longer than a page-table row"
        rid = self._next_rid
        self._next_rid += 1
        self.queue.append(Request(rid, list(prompt), max_new_tokens))
        return rid

    @property
    def active(self) -> int:
        return sum(r is not None for r in self.slots)

    def done(self) -> bool:
        return not self.queue and self.active == 0

    def step(self) -> list[int]:
        """Admit what fits, grow pages, decode one token for every active slot.  Returns the ids that finished."""
        pages = self.engine.pages
        finished_now: list[int] = []
        # ---- admission: FIFO into free slots while the prompt's pages (plus the first generated token's) are there
        newcomers: list[tuple[int, Request]] = []
        for slot in range(len(self.slots)):
            if self.slots[slot] is not None or not self.queue:
                continue
            req = self.queue[0]
            if not pages.can_hold(slot, len(req.tokens_so_far) + 1):
                break                                           # keep arrival order: nobody overtakes the head
            self.queue.popleft()
            pages.ensure(slot, len(req.tokens_so_far) + 1)
            req.arrival = self._admissions
            self._admissions += 1
            self.slots[slot] = req
            newcomers.append((slot, req))
        if newcomers:
            firsts = self.engine.prefill_slots([s for s, _ in newcomers], [r.tokens_so_far for _, r in newcomers])
            self.stats["prefills"] += 1
            for (slot, req), tok in zip(newcomers, firsts):
                self.stats["prefill_tokens"] += len(req.tokens_so_far)
                self.context[slot] = len(req.tokens_so_far)
                req.generated.append(int(tok))
                if self._is_finished(req):
                    finished_now.append(self._retire(slot))
        if self.active == 0:
            return finished_now
        # ---- growth: the step appends one token per active slot at index context[slot]
        for slot, req in enumerate(self.slots):
            if req is None:
                continue
            while True:
                try:
                    pages.ensure(slot, self.context[slot] + 1)
                    break
                except PoolExhausted:
                    if not self._evict_youngest(exclude=slot):
                        raise
        self.stats["peak_pages"] = max(self.stats["peak_pages"], pages.num_pages - 1 - pages.num_free)
        if self.check_invariants:
            pages.check()
        # ---- one decode step over all slots (idle ones are masked out and only ever touch the spare page)
        self.engine.set_active([r is not None for r in self.slots])
        tokens = self.engine.step()
        self.steps += 1
        self.stats["decode_steps"] += 1
        for slot, req in enumerate(self.slots):
            if req is None:
                continue
            self.context[slot] += 1
            req.generated.append(int(tokens[slot]))
            if self._is_finished(req):
                finished_now.append(self._retire(slot))
        return finished_now

    def run(self, max_steps: int = 1 << 30) -> dict[int, list[int]]:
        """Step until every submitted request has finished; returns {request id: generated tokens}."""
        while not self.done() and max_steps > 0:
            before = (len(self.queue), self.active, self.steps)
            self.step()
            max_steps -= 1
            if (len(self.queue), self.active, self.steps) == before and self.active == 0:
                raise PoolExhausted("the head of the queue does not fit into an empty pool")
        return self.finished

    # ----------------------------------------------------------------------------------------------- internals
    def _is_finished(self, req: Request) -> bool:
        return len(req.generated) >= req.max_new_tokens or (req.generated and req.generated[-1] in self.stop_ids)

    def _retire(self, slot: int) -> int:
        req = self.slots[slot]
        self.finished[req.rid] = list(req.generated)
        self.slots[slot] = None
        self.context[slot] = 0
        self.engine.pages.release(slot)
        return req.rid

    def _evict_youngest(self, exclude: int) -> bool:
        """Free the pages of the most recently admitted request other than `exclude` and put it back at the head of the
        queue; it is later prefilled again over its prompt plus what it has generated (recomputation)."""
        victims = [(req.arrival, slot) for slot, req in enumerate(self.slots) if req is not None and slot != exclude]
        if not victims:
            return False
        _, slot = max(victims)
        req = self.slots[slot]
        req.evictions += 1
        self.stats["evictions"] += 1
        self.slots[slot] = None
        self.context[slot] = 0
        self.engine.pages.release(slot)
        self.queue.appendleft(req)
        return True
