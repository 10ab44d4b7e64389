"""Host logic of on-demand paging and continuous batching (b200attn/serving.py) against a stand-in engine on the CPU:
page accounting, admission order, growth across page boundaries, eviction with recomputation, stop ids."""
import pytest
import torch

from b200attn.serving import ContinuousBatcher, PageAllocator, PoolExhausted


class StandInEngine:
    """Deterministic toy 'model': the next token of a sequence is (sum of its tokens * 31 + its length) % 997, so a
    request's output depends on its own history only - what continuous batching must preserve."""

    def __init__(self, batch, max_context, num_pages):
        self.batch, self.max_context = batch, max_context
        self.pages = PageAllocator(num_pages, batch, (max_context + 15) // 16, device="cpu")
        self.history = [None] * batch
        self.mask = [False] * batch

    @staticmethod
    def next_token(history):
        return (sum(history) * 31 + len(history)) % 997

    def prefill_slots(self, slots, prompts):
        out = []
        for slot, prompt in zip(slots, prompts):
            assert len(self.pages.owned[slot]) * 16 >= len(prompt) + 1, "prefill without pages"
            self.history[slot] = list(prompt)
            out.append(self.next_token(self.history[slot]))
            self.history[slot].append(out[-1])
        return torch.tensor(out)

    def set_active(self, mask):
        self.mask = list(mask)

    def step(self):
        toks = []
        for slot in range(self.batch):
            if self.mask[slot]:
                assert len(self.pages.owned[slot]) * 16 >= len(self.history[slot]), "decode past the owned pages"
                t = self.next_token(self.history[slot])
                self.history[slot].append(t)
                toks.append(t)
            else:
                toks.append(0)
        return torch.tensor(toks)


def solo(prompt, n, stop=()):
    hist, out = list(prompt), []
    for _ in range(n):
        t = StandInEngine.next_token(hist)
        hist.append(t)
        out.append(t)
        if t in stop:
            break
    return out


def test_page_allocator_grows_on_demand_and_returns_everything():
    pa = PageAllocator(num_pages=8, max_batch=2, max_pages_per_seq=4, device="cpu")
    assert pa.num_free == 7 and (pa.block_table == 7).all()           # page 7 is the spare page
    assert pa.ensure(0, 16) == 1 and pa.ensure(0, 16) == 0 and pa.ensure(0, 17) == 1
    assert pa.ensure(1, 40) == 3
    pa.check()
    assert pa.block_table[0, :2].tolist() == pa.owned[0] and pa.block_table[0, 2:].tolist() == [7, 7]
    assert set(pa.owned[0]).isdisjoint(pa.owned[1]) and pa.num_free == 2
    with pytest.raises(AssertionError):
        pa.ensure(1, 65)                                               # more than a table row holds
    assert pa.ensure(0, 64) == 2 and pa.num_free == 0
    assert not pa.can_hold(1, 64)
    with pytest.raises(PoolExhausted):
        pa.ensure(1, 64)
    assert len(pa.owned[1]) == 3                                       # a refused request changes nothing
    pa.release(0)
    pa.check()
    assert pa.num_free == 4 and (pa.block_table[0] == 7).all()
    pa.release(1)
    assert pa.num_free == 7
    first = sorted(pa.owned[0]) if pa.ensure(0, 17) else None
    pa.release(0)
    pa.ensure(0, 17)
    assert sorted(pa.owned[0]) == first                                # the same schedule takes the same pages again


def test_continuous_batching_preserves_every_request():
    eng = StandInEngine(batch=3, max_context=96, num_pages=3 * 6 + 1)
    cb = ContinuousBatcher(eng, check_invariants=True)
    gen = torch.Generator().manual_seed(0)
    reqs = {}
    for i in range(8):
        prompt = torch.randint(1, 900, (int(torch.randint(1, 40, (1,), generator=gen)),), generator=gen).tolist()
        n = int(torch.randint(1, 30, (1,), generator=gen))
        reqs[cb.submit(prompt, n)] = (prompt, n)
        if i % 3 == 2:
            cb.step()                                                  # arrivals interleave with decoding
    out = cb.run()
    assert set(out) == set(reqs)
    for rid, (prompt, n) in reqs.items():
        assert out[rid] == solo(prompt, n), rid
    assert cb.active == 0 and eng.pages.num_free == eng.pages.num_pages - 1
    eng.pages.check()
    assert cb.stats["evictions"] == 0 and cb.stats["prefills"] >= 3


def test_stop_ids_and_single_token_requests():
    eng = StandInEngine(batch=2, max_context=64, num_pages=9)
    prompt = [5, 6, 7]
    full = solo(prompt, 12)
    stop = full[4]
    cb = ContinuousBatcher(eng, stop_ids=(stop,))
    a = cb.submit(prompt, 12)
    b = cb.submit([9], 1)
    out = cb.run()
    assert out[a] == full[:full.index(stop) + 1] and out[b] == solo([9], 1)
    assert eng.pages.num_free == 8


def test_pool_pressure_evicts_the_youngest_and_recomputes():
    """Two long-running requests in a pool that cannot hold both to the end: the younger one is evicted, re-queued with
    its tokens so far, prefilled again later - and still produces exactly its solo output."""
    eng = StandInEngine(batch=2, max_context=80, num_pages=6)         # 5 usable pages = 80 tokens in all
    cb = ContinuousBatcher(eng, check_invariants=True)
    a = cb.submit(list(range(1, 20)), 40)       # grows to 59 tokens: 4 pages
    b = cb.submit(list(range(30, 45)), 30)      # grows to 45 tokens: 3 pages
    out = cb.run()
    assert out[a] == solo(list(range(1, 20)), 40) and out[b] == solo(list(range(30, 45)), 30)
    assert cb.stats["evictions"] >= 1
    assert eng.pages.num_free == 5


def test_request_that_can_never_fit_is_reported():
    eng = StandInEngine(batch=1, max_context=64, num_pages=3)          # 2 usable pages = 32 tokens
    cb = ContinuousBatcher(eng)
    cb.submit(list(range(40)), 2)
    with pytest.raises(PoolExhausted):
        cb.run()
