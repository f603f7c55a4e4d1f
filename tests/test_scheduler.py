"""The scheduler's decisions, with a fake step function over a real cache manager:
portions under a token budget, admission, mixing, finishing and freeing, and what
happens when pages run out."""
import hashlib

import pytest
import torch

from inferflux_b200.cache import CacheManager
from inferflux_b200.engine.scheduler import Request, Scheduler, SchedulerConfig
from inferflux_b200.parts import KVCacheSpec
from inferflux_b200.sampling import SamplingParams

VOCAB = 1000


def next_token(prefix):
    """The fake model: the next token is a hash of everything before it."""
    h = hashlib.sha256(",".join(map(str, prefix)).encode()).digest()
    return int.from_bytes(h[:4], "little") % VOCAB


class FakeEngine:
    """Drives Scheduler like Engine does, but the 'model' only keeps each request's
    tokens as the steps deliver them, and checks they arrive in order."""

    def __init__(self, num_pages=64, page=4, max_seqs=8, max_len=4096, **cfg):
        self.cache = CacheManager([(KVCacheSpec(1, 8, None), None)], page_size=page, num_pages=num_pages,
                                  max_seqs=max_seqs, max_seq_len=max_len, dtype=torch.float32, device="cpu")
        self.sched = Scheduler(SchedulerConfig(**cfg), self.cache, max_len)
        self.seen = {}
        self.log = []
        self.n = 0

    def add(self, prompt, max_tokens=8, eos=(), rid=None):
        rid = rid if rid is not None else f"r{self.n}"
        self.n += 1
        self.sched.add(Request(rid, list(prompt), SamplingParams(temperature=0.0), max_tokens=max_tokens,
                               eos_token_ids=eos))
        return rid

    def step(self):
        plan = self.sched.schedule()
        for r in plan.preempted:
            self.seen.pop(r.request_id, None)
        sampled = []
        for e, se in zip(plan.entries, plan.step_entries()):
            rid = e.request.request_id
            if rid not in self.cache:
                self.cache.add_request(rid)
            have = self.seen.setdefault(rid, [])
            assert e.start == len(have) == self.cache.length(rid), "a portion does not start where the last ended"
            self.cache.reserve(rid, e.start + e.count)          # must succeed: the scheduler promised the pages
            self.cache.commit(rid, e.start + e.count)
            have.extend(se.tokens)
            assert (se.want == [e.count - 1]) == e.wants_logits
            if e.wants_logits:
                sampled.append(next_token(have))
        self.log.append([(e.request.request_id, e.start, e.count, e.wants_logits) for e in plan.entries])
        done = self.sched.update(plan, sampled)
        self.cache.check()
        return plan, done

    def run(self, limit=10000):
        out = {}
        for _ in range(limit):
            if not self.sched.has_unfinished():
                break
            plan, done = self.step()
            for r in list(done) + list(plan.failed):
                out[r.request_id] = r
        assert not self.sched.has_unfinished(), "the scheduler did not finish"
        return out


def expected(prompt, n, eos=()):
    seq, out = list(prompt), []
    for _ in range(n):
        t = next_token(seq)
        seq.append(t); out.append(t)
        if t in eos:
            break
    return out


def test_prompt_is_cut_into_portions_and_only_the_last_asks_for_logits():
    e = FakeEngine(num_pages=400, chunked_prefill_tokens=512, max_batch_tokens=16384)
    e.add(range(1200), max_tokens=2)
    e.run()
    first = [entry for step in e.log for entry in step][:4]
    assert [(s, c, w) for _r, s, c, w in first] == [(0, 512, False), (512, 512, False), (1024, 176, True),
                                                    (1200, 1, True)]


def test_token_budget_and_mixing_of_portions_with_decoding():
    e = FakeEngine(num_pages=400, chunked_prefill_tokens=64, max_batch_tokens=100, max_batch_size=8)
    a = e.add(range(10), max_tokens=30)
    e.step()                                                     # a is decoding from now on
    b = e.add(range(100, 400), max_tokens=4)
    c = e.add(range(500, 560), max_tokens=4)
    plan, _ = e.step()
    got = {(x.request.request_id, x.count) for x in plan.entries}
    assert (a, 1) in got and (b, 64) in got and (c, 35) in got    # decode first, then portions up to the budget
    assert plan.num_tokens == 100
    for step in e.log:
        assert sum(c for _r, _s, c, _w in step) <= 100
    res = e.run()
    assert res[a].output == expected(range(10), 30) and res[b].output == expected(range(100, 400), 4)
    assert res[c].output == expected(range(500, 560), 4)


def test_prefill_share_of_the_budget():
    e = FakeEngine(num_pages=400, chunked_prefill_tokens=512, max_batch_tokens=200, mixed_prefill_budget_ratio=0.5)
    e.add(range(300), max_tokens=1)
    plan, _ = e.step()
    assert plan.num_tokens == 100


def test_admission_waits_for_a_free_place():
    e = FakeEngine(num_pages=400, max_batch_size=2, max_seqs=8)
    ids = [e.add(range(i * 10, i * 10 + 5), max_tokens=3) for i in range(4)]
    plan, _ = e.step()
    assert [x.request.request_id for x in plan.entries] == ids[:2]
    res = e.run()
    assert all(res[i].finish_reason == "length" and len(res[i].output) == 3 for i in ids)
    assert max(len(step) for step in e.log) == 2


def test_finishing_frees_pages_and_slots_and_eos_stops():
    prompt = list(range(7))
    stop = expected(prompt, 3)[-1]
    e = FakeEngine(num_pages=16)
    a = e.add(prompt, max_tokens=10, eos=(stop,))
    b = e.add(range(50, 60), max_tokens=0)                        # max_tokens <= 0 counts as 1
    res = e.run()
    assert res[a].finish_reason == "stop" and res[a].output == expected(prompt, 10, eos=(stop,))
    assert res[b].finish_reason == "length" and len(res[b].output) == 1
    assert e.cache.free_pages() == [16] and e.cache.num_free_slots == 8 and not e.cache.live_requests()


def test_out_of_pages_preempts_the_newest_and_recomputes():
    prompts = [list(range(i * 100, i * 100 + 20 + 3 * i)) for i in range(4)]
    small = FakeEngine(num_pages=24, page=4, chunked_prefill_tokens=16)       # 96 tokens of cache for ~190 needed
    big = FakeEngine(num_pages=400, page=4, chunked_prefill_tokens=16)
    for eng in (small, big):
        for p in prompts:
            eng.add(p, max_tokens=24)
    rs, rb = small.run(), big.run()
    assert small.sched.num_preemptions > 0 and big.sched.num_preemptions == 0
    for rid in rb:
        assert rs[rid].output == rb[rid].output == expected(prompts[int(rid[1:])], 24)
    victims = [r for r in rs.values() if r.preemptions]
    assert victims and rs["r0"].preemptions == 0                 # the oldest request is never the victim
    assert small.cache.free_pages() == [24]


def test_a_request_that_can_never_fit_fails_and_the_rest_goes_on():
    e = FakeEngine(num_pages=8, page=4, max_len=64)
    a = e.add(range(100), max_tokens=4)                          # longer than the longest sequence
    b = e.add(range(20), max_tokens=20)                          # 40 tokens need 10 pages, the pool has 8
    c = e.add(range(10), max_tokens=4)
    res = e.run()
    assert res[a].finish_reason.startswith("context_overflow") and not res[a].output
    assert res[b].finish_reason.startswith("context_overflow")
    assert res[c].output == expected(range(10), 4)


def test_context_limit_ends_generation():
    e = FakeEngine(num_pages=64, page=4, max_len=16)
    a = e.add(range(10), max_tokens=100)
    res = e.run()
    assert res[a].finish_reason == "length" and len(res[a].output) == 6      # 10 + 6 = the longest sequence


@pytest.mark.parametrize("cfg", [dict(chunked_prefill_tokens=7, max_batch_tokens=20),
                                 dict(chunked_prefill_tokens=512, max_batch_tokens=16384),
                                 dict(chunked_prefill_tokens=2, max_batch_tokens=9, max_batch_size=3)])
@pytest.mark.parametrize("order", [0, 1])
def test_results_do_not_depend_on_budget_portion_size_or_arrival_order(cfg, order):
    prompts = {f"p{i}": list(range(i * 37, i * 37 + n)) for i, n in enumerate([1, 4, 50, 97, 130])}
    e = FakeEngine(num_pages=200, **cfg)
    names = list(prompts) if order == 0 else list(reversed(prompts))
    for n in names:
        e.add(prompts[n], max_tokens=12, rid=n)
    res = e.run()
    for n, p in prompts.items():
        assert res[n].output == expected(p, 12)


def test_validation():
    with pytest.raises(ValueError):
        SchedulerConfig(max_batch_tokens=0).validate()
    e = FakeEngine()
    with pytest.raises(ValueError):
        e.add([], max_tokens=3)
    with pytest.raises(ValueError):
        e.sched.add(Request("x", [1], SamplingParams(top_p=0.0)))


def test_abort_frees_pages_now_or_when_the_step_in_flight_is_read():
    """A waiting request leaves the queue; a running one gives its pages back at once and the pool
    serves the others with them; one that is owed a token by a step in flight is freed when that
    step's tokens are read, and its token is dropped."""
    eng = FakeEngine(num_pages=12, page=4, max_seqs=3, max_batch_size=3, chunked_prefill_tokens=16)
    a = eng.add(list(range(1, 17)), max_tokens=20)          # 16 tokens = 4 pages, grows to 9
    b = eng.add(list(range(20, 36)), max_tokens=20)
    c = eng.add(list(range(40, 56)), max_tokens=20)
    w = eng.add(list(range(60, 70)), max_tokens=4)          # waits: three slots
    eng.step()
    assert {r.request_id for r in eng.sched.running} == {a, b, c}
    # waiting -> gone
    r = eng.sched.abort(w)
    assert r is not None and r.finish_reason == "abort" and not eng.sched.waiting
    # running, nothing pending -> freed at once
    free_before = eng.cache.free_pages()[0]
    r = eng.sched.abort(b)
    assert r is not None and r.finish_reason == "abort" and b not in eng.cache
    assert eng.cache.free_pages()[0] == free_before + 4     # the 16 prompt tokens it had stored
    eng.cache.check()
    # pending (a step in flight): advance without resolve, abort, then resolve
    plan = eng.sched.schedule()
    for e in plan.entries:
        eng.cache.reserve(e.request.request_id, e.start + e.count)
        eng.cache.commit(e.request.request_id, e.start + e.count)
    eng.sched.advance(plan)
    assert eng.sched.abort(a) is None                        # its token is still coming
    assert a in eng.cache and eng.sched.has_unfinished()
    nxt = eng.sched.schedule(inflight=True)                  # the next step goes on without it
    assert a not in {e.request.request_id for e in nxt.entries}
    done = eng.sched.resolve(plan, [7] * sum(e.wants_logits for e in plan.entries))
    assert [r.request_id for r in done] == [a] and done[0].finish_reason == "abort" and a not in eng.cache
    assert -1 not in done[0].output
    eng.cache.check()
    assert eng.sched.abort("nobody") is None
    # the rest finishes with the pages that came back
    for e in nxt.entries:
        eng.cache.reserve(e.request.request_id, e.start + e.count)
        eng.cache.commit(e.request.request_id, e.start + e.count)
    eng.sched.update(nxt, [3] * sum(e.wants_logits for e in nxt.entries))
    eng.seen.clear()
    eng.cache.check()
