"""The scheduler's decisions, on the CPU: the step function is replaced by the cache manager's own
reserve/commit, the sampler by a rule on token ids."""
import pytest

from liyab_b200 import ErrorCode, SamplingParams
from liyab_b200.cache import CacheManager, KvNeed
from liyab_b200.engine import Request, Scheduler


def make(num_pages=16, page_size=4, max_batched_tokens=16, max_requests=4, max_positions=64, eos=None):
    cache = CacheManager({0: KvNeed(1, 16, 0)}, {}, page_size, num_pages, max_requests)
    return cache, Scheduler(cache, max_positions, max_batched_tokens, max_requests, eos_token_id=eos)


def run_step(cache, sched, next_token=lambda r: 1):
    """One plan/step/update round with the cache bookkeeping a real step does; returns (plan, finished)."""
    plan, finished = sched.plan()
    for e in plan.entries:
        cache.reserve(e.request.id, e.count)
    for e in plan.entries:
        cache.commit(e.request.id, e.count)
    sampled = [next_token(e.request) for e in plan.entries if e.sample]
    finished += sched.update(plan, sampled)
    cache.check()
    return plan, finished


def req(i, n_prompt, max_tokens=4, **kw):
    return Request(id=f"r{i}", prompt=list(range(2, 2 + n_prompt)), params=SamplingParams(temperature=0.0, max_tokens=max_tokens, **kw))


def test_prompt_is_cut_under_the_budget_and_decodes_go_first():
    cache, sched = make(max_batched_tokens=8, num_pages=64)
    a, b = req(0, 19), req(1, 3)
    sched.add(a); sched.add(b)
    plan, _ = run_step(cache, sched)
    assert [(e.request.id, e.count, e.sample) for e in plan.entries] == [("r0", 8, False)]    # budget spent on a
    plan, _ = run_step(cache, sched)
    assert [(e.request.id, e.count, e.sample) for e in plan.entries] == [("r0", 8, False)]
    plan, _ = run_step(cache, sched)       # a's last 3, then b is admitted and fits whole
    assert [(e.request.id, e.count, e.sample) for e in plan.entries] == [("r0", 3, True), ("r1", 3, True)]
    assert len(a.generated) == 1 and len(b.generated) == 1
    c = req(2, 20)
    sched.add(c)
    plan, _ = run_step(cache, sched)       # decodes first (1 token each), the new prompt gets the rest
    assert [(e.request.id, e.count) for e in plan.entries] == [("r0", 1), ("r1", 1), ("r2", 6)]
    assert [e.tokens for e in plan.entries][0] == [a.tokens[-2]]
    assert sched.stats["decode_tokens"] == 2


def test_portions_down_to_one_token():
    cache, sched = make(max_batched_tokens=5, num_pages=64)
    a, b = req(0, 4, max_tokens=8), req(1, 7)
    sched.add(a)
    run_step(cache, sched)
    sched.add(b)
    counts = []
    for _ in range(3):
        plan, _ = run_step(cache, sched)
        counts.append([(e.request.id, e.count) for e in plan.entries])
    assert counts == [[("r0", 1), ("r1", 4)], [("r0", 1), ("r1", 3)], [("r0", 1), ("r1", 1)]]


def test_finish_reasons_free_everything():
    cache, sched = make(eos=9, num_pages=64)
    a = req(0, 3, max_tokens=3)
    b = req(1, 3, max_tokens=50)
    c = req(2, 3, max_tokens=50, ignore_eos=True)
    stopped = []
    d = Request(id="r3", prompt=[2, 3], params=SamplingParams(temperature=0.0, max_tokens=50),
                callback=lambda t: stopped.append(t) or len(stopped) < 2)
    for r in (a, b, c, d):
        sched.add(r)
    done = {}
    step = 0
    while sched.has_work() and step < 20:
        _, fin = run_step(cache, sched, next_token=lambda r: 9 if (r.id in ("r1", "r2") and len(r.generated) == 1) else 5)
        for r in fin:
            done[r.id] = (r.finish_reason, len(r.generated))
        step += 1
        if step == 6:
            sched.cancel("r2")
    assert done == {"r0": ("length", 3), "r1": ("eos", 2), "r3": ("stopped", 2), "r2": ("cancelled", 6)}
    assert all(v == 0 for v in cache.pages_in_use().values()) and not cache.lengths


def test_context_limit_ends_a_request():
    cache, sched = make(max_positions=8, num_pages=64)
    a = req(0, 6, max_tokens=100)
    sched.add(a)
    while sched.has_work():
        run_step(cache, sched)
    # 6 prompt tokens + 2 generated fill the 8 positions; the third generated token has no position to run at
    assert a.finish_reason == "context" and len(a.generated) == 3 and a.n_computed == 8


def test_admission_waits_for_pages_and_takes_first_come_first():
    cache, sched = make(num_pages=6, page_size=4, max_batched_tokens=64)     # 24 positions in all
    a, b, c = req(0, 10, max_tokens=3), req(1, 10, max_tokens=3), req(2, 2, max_tokens=3)
    for r in (a, b, c):
        sched.add(r)
    plan, _ = run_step(cache, sched)
    # a (11 -> 3 pages) and b (3 pages) fit; c would fit too but waits its turn only if pages are short: 6 pages are gone
    assert [e.request.id for e in plan.entries] == ["r0", "r1"] and c.state == "waiting"
    order = []
    while sched.has_work():
        plan, fin = run_step(cache, sched)
        order += [r.id for r in fin]
    assert order == ["r0", "r1", "r2"] and c.finish_reason == "length"


def test_preemption_when_pages_run_out_then_recompute():
    cache, sched = make(num_pages=4, page_size=4, max_batched_tokens=64)       # 16 positions
    a, b = req(0, 6, max_tokens=9), req(1, 5, max_tokens=9)                    # each admitted with 2 pages
    sched.add(a); sched.add(b)
    log = []
    preempted = 0
    while sched.has_work() and len(log) < 60:
        plan, fin = run_step(cache, sched, next_token=lambda r: 100 + len(r.generated))
        preempted += len(plan.preempted)
        log.append([(e.request.id, e.start, e.count) for e in plan.entries])
    assert preempted >= 1 and b.preemptions >= 1 and a.preemptions == 0      # the most recently admitted one yields
    assert sched.stats["preemptions"] == preempted
    assert a.finish_reason == "length" and b.finish_reason == "length"
    assert a.generated == [100 + i for i in range(9)] and b.generated == [100 + i for i in range(9)]
    # after preemption b was recomputed from its prompt and the tokens it had generated
    starts = [s for step in log for (rid, s, n) in step if rid == "r1" and s == 0]
    assert len(starts) >= 2
    assert all(v == 0 for v in cache.pages_in_use().values())


def test_a_request_that_can_never_fit_ends_with_context_full():
    cache, sched = make(num_pages=2, page_size=4, max_batched_tokens=64)
    big = req(0, 9)
    sched.add(big)
    _, fin = run_step(cache, sched)
    assert fin == [big] and big.finish_reason == "error" and big.error.code == ErrorCode.CONTEXT_FULL
    grow = req(1, 6, max_tokens=10)          # fits at admission (7 -> 2 pages), outgrows the cache while decoding
    sched.add(grow)
    while sched.has_work():
        run_step(cache, sched)
    assert grow.finish_reason == "error" and grow.error.code == ErrorCode.CONTEXT_FULL and len(grow.generated) >= 2
    assert all(v == 0 for v in cache.pages_in_use().values())


def test_bad_requests_are_refused():
    cache, sched = make(max_positions=8)
    with pytest.raises(Exception):
        sched.add(Request(id="e", prompt=[], params=SamplingParams()))
    with pytest.raises(Exception) as e:
        sched.add(req(0, 9))
    assert e.value.code == ErrorCode.CONTEXT_FULL
    with pytest.raises(Exception):
        sched.add(Request(id="m", prompt=[1], params=SamplingParams(max_tokens=0)))


def test_draws_do_not_depend_on_batching():
    """A request's n-th draw is uniform(seed, its stream, n): streams are handed out in order of arrival and a seed of
    0 is replaced by a random one, so nothing about a batch enters a draw."""
    from liyab_b200.sampling import uniform_draw
    cache, sched = make()
    a, b, c = (Request(id=n, prompt=[1, 2], params=SamplingParams(seed=s)) for n, s in (("a", 7), ("b", 7), ("c", 0)))
    for r in (a, b, c):
        sched.add(r)
    assert (a.seed, a.stream) == (7, 0) and (b.seed, b.stream) == (7, 1) and c.seed != 0 and c.stream == 2
    draws = [uniform_draw(7, 0, 0), uniform_draw(7, 0, 1), uniform_draw(7, 1, 0)]
    assert len(set(draws)) == 3 and all(0.0 <= u < 1.0 for u in draws)
    # the reference values of the documented generator (SplitMix64 of seed, stream and counter; top 53 bits)
    def plain(seed, stream, counter):
        m = (1 << 64) - 1
        z = (seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03 + counter * 0x8CB92BA72F3D8DD7 + 0x9E3779B97F4A7C15) & m
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        return ((z ^ (z >> 31)) >> 11) / 9007199254740992.0
    assert draws == [plain(7, 0, 0), plain(7, 0, 1), plain(7, 1, 0)]


def run_pipelined(cache, sched, token_of):
    """The host one step ahead: plan and begin step n+1 before step n's tokens are known (finish_step)."""
    inflight = None
    guard = 0
    while (sched.has_work() or inflight is not None) and guard < 500:
        guard += 1
        launched = None
        if sched.has_work():
            plan, _ = sched.plan()
            if plan.entries:
                for e in plan.entries:
                    toks = e.tokens
                    assert all(t >= 0 for t in toks[:-1]) and (toks[-1] >= 0 or e.count == 1), "only a lone token may be unknown"
                    cache.reserve(e.request.id, e.count)
                    cache.commit(e.request.id, e.count)
                # the ids depend on nothing the host has not seen: index of the token in its request
                ids = [token_of(e.request, len(e.request.tokens) - len(e.request.prompt)) for e in plan.entries if e.sample]
                sched.begin_step(plan)
                launched = (plan, ids)
        if inflight is not None:
            sched.finish_step(*inflight)
        inflight = launched
        cache.check()
    assert guard < 500


@pytest.mark.parametrize("num_pages", [64, 5])
def test_pipelined_protocol_gives_the_same_tokens(num_pages):
    def token_of(r, index):
        return 9 if (r.id == "r1" and index == 3) else 100 + index      # r1 meets its end-of-sequence at its 4th token

    outputs = []
    for pipelined in (False, True):
        cache, sched = make(eos=9, num_pages=num_pages, page_size=4, max_batched_tokens=6)
        stops = []
        reqs = [req(0, 7, max_tokens=6), req(1, 3, max_tokens=12), req(2, 5, max_tokens=5, ignore_eos=True),
                Request(id="r3", prompt=[2, 3], params=SamplingParams(temperature=0.0, max_tokens=20),
                        callback=lambda t: stops.append(t) or len(stops) < 4)]
        for r in reqs:
            sched.add(r)
        if pipelined:
            run_pipelined(cache, sched, token_of)
        else:
            while sched.has_work():
                run_step(cache, sched, next_token=lambda r: token_of(r, len(r.generated)))
        outputs.append([(r.generated, r.finish_reason) for r in reqs])
        assert all(v == 0 for v in cache.pages_in_use().values()) and not cache.lengths
        assert all(t >= 0 for r in reqs for t in r.tokens)
    assert outputs[0] == outputs[1]
    assert outputs[0][1] == ([100, 101, 102, 9], "eos") and outputs[0][3][1] == "stopped" and len(outputs[0][3][0]) == 4
