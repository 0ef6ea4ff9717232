"""The scheduler's decisions (no GPU): a fake step function that drives the real cache
manager and returns planned tokens, a hand-driven clock."""
from __future__ import annotations

import pytest

from pylon_b200.cache import CacheManager, OutOfPages
from pylon_b200.engine.scheduler import QueueFullError, Scheduler
from pylon_b200.parts.base import CacheNeed, KVNeed
from pylon_b200.sampling import SamplingParams


class FakeClock:
    def __init__(self):
        self.now = 0.0

    def __call__(self):
        return self.now


class FakeStep:
    """Does the cache bookkeeping of a step like the real one; 'logits' are the row ids."""

    def __init__(self, cache, fail_on=None):
        self.cache = cache
        self.calls = []
        self.fail_on = fail_on

    def __call__(self, entries):
        batch = [(entry.request, len(entry.tokens)) for entry in entries]
        self.cache.prepare(batch)
        if self.fail_on is not None and len(self.calls) == self.fail_on:
            for request, _ in batch:
                self.cache.rollback(request)
            self.calls.append("failed")
            raise RuntimeError("injected")
        for request, _ in batch:
            self.cache.commit(request)
        self.calls.append([(entry.request.request_id, list(entry.tokens), tuple(entry.want)) for entry in entries])
        self.cache.check()
        return [entry.request.request_id for entry in entries if entry.want]


def planned_sampler(plan):
    """plan: request id -> list of tokens it will be given, in order."""
    cursor = {key: 0 for key in plan}

    def sample(logits, params, randoms):
        out = []
        for request_id in logits:
            out.append(plan[request_id][cursor[request_id]])
            cursor[request_id] += 1
        return out

    return sample


def make(num_pages=16, page_size=4, slots=4, plan=None, fail_on=None, **options):
    cache = CacheManager([CacheNeed(kv=KVNeed(1, 4))], [None], page_size=page_size, num_pages=num_pages, max_requests=slots)
    clock = FakeClock()
    step = FakeStep(cache, fail_on)
    options.setdefault("max_batch_size", slots)
    options.setdefault("free_page_floor", False)
    scheduler = Scheduler(cache, step, planned_sampler(plan or {}), clock=clock, **options)
    return scheduler, step, clock, cache


GREEDY3 = SamplingParams(max_new_tokens=3, temperature=0.0)


def test_prompt_is_cut_under_the_token_budget_and_first_token_comes_with_the_last_portion():
    scheduler, step, _, cache = make(plan={"a": [50, 51, 52]}, prefill_chunk_size=4)
    scheduler.add("a", list(range(10)), GREEDY3)
    results = scheduler.run()
    assert [call[0][1] for call in step.calls[:3]] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]]
    assert [call[0][2] for call in step.calls[:3]] == [(), (), (1,)]       # the head runs only where a token is chosen
    assert [call[0][1] for call in step.calls[3:]] == [[50], [51]]          # then one decoded token a step
    assert results[0].output_ids == [50, 51, 52] and results[0].finish_reason == "length"
    assert cache.free_pages() == [16] and cache.free_slots() == 4


def test_decoded_tokens_ride_beside_prompt_portions_and_do_not_use_the_budget():
    scheduler, step, _, _ = make(plan={"a": [9, 9, 9, 9, 9], "b": [8, 8]}, prefill_chunk_size=4)
    scheduler.add("a", [1, 2], SamplingParams(max_new_tokens=5, temperature=0.0))
    scheduler.tick()
    scheduler.add("b", list(range(6)), SamplingParams(max_new_tokens=2, temperature=0.0))
    scheduler.tick()
    assert step.calls[1] == [("a", [9], (0,)), ("b", [0, 1, 2, 3], ())]       # decode row first, full budget for b
    scheduler.tick()
    assert step.calls[2] == [("a", [9], (0,)), ("b", [4, 5], (1,))]


def test_one_tick_packs_several_prompts_and_prefers_one_that_finishes():
    scheduler, step, _, _ = make(plan={"a": [1], "b": [1], "c": [1]}, prefill_chunk_size=8)
    one = SamplingParams(max_new_tokens=1, temperature=0.0)
    scheduler.add("a", list(range(12)), one)
    scheduler.add("b", list(range(5)), one)
    scheduler.add("c", list(range(3)), one)
    scheduler.tick()
    # b fits the budget whole and goes first, then c, the rest of the budget is none: a waits
    assert [(rid, len(tokens)) for rid, tokens, _ in step.calls[0]] == [("b", 5), ("c", 3)]


def test_a_prompt_that_waited_100_ms_goes_first():
    scheduler, step, clock, _ = make(plan={"a": [1], "b": [1]}, prefill_chunk_size=8)
    one = SamplingParams(max_new_tokens=1, temperature=0.0)
    scheduler.add("a", list(range(12)), one)
    scheduler.add("b", list(range(5)), one)
    clock.now = 0.2
    scheduler.tick()
    assert [(rid, len(tokens)) for rid, tokens, _ in step.calls[0]] == [("a", 8)]


def test_stop_token_ends_without_being_returned_and_frees_at_once():
    scheduler, _, _, cache = make(plan={"a": [5, 6, 99, 7]})
    scheduler.add("a", [1, 2, 3], SamplingParams(max_new_tokens=8, temperature=0.0), stop_ids=[99])
    results = scheduler.run()
    assert results[0].output_ids == [5, 6] and results[0].finish_reason == "eos"
    assert cache.free_pages() == [16]
    scheduler2, _, _, _ = make(plan={"a": [5, 99, 7]})
    scheduler2.add("a", [1], SamplingParams(max_new_tokens=3, temperature=0.0, ignore_eos=True), stop_ids=[99])
    assert scheduler2.run()[0].output_ids == [5, 99, 7]


def test_admission_reserves_the_whole_life_and_later_requests_wait_for_pages():
    # 6 pages of 4 tokens.  a needs ceil((6+6)/4) = 3 pages, b needs 3, c needs 2: c must wait.
    plan = {"a": [1] * 6, "b": [1] * 6, "c": [1] * 2}
    scheduler, step, _, cache = make(num_pages=6, plan=plan, admit_skip=0)
    six = SamplingParams(max_new_tokens=6, temperature=0.0)
    scheduler.add("a", list(range(6)), six)
    scheduler.add("b", list(range(6)), six)
    scheduler.add("c", list(range(6)), SamplingParams(max_new_tokens=2, temperature=0.0))
    scheduler.tick()
    assert [r.request_id for r in scheduler.active] == ["a", "b"] and [r.request_id for r in scheduler.waiting] == ["c"]
    results = scheduler.run()
    assert {r.request_id: r.finish_reason for r in results} == {"a": "length", "b": "length", "c": "length"}
    assert cache.free_pages() == [6]
    # c started only after a page reservation was released, and used pages again
    assert cache.groups[0].pool.acquired_total > 6


def test_a_request_larger_than_the_pool_is_refused_at_once():
    scheduler, _, _, _ = make(num_pages=2)
    with pytest.raises(ValueError, match="cache pages"):
        scheduler.add("big", list(range(6)), SamplingParams(max_new_tokens=6, temperature=0.0))


def test_skip_ahead_admission_and_its_100_ms_limit():
    plan = {"a": [1] * 4, "big": [1] * 4, "small": [1]}
    scheduler, _, clock, _ = make(num_pages=6, plan=plan, admit_skip=4)
    scheduler.add("a", list(range(8)), SamplingParams(max_new_tokens=4, temperature=0.0))       # 3 pages
    scheduler.add("big", list(range(12)), SamplingParams(max_new_tokens=4, temperature=0.0))    # 4 pages: does not fit beside a
    scheduler.add("small", [1, 2], SamplingParams(max_new_tokens=1, temperature=0.0))            # 1 page
    scheduler.admit()
    assert [r.request_id for r in scheduler.active] == ["a", "small"] and scheduler.overtakes == 1
    scheduler2, _, clock2, _ = make(num_pages=6, plan=plan, admit_skip=4)
    scheduler2.add("a", list(range(8)), SamplingParams(max_new_tokens=4, temperature=0.0))
    scheduler2.add("big", list(range(12)), SamplingParams(max_new_tokens=4, temperature=0.0))
    scheduler2.add("small", [1, 2], SamplingParams(max_new_tokens=1, temperature=0.0))
    clock2.now = 0.5                                       # the head has waited long enough: nobody passes it
    scheduler2.admit()
    assert [r.request_id for r in scheduler2.active] == ["a"]


def test_free_page_floor_keeps_a_page_per_decoding_request():
    plan = {"a": [1] * 4, "b": [1]}
    scheduler, _, _, _ = make(num_pages=4, plan=plan, free_page_floor=True, admit_skip=0)
    scheduler.add("a", [1, 2, 3], SamplingParams(max_new_tokens=4, temperature=0.0))   # 2 pages
    scheduler.tick()                                                                  # a decodes now
    scheduler.add("b", list(range(7)), SamplingParams(max_new_tokens=1, temperature=0.0))   # 2 pages: would leave 0 < 1
    scheduler.admit()
    assert [r.request_id for r in scheduler.active] == ["a"]


def test_slots_limit_the_batch_and_a_full_decoding_batch_holds_prompts_off_for_100_ms():
    plan = {"a": [1] * 8, "b": [1] * 8, "c": [1]}
    scheduler, step, clock, _ = make(slots=3, max_batch_size=2, plan=plan)
    eight = SamplingParams(max_new_tokens=8, temperature=0.0)
    scheduler.add("a", [1], eight)
    scheduler.add("b", [1], eight)
    scheduler.add("c", [1, 2], SamplingParams(max_new_tokens=1, temperature=0.0))
    scheduler.tick()
    assert [r.request_id for r in scheduler.active] == ["a", "b"] and len(scheduler.waiting) == 1


def test_queue_limit_and_abort():
    scheduler, _, _, cache = make(max_queue_size=2, plan={"a": [1] * 5})
    scheduler.add("a", [1], SamplingParams(max_new_tokens=5, temperature=0.0))
    scheduler.add("b", [1], GREEDY3)
    with pytest.raises(QueueFullError):
        scheduler.add("c", [1], GREEDY3)
    assert scheduler.abort("b") and not scheduler.abort("zzz")
    scheduler.tick()
    assert scheduler.abort("a") and cache.free_pages() == [16] and not scheduler.has_work()
    with pytest.raises(ValueError, match="at least one token"):
        scheduler.add("d", [], GREEDY3)


def test_a_failing_step_fails_its_requests_only_and_gives_their_pages_back():
    plan = {"a": [1] * 3, "b": [1] * 3}
    scheduler, step, _, cache = make(plan=plan, fail_on=1)
    scheduler.add("a", [1, 2], GREEDY3)
    scheduler.tick()                          # step 0: a prefills and gets its first token
    scheduler.add("b", [3, 4], GREEDY3)
    finished = scheduler.tick()               # step 1 fails: a (decoding) and b (prefilling) were in it
    assert {r.request_id: r.finish_reason for r in finished} == {"a": "error", "b": "error"}
    assert all(isinstance(r.error, RuntimeError) for r in finished)
    assert cache.free_pages() == [16] and cache.free_slots() == 4 and not scheduler.has_work()
    scheduler.sample = planned_sampler({"c": [7, 7, 7]})
    scheduler.add("c", [5], GREEDY3)
    assert scheduler.run()[0].output_ids == [7, 7, 7]   # the engine goes on


def test_running_out_of_pages_inside_a_step_fails_that_step_only():
    """Reservations make this impossible for admitted requests; a pool that someone else
    drained shows what happens anyway."""
    scheduler, _, _, cache = make(num_pages=4, plan={"a": [1, 1]})
    scheduler.add("a", list(range(8)), SamplingParams(max_new_tokens=2, temperature=0.0))
    thief = cache.open("thief", 12)
    cache.prepare([(thief, 12)])
    cache.commit(thief)
    finished = scheduler.tick()
    assert finished[0].finish_reason == "error" and isinstance(finished[0].error, OutOfPages)
    cache.close(thief)
    assert cache.free_pages() == [4]


def test_sampling_options_are_checked():
    with pytest.raises(ValueError):
        SamplingParams(max_new_tokens=0)
    with pytest.raises(ValueError):
        SamplingParams(temperature=2.5)
    with pytest.raises(ValueError):
        SamplingParams(top_p=0.0)
    defaults = SamplingParams()
    assert (defaults.max_new_tokens, defaults.temperature, defaults.top_p) == (256, 0.2, 0.95)


def test_rows_alike_is_a_matter_of_the_longest_against_the_mean():
    """The hint the step function gives the parts: the requests of a step hold about equally many
    tokens after it when the longest is at most an eighth above the mean."""
    from types import SimpleNamespace

    from pylon_b200.engine.step import StepFunction

    def entries(*pairs):   # (tokens held, tokens brought)
        return [SimpleNamespace(request=SimpleNamespace(length=held), tokens=[0] * brought) for held, brought in pairs]

    assert StepFunction.rows_alike(entries((4000, 1)))
    assert StepFunction.rows_alike(entries((4095, 1), (4095, 1), (4090, 1)))
    assert StepFunction.rows_alike(entries((0, 1), (0, 1)))
    assert StepFunction.rows_alike(entries((800, 1), (1000, 1)))            # 1001 against a mean of 901
    assert not StepFunction.rows_alike(entries((700, 1), (1000, 1)))        # 1001 against a mean of 851
    assert not StepFunction.rows_alike(entries((4000, 1), (10, 1), (10, 1)))
    assert StepFunction.rows_alike(entries((2000, 48), (2047, 1)))           # what a request brings counts as held


# -- running ahead: a tick queues its step before it waits for the tokens of the step before --------------------------
class FakeDeviceTokens:
    """Stands for the tensor of sampled tokens on the device: the step function may look into it, the scheduler may not."""

    def __init__(self, tokens):
        self.tokens = list(tokens)
        self.shape = (len(self.tokens),)


class LaunchingSampler:
    """A sampler with ``launch``: the tokens are 'on the device' at once and reach the host when ``result`` is called.
    Keeps the order of launches and results in ``events``."""

    def __init__(self, plan, events):
        self.choose = planned_sampler(plan)
        self.events = events

    def launch(self, logits, params, randoms):
        sampler, tokens = self, self.choose(logits, params, randoms)
        number = sum(1 for event in self.events if event[0] == "launch")
        self.events.append(("launch", number))

        class Handle:
            device = FakeDeviceTokens(tokens)

            def result(self):
                sampler.events.append(("result", number))
                return tokens

        return Handle()

    def __call__(self, logits, params, randoms):
        return self.launch(logits, params, randoms).result()


class FakeStepWithSources(FakeStep):
    """Takes the tokens that entries name on the 'device' from there, as the real step function's kernel does."""

    def __call__(self, entries):
        for entry in entries:
            if entry.source is not None:
                tensor, row = entry.source
                assert len(entry.tokens) == 1
                entry.tokens = [tensor.tokens[row]]
        return super().__call__(entries)


def make_ahead(plan, run_ahead, num_pages=64, page_size=4, slots=4, **options):
    cache = CacheManager([CacheNeed(kv=KVNeed(1, 4))], [None], page_size=page_size, num_pages=num_pages, max_requests=slots)
    events = []
    step = FakeStepWithSources(cache)
    options.setdefault("max_batch_size", slots)
    options.setdefault("free_page_floor", False)
    scheduler = Scheduler(cache, step, LaunchingSampler(plan, events), clock=FakeClock(), run_ahead=run_ahead, **options)
    return scheduler, step, events, cache


def test_running_ahead_queues_the_next_step_before_it_reads_the_tokens_of_the_last():
    scheduler, step, events, cache = make_ahead({"a": [50, 51, 52, 53]}, run_ahead=True, prefill_chunk_size=4)
    scheduler.add("a", list(range(6)), SamplingParams(max_new_tokens=4, temperature=0.0))
    results = scheduler.run()
    assert results[0].output_ids == [50, 51, 52, 53] and results[0].finish_reason == "length"
    # the prompt's two portions, then three decoded tokens, each taken on the device; max_new_tokens is never overrun
    assert [call[0][1] for call in step.calls] == [[0, 1, 2, 3], [4, 5], [50], [51], [52]]
    # every result is read after the launch of the step behind it
    assert events == [("launch", 0), ("launch", 1), ("result", 0), ("launch", 2), ("result", 1), ("launch", 3), ("result", 2), ("result", 3)]
    assert cache.free_pages() == [64] and cache.free_slots() == 4


def test_running_ahead_drops_the_token_of_the_step_behind_a_stop_id():
    scheduler, step, events, cache = make_ahead({"a": [5, 6, 99, 7, 8], "b": [1, 2, 3, 4, 5, 6]}, run_ahead=True)
    scheduler.add("a", [1, 2, 3], SamplingParams(max_new_tokens=8, temperature=0.0), stop_ids=[99])
    scheduler.add("b", [4, 5], SamplingParams(max_new_tokens=6, temperature=0.0))
    results = {result.request_id: result for result in scheduler.run()}
    assert results["a"].output_ids == [5, 6] and results["a"].finish_reason == "eos"
    assert results["b"].output_ids == [1, 2, 3, 4, 5, 6] and results["b"].finish_reason == "length"
    # a was given one step with its stop id as input (queued before the host had seen it), and none after that
    fed_to_a = [tokens for call in step.calls for rid, tokens, _ in call if rid == "a"]
    assert fed_to_a == [[1, 2, 3], [5], [6], [99]]
    assert cache.free_pages() == [64] and cache.free_slots() == 4


def test_a_scheduler_that_runs_ahead_needs_a_sampler_that_launches():
    cache = CacheManager([CacheNeed(kv=KVNeed(1, 4))], [None], page_size=4, num_pages=8, max_requests=2)
    with pytest.raises(ValueError, match="launch"):
        Scheduler(cache, FakeStep(cache), planned_sampler({}), max_batch_size=2, run_ahead=True)


@pytest.mark.parametrize("seed", range(6))
def test_running_ahead_generates_what_waiting_generates(seed):
    """Random requests (prompt lengths, limits, stop ids that do and do not come up, arrival ticks) through a tight pool,
    with and without running ahead: the same output for every request, every page and slot given back, and at most one
    step more per request that met a stop id."""
    import random

    rng = random.Random(seed)
    requests = []
    for index in range(14):
        prompt = [rng.randrange(100) for _ in range(rng.randrange(1, 19))]
        limit = rng.randrange(1, 12)
        plan = [rng.randrange(100, 120) for _ in range(limit + 2)]
        requests.append((f"r{index}", prompt, limit, plan, [rng.choice(plan)] if rng.random() < 0.5 else [], rng.randrange(0, 12)))
    outcomes = {}
    for run_ahead in (False, True):
        scheduler, step, events, cache = make_ahead({rid: plan for rid, _, _, plan, _, _ in requests}, run_ahead, num_pages=24, slots=3,
                                                    prefill_chunk_size=7, max_queue_size=14)
        waiting = sorted(requests, key=lambda request: request[5])
        results = {}
        tick = 0
        while waiting or scheduler.has_work():
            while waiting and waiting[0][5] <= tick:
                rid, prompt, limit, _, stops, _ = waiting.pop(0)
                scheduler.add(rid, prompt, SamplingParams(max_new_tokens=limit, temperature=0.0), stop_ids=stops)
            for result in scheduler.tick():
                results[result.request_id] = (result.output_ids, result.finish_reason)
            cache.check()
            tick += 1
            assert tick < 2_000
        assert cache.free_pages() == [24] and cache.free_slots() == 3
        outcomes[run_ahead] = (results, len(step.calls))
    assert outcomes[True][0] == outcomes[False][0]
    # A request that ends by its length gives back slot and pages when its last token is launched, so nothing waits for
    # it; the host learns of a stop id one tick late, so a slot may stand empty for a tick each time a request ends by one.
    stopped = sum(1 for _, reason in outcomes[False][0].values() if reason == "eos")
    assert outcomes[True][1] <= outcomes[False][1] + stopped + 1


def test_running_ahead_a_step_that_fails_at_launch_fails_its_requests_only():
    scheduler, step, events, cache = make_ahead({"a": [1, 2, 3, 4, 5, 6], "b": [7, 8, 9]}, run_ahead=True)
    step.fail_on = 3     # the fourth call of the step function raises, with the third step still in flight
    scheduler.add("a", [1, 2, 3], SamplingParams(max_new_tokens=6, temperature=0.0))
    for _ in range(3):
        scheduler.tick()
    scheduler.add("b", [4, 5], SamplingParams(max_new_tokens=3, temperature=0.0))   # joins at the failing step
    results = {result.request_id: result for result in scheduler.run()}
    assert results["a"].finish_reason == "error" and results["b"].finish_reason == "error"
    assert results["a"].output_ids == [1, 2]      # what had been read back before the step failed; the token in flight is dropped
    assert cache.free_pages() == [64] and cache.free_slots() == 4
    cache.check()
    scheduler.add("c", [1], SamplingParams(max_new_tokens=2, temperature=0.0))
    scheduler.sample.choose = planned_sampler({"c": [11, 12]})
    assert scheduler.run()[0].output_ids == [11, 12]


def test_running_ahead_a_request_dropped_while_its_step_is_in_flight():
    scheduler, step, events, cache = make_ahead({"a": [1, 2, 3, 4, 5, 6], "b": [7, 8, 9, 10]}, run_ahead=True)
    scheduler.add("a", [1, 2, 3], SamplingParams(max_new_tokens=6, temperature=0.0))
    scheduler.add("b", [4, 5], SamplingParams(max_new_tokens=4, temperature=0.0))
    scheduler.tick()
    scheduler.tick()
    assert scheduler.abort("a")           # a step with a row for it is queued; its token will be dropped
    assert cache.free_slots() == 3
    results = scheduler.run()
    assert [(result.request_id, result.output_ids) for result in results] == [("b", [7, 8, 9, 10])]
    assert cache.free_pages() == [64] and cache.free_slots() == 4
    cache.check()


def test_running_ahead_tokens_that_come_back_void_fail_the_requests_of_that_step():
    scheduler, step, events, cache = make_ahead({"a": [1, 2, 3, 4, 5, 6, 7, 8], "b": [7, 8, 9]}, run_ahead=True)
    launch = scheduler.sample.launch
    count = [0]

    def launch_with_one_void_result(logits, params, randoms):
        handle = launch(logits, params, randoms)
        count[0] += 1
        if count[0] == 3:
            def void():
                raise RuntimeError("the results of that step are void")
            handle.result = void
        return handle

    scheduler.sample.launch = launch_with_one_void_result
    scheduler.add("a", [1, 2, 3], SamplingParams(max_new_tokens=8, temperature=0.0))
    results = scheduler.run()
    assert results[0].finish_reason == "error" and results[0].output_ids == [1, 2]
    assert cache.free_pages() == [64] and cache.free_slots() == 4
    scheduler.add("b", [4], SamplingParams(max_new_tokens=3, temperature=0.0))
    assert scheduler.run()[0].output_ids == [7, 8, 9]


def test_running_ahead_a_request_that_ends_by_length_makes_room_when_its_last_token_is_launched():
    """One slot, two requests: the step that chooses the first one's last token gives its slot and pages back, so the
    second's prompt goes into the very next step, while the first one's last token is still on its way to the host."""
    scheduler, step, events, cache = make_ahead({"a": [1, 2, 3], "b": [7, 8]}, run_ahead=True, slots=1)
    scheduler.add("a", [1, 2, 3], SamplingParams(max_new_tokens=3, temperature=0.0))
    scheduler.add("b", [4, 5], SamplingParams(max_new_tokens=2, temperature=0.0))
    results = {result.request_id: result for result in scheduler.run()}
    assert results["a"].output_ids == [1, 2, 3] and results["b"].output_ids == [7, 8]
    assert [[rid for rid, _, _ in call] for call in step.calls] == [["a"], ["a"], ["a"], ["b"], ["b"]]   # no step stands empty in between
    assert events.index(("launch", 3)) < events.index(("result", 2))      # b's prompt is queued before a's last token is read
    assert cache.free_pages() == [64] and cache.free_slots() == 1
    # a request dropped while its last token is on its way
    scheduler.sample.choose = planned_sampler({"c": [5, 6]})
    scheduler.add("c", [9], SamplingParams(max_new_tokens=2, temperature=0.0))
    scheduler.tick()
    scheduler.tick()
    assert [request.request_id for request in scheduler.leaving] == ["c"] and cache.free_slots() == 1
    assert scheduler.abort("c") and not scheduler.leaving
    assert scheduler.run() == [] and not scheduler.has_work()
