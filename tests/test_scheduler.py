"""The scheduler's decisions, on the host with a stand-in for the model step."""
import random

import pytest

from flyweight_b200.cache import PAGE_SIZE, CacheManager
from flyweight_b200.engine.runner import StepPlanner
from flyweight_b200.engine.scheduler import (EVENT_ERROR, EVENT_FINISHED, EVENT_TOKEN, Scheduler)
from flyweight_b200.parts import FixedState, PagedKV
from flyweight_b200.sampling import GREEDY

VOCAB = 50


def make(num_pages=8, num_slots=4, budget=32, max_len=512):
    cache = CacheManager([PagedKV(1, 16), FixedState((4, 2))], num_pages, num_slots, device=None)
    planner = StepPlanner(cache, VOCAB, max_len, budget)
    return Scheduler(planner, budget, max_len), planner


def fake_token(task):
    """A deterministic 'model': the next token depends on the whole text so far."""
    return (sum(task.text) * 31 + len(task.text)) % VOCAB


def run_step(sched, planner, log=None):
    step = sched.schedule()
    if step.entries:
        planner.plan(step.entries)            # what the runner does before the kernels
        for task in sched.advance(step):
            sched.accept(task, fake_token(task))
    planner.cache.check()
    if log is not None:
        log.append(step)
    return step


def test_prompt_is_cut_into_portions_under_the_budget():
    sched, planner = make(budget=32)
    tid = sched.submit(list(range(40)) * 2, 3, (), GREEDY)      # 80 prompt tokens
    sizes = []
    while sched.has_work():
        step = run_step(sched, planner)
        sizes.append([len(e[1]) for e in step.entries])
    assert sizes[:3] == [[32], [32], [16]]                      # 80 = 32 + 32 + 16
    assert sizes[3:] == [[1], [1]]                              # then one token per step
    task = sched.tasks[tid]
    assert len(task.generated) == 3 and task.finish_reason == "length"
    assert planner.cache.free_slots == 4 and planner.cache.groups[0].pool.n_used == 0


def test_logits_are_wanted_only_at_the_end_of_the_known_text():
    sched, planner = make(budget=16)
    sched.submit(list(range(20)), 2, (), GREEDY)
    first = sched.schedule()
    assert first.entries[0][2] == []                            # mid-prompt portion: none
    planner.plan(first.entries)
    sched.advance(first)
    second = sched.schedule()
    assert len(second.entries[0][1]) == 4 and second.entries[0][2] == [3]


def test_decodes_come_first_and_share_the_step_with_a_prompt_portion():
    sched, planner = make(budget=16, num_slots=4)
    a = sched.submit([1, 2, 3], 8, (), GREEDY)
    run_step(sched, planner)                                    # a: prompt done, one token
    b = sched.submit(list(range(30)), 2, (), GREEDY)
    step = run_step(sched, planner)
    assert [e[0] for e in step.entries] == [a, b]
    assert [len(e[1]) for e in step.entries] == [1, 15]         # budget 16 = 1 decode + 15
    step = run_step(sched, planner)
    assert [len(e[1]) for e in step.entries] == [1, 15]


def test_admission_is_fifo_and_waits_for_a_slot():
    sched, planner = make(num_slots=2, budget=64)
    ids = [sched.submit([i + 1] * 5, 4, (), GREEDY) for i in range(4)]
    step = run_step(sched, planner)
    assert [e[0] for e in step.entries] == ids[:2]
    assert [t.id for t in sched.waiting] == ids[2:]
    while sched.has_work():
        run_step(sched, planner)
    order = sorted(ids, key=lambda i: sched.tasks[i].admitted_at)
    assert order == ids


def test_stop_token_is_emitted_then_finishes():
    sched, planner = make()
    tid = sched.submit([4, 5, 6], 10, (), GREEDY)
    step = sched.schedule()
    planner.plan(step.entries)
    (task,) = sched.advance(step)
    task.stop_tokens = (17,)
    events = sched.accept(task, 17)
    assert events == [(tid, 17, EVENT_TOKEN), (tid, 0, EVENT_FINISHED)]
    assert task.finish_reason == "stop" and not sched.has_work()


def test_submit_checks():
    sched, _ = make(num_pages=2, max_len=200)
    with pytest.raises(ValueError, match="must not be empty"):
        sched.submit([], 4)
    with pytest.raises(ValueError, match="max_tokens must be positive"):
        sched.submit([1], 0)
    with pytest.raises(ValueError, match="context limit"):
        sched.submit([1] * 150, 100)
    with pytest.raises(ValueError, match="cache pages"):
        sched.submit([1] * 100, 60)                             # 160 tokens = 3 pages > 2
    with pytest.raises(ValueError, match="outside"):
        sched.submit([VOCAB], 1)


def test_cancel_frees_everything():
    sched, planner = make()
    a = sched.submit([1] * 70, 50, (), GREEDY)
    run_step(sched, planner)
    run_step(sched, planner)
    sched.cancel(a)
    step = run_step(sched, planner)
    assert (a, 0, EVENT_FINISHED) in step.events
    assert sched.tasks[a].finish_reason == "cancelled"
    assert planner.cache.groups[0].pool.n_used == 0 and planner.cache.free_slots == 4


def test_out_of_pages_preempts_the_newest_and_it_finishes_the_same():
    def outputs(num_pages):
        sched, planner = make(num_pages=num_pages, num_slots=3, budget=64, max_len=400)
        ids = [sched.submit([i + 2] * 50, 100, (), GREEDY) for i in range(3)]
        log = []
        while sched.has_work():
            run_step(sched, planner, log)
        return sched, ids, log

    roomy, ids, _ = outputs(num_pages=16)
    tight, ids2, log = outputs(num_pages=5)         # 3 x 150 tokens = 9 pages do not fit in 5
    assert roomy.stats["preemptions"] == 0
    assert tight.stats["preemptions"] > 0
    preempted = [tid for step in log for tid in step.preempted]
    first = next(step for step in log if step.preempted)
    running_then = sorted(t.id for t in tight.tasks.values() if t.admitted_at >= 0)
    assert first.preempted[0] == max(ids2)          # the most recently admitted goes first
    for a, b in zip(ids, ids2):
        assert roomy.tasks[a].generated == tight.tasks[b].generated
        assert tight.tasks[b].finish_reason == "length"
    assert tight.cache.groups[0].pool.n_used == 0
    assert set(preempted) <= set(ids2) and running_then


def test_a_request_larger_than_the_pool_fails_alone():
    sched, planner = make(num_pages=2, max_len=400)
    # passes the submit check (prompt + max_tokens = 2 pages) but cannot get the spare page
    tid = sched.submit([3] * 100, 28, (), GREEDY)
    seen = []
    for _ in range(200):
        if not sched.has_work():
            break
        seen.extend(run_step(sched, planner).events)
    task = sched.tasks[tid]
    assert task.state == "finished"
    assert task.finish_reason in ("length", "error")
    if task.error:
        assert (tid, 0, EVENT_ERROR) in seen
    assert planner.cache.groups[0].pool.n_used == 0


def test_random_workloads_always_drain():
    rng = random.Random(3)
    for _ in range(10):
        sched, planner = make(num_pages=rng.randint(4, 10), num_slots=rng.randint(1, 4),
                              budget=rng.choice([8, 33, 64]), max_len=256)
        ids = [sched.submit([rng.randrange(VOCAB) for _ in range(rng.randint(1, 120))],
                            rng.randint(1, 60), (), GREEDY) for _ in range(8)]
        for _ in range(5000):
            if not sched.has_work():
                break
            step = run_step(sched, planner)
            assert sum(len(e[1]) for e in step.entries) <= sched.max_batched_tokens
        assert not sched.has_work()
        assert all(sched.tasks[i].state == "finished" for i in ids)
        assert planner.cache.groups[0].pool.n_used == 0


def test_a_request_whose_bookkeeping_raises_between_steps_fails_alone():
    """An exception raised for one request while the scheduler plans a step (here: the page
    arithmetic of that request, made to raise by the planner stand-in) ends that request with an
    error event and gives back what it held; the others run to the end with the tokens they would
    have had anyway (native/src/v2_runtime.cpp:33788-33797)."""
    class FaultyPlanner(StepPlanner):
        poisoned = None

        def pages_short(self, entries):
            for request, _, _ in entries:
                if request == self.poisoned:
                    error = RuntimeError("injected: this request's page table is broken")
                    error.request = request
                    raise error
            return super().pages_short(entries)

    def run(poison_at):
        cache = CacheManager([PagedKV(1, 16), FixedState((4, 2))], 12, 4, device=None)
        planner = FaultyPlanner(cache, VOCAB, 512, 32)
        sched = Scheduler(planner, 32, 512)
        ids = [sched.submit([3 + i] * (20 + 7 * i), 12, (), GREEDY) for i in range(4)]
        events, steps = [], 0
        while sched.has_work():
            if steps == poison_at:
                planner.poisoned = ids[1]
            step = sched.schedule()
            events.extend(step.events)
            if step.entries:
                planner.plan(step.entries)
                for task in sched.advance(step):
                    events.extend(sched.accept(task, fake_token(task)))
            planner.cache.check()
            steps += 1
            assert steps < 200
        return sched, ids, events

    clean, ids, _ = run(None)
    for when in (0, 2, 6):                     # before admission, in its prompt, while decoding
        sched, ids, events = run(when)
        victim = sched.tasks[ids[1]]
        assert victim.state == "finished" and victim.finish_reason == "error"
        assert "injected" in victim.error
        assert events.count((ids[1], 0, EVENT_ERROR)) == 1
        for tid in (ids[0], ids[2], ids[3]):
            assert sched.tasks[tid].generated == clean.tasks[tid].generated
            assert sched.tasks[tid].finish_reason == "length"
        assert sched.planner.cache.free_slots == 4 and sched.planner.cache.groups[0].pool.n_used == 0
        assert sched.stats["failed"] == 1


def test_fail_takes_a_task_off_the_lists_even_if_the_release_raises():
    sched, planner = make()
    tid = sched.submit([1, 2, 3], 4, (), GREEDY)
    run_step(sched, planner)
    task = sched.tasks[tid]
    original = planner.finish
    planner.finish = lambda request: (_ for _ in ()).throw(RuntimeError("release failed"))
    assert sched.fail(task, "first fault") == [(tid, 0, EVENT_ERROR)]
    planner.finish = original
    assert task.state == "finished" and "first fault" in task.error and "release failed" in task.error
    assert not sched.has_work() and sched.fail(task, "again") == []


def test_the_default_pool_runs_two_requests_that_fill_the_context_side_by_side():
    """The default pool keeps one page to spare per sequence, so that admission's spare page does
    not make requests that reach the context limit wait for one another."""
    from flyweight_b200.engine.runtime import EngineConfig
    config = EngineConfig(context_limit=256, parallel_sequences=2, max_batched_tokens=512)
    assert config.pool_tokens == 2 * (256 // PAGE_SIZE + 1) * PAGE_SIZE
    sched, planner = make(num_pages=config.pool_tokens // PAGE_SIZE, num_slots=2, budget=512, max_len=256)
    ids = [sched.submit([1 + i] * 200, 56, (), GREEDY) for i in range(2)]
    step = run_step(sched, planner)
    assert [entry[0] for entry in step.entries] == ids          # both admitted in the first step
    while sched.has_work():
        run_step(sched, planner)
    assert all(len(sched.tasks[i].generated) == 56 for i in ids) and sched.stats["preemptions"] == 0
    with pytest.raises(ValueError):
        EngineConfig(context_limit=0)


def test_the_queue_refuses_past_its_limit_and_the_limit_follows_the_parallel_sequences():
    from flyweight_b200.engine.runtime import EngineConfig
    from flyweight_b200.engine.scheduler import QueueFull
    cache = CacheManager([PagedKV(1, 16), FixedState((4, 2))], 8, 4, device=None)
    planner = StepPlanner(cache, VOCAB, 512, 32)
    sched = Scheduler(planner, 32, 512, max_queued=3)
    for _ in range(3):
        sched.submit([1, 2, 3], 4)
    with pytest.raises(QueueFull):
        sched.submit([1, 2, 3], 4)
    run_step(sched, planner)                      # nothing finished: still full
    with pytest.raises(QueueFull):
        sched.submit([1], 1)
    while sched.has_work():
        run_step(sched, planner)
    sched.submit([1], 1)                          # room again
    assert EngineConfig().queue_limit == 256      # native/src/v2_runtime.cpp:32588
    assert EngineConfig(parallel_sequences=512).queue_limit == 512
    assert EngineConfig(parallel_sequences=4, max_queued=16).queue_limit == 16
