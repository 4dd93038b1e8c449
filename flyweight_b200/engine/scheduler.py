"""The scheduler: which requests run in the next step, and with which tokens.

Decisions, in order, for every step:

1. every running request that is decoding contributes its one next token;
2. running requests still in their prompt get the next portion, as large as the token
   budget leaves (a portion may be cut anywhere, down to one token);
3. waiting requests are admitted first-come first-served while a state slot is free, the
   budget is not used up and the pool has pages for their whole known text plus one
   spare page; an admitted request starts its prompt in the same step;
4. if the pages for the step are lacking, the most recently admitted running request is
   *preempted*: everything it holds goes back to the pools and it returns to the front of
   the waiting queue with its prompt and the tokens it has generated so far as its text;
   when it is admitted again that text is recomputed, and its random generator continues
   where it was, so its output is the same as without the preemption.  This repeats until
   the step fits; a single request that does not fit an empty pool fails with an error.

flyweight reserves a whole context per slot at start-up, so it never runs out in the
middle of a request (native/src/v2_runtime.cpp:33578-33609); its queue (cap 256, :32588-32591),
submit-time checks (:32511-32535), one-token-per-cycle decoding (:33770-33787) and finish
rules (:33777-33780) are kept.  Everything here is host logic and runs without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..cache.manager import PAGE_SIZE
from ..sampling.config import SamplingConfig
from ..sampling.rng import XorShift64Star

MAX_QUEUED = 256          # native/src/v2_runtime.cpp:32588

# event kinds, as in native/include/flyweight_v2.h:413-417
EVENT_TOKEN, EVENT_FINISHED, EVENT_ERROR, EVENT_PROGRESS = 0, 1, 2, 3
IN_FLIGHT = 0             # placeholder id of a token whose value is still on the device


class QueueFull(RuntimeError):
    pass


@dataclass(eq=False)
class Task:
    id: int
    prompt: List[int]
    max_tokens: int
    stop_tokens: Tuple[int, ...]
    sampling: SamplingConfig
    rng: XorShift64Star
    generated: List[int] = field(default_factory=list)
    computed: int = 0              # tokens of (prompt + generated) that are in the cache
    state: str = "waiting"         # waiting | running | finished
    finish_reason: Optional[str] = None
    error: Optional[str] = None
    cancelled: bool = False
    preemptions: int = 0
    admitted_at: int = -1          # admission counter value (larger = admitted later)
    in_flight: int = 0             # 1: its next token is sampled on the device but not read yet
    greedy: bool = field(init=False, default=True)       # of its sampling settings, read once: they
    penalizes: bool = field(init=False, default=False)   # are asked of every running task on every step

    def __post_init__(self):
        self.greedy = bool(self.sampling.greedy)
        self.penalizes = bool(self.sampling.penalizes)

    @property
    def text(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def pending(self) -> int:
        """Tokens of its text that are not in the cache yet; a token still in flight counts: it is
        the text's next token, only its value is not on the host yet."""
        return len(self.prompt) + len(self.generated) + self.in_flight - self.computed

    def ends_with_the_token_in_flight(self, max_model_len: int) -> bool:
        """Whether the token in flight is known to be its last (token count or context limit)."""
        return (len(self.generated) + self.in_flight >= self.max_tokens
                or len(self.prompt) + len(self.generated) + self.in_flight >= max_model_len)

    def tokens_from(self, start: int, count: int) -> List[int]:
        """``text[start:start + count]`` without joining the two lists first (a long prompt
        would be copied once per step and request).  A token in flight stands as ``IN_FLIGHT``:
        the step function puts the value in on the device."""
        known = len(self.prompt)
        if start + count <= known:
            return self.prompt[start:start + count]
        if start >= known:
            out = self.generated[start - known:start - known + count]
        else:
            out = self.prompt[start:] + self.generated[:start + count - known]
        if len(out) < count:
            out = out + [IN_FLIGHT] * (count - len(out))
        return out


@dataclass
class ScheduledStep:
    entries: List[Tuple[int, List[int], List[int]]]     # (task id, tokens, want)
    tasks: List[Task]                                   # same order as entries
    preempted: List[int] = field(default_factory=list)
    failed: List[int] = field(default_factory=list)
    events: List[Tuple[int, int, int]] = field(default_factory=list)   # made while scheduling
    in_flight: List[Task] = field(default_factory=list)   # tasks whose entry ends in a token still on the device


class Scheduler:
    def __init__(self, planner, max_batched_tokens: int, max_model_len: int, max_queued: int = MAX_QUEUED):
        """``planner`` is a ``StepPlanner`` (the runner, or a device-free stand-in): the
        scheduler asks it how many pages a step lacks and tells it when a request ends.
        ``max_queued``: most requests waiting and running together before ``submit`` refuses."""
        self.planner = planner
        self.max_queued = int(max_queued)
        self.cache = planner.cache
        self.max_batched_tokens = int(max_batched_tokens)
        self.max_model_len = int(max_model_len)
        self.waiting: Deque[Task] = deque()
        self.running: List[Task] = []
        self.tasks: Dict[int, Task] = {}
        self._next_id = 1
        self._admissions = 0
        self.stats = {"preemptions": 0, "admitted": 0, "finished": 0, "failed": 0,
                      "prefill_tokens": 0, "decode_tokens": 0, "steps": 0}
        self.penalizing = 0         # live tasks (waiting or running) whose sampling has a penalty

    # ------------------------------------------------------------------ submit / cancel
    def submit(self, prompt: Sequence[int], max_tokens: int, stop_tokens: Sequence[int] = (),
               sampling: Optional[SamplingConfig] = None) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("prompt_tokens must not be empty")
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        if len(prompt) + max_tokens > self.max_model_len:          # v2_runtime.cpp:32511-32514
            raise ValueError(f"prompt ({len(prompt)}) + max_tokens ({max_tokens}) exceeds the "
                             f"context limit {self.max_model_len}")
        pages = -(-(len(prompt) + max_tokens) // PAGE_SIZE)
        if any(pages > group.pool.num_pages for group in self.cache.groups):
            raise ValueError(f"the request needs {pages} cache pages, the pool has "
                             f"{self.cache.num_pages}")
        vocab = self.planner.vocab_size
        for token in prompt:
            if not 0 <= token < vocab:
                raise ValueError(f"token id {token} is outside [0, {vocab})")
        if len(self.waiting) + len(self.running) >= self.max_queued:
            raise QueueFull("the engine queue is full")
        sampling = sampling or SamplingConfig()
        task = Task(self._next_id, prompt, int(max_tokens), tuple(int(t) for t in stop_tokens),
                    sampling, XorShift64Star(sampling.seed, self._next_id))
        self._next_id += 1
        self.tasks[task.id] = task
        self.waiting.append(task)
        self.penalizing += task.penalizes
        return task.id

    def cancel(self, task_id: int) -> None:
        task = self.tasks.get(task_id)
        if task is not None and task.state != "finished":
            task.cancelled = True

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ one scheduling round
    def _finish(self, task: Task, reason: str, error: Optional[str] = None) -> None:
        if task.state == "running":
            self.running.remove(task)
            self.planner.finish(task.id)
        elif task.state == "waiting" and task in self.waiting:
            self.waiting.remove(task)
        if task.state != "finished":
            self.penalizing -= task.penalizes
        task.state = "finished"
        task.finish_reason = reason
        task.error = error
        self.stats["failed" if error else "finished"] += 1

    def fail(self, task: Task, message: str) -> List[Tuple[int, int, int]]:
        """Give up ``task`` alone with an error event: what it holds goes back, the others go on
        (per-task catch of native/src/v2_runtime.cpp:33788-33797).  If even the release of what it
        holds raises, the task is still taken off the lists, so that it cannot be scheduled again."""
        if task.state == "finished":
            return []
        try:
            self._finish(task, "error", message)
        except Exception as error:                         # its own bookkeeping is what is broken
            if task in self.running:
                self.running.remove(task)
            if task in self.waiting:
                self.waiting.remove(task)
            if task.state != "finished":
                self.penalizing -= task.penalizes
            task.state, task.finish_reason = "finished", "error"
            task.error = f"{message}; while giving back what it held: {error}"
            self.stats["failed"] += 1
        return [(task.id, 0, EVENT_ERROR)]

    def fail_scheduled(self, step: "ScheduledStep", request, message: str) -> bool:
        """The step function refused the entry of ``request``: fail that task, take its entry out
        of the step.  False if the step holds no such entry."""
        for index, task in enumerate(step.tasks):
            if task.id == request:
                del step.tasks[index], step.entries[index]
                step.events.extend(self.fail(task, message))
                step.failed.append(task.id)
                return True
        return False

    def _pages_short(self, entries, chosen: List[Task], step: "ScheduledStep", extra=()) -> int:
        """``planner.pages_short`` for the step's entries (and ``extra`` ones, asked about but not
        part of the step).  A request whose own bookkeeping raises there fails alone: its entry
        leaves the step, and the question is asked again without it."""
        while True:
            try:
                return self.planner.pages_short(entries + list(extra))
            except Exception as error:
                task = self.tasks.get(getattr(error, "request", None))
                if task is None or task.state == "finished":
                    raise
                step.events.extend(self.fail(task, f"{type(error).__name__}: {error}"))
                step.failed.append(task.id)
                if task in chosen:
                    index = chosen.index(task)
                    del chosen[index], entries[index]
                extra = [entry for entry in extra if entry[0] != task.id and entry[0] != ("spare", task.id)]

    def _preempt(self, task: Task) -> None:
        self.running.remove(task)
        self.planner.finish(task.id)
        task.state = "waiting"
        task.computed = 0
        task.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(task)

    def _portion(self, task: Task, budget: int):
        n = min(task.pending, budget)
        tokens = task.tokens_from(task.computed, n)
        want = [n - 1] if n == task.pending else []
        return (task.id, tokens, want)

    def schedule(self) -> ScheduledStep:
        step = ScheduledStep([], [])
        for task in [t for t in list(self.waiting) + list(self.running) if t.cancelled]:
            self._finish(task, "cancelled")
            step.events.append((task.id, 0, EVENT_FINISHED))
        budget = self.max_batched_tokens
        chosen: List[Task] = []
        entries = []
        # the running requests in two turns: those that decode (one token each) first, then the
        # portions of prompts; a request's pending count is taken once (hundreds may be running)
        reading = []
        max_model_len = self.max_model_len
        for task in self.running:
            generated = task.generated
            known = len(task.prompt) + len(generated) + task.in_flight
            if known - task.computed != 1:           # (its ``pending``, spelt out: this loop is the hot one)
                reading.append(task)
                continue
            if budget <= 0:
                continue
            if task.in_flight:
                if len(generated) + 1 >= task.max_tokens or known >= max_model_len:
                    continue                        # it ends when that token is read: nothing more to run
                token = IN_FLIGHT
            else:
                token = generated[-1] if generated else task.prompt[-1]
            budget -= 1
            chosen.append(task)
            entries.append((task.id, [token], [0]))
        for task in reading:
            if budget <= 0:
                break
            if task.in_flight and task.ends_with_the_token_in_flight(max_model_len):
                continue
            try:
                entry = self._portion(task, budget)
            except Exception as error:
                step.events.extend(self.fail(task, f"{type(error).__name__}: {error}"))
                step.failed.append(task.id)
                continue
            budget -= len(entry[1])
            chosen.append(task)
            entries.append(entry)
        # make the step of the running requests fit, preempting the newest if it does not
        while entries and self._pages_short(entries, chosen, step):
            victim = max(self.running, key=lambda t: t.admitted_at)
            if len(self.running) == 1:
                self._finish(victim, "error", "the request does not fit the cache pool")
                step.failed.append(victim.id)
                step.events.append((victim.id, 0, EVENT_ERROR))
            else:
                self._preempt(victim)
                step.preempted.append(victim.id)
            if victim in chosen:
                index = chosen.index(victim)
                budget += len(entries[index][1])
                del chosen[index], entries[index]
        # admit waiting requests, first come first served
        admitting = 0                                   # requests of this step that take a slot when it runs
        while self.waiting and budget > 0 and self.cache.free_slots > admitting:
            task = self.waiting[0]
            if step.preempted and task.id in step.preempted:
                break                                   # just evicted: not in the same step
            whole = (task.id, range(len(task.prompt) + len(task.generated)), [])   # only its length counts
            spare = [(("spare", task.id), [0] * PAGE_SIZE, [])]
            short = self._pages_short(entries, chosen, step, [whole] + spare)
            if task.state == "finished":
                continue                                # its own bookkeeping failed: it is gone
            if short:
                if chosen or self.running:
                    break                               # wait until someone finishes
                # nothing else is live: it gets the pool to itself, or can never run
                if self.planner.pages_short([whole]):
                    self.waiting.popleft()
                    self._finish(task, "error", "the request does not fit the cache pool")
                    step.failed.append(task.id)
                    step.events.append((task.id, 0, EVENT_ERROR))
                    continue
            entry = self._portion(task, budget)
            budget -= len(entry[1])
            self.waiting.popleft()
            chosen.append(task)
            entries.append(entry)
            admitting += 1
        for task in chosen:
            if task.state == "waiting":
                task.state = "running"
                task.admitted_at = self._admissions
                self._admissions += 1
                self.running.append(task)
                self.stats["admitted"] += 1
        step.entries, step.tasks = entries, chosen
        step.in_flight = [task for task in chosen if task.in_flight]
        return step

    # ------------------------------------------------------------------ after the step ran
    def advance(self, step: ScheduledStep) -> List[Task]:
        """Account for the tokens the step computed; returns the tasks that now need a
        token sampled (those whose last known token was in the step), in entry order."""
        need = []
        for task, (_, tokens, want) in zip(step.tasks, step.entries):
            if task.computed < len(task.prompt):
                self.stats["prefill_tokens"] += len(tokens)
            else:
                self.stats["decode_tokens"] += len(tokens)
            task.computed += len(tokens)
            if want:
                need.append(task)
        self.stats["steps"] += 1
        return need

    def advance_decode(self, tasks: Sequence[Task]) -> None:
        """``advance`` for a step in which every running task decoded one token."""
        for task in tasks:
            task.computed += 1
        self.stats["decode_tokens"] += len(tasks)
        self.stats["steps"] += 1

    def accept(self, task: Task, token: int) -> List[Tuple[int, int, int]]:
        """A sampled token for ``task``: emit it, then finish on a stop token, on
        ``max_tokens`` or at the context limit (emit-then-stop order of
        native/src/v2_runtime.cpp:33775-33780)."""
        token = int(token)
        task.generated.append(token)
        if task.in_flight:
            task.in_flight -= 1
        events = [(task.id, token, EVENT_TOKEN)]
        reason = None
        if token in task.stop_tokens:
            reason = "stop"
        elif len(task.generated) >= task.max_tokens:
            reason = "length"
        elif len(task.prompt) + len(task.generated) >= self.max_model_len:
            reason = "context"
        if reason:
            self._finish(task, reason)
            events.append((task.id, 0, EVENT_FINISHED))
        return events
