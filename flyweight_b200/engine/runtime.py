"""The Python entry point, in flyweight's manner (src/flyweight/v2.py: ``V2Model`` :2188,
``V2QwenRuntime`` :3297): open a model folder, ask it for a runtime, then either call the
blocking ``generate`` or queue tasks and pump ``engine_step``.

    model = Model("path/to/folder", dtype="bfloat16")
    with model.native_runtime(context_limit=4096, parallel_sequences=8) as runtime:
        runtime.generate([1, 2, 3], 16, print)                     # greedy, blocking
        tid = runtime.task_submit([1, 2, 3], 16, stop_tokens=(7,), temperature=0.8, seed=1)
        while runtime.has_work():
            for task_id, token, kind in runtime.engine_step():     # 0 token, 1 finished,
                ...                                                # 2 error, 3 progress
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch

from ..cache.manager import PAGE_SIZE
from ..config.registry import load_config
from ..kernels import lib as kernel_lib
from ..sampling import sampler as device_sampler
from ..sampling.config import GREEDY, SamplingConfig
from .loading import load_model, parse_dtype, random_model
from .runner import ModelRunner, StepError
from .scheduler import (EVENT_ERROR, EVENT_FINISHED, EVENT_PROGRESS, EVENT_TOKEN, Scheduler, Task)


@dataclass(frozen=True)
class GenerationResult:
    """As src/flyweight/generation.py:9-24, without the text fields (token ids in, out)."""
    prompt_ids: Tuple[int, ...]
    generated_ids: Tuple[int, ...]
    finish_reason: str
    stopped_on_eos: bool
    preemptions: int = 0


@dataclass(frozen=True)
class EngineConfig:
    """The limits and switches of one runtime, in one place (no environment variables on the
    forward path).  ``context_limit``: most tokens (prompt + output) of one request;
    ``parallel_sequences``: most requests live at a time (flyweight's ``--parallel``);
    ``cache_tokens``: size of the KV pool in tokens (None: every live request at the context limit,
    plus the spare page the scheduler keeps per admission); ``max_batched_tokens``: token budget of
    one step; ``max_queued``: most requests queued and running before ``task_submit`` refuses (raised to
    ``parallel_sequences`` when that is larger); ``graph_after``: how many decode steps in a row must have
    the same batch size and table width before a graph is recorded for that shape (recording costs ten to
    thirty steps' time; a batch whose size wanders never pays it back); ``use_graphs``: CUDA graphs for steps of single tokens; ``use_plan``: the native step
    plan for the others; ``steady_decode`` / ``run_ahead``: the short ways of ``engine_step``."""
    context_limit: int = 4096
    parallel_sequences: int = 1
    cache_tokens: Optional[int] = None
    max_batched_tokens: int = 2048
    use_graphs: bool = True
    use_plan: bool = True
    steady_decode: bool = True
    run_ahead: bool = True
    max_queued: int = 256          # flyweight's queue limit (native/src/v2_runtime.cpp:32588)
    graph_after: int = 16          # decode steps of one shape in a row before a CUDA graph is recorded for it

    def __post_init__(self):
        if self.context_limit <= 0 or self.parallel_sequences <= 0 or self.max_batched_tokens <= 0:
            raise ValueError("context_limit, parallel_sequences and max_batched_tokens must be positive")
        if self.cache_tokens is not None and self.cache_tokens < PAGE_SIZE:
            raise ValueError(f"cache_tokens must hold at least one page of {PAGE_SIZE} tokens")

    @property
    def queue_limit(self) -> int:
        """Requests waiting and running together before a submit is refused: ``max_queued``, and
        never fewer than can run side by side."""
        return max(int(self.max_queued), self.parallel_sequences)

    @property
    def pool_tokens(self) -> int:
        if self.cache_tokens is not None:
            return int(self.cache_tokens)
        return self.parallel_sequences * (-(-self.context_limit // PAGE_SIZE) + 1) * PAGE_SIZE


class Model:
    """A model folder (``config.json`` + ``model.safetensors``) opened on one GPU, or a
    configuration with seeded random weights (``Model.random``)."""

    def __init__(self, path=None, dtype="bfloat16", device="cuda:0", *, _model=None):
        if _model is None:
            _model = load_model(path, dtype, device)
        self.path = path
        self.module = _model
        self.config = getattr(_model, "config", None)
        self.precision = _model.precision

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0",
               preset: str = "baseline") -> "Model":
        return cls(_model=random_model(config, seed, dtype, device, preset))

    def native_runtime(self, context_limit: int = 4096, parallel_sequences: int = 1,
                       cache_tokens: Optional[int] = None, max_batched_tokens: int = 2048,
                       config: Optional[EngineConfig] = None, **switches) -> "Runtime":
        """A runtime over this model: pass an ``EngineConfig``, or its fields by name (flyweight's
        ``native_runtime(context_limit=..., parallel_sequences=...)``, src/flyweight/v2.py:3297)."""
        if config is None:
            config = EngineConfig(context_limit=int(context_limit), parallel_sequences=max(1, int(parallel_sequences)),
                                  cache_tokens=cache_tokens, max_batched_tokens=int(max_batched_tokens),
                                  **switches)
        return Runtime(self, config)


class Runtime:
    def __init__(self, model: Model, config: EngineConfig):
        self.model = model
        self.config = config
        self.context_limit = config.context_limit
        self.parallel_sequences = config.parallel_sequences
        # the default pool has a page to spare per sequence: admission keeps one free page in hand,
        # and requests that fill the context limit must still run side by side
        self.cache_tokens = config.pool_tokens
        self.max_batched_tokens = config.max_batched_tokens
        self.runner: Optional[ModelRunner] = None
        self.scheduler: Optional[Scheduler] = None
        self._token_buffer: Optional[torch.Tensor] = None
        self._token_event = None
        self._counters = {"engine_steps": 0, "steady_steps": 0, "pipelined_steps": 0, "step_seconds": 0.0,
                          "sampling_seconds": 0.0, "d2h_bytes": 0}
        self.steady_decode = config.steady_decode    # take the short way when a step repeats the last one
        self.run_ahead = config.run_ahead            # ... and launch the step after it before reading this one's tokens
        self._ahead = None                 # a decode step already launched whose tokens were not read yet
        self._flight = None                # the same for a step of any kind (the pipelined way)
        self._token_ring = None            # pinned buffers for the sampled ids of two steps in flight
        self._health_due, self._steps_unchecked = True, 0
        # tracing hook: called as observer(tasks, logits) with the fp32 logits [len(tasks)][vocab]
        # every time tokens are about to be sampled from them (the tensor is overwritten by the
        # next step: copy what is to be kept)
        self.logits_observer: Optional[Callable] = None
        self.prepare()

    # ------------------------------------------------------------------ life cycle
    def prepare(self) -> None:
        if self.runner is not None:
            return
        self.runner = ModelRunner(self.model.module, num_pages=max(1, self.cache_tokens // PAGE_SIZE),
                                  num_slots=self.parallel_sequences,
                                  max_model_len=self.context_limit,
                                  max_batched_tokens=self.max_batched_tokens,
                                  use_graphs=self.config.use_graphs, use_plan=self.config.use_plan,
                                  graph_after=self.config.graph_after)
        self.scheduler = Scheduler(self.runner, self.max_batched_tokens, self.context_limit,
                                   self.config.queue_limit)

    def reset(self) -> None:
        """Forget every request and give back everything the cache holds."""
        self._ahead = self._flight = None
        self.runner.cache.reset()
        self.scheduler = Scheduler(self.runner, self.max_batched_tokens, self.context_limit,
                                   self.config.queue_limit)

    def close(self) -> None:
        runner, self.runner, self.scheduler = self.runner, None, None
        self._ahead = self._flight = None
        if runner is not None:
            runner.check_health()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    # ------------------------------------------------------------------ tasks
    def task_submit(self, prompt_tokens: Sequence[int], max_tokens: int,
                    stop_tokens: Sequence[int] = (), *, temperature: float = 0.0, top_k: int = 20,
                    top_p: float = 0.95, min_p: float = 0.0, repetition_penalty: float = 1.0,
                    presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
                    penalty_window: int = 64, seed: Optional[int] = None) -> int:
        """Queue a request; returns its task id (names and defaults of
        src/flyweight/v2.py:3878-3896)."""
        sampling = SamplingConfig(temperature=temperature, top_k=top_k, top_p=top_p, min_p=min_p,
                                  seed=seed, repetition_penalty=repetition_penalty,
                                  presence_penalty=presence_penalty,
                                  frequency_penalty=frequency_penalty,
                                  penalty_window=penalty_window)
        return self.scheduler.submit(prompt_tokens, max_tokens, stop_tokens, sampling)

    def task_cancel(self, task_id: int) -> None:
        self.scheduler.cancel(task_id)

    def task(self, task_id: int) -> Task:
        return self.scheduler.tasks[task_id]

    def task_error(self, task_id: int) -> Optional[str]:
        return self.scheduler.tasks[task_id].error

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._flight is not None

    def engine_step(self) -> List[Tuple[int, int, int]]:
        """One scheduling cycle: one batched model step and one token for every request
        that was due.  Returns events ``(task id, token or count, kind)``.

        Three ways, the shortest that applies: steady decoding (the same requests one token further:
        no scheduling at all, see ``_steady_step``); the pipelined way (``run_ahead``): the step
        after this one is scheduled and launched before this one's tokens are read -- the ids it
        needs are still on the device and go from the sampler's output into its batch there -- so
        the host's scheduling, packing and launching overlap the device's work; and the plain way,
        which reads every step's tokens before it plans the next."""
        started = time.perf_counter()
        if self._flight is None and (self._ahead is not None or self.steady_decode):
            events = self._steady_step()
            if events is not None:
                self._counters["steady_steps"] += 1
                self._counters["engine_steps"] += 1
                self._counters["step_seconds"] += time.perf_counter() - started
                return events
        events: List[Tuple[int, int, int]] = []
        current = self._flight
        self._flight = None
        if current is None:
            current = self._launch_scheduled(events, None)
        if current is not None:
            if self._may_pipeline(current):
                if self.scheduler.penalizing:
                    # penalties want the ids of step k on the host before step k+1 is SAMPLED, not
                    # before it is launched: launch its forward pass, read step k's ids while it
                    # runs, then queue its sampling behind it
                    launched = self._launch_scheduled(events, current, sample=False)
                    events.extend(self._accept_flight(current))
                    current = None
                    if launched is not None:
                        self._flight = self._sample_async(launched["need"], launched["logits"])
                        self._flight["graph_step"] = launched["graph_step"]
                else:
                    self._flight = self._launch_scheduled(events, current)
                if self._flight is not None:
                    self._counters["pipelined_steps"] += 1
            if current is not None:
                events.extend(self._accept_flight(current))
        self._counters["engine_steps"] += 1
        self._counters["step_seconds"] += time.perf_counter() - started
        return events

    def _launch_scheduled(self, events, after, sample=True):
        """Schedule a step, launch it and its sampling; nothing is waited for.  ``after``: the step
        launched before it whose tokens are not read yet (its requests' next ids are taken from its
        sampler's output on the device).  Returns the launched step's record, or None when the
        step samples nothing (no tokens to read: nothing to wait for later either).  ``sample``
        False: the sampling is left to the caller, who gets the requests to sample and the logits."""
        scheduler, runner = self.scheduler, self.runner
        step = scheduler.schedule()
        logits = None
        while step.entries and logits is None:
            patch = None
            if after is not None and step.in_flight:
                rows = {id(task): row for row, task in enumerate(after["tasks"])}
                patch = [(index, rows[id(task)]) for index, task in enumerate(step.tasks) if task.in_flight]
            try:
                logits = runner.step(step.entries, pages_checked=True, own_entries=True,
                                     patch_source=after["device"] if patch else None, patch=patch)
            except StepError as error:
                # the step function refuses one request's entry before anything is launched or
                # mapped: that request fails alone, the step runs without it
                if not scheduler.fail_scheduled(step, error.request, str(error)):
                    raise
        events.extend(step.events)
        if not step.entries:
            return None
        need = scheduler.advance(step)
        if len(need) != len(step.tasks):
            sampled = {id(task) for task in need}
            for task in step.tasks:
                if id(task) not in sampled:
                    events.append((task.id, task.computed, EVENT_PROGRESS))
        if not need:
            return None
        if not sample:
            return {"need": need, "logits": logits, "graph_step": runner.last_decode_graph is not None}
        flight = self._sample_async(need, logits)
        flight["graph_step"] = runner.last_decode_graph is not None
        return flight

    def _may_pipeline(self, current) -> bool:
        """Whether the step after ``current`` may be planned before ``current``'s tokens are read.
        Not when steady decoding is about to take over (the same requests, everybody decoding,
        nobody waiting): that way is shorter still and starts from a step whose tokens have been
        read."""
        if not self.run_ahead:
            return False
        scheduler = self.scheduler
        if (self.steady_decode and current.get("graph_step") and not scheduler.waiting
                and len(current["tasks"]) == len(scheduler.running)
                and self._same_requests_again() is not None):
            return False                 # (with hundreds running, somebody needs a page every step: then not)
        return True

    def _sample_async(self, need, logits):
        """Sampling (arg-max or draws) and the copy of the ids to pinned memory, both queued;
        nobody waits here.  The requests' tokens are in flight from now until ``_accept_flight``."""
        if self.logits_observer is not None:
            self.logits_observer(need, logits)
        if all(task.greedy for task in need):
            tokens = device_sampler.argmax(logits)
        else:
            uniforms = [0.0 if task.greedy else task.rng.uniform() for task in need]
            tokens = device_sampler.sample(logits, [task.sampling for task in need], uniforms,
                                           [task.generated for task in need])
        flight = self._queue_read(need, tokens)
        for task in need:
            task.in_flight += 1
        return flight

    def _accept_flight(self, flight) -> List[Tuple[int, int, int]]:
        """Wait for the ids of a launched step and hand them to their requests.  A request that
        ended meanwhile (a stop token in the step before, a cancellation, a failure) drops its id; one
        that was preempted meanwhile keeps it: it is part of its text when it is admitted again."""
        sampled = time.perf_counter()
        flight["event"].synchronize()
        host = flight["host"].tolist()
        self._counters["d2h_bytes"] += 4 * len(host)
        self._counters["sampling_seconds"] += time.perf_counter() - sampled
        if flight["health"][0] or flight["health"][1]:
            self.runner.check_health()          # kernels fail loudly: raises, for the whole engine
        events: List[Tuple[int, int, int]] = []
        for task, token in zip(flight["tasks"], host):
            if task.state == "finished":
                task.in_flight = 0
                continue
            events.extend(self._accept(task, token))
        if len(events) != len(host):
            self._health_due = True             # somebody ended (or had ended): look at the next step's words
        return events

    def _sample_and_accept(self, need, logits, events) -> None:
        sampled = time.perf_counter()
        if self.logits_observer is not None:
            self.logits_observer(need, logits)
        if all(task.greedy for task in need):
            tokens = device_sampler.argmax(logits)
        else:
            uniforms = [0.0 if task.greedy else task.rng.uniform() for task in need]
            tokens = device_sampler.sample(logits, [task.sampling for task in need], uniforms,
                                           [task.generated for task in need])
        host = self._read_tokens(tokens)              # the step's only device->host read
        self._counters["d2h_bytes"] += 4 * len(host)
        self._counters["sampling_seconds"] += time.perf_counter() - sampled
        finished = False
        for task, token in zip(need, host):
            accepted = self._accept(task, token)
            finished = finished or len(accepted) > 1
            events.extend(accepted)
        if finished:
            self.runner.check_health()          # once per finished request: kernels fail loudly

    def _accept(self, task, token) -> List[Tuple[int, int, int]]:
        """Hand a sampled token to its request.  An exception in one request's host bookkeeping
        ends that request with an error event; the others are not touched.  (A device error is
        another matter: ``check_health`` raises for the whole engine.)"""
        try:
            return self.scheduler.accept(task, token)
        except Exception as error:
            return self.scheduler.fail(task, f"{type(error).__name__}: {error}")

    # ------------------------------------------------------------------ steady decoding
    def _steady_step(self):
        """Steady decoding: nothing to schedule, no page to map, the captured graph replayed one
        position further.  The step after this one is launched as well before this one's tokens
        are read: its token ids go from the sampler's output to the embedding on the device, so the
        device does not wait for the host between steps (with penalties in the batch the next
        step's sampling, not its forward pass, waits until this step's ids have been read).  Returns the events
        of one step, or None when the next step is not a repeat of the last one."""
        current = self._ahead
        self._ahead = None
        if current is None:
            need = self._same_requests_again()
            if need is None:
                return None
            logits = self.runner.step_same_requests([task.generated[-1] for task in need])
            self.scheduler.advance_decode(need)
            if not self.run_ahead:
                events = []
                self._sample_and_accept(need, logits, events)
                return events
            current = self._sample_ahead(need, logits)
        if self.run_ahead and self.steady_decode and self._may_follow(current["tasks"]):
            logits = self.runner.step_same_requests(device_tokens=current["device"])
            self.scheduler.advance_decode(current["tasks"])
            if self.scheduler.penalizing:
                # penalties want this step's ids on the host before the next step is SAMPLED: its
                # forward pass is running, read the ids now, then queue its sampling behind it
                events = self._accept_async(current)
                self._ahead = self._sample_ahead(current["tasks"], logits)
                return events
            self._ahead = self._sample_ahead(current["tasks"], logits)
        return self._accept_async(current)

    def _may_follow(self, tasks) -> bool:
        """Whether the step after the one in flight may be launched now: the same requests go
        on (nobody waits, is cancelled, or is known to end with the token in flight), none reaches
        the limit, and those at a page's edge all find a page."""
        scheduler, runner = self.scheduler, self.runner
        if scheduler.waiting or len(scheduler.running) != len(tasks):
            return False
        cache = runner.cache
        for task, running in zip(tasks, scheduler.running):
            if task is not running or task.cancelled or len(task.generated) + 1 >= task.max_tokens:
                return False
            if cache.length(task.id) + 1 > runner.max_model_len:
                return False
            if len(task.prompt) + len(task.generated) + 1 >= self.scheduler.max_model_len:
                return False
        graph = runner.last_decode_graph
        return graph is not None and cache.room_for_one_more([task.id for task in tasks], graph.batch.width)

    def _sample_ahead(self, tasks, logits):
        """Sampling on the device (arg-max, or draws with uniform numbers taken from the requests'
        generators now: they do not depend on the tokens) and the copy of the ids to pinned memory,
        both queued; nobody waits here.  Requests with penalties are sampled with the tokens the
        host knows at this moment: the caller has read the step before."""
        if self.logits_observer is not None:
            self.logits_observer(tasks, logits)
        if all(task.greedy for task in tasks):
            tokens = device_sampler.argmax(logits)
        else:
            uniforms = [0.0 if task.greedy else task.rng.uniform() for task in tasks]
            recents = [task.generated for task in tasks] if self.scheduler.penalizing else None
            tokens = device_sampler.sample(logits, [task.sampling for task in tasks], uniforms, recents)
        return self._queue_read(tasks, tokens)

    def _queue_read(self, tasks, tokens):
        """The copy of sampled ids (int32 on the device) to one of two pinned buffers, queued."""
        if self._token_ring is None:
            self._token_ring = {"buffers": [torch.empty(256, dtype=torch.int32).pin_memory() for _ in range(2)],
                                "events": [torch.cuda.Event() for _ in range(2)], "turn": 0}
        ring = self._token_ring
        turn = ring["turn"]
        ring["turn"] = turn ^ 1
        count = tokens.numel()
        if ring["buffers"][turn].numel() < count + 2:
            ring["buffers"][turn] = torch.empty(2 * count + 2, dtype=torch.int32).pin_memory()
        buffer = ring["buffers"][turn]
        view = buffer[:count]
        view.copy_(tokens, non_blocking=True)
        # The two words of the health check (a kernel that gave up, a token id outside the
        # vocabulary) ride along behind the ids, so that a failure is known when the ids are read,
        # without a wait of its own: after every step in which a request ended, and every 32nd step
        # (two small copies more would cost a decode step of eight requests 2 % of its time).
        buffer[count] = buffer[count + 1] = 0
        self._steps_unchecked += 1
        if self._health_due or self._steps_unchecked >= 32:
            self._health_due, self._steps_unchecked = False, 0
            kernel_lib.call("fwb_health_peek_async", buffer.data_ptr() + 4 * count,
                            kernel_lib.ptr(self.runner.bad_token_flag), kernel_lib.stream())
        ring["events"][turn].record()
        return {"tasks": list(tasks), "device": tokens, "host": view, "health": buffer[count:count + 2],
                "event": ring["events"][turn]}

    def _accept_async(self, step) -> List[Tuple[int, int, int]]:
        """Wait for the ids of a launched step and hand them to their requests.  A request that
        ended while the step was in flight (a stop token in the step before, a cancellation)
        drops its id."""
        sampled = time.perf_counter()
        step["event"].synchronize()
        host = step["host"].tolist()
        self._counters["d2h_bytes"] += 4 * len(host)
        self._counters["sampling_seconds"] += time.perf_counter() - sampled
        if step["health"][0] or step["health"][1]:
            self.runner.check_health()          # kernels fail loudly: raises, for the whole engine
        events: List[Tuple[int, int, int]] = []
        for task in step["tasks"]:
            if task.cancelled and task.state == "running":     # cancelled while the step was in flight
                self.scheduler._finish(task, "cancelled")
                events.append((task.id, 0, EVENT_FINISHED))
        for task, token in zip(step["tasks"], host):
            if task.state != "running":
                continue
            events.extend(self._accept(task, token))
        if len(events) != len(host):
            self._health_due = True
        return events

    def _same_requests_again(self):
        """The running tasks, if the next step is the last one moved on by one token: nobody
        waits, everybody decodes, the last step replayed a graph for exactly these requests in
        this order, nobody reaches a limit, and those at a page's edge all find a page.  Else None."""
        scheduler, runner = self.scheduler, self.runner
        graph = runner.last_decode_graph
        tasks = scheduler.running
        if graph is None or graph.graph is None or scheduler.waiting or not tasks:
            return None
        segments = graph.batch.segments
        if len(segments) != len(tasks):
            return None
        cache = runner.cache
        for task, segment in zip(tasks, segments):
            if segment.request != task.id or task.cancelled or task.pending != 1:
                return None
            if cache.length(task.id) + 1 > runner.max_model_len:
                return None
        if not cache.room_for_one_more([task.id for task in tasks], graph.batch.width):
            return None                      # pages are short (the scheduler decides who waits) or the table outgrows the graph
        return list(tasks)

    def _read_tokens(self, tokens: torch.Tensor) -> List[int]:
        """Sampled token ids to the host through a pinned buffer (no allocation per step)."""
        count = tokens.numel()
        if self._token_buffer is None or self._token_buffer.numel() < count:
            self._token_buffer = torch.empty(max(count, 256), dtype=torch.int32).pin_memory()
            self._token_event = torch.cuda.Event()
        view = self._token_buffer[:count]
        view.copy_(tokens, non_blocking=True)
        self._token_event.record()
        self._token_event.synchronize()
        return view.tolist()

    # ------------------------------------------------------------------ blocking calls
    def generate(self, prompt_tokens: Sequence[int], max_tokens: int,
                 callback: Optional[Callable[[int], object]] = None) -> List[int]:
        """Greedy decode of one prompt to ``max_tokens`` (no stop set); ``callback(token)``
        returning False stops it (src/flyweight/v2.py:3837-3849).  Returns the tokens."""
        if not prompt_tokens:
            raise ValueError("prompt_tokens must not be empty")
        if max_tokens <= 0:
            raise ValueError("max_tokens must be positive")
        task_id = self.scheduler.submit(prompt_tokens, max_tokens, (), GREEDY)
        out: List[int] = []
        while self.scheduler.tasks[task_id].state != "finished":
            for tid, token, kind in self.engine_step():
                if tid != task_id:
                    continue
                if kind == EVENT_TOKEN:
                    out.append(token)
                    if callback is not None and callback(token) is False:
                        self.scheduler.cancel(task_id)
                elif kind == EVENT_ERROR:
                    raise RuntimeError(self.scheduler.tasks[task_id].error or "generation failed")
        return out

    def generate_batch(self, prompts: Sequence[Sequence[int]], max_tokens: int,
                       sampling: Optional[SamplingConfig] = None,
                       stop_tokens: Sequence[int] = (), seeds: Optional[Sequence[int]] = None
                       ) -> List[GenerationResult]:
        """Run several requests to the end through the scheduler; results in input order."""
        sampling = sampling or GREEDY
        ids = []
        for index, prompt in enumerate(prompts):
            cfg = sampling
            if seeds is not None:
                cfg = SamplingConfig(**{**sampling.__dict__, "seed": seeds[index]})
            ids.append(self.scheduler.submit(prompt, max_tokens, stop_tokens, cfg))
        while any(self.scheduler.tasks[i].state != "finished" for i in ids):
            self.engine_step()
        results = []
        for i in ids:
            task = self.scheduler.tasks[i]
            if task.error:
                raise RuntimeError(f"task {i}: {task.error}")
            results.append(GenerationResult(tuple(task.prompt), tuple(task.generated),
                                            task.finish_reason or "", task.finish_reason == "stop",
                                            task.preemptions))
        return results

    # ------------------------------------------------------------------ counters
    @property
    def info(self) -> Dict[str, object]:
        out: Dict[str, object] = dict(self._counters)
        out.update(self.scheduler.stats)
        out["cache"] = self.runner.cache.stats()
        out["model_steps"] = self.runner.steps
        out["tokens_run"] = self.runner.tokens_run
        out["h2d_bytes"] = self.runner.h2d_bytes
        out["graphs_recorded"] = self.runner.graphs_recorded
        out["graph_replays"] = self.runner.graph_replays
        out["graphs_held"] = len(self.runner._graphs)
        return out
