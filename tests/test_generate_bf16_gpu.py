"""bfloat16, the precision that serves, driven through the scheduler with many requests: random
workloads whose batches cross 16 live requests (where norms start to be folded into the
products), preemption with a small pool, seeded sampling, steady decoding with and without the
step launched ahead, and decoding across 1,024 tokens of context, where a second CUDA graph
(a wider block table, another split of the context) takes over.

bfloat16 may flip a near-tie against the float64 oracle, so generated tokens are not compared
with the oracle's own greedy run.  The criterion is on logits: the oracle reads the text the
engine actually produced, and at every generated position the chosen token's oracle logit must
be within the bfloat16 bound of the oracle's best."""
import random

import numpy as np
import pytest

import plain_lfm2 as P
from gpu_util import TOL_ORACLE, assert_close, model_dir, new_runner, plain_logits, plain_model, random_tokens
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
DTYPE = "bfloat16"
BOUND = 2 * TOL_ORACLE[DTYPE]          # two bfloat16 computations of a near-tie may disagree


def open_runtime(name, **kwargs):
    from flyweight_b200 import Model
    return Model(model_dir(name, DTYPE), dtype=DTYPE).native_runtime(**kwargs)


def assert_follows_its_logits(name, prompt, generated, what=""):
    """Every generated token is (nearly) the oracle's best at its position, given the text so far."""
    assert generated, f"{what}: nothing was generated"
    logits = plain_logits(name, DTYPE, list(prompt) + list(generated))
    scale = max(1.0, float(np.abs(logits).max()))
    for i, token in enumerate(generated):
        row = logits[len(prompt) - 1 + i]
        assert row.max() - row[token] <= BOUND * scale, \
            f"{what}: token {i} ({token}) is {row.max() - row[token]:.4g} below the best logit (scale {scale:.3g})"


def drain(runtime, limit=20000):
    log = []
    steps = 0
    while runtime.has_work():
        events = runtime.engine_step()
        for task, _, kind in events:
            assert kind != 2, runtime.task_error(task)
        log.extend(events)
        steps += 1
        assert steps < limit, "the runtime does not finish"
    return log


@pytest.mark.parametrize("name", ["A", "B"])
def test_random_workloads_in_bfloat16_with_up_to_twenty_live_requests(name):
    rnd = random.Random(23)
    vocab = TINY[name]["vocab_size"]
    from flyweight_b200 import Model
    model = Model(model_dir(name, DTYPE), dtype=DTYPE)
    most_live = 0
    for round_ in range(8):
        limit = rnd.choice([128, 192, 320])
        parallel = rnd.choice([3, 17, 20, 24]) if round_ else 20
        runtime = model.native_runtime(context_limit=limit, parallel_sequences=parallel,
                                       max_batched_tokens=rnd.choice([16, 48, 256]))
        requests = {}

        def submit(count):
            for _ in range(count):
                new = rnd.randint(1, 40)
                prompt = [rnd.randrange(vocab) for _ in range(min(rnd.randint(1, 90), limit - new - 1))]
                requests[runtime.task_submit(prompt, new)] = (prompt, new)

        submit(rnd.randint(1, 6) if parallel == 3 else 15)
        steps = 0
        while runtime.has_work():
            for task, _, kind in runtime.engine_step():
                assert kind != 2, runtime.task_error(task)
            steps += 1
            most_live = max(most_live, len(runtime.scheduler.running))
            if steps == 12 and parallel > 3:
                submit(rnd.randint(2, 9))               # 15 live requests become 17 and more
            assert steps < 5000, "the runtime does not finish"
        for task, (prompt, new) in requests.items():
            got = runtime.task(task).generated
            assert len(got) == new
            assert_follows_its_logits(name, prompt, got, f"{name} workload {round_}, {len(prompt)} + {new} tokens")
        assert runtime.info["cache"]["groups"][0]["pages_in_use"] == 0
        runtime.close()
    assert most_live > 16


def test_preemption_in_bfloat16():
    name = "A"
    prompts = [random_tokens(name, n, seed=160 + n) for n in (50, 60, 70)]
    with open_runtime(name, context_limit=256, parallel_sequences=3, cache_tokens=6 * 64) as runtime:
        results = runtime.generate_batch(prompts, 120)     # 3 x 170..190 tokens need 9 pages of 6
        assert runtime.info["preemptions"] > 0
    for prompt, result in zip(prompts, results):
        assert len(result.generated_ids) == 120
        assert_follows_its_logits(name, prompt, result.generated_ids, f"preempted {result.preemptions} times")


def test_seeded_sampling_in_bfloat16_draws_what_the_plain_sampler_draws():
    """The runtime's tracing hook hands over the very logits each token was sampled from.  Those
    rows must be the oracle's logits of the text so far (within the bfloat16 bound), and the plain
    sampler, given the same rows and the request's own random numbers in order, must draw the
    very tokens the engine produced: the right row reaches the right request, its generator
    advances once per token, whatever else is in the batch."""
    name = "B"
    prompts = [random_tokens(name, n, seed=140 + n) for n in (1, 7, 64, 100, 129)]
    settings = dict(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05)
    seen = {}

    def observer(tasks, logits):
        rows = logits.cpu().numpy()
        for task, row in zip(tasks, rows):
            seen.setdefault(task.id, []).append(row.copy())

    with open_runtime(name, context_limit=192, parallel_sequences=4, max_batched_tokens=16) as runtime:
        runtime.logits_observer = observer
        ids = [runtime.task_submit(p, 24, seed=7 + i, **settings) for i, p in enumerate(prompts)]
        drain(runtime)
        texts = [runtime.task(i).generated for i in ids]
    for i, (tid, prompt, generated) in enumerate(zip(ids, prompts, texts)):
        assert len(generated) == 24 and len(seen[tid]) == 24
        want = plain_logits(name, DTYPE, prompt + generated)[len(prompt) - 1:-1]
        assert_close(np.stack(seen[tid]), want, TOL_ORACLE[DTYPE], f"request {i}: the logits it was sampled from")
        rng = P.XorShift64Star(7 + i)
        drawn = [P.sample(row, rng=rng, **settings) for row in seen[tid]]
        assert drawn == generated, f"request {i}"


def test_steady_decoding_and_the_step_launched_ahead_in_bfloat16():
    """Steady decoding replays the graph the long way would have replayed, so in bfloat16 too the
    tokens are the same with it, with the next step launched ahead, and without either."""
    name = "B"
    prompts = [random_tokens(name, n, seed=180 + n) for n in (30, 61, 64, 100)]

    def run(steady, ahead):
        with open_runtime(name, context_limit=256, parallel_sequences=4, graph_after=0) as runtime:
            runtime.steady_decode = steady
            runtime.run_ahead = ahead
            ids = [runtime.task_submit(p, 40 + 17 * i) for i, p in enumerate(prompts)]
            log = drain(runtime)
            return [runtime.task(i).generated for i in ids], log, runtime.info["steady_steps"]

    slow, slow_log, none = run(False, False)
    steady, steady_log, steady_steps = run(True, False)
    ahead, ahead_log, ahead_steps = run(True, True)
    assert none == 0 and steady_steps > 40 and ahead_steps > 40
    assert steady == slow and steady_log == slow_log
    assert ahead == slow and ahead_log == slow_log
    for prompt, generated in zip(prompts, slow):
        assert_follows_its_logits(name, prompt, generated, "steady decoding")


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "bfloat16")])
def test_decoding_across_1024_tokens_of_context_changes_the_graph(name, dtype):
    """Decode graphs are keyed by the block-table width rounded up to 16 pages.  Two requests
    decode together, one of them from position 1,000 to 1,060: at 1,024 tokens its table grows to
    17 pages, a second graph is recorded, and the context is cut into other slices.  Logits on
    both sides of the edge against the oracle."""
    runner = new_runner(name, dtype, num_pages=24, num_slots=2, max_model_len=1100)
    long_tokens = random_tokens(name, 1060, seed=5)
    short_tokens = random_tokens(name, 40 + 60, seed=6)
    want_long = plain_logits(name, dtype, long_tokens)
    want_short = plain_logits(name, dtype, short_tokens)
    runner.step([("long", long_tokens[:1000], []), ("short", short_tokens[:40], [])])
    got_long, got_short = [], []
    for i in range(60):
        out = runner.step([("long", [long_tokens[1000 + i]], [0]), ("short", [short_tokens[40 + i]], [0])])
        out = out.cpu().numpy()
        got_long.append(out[0])
        got_short.append(out[1])
    assert sorted(runner._graphs) == [(2, 16), (2, 32)]
    assert runner.graph_replays >= 56
    assert_close(np.stack(got_long), want_long[1000:], TOL_ORACLE[dtype], f"{name} {dtype}: across the bucket edge")
    assert_close(np.stack(got_short), want_short[40:], TOL_ORACLE[dtype], f"{name} {dtype}: its short neighbour")
    runner.finish("long")
    runner.finish("short")
    runner.cache.check()
    runner.check_health()


def test_a_request_generated_across_1024_tokens_through_the_runtime():
    name = "A"
    prompt = random_tokens(name, 990, seed=9)
    other = random_tokens(name, 20, seed=10)
    with open_runtime(name, context_limit=1100, parallel_sequences=2, max_batched_tokens=512) as runtime:
        ids = [runtime.task_submit(prompt, 70), runtime.task_submit(other, 90)]
        drain(runtime)
        texts = [runtime.task(i).generated for i in ids]
        assert len(runtime.runner._graphs) >= 2
    assert_follows_its_logits(name, prompt, texts[0], "across 1,024 tokens")
    assert_follows_its_logits(name, other, texts[1], "its neighbour")
