"""Generation through the Python entry point and the command line: greedy tokens against the
plain implementation, seeded sampling against the plain sampler, preemption without a change
of output."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_lfm2 as P
from gpu_util import model_dir, plain_logits, plain_model, random_tokens
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def open_runtime(name, dtype, **kwargs):
    from flyweight_b200 import Model
    return Model(model_dir(name, dtype), dtype=dtype).native_runtime(**kwargs)


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_equals_the_plain_implementation(name):
    cfg, w = plain_model(name, "float32")
    prompts = [random_tokens(name, n, seed=20 + n) for n in (5, 17, 33)]
    with open_runtime(name, "float32", context_limit=128, parallel_sequences=3) as runtime:
        seen = []
        first = runtime.generate(prompts[0], 16, seen.append)
        assert first == seen == P.greedy_generate(cfg, w, prompts[0], 16)
        results = runtime.generate_batch(prompts, 16)
        for prompt, result in zip(prompts, results):
            assert list(result.generated_ids) == P.greedy_generate(cfg, w, prompt, 16)
            assert result.finish_reason == "length"
        info = runtime.info
        assert info["cache"]["groups"][0]["pages_in_use"] == 0 and info["decode_tokens"] > 0


def test_bfloat16_generation_follows_its_own_logits():
    """bfloat16 may flip a near-tie against the oracle, so the check is on logits: at every
    generated position the chosen token's oracle logit is within the bfloat16 bound of the
    oracle's best."""
    name, dtype = "B", "bfloat16"
    prompt = random_tokens(name, 40, seed=3)
    with open_runtime(name, dtype, context_limit=128, parallel_sequences=1) as runtime:
        tokens = runtime.generate(prompt, 12)
    logits = plain_logits(name, dtype, prompt + tokens)
    scale = max(1.0, np.abs(logits).max())
    for i, token in enumerate(tokens):
        row = logits[len(prompt) - 1 + i]
        assert row.max() - row[token] <= 2 * 10 * 2.0 ** -9 * scale


def test_callback_returning_false_stops_and_stop_tokens_end_a_task():
    cfg, w = plain_model("A", "float32")
    prompt = random_tokens("A", 9, seed=1)
    expected = P.greedy_generate(cfg, w, prompt, 8)
    with open_runtime("A", "float32", context_limit=64, parallel_sequences=2) as runtime:
        got = []
        runtime.generate(prompt, 8, lambda t: (got.append(t), len(got) < 3)[1])
        assert got == expected[:3]
        tid = runtime.task_submit(prompt, 8, stop_tokens=(expected[4],))
        events = []
        while runtime.has_work():
            events.extend(runtime.engine_step())
        tokens = [t for i, t, kind in events if i == tid and kind == 0]
        stop_at = expected.index(expected[4])
        assert tokens == expected[:stop_at + 1] and runtime.task(tid).finish_reason == "stop"
        assert (tid, 0, 1) in events


def test_seeded_sampling_equals_the_plain_sampler_and_ignores_batching():
    name = "B"
    cfg, w = plain_model(name, "float32")
    prompts = [random_tokens(name, n, seed=40 + n) for n in (1, 7, 64, 100, 129)]
    settings = dict(temperature=0.8, top_k=40, top_p=0.95, min_p=0.05)

    def plain_run(prompt, seed, count):
        rng = P.XorShift64Star(seed)
        text, out = list(prompt), []
        for _ in range(count):
            token = P.sample(P.forward(cfg, w, text)[-1].astype(np.float32), rng=rng, **settings)
            out.append(token)
            text.append(token)
        return out

    with open_runtime(name, "float32", context_limit=192, parallel_sequences=4,
                      max_batched_tokens=16) as runtime:       # prompts enter in portions of <= 16
        ids = [runtime.task_submit(p, 24, seed=7 + i, **settings) for i, p in enumerate(prompts)]
        while runtime.has_work():
            runtime.engine_step()
        batched = [runtime.task(i).generated for i in ids]
        solo = []
        for i, p in enumerate(prompts[:2]):
            tid = runtime.task_submit(p, 24, seed=7 + i, **settings)
            while runtime.has_work():
                runtime.engine_step()
            solo.append(runtime.task(tid).generated)
    assert batched[:2] == solo                                # same seed, same tokens, alone or not
    # against the oracle: equal as long as no near-tie in float32 vs float64 decides a draw
    for i in (0, 1, 2):
        assert batched[i] == plain_run(prompts[i], 7 + i, 24)


def test_preemption_does_not_change_the_output():
    name = "A"
    prompts = [random_tokens(name, n, seed=60 + n) for n in (50, 60, 70)]
    with open_runtime(name, "float32", context_limit=256, parallel_sequences=3,
                      cache_tokens=3 * 256) as runtime:
        roomy = [list(r.generated_ids) for r in runtime.generate_batch(prompts, 120)]
        assert runtime.info["preemptions"] == 0
    with open_runtime(name, "float32", context_limit=256, parallel_sequences=3,
                      cache_tokens=6 * 64) as runtime:         # 3 x 170..190 tokens need 9 pages
        results = runtime.generate_batch(prompts, 120)
        assert runtime.info["preemptions"] > 0
        assert sum(r.preemptions for r in results) == runtime.info["preemptions"]
    assert [list(r.generated_ids) for r in results] == roomy


def test_command_line_generate_and_inspect():
    cfg, w = plain_model("A", "float32")
    prompt = random_tokens("A", 6, seed=2)
    run = lambda *args: subprocess.run([sys.executable, "-m", "flyweight_b200", *args], cwd=ROOT,
                                       capture_output=True, text=True, timeout=600)
    proc = run("generate", str(model_dir("A", "float32")), "--prompt", ",".join(map(str, prompt)),
               "--max-tokens", "5", "--temperature", "0", "--dtype", "float32")
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [int(t) for t in proc.stdout.split()] == P.greedy_generate(cfg, w, prompt, 5)
    proc = run("inspect", str(model_dir("A", "float32")))
    assert proc.returncode == 0 and '"ffn_dim": 192' in proc.stdout


def test_the_steady_decode_shortcut_changes_nothing():
    """When a step has the same requests as the last one and nobody needs a page, the runtime
    skips scheduling and replays the captured graph one position further.  Same tokens as the
    long way, sampled or greedy, across page edges and with requests that end at different times."""
    name = "B"
    prompts = [random_tokens(name, n, seed=80 + n) for n in (30, 61, 64, 100)]
    settings = dict(temperature=0.7, top_k=30, top_p=0.9, min_p=0.02)

    def run(steady):
        with open_runtime(name, "float32", context_limit=256, parallel_sequences=4, graph_after=0) as runtime:
            runtime.steady_decode = steady
            ids = [runtime.task_submit(p, 40 + 17 * i, seed=3 + i, **(settings if i % 2 else {}))
                   for i, p in enumerate(prompts)]
            while runtime.has_work():
                runtime.engine_step()
            return [runtime.task(i).generated for i in ids], runtime.info["steady_steps"]

    fast, steady_steps = run(True)
    slow, none = run(False)
    assert fast == slow
    assert steady_steps > 40 and none == 0


def test_launching_the_next_step_before_reading_this_one_changes_nothing():
    """Greedy requests in steady decoding: the runtime launches step k+1, fed on the device from
    the sampler of step k, before it reads step k's tokens.  Requests that end on a stop token
    (seen one step late), on their token count, across page edges, and one that is cancelled
    half way must produce the same tokens and events as without it."""
    name = "A"
    prompts = [random_tokens(name, n, seed=90 + n) for n in (20, 50, 63, 90)]

    def run(ahead, stop):
        with open_runtime(name, "float32", context_limit=256, parallel_sequences=4, graph_after=0) as runtime:
            runtime.run_ahead = ahead
            ids = [runtime.task_submit(p, 60 + 13 * i, stop) for i, p in enumerate(prompts)]
            log = []
            steps = 0
            while runtime.has_work():
                log.extend(runtime.engine_step())
                steps += 1
                if steps == 30:
                    runtime.task_cancel(ids[1])
            return [runtime.task(i).generated for i in ids], log, runtime.info["steady_steps"]

    plain, _, _ = run(False, ())
    # a token that request 2 produces half way becomes everybody's stop token
    stop = (plain[2][25],)
    slow, slow_log, _ = run(False, stop)
    fast, fast_log, steady = run(True, stop)
    assert fast == slow and fast_log == slow_log
    assert steady > 20
    assert len(slow[2]) <= 26 and any(len(a) < len(b) for a, b in zip(slow, plain))


@pytest.mark.parametrize("name", ["A", "B"])
def test_random_workloads_through_the_runtime(name):
    """A few dozen random workloads (how many requests at a time, how many pages, which token
    budget, which lengths are all drawn): every request's greedy tokens equal the plain
    implementation's, whatever the scheduler made of them (portions, mixed steps, graphs,
    steady decoding one step ahead, pages used again)."""
    import random
    cfg, w = plain_model(name, "float32")
    rnd = random.Random(17)
    from flyweight_b200 import Model
    model = Model(model_dir(name, "float32"), dtype="float32")
    checked = 0
    for _ in range(12):
        limit = rnd.choice([128, 192, 320])
        runtime = model.native_runtime(context_limit=limit, parallel_sequences=rnd.choice([1, 2, 3, 4]),
                                       max_batched_tokens=rnd.choice([16, 48, 256]))
        requests = {}
        for _ in range(rnd.randint(1, 6)):
            new = rnd.randint(1, 40)
            prompt = [rnd.randrange(cfg["vocab_size"]) for _ in range(min(rnd.randint(1, 90), limit - new - 1))]
            requests[runtime.task_submit(prompt, new)] = (prompt, new, [])
        steps = 0
        while runtime.has_work():
            for task, token, kind in runtime.engine_step():
                assert kind != 2, runtime.task_error(task)
                if kind == 0:
                    requests[task][2].append(token)
            steps += 1
            assert steps < 5000, "the runtime does not finish"
        runtime.close()
        for prompt, new, got in requests.values():
            want = P.greedy_generate(cfg, w, prompt, new)
            if got != want:
                # 32-bit against float64: only a near-tie between the two best logits may differ
                k = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), min(len(got), len(want)))
                top = np.sort(P.forward(cfg, w, prompt + want[:k])[-1])[-2:]
                assert len(got) == len(want) and top[1] - top[0] <= 1e-4 * max(1.0, abs(top[1])), \
                    f"{name}: request of {len(prompt)} + {new} tokens: got {got}, want {want}"
            checked += 1
    assert checked >= 12


def test_one_bad_request_fails_alone():
    """A request whose text is damaged after it was queued (a token id outside the vocabulary: the
    step function refuses the entry before anything is launched), and one whose host bookkeeping
    raises when its token is accepted: each ends with an error event and its message, what it held
    goes back, and the other requests produce the tokens they produce without them."""
    name = "A"
    cfg, w = plain_model(name, "float32")
    prompts = [random_tokens(name, n, seed=70 + n) for n in (12, 30, 45, 9)]
    with open_runtime(name, "float32", context_limit=128, parallel_sequences=4,
                      max_batched_tokens=16) as runtime:
        ids = [runtime.task_submit(p, 10) for p in prompts]
        runtime.task(ids[1]).prompt[20] = cfg["vocab_size"] + 5      # reached in its second portion
        runtime.task(ids[3]).stop_tokens = None                      # `token in None` raises
        events = []
        steps = 0
        while runtime.has_work():
            events.extend(runtime.engine_step())
            steps += 1
            assert steps < 500
        assert events.count((ids[1], 0, 2)) == 1 and events.count((ids[3], 0, 2)) == 1
        assert "outside" in runtime.task_error(ids[1])
        assert "TypeError" in runtime.task_error(ids[3])
        for i in (0, 2):
            assert runtime.task(ids[i]).generated == P.greedy_generate(cfg, w, prompts[i], 10)
            assert runtime.task_error(ids[i]) is None
        info = runtime.info
        assert info["failed"] == 2 and info["cache"]["slots_in_use"] == 0
        assert info["cache"]["groups"][0]["pages_in_use"] == 0
        # the runtime goes on serving
        assert runtime.generate(prompts[0], 10) == P.greedy_generate(cfg, w, prompts[0], 10)


def test_penalties_with_the_whole_vocabulary_as_candidates_run_to_the_end():
    """top_k 0 (every token a candidate) or above 1,024 together with penalties: accepted at
    submit and sampled on the device like any other request, beside a greedy neighbour."""
    name = "B"
    cfg, w = plain_model(name, "float32")
    prompts = [random_tokens(name, n, seed=75 + n) for n in (8, 20, 14)]
    with open_runtime(name, "float32", context_limit=96, parallel_sequences=3) as runtime:
        a = runtime.task_submit(prompts[0], 30, temperature=0.7, top_k=0, top_p=0.9, min_p=0.0, seed=4,
                                repetition_penalty=1.4, frequency_penalty=0.3)
        b = runtime.task_submit(prompts[1], 30)
        c = runtime.task_submit(prompts[2], 30, temperature=0.0, top_k=0, repetition_penalty=2.0,
                                presence_penalty=1.0)
        steps = 0
        while runtime.has_work():
            for task, _, kind in runtime.engine_step():
                assert kind != 2, runtime.task_error(task)
            steps += 1
            assert steps < 200
        assert len(runtime.task(a).generated) == 30 and len(runtime.task(c).generated) == 30
        assert runtime.task(b).generated == P.greedy_generate(cfg, w, prompts[1], 30)
        # greedy under a strong repetition penalty does not settle into a loop of one token
        tail = runtime.task(c).generated[-10:]
        assert len(set(tail)) > 1


@pytest.mark.parametrize("name", ["A", "B"])
def test_planning_the_next_step_before_this_one_is_read_changes_nothing(name):
    """The pipelined way of ``engine_step``: prompts in portions beside decoding requests, sampled
    and greedy requests, stop tokens (seen one step late), a cancellation, requests that end on their
    token count, a pool so small that requests are preempted while a token of theirs is in flight.
    Every request's tokens and its reason to finish equal the plain way's."""
    import random
    rnd = random.Random(5)
    vocab = TINY[name]["vocab_size"]
    prompts = [[rnd.randrange(vocab) for _ in range(n)] for n in (3, 70, 20, 130, 64, 1, 45, 90)]
    settings = dict(temperature=0.9, top_k=50, top_p=0.95, min_p=0.0)

    def run(ahead, stop, cache_tokens):
        with open_runtime(name, "float32", context_limit=320, parallel_sequences=5, max_batched_tokens=48,
                          cache_tokens=cache_tokens, run_ahead=ahead, steady_decode=ahead) as runtime:
            ids = [runtime.task_submit(p, 40 + 12 * i, stop, seed=11 + i, **(settings if i % 3 == 0 else
                                                                          dict(temperature=0.0)))
                   for i, p in enumerate(prompts)]
            steps = 0
            while runtime.has_work():
                runtime.engine_step()
                steps += 1
                if steps == 25:
                    runtime.task_cancel(ids[3])
                assert steps < 3000
            info = runtime.info
            assert info["cache"]["groups"][0]["pages_in_use"] == 0 and info["cache"]["slots_in_use"] == 0
            tasks = [runtime.task(i) for i in ids]
            return ([t.generated for t in tasks], [t.finish_reason for t in tasks], info)

    plain, _, _ = run(False, (), None)
    stop = (plain[1][12], plain[6][20])
    for cache_tokens in (None, 6 * 64):
        slow, slow_reasons, slow_info = run(False, stop, cache_tokens)
        fast, fast_reasons, fast_info = run(True, stop, cache_tokens)
        assert fast_info["pipelined_steps"] > 20 and slow_info["pipelined_steps"] == 0
        if cache_tokens is None:
            # the same schedule in both ways: the same tokens, bit for bit
            assert fast == slow and fast_reasons == slow_reasons
            assert "stop" in fast_reasons and "cancelled" in fast_reasons and "length" in fast_reasons
        else:
            # a small pool: the two ways preempt at different moments (a request that ends on a stop
            # token holds its pages one step longer in the pipelined way), so recomputed prompts may
            # differ in the last bits; greedy requests still produce the plain implementation's tokens
            assert fast_info["preemptions"] > 0
            cfg, w = plain_model(name, "float32")
            for i, prompt in enumerate(prompts):
                if i % 3 and fast_reasons[i] == "length":
                    assert fast[i] == P.greedy_generate(cfg, w, prompt, len(fast[i]))


def test_a_graph_is_recorded_only_for_a_batch_that_stays():
    """Recording a CUDA graph costs ten to thirty decode steps, so the runtime records one for a
    (batch size, table width) only after 16 decode steps in a row have had that shape; a batch whose
    size changes every few steps runs through the native plan and records none.  Same tokens."""
    name = "A"
    cfg, w = plain_model(name, "float32")
    prompts = [random_tokens(name, n, seed=300 + n) for n in (9, 14, 11)]
    with open_runtime(name, "float32", context_limit=128, parallel_sequences=3) as runtime:
        assert runtime.config.graph_after == 16
        ids = [runtime.task_submit(p, n) for p, n in zip(prompts, (50, 12, 6))]    # 3, then 2, then 1 decoding
        seen = []
        while runtime.has_work():
            runtime.engine_step()
            seen.append(sorted(runtime.runner._graphs))
        for i, p, n in zip(ids, prompts, (50, 12, 6)):
            assert runtime.task(i).generated == P.greedy_generate(cfg, w, p, n)
        assert seen[10] == [] and seen[-1] == [(1, 16)]       # three and two together never lasted 16 steps
        assert runtime.info["steady_steps"] > 10 and runtime.info["graphs_recorded"] == 1


def test_a_kernel_that_gave_up_is_noticed_while_requests_keep_running():
    """The two words of the health check ride behind the sampled ids (after a step in which a request
    ended, and every 32nd step), so a failure is raised without a wait of its own: here the status
    word is set by the self-test kernel (a bounded wait on a barrier nobody arrives on) while two
    requests decode, and the engine raises within the next 33 steps."""
    from flyweight_b200.kernels import KernelError, lib, tensorcore
    from flyweight_b200.kernels.lib import stream
    name = "A"
    prompts = [random_tokens(name, n, seed=400 + n) for n in (10, 12)]
    runtime = open_runtime(name, "float32", context_limit=256, parallel_sequences=2)
    try:
        for p in prompts:
            runtime.task_submit(p, 200)
        for _ in range(40):
            runtime.engine_step()
        assert tensorcore.status() == 0
        lib.call("fwb_selftest_bounded_wait", 91, stream())
        with pytest.raises(KernelError, match="gave up"):
            for _ in range(34):
                runtime.engine_step()
    finally:
        assert tensorcore.status() == 0          # the check that raised has read and cleared the word
        runtime.runner = None                    # (closing would run the health check once more)


def windowed_toy_architecture():
    """Defined only here, from the framework's own parts (so its decode steps are recorded as graphs):
    two attention layers, the first with a sliding window of 70 keys and so with pages of its own."""
    from flyweight_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from flyweight_b200.parts.model import DecoderModel

    class WindowConfig:
        architectures = ("ToyWindowForCausalLM",)

        def __init__(self, raw):
            self.raw = dict(raw)

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

        def to_dict(self):
            return dict(self.raw)

        def model_spec(self):
            H, V = self.raw["hidden_size"], self.raw["vocab_size"]
            norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-5}, {"weight": name})
            attn = lambda i, window: PartSpec("gqa_attention", {
                "hidden_size": H, "num_heads": 2, "num_kv_heads": 1, "head_dim": H // 2, "qk_norm_eps": 1e-5,
                "window": window, "position": PartSpec("rope_half_split", {"theta": 100.0, "rotary_dim": H // 2})},
                {k: f"l{i}.attn.{k}" for k in ("q", "k", "v", "o", "q_norm", "k_norm")})
            ffn = lambda i: PartSpec("swiglu", {"hidden_size": H, "ffn_dim": 2 * H},
                                     {"gate": f"l{i}.gate", "up": f"l{i}.up", "down": f"l{i}.down"})
            layers = tuple(LayerSpec("prenorm_residual", norm(f"l{i}.n1"), attn(i, window), norm(f"l{i}.n2"), ffn(i))
                           for i, window in enumerate((self.raw["window"], 0)))
            return ModelSpec("ToyWindowForCausalLM", H, V, 512, "embed", norm("final"), None, layers,
                             (ScheduleEntry(0), ScheduleEntry(1)))

    class ToyWindowForCausalLM(DecoderModel):
        def __init__(self, config, precision, device):
            self.config = config
            super().__init__(config.model_spec(), precision, device)

    register_architecture("ToyWindowForCausalLM", WindowConfig, ToyWindowForCausalLM)
    return {"architectures": ["ToyWindowForCausalLM"], "hidden_size": 32, "vocab_size": 50, "window": 70}


def test_steady_decoding_with_a_sliding_window(tmp_path):
    """A model with a window group goes the short ways too: the graph is replayed for the same requests
    while the window hands pages back and page edges bring new ones.  Same tokens as the long way, and
    the window's group holds fewer pages than the group that keeps every key."""
    from flyweight_b200 import Model
    from tiny_configs import make_model_dir
    folder = make_model_dir(tmp_path / "toy_window", windowed_toy_architecture(), seed=4, dtype=torch.float32)
    rng = np.random.default_rng(5)
    prompts = [[int(t) for t in rng.integers(0, 50, size=n)] for n in (30, 100, 130)]
    settings = dict(temperature=0.9, top_k=0, top_p=0.95)

    def run(steady):
        with Model(folder, dtype="float32").native_runtime(context_limit=512, parallel_sequences=3,
                                                           graph_after=0) as runtime:
            assert runtime.runner.model.graph_safe
            runtime.steady_decode = steady
            ids = [runtime.task_submit(p, 200 + 10 * i, seed=11 + i, **(settings if i else {}))
                   for i, p in enumerate(prompts)]
            groups = runtime.runner.cache.groups
            assert [g.window for g in groups] == [70, 0]
            windowed = kept = 0
            while runtime.has_work():
                runtime.engine_step()
                windowed, kept = max(windowed, groups[0].pool.n_used), max(kept, groups[1].pool.n_used)
                runtime.runner.cache.check()
            assert groups[0].pool.n_used == 0 and groups[1].pool.n_used == 0
            return [runtime.task(i).generated for i in ids], runtime.info["steady_steps"], windowed, kept

    fast, steady_steps, windowed, kept = run(True)
    slow, none, windowed_slow, kept_slow = run(False)
    assert fast == slow and [len(g) for g in fast] == [200, 210, 220]
    assert steady_steps > 150 and none == 0
    assert windowed <= 9 < kept == kept_slow              # three requests, at most three pages of a window each
