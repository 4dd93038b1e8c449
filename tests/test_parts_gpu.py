"""Each part alone against the plain implementation's function for that part, and the
generality of the layer description: a toy mixer with state of its own that a test defines
and registers, a layer that runs twice, and a layer that reads another layer's cache."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda:0")


def tensors_for(part, seed, dtype=torch.float32):
    from flyweight_b200.weights import random_tensors
    return random_tensors(part.declare(), seed, "unit", dtype, "cpu")


def as_numpy(tensors):
    return {k: v.double().numpy() for k, v in tensors.items()}


def simple_batch(lengths_new, lengths_old, n_groups=1, slots=None):
    """A StepContext for segments with ``lengths_old`` cached tokens and ``lengths_new`` new
    ones; pages are handed out in order."""
    from flyweight_b200.engine import Segment, StepBatch, StepContext
    segments, tables, page = [], [], 0
    for i, (n, old) in enumerate(zip(lengths_new, lengths_old)):
        segments.append(Segment(f"s{i}", slots[i] if slots else i, old, [0] * n, []))
        count = -(-(old + n) // 64)
        tables.append(list(range(page, page + count)))
        page += count
    width = max(len(t) for t in tables)
    rows = [t + [-1] * (width - len(t)) for t in tables]
    return StepBatch(segments, [rows] * n_groups, DEV), page


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_rmsnorm_part(dtype):
    from flyweight_b200.config import PartSpec
    from flyweight_b200.engine import StepContext
    from flyweight_b200.parts import Precision, build_norm
    part = build_norm(PartSpec("rmsnorm", {"size": 100, "eps": 1e-4}, {"weight": "n.weight"}))
    tensors = tensors_for(part, 1)
    precision = Precision(dtype)
    part.bind(tensors.__getitem__, precision, DEV)
    x = torch.randn(7, 100)
    got = part.forward(StepContext(None, precision, DEV), x.to(DEV))
    want = P.rms_norm(x.double().numpy(), as_numpy(tensors)["n.weight"], 1e-4)
    np.testing.assert_allclose(got.double().cpu().numpy(), want,
                               atol=1e-5 if dtype == "float32" else 2 ** -7 * np.abs(want).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,F", [(64, 192), (96, 320), (40, 72)])
def test_swiglu_part(dtype, H, F):
    from flyweight_b200.config import PartSpec
    from flyweight_b200.engine import StepContext
    from flyweight_b200.parts import Precision, build_feed_forward
    part = build_feed_forward(PartSpec(
        "swiglu", {"hidden_size": H, "ffn_dim": F},
        {"gate": "f.feed_forward.w1.weight", "up": "f.feed_forward.w3.weight",
         "down": "f.feed_forward.w2.weight"}))
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = tensors_for(part, 2, stored)
    precision = Precision(dtype)
    part.bind(tensors.__getitem__, precision, DEV)
    h = torch.randn(9, H).to(stored)
    got = part.forward(StepContext(None, precision, DEV), h.to(DEV))
    want = P.swiglu(h.double().numpy(), as_numpy(tensors), "f.")
    assert got.dtype == torch.float32
    tol = 1e-5 if dtype == "float32" else 2 ** -6
    assert np.abs(got.double().cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,L,bias", [(64, 3, False), (96, 4, True)])
def test_short_conv_part_carries_its_state_across_portions(dtype, H, L, bias):
    from flyweight_b200.cache import CacheManager
    from flyweight_b200.config import PartSpec
    from flyweight_b200.engine import StepContext
    from flyweight_b200.parts import Precision, build_mixer
    names = {"in_proj": "c.conv.in_proj.weight", "taps": "c.conv.conv.weight",
             "out_proj": "c.conv.out_proj.weight"}
    if bias:
        names["bias"] = "c.conv.conv.bias"
    part = build_mixer(PartSpec("gated_short_conv", {"hidden_size": H, "taps": L, "bias": bias}, names))
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = tensors_for(part, 3, stored)
    precision = Precision(dtype)
    part.bind(tensors.__getitem__, precision, DEV)
    cache = CacheManager([part.state_spec()], 4, 3, precision.cache_dtype, DEV)
    h = torch.randn(40, H).to(stored)
    want = P.shortconv_mixer(h.double().numpy(), as_numpy(tensors), "c.", taps_len=L, has_bias=bias)
    outs, pos = [], 0
    for n in (1, 2, L - 1, 17, 1, 40):
        n = min(n, 40 - pos)
        if n <= 0:
            break
        batch, _ = simple_batch([n], [pos], slots=[2])
        outs.append(part.forward(StepContext(batch, precision, DEV), h[pos:pos + n].to(DEV),
                                 cache.layer_caches[0]))
        pos += n
    got = torch.cat(outs).double().cpu().numpy()
    tol = 1e-5 if dtype == "float32" else 2 ** -6
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,nh,nkv,hd,theta,eps", [(64, 4, 2, 16, 1e4, 1e-5), (96, 3, 1, 32, 1e6, 1e-6),
                                                   (160, 2, 2, 80, 100.0, 1e-5)])
def test_attention_part_over_portions(dtype, H, nh, nkv, hd, theta, eps):
    from flyweight_b200.cache import CacheManager
    from flyweight_b200.config import PartSpec
    from flyweight_b200.engine import StepContext
    from flyweight_b200.parts import Precision, build_mixer
    names = {k: f"a.self_attn.{v}.weight" for k, v in
             dict(q="q_proj", k="k_proj", v="v_proj", o="out_proj", q_norm="q_layernorm",
                  k_norm="k_layernorm").items()}
    part = build_mixer(PartSpec("gqa_attention", {
        "hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qk_norm_eps": eps,
        "position": PartSpec("rope_half_split", {"theta": theta, "rotary_dim": hd}), "window": 0}, names))
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    tensors = tensors_for(part, 4, stored)
    precision = Precision(dtype)
    part.bind(tensors.__getitem__, precision, DEV)
    part.prepare(512, DEV)
    cache = CacheManager([part.state_spec()], 4, 2, precision.cache_dtype, DEV)
    T = 150
    h = torch.randn(T, H).to(stored)
    want = P.attention_mixer(h.double().numpy(), as_numpy(tensors), "a.", n_heads=nh, n_kv_heads=nkv,
                             head_dim=hd, eps=eps, theta=theta)
    outs, pos = [], 0
    for n in (70, 1, 1, 60, 2, 16):
        batch, _ = simple_batch([n], [pos])
        outs.append(part.forward(StepContext(batch, precision, DEV), h[pos:pos + n].to(DEV),
                                 cache.layer_caches[0]))
        pos += n
    got = torch.cat(outs).double().cpu().numpy()
    tol = 1e-5 if dtype == "float32" else 2 ** -6
    assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())


# ------------------------------------------------------------------ generality of the description
def toy_architecture():
    """A toy architecture defined entirely here: its mixer keeps a running sum of its inputs in
    a fixed-size state slot (``y_t = W (s + x_0 + ... + x_t) / (count)`` would need a count;
    this one decays: s_t = 0.5 * s_{t-1} + x_t, y_t = W s_t).  It is registered, built and
    stepped through the framework's registries, model, cache manager and step function."""
    from flyweight_b200.config import (LayerSpec, ModelSpec, PartSpec, ScheduleEntry,
                                       register_architecture)
    from flyweight_b200.parts import FixedState, Mixer, register_mixer
    from flyweight_b200.parts.model import DecoderModel
    from flyweight_b200.weights import TensorDecl

    @register_mixer("toy_decay")
    class ToyDecay(Mixer):
        def __init__(self, spec):
            super().__init__(spec)
            self.hidden = int(self.params["hidden_size"])
            self.decay = float(self.params["decay"])

        def declare(self):
            return {self.names["w"]: TensorDecl((self.hidden, self.hidden))}

        def bind(self, get, precision, device):
            self.w = get(self.names["w"]).to(device=device, dtype=torch.float32)

        def state_spec(self):
            return FixedState((self.hidden,), dtype=torch.float64)     # a state that is not fp32

        def forward(self, ctx, h, cache):
            out = torch.empty(h.shape, dtype=torch.float32, device=h.device)
            start = 0
            for seg in ctx.batch.segments:          # test code: plain torch, token by token
                s = cache.state[seg.slot]
                for t in range(start, start + len(seg.tokens)):
                    assert s.dtype == torch.float64
                    s.mul_(self.decay).add_(h[t].double())
                    out[t] = self.w @ s.float()
                start += len(seg.tokens)
            return out

    class ToyConfig:
        architectures = ("ToyForCausalLM",)

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
            attn = lambda i, shares=False: PartSpec("gqa_attention", {
                "hidden_size": H, "num_heads": 2, "num_kv_heads": 1, "head_dim": H // 2,
                "qk_norm_eps": None, "shares_cache": shares, "window": self.raw.get("window", 0),
                "position": PartSpec("rope_half_split", {"theta": 100.0, "rotary_dim": H // 4})},
                {k: f"l{i}.attn.{k}" for k in ("q", "k", "v", "o")})
            ffn = lambda i: PartSpec("swiglu", {"hidden_size": H, "ffn_dim": 2 * H},
                                     {"gate": f"l{i}.gate", "up": f"l{i}.up", "down": f"l{i}.down"})
            mixers = [PartSpec("toy_decay", {"hidden_size": H, "decay": 0.5}, {"w": "l0.toy.w"}),
                      attn(1), attn(2, shares=True)]
            layers = tuple(LayerSpec("prenorm_residual", norm(f"l{i}.n1"), m, norm(f"l{i}.n2"), ffn(i))
                           for i, m in enumerate(mixers))
            # layer 0 runs twice (two states), layer 2 reads the cache that layer 1 wrote
            schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2, cache_of=1), ScheduleEntry(0))
            return ModelSpec("ToyForCausalLM", H, V, 512, "embed", norm("final"), None, layers, schedule,
                             embedding_scale=1.5, logit_softcap=6.0)

    class ToyForCausalLM(DecoderModel):
        def __init__(self, config, precision, device):
            self.config = config
            super().__init__(config.model_spec(), precision, device)

    register_architecture("ToyForCausalLM", ToyConfig, ToyForCausalLM)
    return {"architectures": ["ToyForCausalLM"], "hidden_size": 32, "vocab_size": 50}


def toy_reference(raw, w, tokens):
    """The same toy model, whole sequence, float64 numpy."""
    H = raw["hidden_size"]
    hd = H // 2
    T = len(tokens)
    x = 1.5 * w["embed"][np.asarray(tokens)]                   # ModelSpec.embedding_scale
    window = raw.get("window", 0)

    def ffn(h, i):
        return (P.silu(h @ w[f"l{i}.gate"].T) * (h @ w[f"l{i}.up"].T)) @ w[f"l{i}.down"].T

    def toy(h):
        s, out = np.zeros(H), np.zeros((T, H))
        for t in range(T):
            s = 0.5 * s + h[t]
            out[t] = w["l0.toy.w"] @ s
        return out

    def rope(v):                                               # rotary over the first hd/2 channels
        rot = hd // 2
        turned = P.rope_half_split(v[..., :rot], np.arange(T), 100.0)
        return np.concatenate([turned, v[..., rot:]], axis=-1)

    def attend(q, k, v):
        out = np.zeros((T, 2, hd))
        idx = np.arange(T)
        ok = idx[None] <= idx[:, None]
        if window:
            ok &= idx[None] > idx[:, None] - window
        for head in range(2):
            s = np.where(ok, q[:, head] @ k[:, 0].T / math.sqrt(hd), -np.inf)
            p = np.exp(s - s.max(-1, keepdims=True))
            out[:, head] = (p / p.sum(-1, keepdims=True)) @ v[:, 0]
        return out.reshape(T, H)

    kv = {}
    for position, layer in enumerate([0, 1, 2, 0]):
        h = P.rms_norm(x, w[f"l{layer}.n1"], 1e-5)
        if layer == 0:
            delta = toy(h)
        else:
            q = rope((h @ w[f"l{layer}.attn.q"].T).reshape(T, 2, hd))
            if layer == 1:
                kv["k"] = rope((h @ w["l1.attn.k"].T).reshape(T, 1, hd))
                kv["v"] = (h @ w["l1.attn.v"].T).reshape(T, 1, hd)
            delta = attend(q, kv["k"], kv["v"]) @ w[f"l{layer}.attn.o"].T
        x = x + delta
        x = x + ffn(P.rms_norm(x, w[f"l{layer}.n2"], 1e-5), layer)
    logits = P.rms_norm(x, w["final"], 1e-5) @ w["embed"].T
    return 6.0 * np.tanh(logits / 6.0)                         # ModelSpec.logit_softcap


@pytest.mark.parametrize("window", [0, 40])
def test_a_toy_architecture_defined_in_the_test(window, tmp_path):
    """Registered mixer with its own state, a layer scheduled twice, a layer reading another
    layer's cache, partial rotary, no q/k norm, a sliding window with its own page group, a state
    that is not fp32, a scaled embedding and soft-capped logits -- without touching a file of the
    framework."""
    from flyweight_b200.engine import ModelRunner, load_model
    from flyweight_b200.weights import load_model_tensors
    from tiny_configs import make_model_dir
    raw = dict(toy_architecture(), window=window)
    folder = make_model_dir(tmp_path / "toy", raw, seed=2, dtype=torch.float32)
    model = load_model(folder, "float32")
    specs = model.state_specs()
    assert [type(s).__name__ for s in specs] == ["FixedState", "PagedKV", "NoneType", "FixedState"]
    runner = ModelRunner(model, num_pages=4, num_slots=2, max_model_len=256)
    assert runner.cache.layer_caches[0].state.dtype == torch.float64
    assert runner.cache.groups[0].window == window
    w = as_numpy(load_model_tensors(folder))
    tokens = [int(t) for t in np.random.default_rng(0).integers(0, 50, size=200)]
    want = toy_reference(raw, w, tokens)
    whole = runner.step([("a", tokens, list(range(200)))]).cpu().numpy()
    runner.finish("a")
    assert np.abs(whole - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    parts, pos = [], 0
    for n in [3, 1, 64, 2, 50, 1, 1, 78]:
        parts.append(runner.step([("b", tokens[pos:pos + n], list(range(n)))]).cpu().numpy())
        pos += n
        runner.cache.check()
    got = np.concatenate(parts)
    assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    if window:
        table = runner.cache.groups[0].tables["b"]
        assert table[0] == -1 and table[1] >= 0             # passed before the last step / during it
        assert runner.cache.release_passed("b") == 1        # what the next step would give back
        assert table[1] == -1 and runner.cache.groups[0].pool.n_used == 2
    runner.finish("b")
    assert runner.cache.groups[0].pool.n_used == 0


# ------------------------------------------------------------------ a second toy: routing, positions
def toy_routed_architecture():
    """Another toy, again defined only here: a feed-forward that routes every token to one of
    three small experts (router logits and softmax in fp32, top-1, the expert's output scaled
    by its probability) and a position encoding of its own (rotary angles at pos / 4, full
    head), in a model whose two layers differ (dense SwiGLU in one, routed experts in the other)."""
    from flyweight_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from flyweight_b200.parts import (Arrangement, FeedForward, PositionEncoding, register_arrangement,
                                      register_feed_forward, register_position)
    from flyweight_b200.parts.model import DecoderModel
    from flyweight_b200.weights import TensorDecl

    @register_position("toy_slow_rope")
    class SlowRope(PositionEncoding):
        def __init__(self, spec):
            super().__init__(spec)
            self.rotary_dim = int(self.params["rotary_dim"])
            self.slowdown = float(self.params["slowdown"])

        def table(self, n_positions, device):
            half = self.rotary_dim // 2
            inv = 50.0 ** (-torch.arange(half, dtype=torch.float64) * 2 / self.rotary_dim)
            angle = (torch.arange(n_positions, dtype=torch.float64) / self.slowdown)[:, None] * inv[None]
            return torch.stack([angle.cos(), angle.sin()], -1).float().contiguous().to(device)

    @register_arrangement("toy_post_norm_ffn_only")
    class PostNormFfnOnly(Arrangement):
        """A layer with no mixer and a norm *after* its feed-forward: x += norm(ffn(x)).  Two parts
        where the pre-norm block has four; it keeps nothing in the cache."""
        ROLES = {"feed_forward": ("feed_forward", True), "post_norm": ("norm", True)}

        def forward(self, ctx, x, pending, cache):
            from flyweight_b200.kernels import ops
            if pending is not None:
                ops.add_(x, pending)
            delta = self.feed_forward.forward(ctx, x)           # this toy's experts read fp32 rows
            normed = self.post_norm.forward(ctx, delta.contiguous())
            return x, normed.float()

    @register_feed_forward("toy_top1_experts")
    class Top1Experts(FeedForward):
        def __init__(self, spec):
            super().__init__(spec)
            self.hidden, self.width, self.n = (int(self.params[k]) for k in ("hidden_size", "width", "experts"))

        def declare(self):
            n = self.names
            return {n["router"]: TensorDecl((self.n, self.hidden)),
                    n["up"]: TensorDecl((self.n * self.width, self.hidden)),
                    n["down"]: TensorDecl((self.n * self.hidden, self.width))}

        def bind(self, get, precision, device):
            f32 = lambda name: get(self.names[name]).to(device=device, dtype=torch.float32)
            self.router = f32("router")
            self.up = f32("up").reshape(self.n, self.width, self.hidden)
            self.down = f32("down").reshape(self.n, self.hidden, self.width)

        def forward(self, ctx, h):                 # test code: plain torch on the device
            h = h.float()
            prob = torch.softmax(h @ self.router.T, dim=-1)
            weight, expert = prob.max(dim=-1)
            hidden = torch.relu(torch.einsum("th,twh->tw", h, self.up[expert]))
            return weight[:, None] * torch.einsum("tw,thw->th", hidden, self.down[expert])

    class RoutedConfig:
        architectures = ("ToyRoutedForCausalLM",)

        def __init__(self, raw):
            self.raw = dict(raw)

        @classmethod
        def from_dict(cls, raw):
            return cls(raw)

        def to_dict(self):
            return dict(self.raw)

        def model_spec(self):
            H, V = self.raw["hidden_size"], self.raw["vocab_size"]
            norm = lambda name: PartSpec("rmsnorm", {"size": H, "eps": 1e-6}, {"weight": name})
            positions = [PartSpec("toy_slow_rope", {"rotary_dim": 16, "slowdown": 4.0}),
                         # the framework's rotary part with the other pairing, on half of the head
                         PartSpec("rope", {"theta": 50.0, "rotary_dim": 8, "pairing": "interleaved"})]
            attn = lambda i: PartSpec("gqa_attention", {
                "hidden_size": H, "num_heads": 3, "num_kv_heads": 3, "head_dim": 16, "qk_norm_eps": None,
                "position": positions[i]},
                {k: f"l{i}.attn.{k}" for k in ("q", "k", "v", "o")})
            routed2 = PartSpec("toy_top1_experts", {"hidden_size": H, "width": 24, "experts": 3},
                               {"router": "l2.router", "up": "l2.experts.up", "down": "l2.experts.down"})
            dense = PartSpec("swiglu", {"hidden_size": H, "ffn_dim": 80},
                             {"gate": "l0.gate", "up": "l0.up", "down": "l0.down"})
            routed = PartSpec("toy_top1_experts", {"hidden_size": H, "width": 24, "experts": 3},
                              {"router": "l1.router", "up": "l1.experts.up", "down": "l1.experts.down"})
            layers = (LayerSpec("prenorm_residual", norm("l0.n1"), attn(0), norm("l0.n2"), dense),
                      LayerSpec("prenorm_residual", norm("l1.n1"), attn(1), norm("l1.n2"), routed),
                      LayerSpec("toy_post_norm_ffn_only", parts={"feed_forward": routed2, "post_norm": norm("l2.post")}))
            return ModelSpec("ToyRoutedForCausalLM", H, V, 512, "embed", norm("final"), "head", layers,
                             (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2)))

    class ToyRoutedForCausalLM(DecoderModel):
        def __init__(self, config, precision, device):
            self.config = config
            super().__init__(config.model_spec(), precision, device)

    register_architecture("ToyRoutedForCausalLM", RoutedConfig, ToyRoutedForCausalLM)
    return {"architectures": ["ToyRoutedForCausalLM"], "hidden_size": 48, "vocab_size": 70}


def toy_routed_reference(raw, w, tokens):
    H, T, hd, nh = raw["hidden_size"], len(tokens), 16, 3
    x = w["embed"][np.asarray(tokens)]
    pos = np.arange(T)

    def rope(v):                                   # [T][nh][hd], angles at pos / 4, base 50
        half = hd // 2
        inv = 50.0 ** (-np.arange(half) * 2.0 / hd)
        ang = (pos / 4.0)[:, None] * inv[None]
        cos, sin = np.cos(ang)[:, None], np.sin(ang)[:, None]
        a, b = v[..., :half], v[..., half:]
        return np.concatenate([a * cos - b * sin, b * cos + a * sin], -1)

    def rope_interleaved(v):                       # pairs (2i, 2i + 1) of the first 8 channels, base 50
        rot = 8
        inv = 50.0 ** (-np.arange(rot // 2) * 2.0 / rot)
        ang = pos[:, None] * inv[None]
        cos, sin = np.cos(ang)[:, None], np.sin(ang)[:, None]
        out = v.copy()
        a, b = v[..., 0:rot:2], v[..., 1:rot:2]
        out[..., 0:rot:2] = a * cos - b * sin
        out[..., 1:rot:2] = b * cos + a * sin
        return out

    def attend(h, i):
        turn = rope if i == 0 else rope_interleaved
        q = turn((h @ w[f"l{i}.attn.q"].T).reshape(T, nh, hd))
        k = turn((h @ w[f"l{i}.attn.k"].T).reshape(T, nh, hd))
        v = (h @ w[f"l{i}.attn.v"].T).reshape(T, nh, hd)
        out = np.zeros((T, nh, hd))
        ok = pos[None] <= pos[:, None]
        for head in range(nh):
            s = np.where(ok, q[:, head] @ k[:, head].T / math.sqrt(hd), -np.inf)
            p = np.exp(s - s.max(-1, keepdims=True))
            out[:, head] = (p / p.sum(-1, keepdims=True)) @ v[:, head]
        return out.reshape(T, nh * hd) @ w[f"l{i}.attn.o"].T

    def experts(h, i=1):
        logits = h @ w[f"l{i}.router"].T
        prob = np.exp(logits - logits.max(-1, keepdims=True))
        prob /= prob.sum(-1, keepdims=True)
        up = w[f"l{i}.experts.up"].reshape(3, 24, H)
        down = w[f"l{i}.experts.down"].reshape(3, H, 24)
        out = np.zeros_like(h)
        for t in range(T):
            e = int(prob[t].argmax())
            out[t] = prob[t, e] * (down[e] @ np.maximum(up[e] @ h[t], 0.0))
        return out

    x = x + attend(P.rms_norm(x, w["l0.n1"], 1e-6), 0)
    h = P.rms_norm(x, w["l0.n2"], 1e-6)
    x = x + (P.silu(h @ w["l0.gate"].T) * (h @ w["l0.up"].T)) @ w["l0.down"].T
    x = x + attend(P.rms_norm(x, w["l1.n1"], 1e-6), 1)
    x = x + experts(P.rms_norm(x, w["l1.n2"], 1e-6))
    x = x + P.rms_norm(experts(x, 2), w["l2.post"], 1e-6)      # the layer without a mixer, norm after
    return P.rms_norm(x, w["final"], 1e-6) @ w["head"].T


def test_a_routed_feed_forward_and_another_position_encoding_defined_in_the_test(tmp_path):
    """A feed-forward with routing, a position encoding of its own and an arrangement of its own
    (no mixer, a norm after the feed-forward: two parts instead of four) are registered here,
    named by a toy configuration layer by layer (one dense, one routed, one without a mixer; one
    attention with the toy's positions, one with the framework's rotary part in interleaved
    pairing), and the model is built, loaded, stepped whole and in portions through the framework."""
    from flyweight_b200.engine import ModelRunner, load_model
    from flyweight_b200.weights import load_model_tensors
    from tiny_configs import make_model_dir
    raw = toy_routed_architecture()
    folder = make_model_dir(tmp_path / "routed", raw, seed=4, dtype=torch.float32)
    model = load_model(folder, "float32")
    assert not model.graph_safe                     # a part defined elsewhere: decode steps run eagerly
    assert [type(spec).__name__ for spec in model.state_specs()] == ["PagedKV", "PagedKV", "NoneType"]
    runner = ModelRunner(model, num_pages=6, num_slots=2, max_model_len=256)
    w = as_numpy(load_model_tensors(folder))
    tokens = [int(t) for t in np.random.default_rng(1).integers(0, 70, size=150)]
    want = toy_routed_reference(raw, w, tokens)
    whole = runner.step([("a", tokens, list(range(150)))]).cpu().numpy()
    runner.finish("a")
    scale = max(1.0, np.abs(want).max())
    assert np.abs(whole - want).max() <= 1e-4 * scale
    parts, at = [], 0
    for n in [5, 64, 2, 40, 1, 1, 37]:
        parts.append(runner.step([("b", tokens[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    runner.finish("b")
    assert np.abs(np.concatenate(parts) - want).max() <= 1e-4 * scale
    runner.cache.check()
