"""The plain implementation against flyweight's own float64 forward (committed outputs of
tests/golden/make_golden.py), and a few properties of its parts (no GPU)."""
import json
from pathlib import Path

import numpy as np
import pytest

import plain_lfm2 as P

GOLDEN = Path(__file__).parent / "golden" / "lfm2_reference_greedy.npz"


@pytest.mark.parametrize("name", ["g1", "g2"])
def test_greedy_tokens_equal_the_reference_forward(name):
    data = np.load(GOLDEN)
    config = json.loads(bytes(data[f"{name}.config"]).decode())
    weights = {key[len(name) + 3:]: data[key].astype(np.float64)
               for key in data.files if key.startswith(f"{name}.w.")}
    prompt = data[f"{name}.prompt"].tolist()
    expected = data[f"{name}.tokens"].tolist()
    assert P.greedy_generate(config, weights, prompt, len(expected)) == expected


def test_conv_is_causal_and_matches_a_token_by_token_state():
    rng = np.random.default_rng(0)
    H, L, T = 6, 4, 11
    w = {"c.conv.in_proj.weight": rng.standard_normal((3 * H, H)),
         "c.conv.conv.weight": rng.standard_normal((H, 1, L)),
         "c.conv.conv.bias": rng.standard_normal(H),
         "c.conv.out_proj.weight": rng.standard_normal((H, H))}
    h = rng.standard_normal((T, H))
    whole = P.shortconv_mixer(h, w, "c.", taps_len=L, has_bias=True)
    # rolling state, one token at a time (native/include/flyweight_v2_native_kernels.hpp:1301-1319)
    state = np.zeros((H, L - 1))
    taps = w["c.conv.conv.weight"].reshape(H, L)
    for t in range(T):
        p = w["c.conv.in_proj.weight"] @ h[t]
        b, c, x = p[:H], p[H:2 * H], p[2 * H:]
        window = np.concatenate([state, (b * x)[:, None]], axis=1)
        state = window[:, 1:]
        y = (taps * window).sum(axis=1) + w["c.conv.conv.bias"]
        np.testing.assert_allclose(w["c.conv.out_proj.weight"] @ (c * y), whole[t], atol=1e-12)
    changed = h.copy()
    changed[7] += 1.0
    again = P.shortconv_mixer(changed, w, "c.", taps_len=L, has_bias=True)
    np.testing.assert_array_equal(again[:7], whole[:7])


def test_rope_rotates_pairs_and_keeps_norms():
    x = np.random.default_rng(1).standard_normal((5, 2, 8))
    out = P.rope_half_split(x, np.arange(5), 100.0)
    np.testing.assert_allclose(out[0], x[0], atol=1e-12)                 # position 0: identity
    np.testing.assert_allclose((out ** 2).sum(-1), (x ** 2).sum(-1), atol=1e-12)
    angle = 3 * 100.0 ** (-2 * 1 / 8)
    a, b = x[3, 0, 1], x[3, 0, 5]                                        # pair (1, 1 + 4)
    np.testing.assert_allclose(out[3, 0, 1], a * np.cos(angle) - b * np.sin(angle), atol=1e-12)
    np.testing.assert_allclose(out[3, 0, 5], b * np.cos(angle) + a * np.sin(angle), atol=1e-12)


def test_attention_is_causal_and_the_window_drops_old_keys():
    rng = np.random.default_rng(2)
    H, nh, nkv, hd, T = 16, 4, 2, 4, 9
    w = {"a.self_attn.q_proj.weight": rng.standard_normal((nh * hd, H)),
         "a.self_attn.k_proj.weight": rng.standard_normal((nkv * hd, H)),
         "a.self_attn.v_proj.weight": rng.standard_normal((nkv * hd, H)),
         "a.self_attn.out_proj.weight": rng.standard_normal((H, nh * hd)),
         "a.self_attn.q_layernorm.weight": np.ones(hd), "a.self_attn.k_layernorm.weight": np.ones(hd)}
    h = rng.standard_normal((T, H))
    kw = dict(n_heads=nh, n_kv_heads=nkv, head_dim=hd, eps=1e-5, theta=50.0)
    full = P.attention_mixer(h, w, "a.", **kw)
    changed = h.copy()
    changed[6] += 1.0
    np.testing.assert_array_equal(P.attention_mixer(changed, w, "a.", **kw)[:6], full[:6])
    windowed = P.attention_mixer(h, w, "a.", window=3, **kw)
    np.testing.assert_allclose(windowed[:3], full[:3], atol=1e-12)       # window not yet full
    assert np.abs(windowed[5:] - full[5:]).max() > 1e-6
    changed = h.copy()
    changed[1] += 5.0                                                    # outside the window of 8
    np.testing.assert_allclose(P.attention_mixer(changed, w, "a.", window=3, **kw)[8], windowed[8],
                               atol=1e-12)


def test_sampler_follows_the_reference_order():
    logits = np.array([1.0, 3.0, 3.0, 2.0, -1.0], dtype=np.float32)
    rng = P.XorShift64Star(9)
    assert P.sample(logits, temperature=0.0, top_k=3, top_p=1.0, min_p=0.0, rng=rng) == 1
    assert rng.state == 9                                # greedy draws no number
    # top_k 2 keeps ids 1 and 2 (equal logits, lower id first); u decides between them
    picks = {P.sample(logits, temperature=1.0, top_k=2, top_p=1.0, min_p=0.0,
                      rng=P.XorShift64Star(seed)) for seed in range(1, 40)}
    assert picks == {1, 2}
    # min_p 0.9 drops everything below 0.9 * p_max: only the two maxima stay even with top_k 0
    picks = {P.sample(logits, temperature=1.0, top_k=0, top_p=1.0, min_p=0.9,
                      rng=P.XorShift64Star(seed)) for seed in range(1, 40)}
    assert picks == {1, 2}
    # top_p smaller than the first candidate's share keeps just that one
    assert all(P.sample(logits, temperature=1.0, top_k=0, top_p=0.2, min_p=0.0,
                        rng=P.XorShift64Star(seed)) == 1 for seed in range(1, 20))
    u = P.XorShift64Star(1).uniform()
    assert 0.0 <= u < 1.0


def test_host_rng_equals_the_plain_one():
    from flyweight_b200.sampling import XorShift64Star
    for seed in (1, 7, 2 ** 63 + 5, 0):
        mine, plain = XorShift64Star(seed), P.XorShift64Star(seed)
        assert [mine.uniform() for _ in range(5)] == [plain.uniform() for _ in range(5)]


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_torch_spelling_of_the_plain_forward_equals_the_numpy_one(name, tmp_path):
    """``plain_lfm2_torch`` (float64 torch, used at real layer sizes on the GPU) and
    ``plain_lfm2`` (float64 numpy) on both tiny configurations: same logits, and the same rows
    when only some positions are asked for."""
    import torch
    import plain_lfm2_torch as PT
    from tiny_configs import TINY, make_model_dir
    folder = make_model_dir(tmp_path / name, TINY[name], seed=5, dtype=torch.bfloat16)
    tokens = [int(t) for t in np.random.default_rng(3).integers(0, TINY[name]["vocab_size"], size=70)]
    cfg, w = P.load_model_dir(folder)
    want = P.forward(cfg, w, tokens)
    cfg_t, w_t = PT.load_model_dir(folder)
    got = PT.forward(cfg_t, w_t, tokens)
    np.testing.assert_allclose(got, want, rtol=0, atol=1e-10 * max(1.0, np.abs(want).max()))
    rows = [0, 1, 33, 69]
    np.testing.assert_allclose(PT.forward(cfg_t, w_t, tokens, rows=rows), want[rows], rtol=0,
                               atol=1e-10 * max(1.0, np.abs(want).max()))
