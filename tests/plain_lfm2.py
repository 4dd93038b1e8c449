"""A plain, slow LFM2 forward pass: whole sequences, no cache, float64 numpy.

This file is the oracle of the test-suite.  It shares no code with the
``flyweight_b200`` package: it parses ``config.json`` itself, reads
``model.safetensors`` itself, and has one function for each part of the model.
Every function cites the place in yairpatch/flyweight that fixes its formula
(paths are relative to that project's root).

The formulas were checked once against flyweight's own float64 numpy forward
(``tests/lfm2_gguf_fixture.py``, function ``reference_greedy``); the script and
its small outputs are under ``tests/golden/``.  What flyweight's fixture cannot
express (a conv bias, an untied head, another eps, a sliding window, logits
instead of token ids) rests on the formulas cited below.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# --------------------------------------------------------------------------- files

def read_safetensors(path) -> dict[str, np.ndarray]:
    """Every tensor of a safetensors file as float64 (integers as int64).

    Container: u64 little-endian header length, a JSON header of
    ``{name: {dtype, shape, data_offsets}}``, then the flat payload
    (native/include/flyweight_v2_safetensors.hpp:50-135).
    """
    raw = Path(path).read_bytes()
    (header_len,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + header_len])
    base = 8 + header_len
    out: dict[str, np.ndarray] = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        blob = raw[base + begin:base + end]
        shape = tuple(entry["shape"])
        kind = entry["dtype"]
        if kind == "F32":
            arr = np.frombuffer(blob, dtype="<f4").astype(np.float64)
        elif kind == "F64":
            arr = np.frombuffer(blob, dtype="<f8").astype(np.float64)
        elif kind == "BF16":
            # bf16 -> f32 is "bits << 16" (native/include/flyweight_v2_native_kernels.hpp:97-108)
            bits = np.frombuffer(blob, dtype="<u2").astype(np.uint32) << 16
            arr = bits.view(np.float32).astype(np.float64)
        elif kind == "F16":
            arr = np.frombuffer(blob, dtype="<f2").astype(np.float64)
        elif kind == "I32":
            arr = np.frombuffer(blob, dtype="<i4").astype(np.int64)
        elif kind == "I64":
            arr = np.frombuffer(blob, dtype="<i8").astype(np.int64)
        else:
            raise ValueError(f"plain reader: unsupported dtype {kind} for {name}")
        out[name] = arr.reshape(shape)
    return out


def ffn_width(cfg: dict) -> int:
    """SwiGLU width from the config keys.

    flyweight reads the width off the gate tensor's shape
    (native/src/v2_runtime.cpp:3527-3535); the rule below is the one the LFM2
    config keys describe: optional x2/3, optional multiplier, round up to a
    multiple of ``block_multiple_of``.
    """
    width = int(cfg["intermediate_size"])
    if cfg.get("block_auto_adjust_ff_dim", False):
        width = int(2 * width / 3)
        mult = cfg.get("block_ffn_dim_multiplier")
        if mult is not None:
            width = int(mult * width)
        multiple = int(cfg.get("block_multiple_of", 256))
        width = multiple * ((width + multiple - 1) // multiple)
    return width


def layer_kinds(cfg: dict) -> list[str]:
    """'attention' or 'conv' for each layer (native/src/v2_runtime.cpp:4203-4209)."""
    n = int(cfg["num_hidden_layers"])
    if cfg.get("layer_types") is not None:
        kinds = []
        for name in cfg["layer_types"]:
            kinds.append("attention" if name in ("full_attention", "attention", "attn") else "conv")
        assert len(kinds) == n
        return kinds
    full = set(cfg.get("full_attn_idxs") or [])
    return ["attention" if i in full else "conv" for i in range(n)]


# --------------------------------------------------------------------------- parts

def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    """x * rsqrt(mean(x^2) + eps) * w over the last axis, plain (not 1+w) weight.

    native/include/flyweight_v2_qwen_kernels.hpp:424-447 (rms_norm), called with
    one_centered=0 at native/src/v2_runtime.cpp:27741.
    """
    inv = 1.0 / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return (x * inv) * weight


def rope_half_split(x: np.ndarray, positions: np.ndarray, theta: float) -> np.ndarray:
    """Half-split (NEOX) rotary embedding over the whole head.

    x: [T, heads, hd]; pair (i, i + hd/2), angle = pos * theta^(-2i/hd);
    out[i] = a cos - b sin, out[i+hd/2] = b cos + a sin
    (native/include/flyweight_v2_native_kernels.hpp:993-1008 angle, :1034-1047
    rotation; tests/lfm2_gguf_fixture.py:252-257).
    """
    hd = x.shape[-1]
    half = hd // 2
    inv_freq = theta ** (-np.arange(half, dtype=np.float64) * 2.0 / hd)
    angle = positions.astype(np.float64)[:, None] * inv_freq[None, :]      # [T, half]
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * cos - b * sin, b * cos + a * sin], axis=-1)


def attention_mixer(h, w, prefix, *, n_heads, n_kv_heads, head_dim, eps, theta,
                    positions=None, window=0):
    """GQA attention with per-head q/k RMSNorm and RoPE over a whole sequence.

    Order: q,k,v projections without bias (native/src/v2_runtime.cpp:28437-28439);
    per-head RMSNorm of q and k with the block eps (:28449-28450,
    native/include/flyweight_v2_native_kernels.hpp:1025-1033); RoPE on q and k,
    v untouched; scores (q.k)/sqrt(hd) of query head j against KV head
    j // (n_heads/n_kv_heads) (native/include/flyweight_v2_qwen_kernels.hpp:12629);
    causal (only positions <= the query's are cached, native/src/v2_runtime.cpp:25553-25558);
    softmax with max subtraction (flyweight_v2_qwen_kernels.hpp:12764-12781);
    output projection, no gate (native/src/v2_mtp_verifier.inc:1837-1841).
    ``window`` > 0 keeps only the last ``window`` keys (the reference's
    attention_window; LFM2 itself uses 0).
    """
    T = h.shape[0]
    if positions is None:
        positions = np.arange(T)
    q = (h @ w[prefix + "self_attn.q_proj.weight"].T).reshape(T, n_heads, head_dim)
    k = (h @ w[prefix + "self_attn.k_proj.weight"].T).reshape(T, n_kv_heads, head_dim)
    v = (h @ w[prefix + "self_attn.v_proj.weight"].T).reshape(T, n_kv_heads, head_dim)
    q = rms_norm(q, w[prefix + "self_attn.q_layernorm.weight"], eps)
    k = rms_norm(k, w[prefix + "self_attn.k_layernorm.weight"], eps)
    q = rope_half_split(q, positions, theta)
    k = rope_half_split(k, positions, theta)
    group = n_heads // n_kv_heads
    out = np.zeros((T, n_heads, head_dim))
    scale = 1.0 / math.sqrt(head_dim)
    idx = np.arange(T)
    allowed = idx[None, :] <= idx[:, None]
    if window and window > 0:
        allowed &= idx[None, :] > (idx[:, None] - window)
    for head in range(n_heads):
        kv = head // group
        scores = (q[:, head, :] @ k[:, kv, :].T) * scale                 # [T, T]
        scores = np.where(allowed, scores, -np.inf)
        scores = scores - scores.max(axis=-1, keepdims=True)
        p = np.exp(scores)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, head, :] = p @ v[:, kv, :]
    return out.reshape(T, n_heads * head_dim) @ w[prefix + "self_attn.out_proj.weight"].T


def shortconv_mixer(h, w, prefix, *, taps_len, has_bias):
    """Gated short convolution over a whole sequence.

    in_proj to 3H split in the order B | C | x
    (native/include/flyweight_v2_native_kernels.hpp:1295-1299,1311,1318;
    tests/lfm2_gguf_fixture.py:290-291); bx = B*x; causal depthwise FIR with the
    oldest tap first and zeros before the sequence start (:1312-1314, state
    zeroed at native/src/v2_runtime.cpp:20438); optional bias added after the
    taps and before the C gate (same place as flyweight_v2_native_kernels.hpp:1370);
    z = C*y; out_proj.
    """
    T, H = h.shape
    p = h @ w[prefix + "conv.in_proj.weight"].T
    B, C, xg = p[:, :H], p[:, H:2 * H], p[:, 2 * H:]
    bx = B * xg
    taps = w[prefix + "conv.conv.weight"].reshape(H, taps_len)            # [H][1][L] -> [H][L]
    padded = np.concatenate([np.zeros((taps_len - 1, H)), bx], axis=0)
    y = np.zeros((T, H))
    for k in range(taps_len):
        y += padded[k:k + T, :] * taps[:, k][None, :]
    if has_bias:
        y = y + w[prefix + "conv.conv.bias"][None, :]
    return (C * y) @ w[prefix + "conv.out_proj.weight"].T


def silu(x):
    """x * sigmoid(x), sigmoid evaluated sign-split for stability
    (native/include/flyweight_v2_qwen_kernels.hpp:1217-1222)."""
    pos = 1.0 / (1.0 + np.exp(-np.abs(x)))
    sig = np.where(x >= 0, pos, 1.0 - pos)
    return x * sig


def swiglu(h, w, prefix):
    """w2( silu(w1 h) * (w3 h) ): gate=w1, up=w3, down=w2
    (native/src/v2_runtime.cpp:28797-28805; tests/lfm2_gguf_fixture.py:165-167,310-311)."""
    gate = h @ w[prefix + "feed_forward.w1.weight"].T
    up = h @ w[prefix + "feed_forward.w3.weight"].T
    return (silu(gate) * up) @ w[prefix + "feed_forward.w2.weight"].T


def block(x, w, layer, kind, cfg):
    """Pre-norm residual block: x += mixer(norm1(x)); x += ffn(norm2(x))
    (native/src/v2_runtime.cpp:4164-4175, :28281-28282, :28476-28477, :29133)."""
    prefix = f"model.layers.{layer}."
    eps = float(cfg.get("norm_eps", 1e-6) or 1e-6)                      # default: v2_runtime.cpp:27558
    h = rms_norm(x, w[prefix + "operator_norm.weight"], eps)
    if kind == "attention":
        n_heads = int(cfg["num_attention_heads"])
        delta = attention_mixer(
            h, w, prefix, n_heads=n_heads, n_kv_heads=int(cfg["num_key_value_heads"]),
            head_dim=int(cfg["hidden_size"]) // n_heads,                 # v2_runtime.cpp:4222
            eps=eps, theta=float(cfg.get("rope_theta", 1e6) or 1e6))     # v2_runtime.cpp:4235
    else:
        delta = shortconv_mixer(h, w, prefix, taps_len=int(cfg.get("conv_L_cache", 3)),
                                has_bias=bool(cfg.get("conv_bias", False)))
    x = x + delta
    h = rms_norm(x, w[prefix + "ffn_norm.weight"], eps)
    return x + swiglu(h, w, prefix)


def forward(cfg: dict, w: dict[str, np.ndarray], tokens) -> np.ndarray:
    """Logits [T, V] for one whole sequence of token ids.

    Embedding rows without scaling (native/src/v2_runtime.cpp:27951-27956), the
    blocks in order, the final norm ``embedding_norm`` (:29176) and the head:
    ``lm_head.weight`` if present, else the embedding table (:4190-4191).
    """
    tokens = np.asarray(tokens, dtype=np.int64)
    if tokens.min() < 0 or tokens.max() >= int(cfg["vocab_size"]):
        raise ValueError("token id out of range")                        # v2_runtime.cpp:27530
    x = w["model.embed_tokens.weight"][tokens]
    for layer, kind in enumerate(layer_kinds(cfg)):
        x = block(x, w, layer, kind, cfg)
    eps = float(cfg.get("norm_eps", 1e-6) or 1e-6)
    n = rms_norm(x, w["model.embedding_norm.weight"], eps)
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return n @ head.T


def load_model_dir(path):
    path = Path(path)
    cfg = json.loads((path / "config.json").read_text())
    return cfg, read_safetensors(path / "model.safetensors")


# --------------------------------------------------------------------------- sampling

MASK64 = (1 << 64) - 1


class XorShift64Star:
    """The reference's per-request generator (native/src/v2_runtime.cpp:29307-29314)."""

    def __init__(self, seed: int):
        self.state = (seed & MASK64) or 0x9E3779B97F4A7C15                # v2_runtime.cpp:32596

    def uniform(self) -> float:
        v = self.state or 0x9E3779B97F4A7C15
        v ^= v >> 12
        v ^= (v << 25) & MASK64
        v ^= v >> 27
        self.state = v
        r = (v * 2685821657736338717) & MASK64
        return (r >> 11) * (1.0 / 9007199254740992.0)


def sample(logits: np.ndarray, *, temperature: float, top_k: int, top_p: float, min_p: float,
           rng: XorShift64Star) -> int:
    """One token from one row of logits, in the reference's order of operations.

    Candidates: the top_k largest logits sorted descending, ties to the lower id
    (top_k == 0 keeps all; native/src/v2_runtime.cpp:29543-29565); temperature 0
    or top_k 1 is greedy (:29356-29358, :29393-29395, :29691-29698); else
    p = exp(l/t - max) in float64, top-p prefix with cumulative mass >= top_p,
    then min-p prefix (p >= min_p * p_max), one uniform draw over the kept mass
    (:29699-29743).
    """
    logits = np.asarray(logits, dtype=np.float32)
    order = np.lexsort((np.arange(logits.size), -logits.astype(np.float64)))
    if top_k and top_k > 0:
        order = order[:top_k]
    if not temperature > 0.0 or order.size == 1:
        return int(order[0])
    cand = logits[order].astype(np.float64) / np.float64(np.float32(temperature))
    probs = np.exp(cand - cand[0])
    total = probs.sum()
    keep = probs.size
    if top_p < 1.0:
        cumulative = 0.0
        for i in range(probs.size):
            cumulative += probs[i] / total
            if cumulative >= np.float64(np.float32(top_p)):
                keep = i + 1
                break
    if min_p > 0.0:
        floor = np.float64(np.float32(min_p)) * probs[0]
        kept = 1
        while kept < keep and probs[kept] >= floor:
            kept += 1
        keep = kept
    kept_total = 0.0
    for i in range(keep):
        kept_total += probs[i]
    threshold = rng.uniform() * kept_total
    cumulative = 0.0
    for i in range(keep):
        cumulative += probs[i]
        if threshold <= cumulative:
            return int(order[i])
    return int(order[keep - 1])


def greedy_generate(cfg, w, prompt, count):
    """Greedy continuation by re-running whole sequences (slow by design)."""
    tokens = list(prompt)
    out = []
    for _ in range(count):
        logits = forward(cfg, w, tokens)[-1]
        nxt = int(np.lexsort((np.arange(logits.size), -logits))[0])
        out.append(nxt)
        tokens.append(nxt)
    return out
