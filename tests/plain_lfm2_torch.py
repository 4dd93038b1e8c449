"""The plain LFM2 forward pass once more, in float64 torch, for sizes at which numpy on the
host would take minutes (hidden 2048, vocabulary 65,536, hundreds of tokens).

Whole sequences, no cache, one function for each part, every tensor float64 on whatever
device the weights were put on.  It imports nothing from the ``flyweight_b200`` package.  The
formulas are those of ``plain_lfm2.py`` (which cites the place in yairpatch/flyweight for each);
``tests/test_plain_reference.py`` checks on the CPU that the two agree on both tiny
configurations, so this file is a second spelling of the same oracle and not a second oracle.
Only the config helpers (layer kinds) are taken from ``plain_lfm2``.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

from plain_lfm2 import layer_kinds

F64 = torch.float64


def read_safetensors(path, device="cpu") -> dict:
    """Every tensor of a safetensors file as float64 on ``device``
    (container: native/include/flyweight_v2_safetensors.hpp:50-135)."""
    raw = np.fromfile(str(path), dtype=np.uint8)
    (header_len,) = struct.unpack("<Q", raw[:8].tobytes())
    header = json.loads(raw[8:8 + header_len].tobytes())
    base = 8 + header_len
    out = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        begin, end = entry["data_offsets"]
        blob = raw[base + begin:base + end]
        kind = entry["dtype"]
        if kind == "F32":
            tensor = torch.from_numpy(blob.view("<f4").copy())
        elif kind == "BF16":
            # bf16 -> f32 is "bits << 16" (native/include/flyweight_v2_native_kernels.hpp:97-108)
            bits = torch.from_numpy(blob.view("<u2").astype(np.int32)) << 16
            tensor = bits.view(torch.float32)
        elif kind == "F16":
            tensor = torch.from_numpy(blob.view("<f2").copy())
        elif kind == "F64":
            tensor = torch.from_numpy(blob.view("<f8").copy())
        else:
            raise ValueError(f"plain reader: unsupported dtype {kind} for {name}")
        out[name] = tensor.to(device).to(F64).reshape(tuple(entry["shape"]))
    return out


def load_model_dir(path, device="cpu"):
    path = Path(path)
    cfg = json.loads((path / "config.json").read_text())
    return cfg, read_safetensors(path / "model.safetensors", device)


def rms_norm(x, weight, eps):
    """(x * rsqrt(mean(x^2) + eps)) * w, plain weight (plain_lfm2.rms_norm)."""
    inv = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return (x * inv) * weight


def rope_half_split(x, positions, theta):
    """Pair (i, i + hd/2) turns by pos * theta^(-2i/hd) (plain_lfm2.rope_half_split)."""
    hd = x.shape[-1]
    half = hd // 2
    inv_freq = torch.tensor(theta, dtype=F64, device=x.device) ** (
        -torch.arange(half, dtype=F64, device=x.device) * 2.0 / hd)
    angle = positions.to(F64)[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :half], x[..., half:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def attention_mixer(h, w, prefix, *, n_heads, n_kv_heads, head_dim, eps, theta):
    """q/k/v, per-head RMSNorm of q and k, rotation, causal softmax((q.k)/sqrt(hd)) v with query
    head j on KV head j // group, output projection (plain_lfm2.attention_mixer)."""
    T = h.shape[0]
    positions = torch.arange(T, device=h.device)
    q = (h @ w[prefix + "self_attn.q_proj.weight"].T).reshape(T, n_heads, head_dim)
    k = (h @ w[prefix + "self_attn.k_proj.weight"].T).reshape(T, n_kv_heads, head_dim)
    v = (h @ w[prefix + "self_attn.v_proj.weight"].T).reshape(T, n_kv_heads, head_dim)
    q = rope_half_split(rms_norm(q, w[prefix + "self_attn.q_layernorm.weight"], eps), positions, theta)
    k = rope_half_split(rms_norm(k, w[prefix + "self_attn.k_layernorm.weight"], eps), positions, theta)
    group = n_heads // n_kv_heads
    allowed = positions[None, :] <= positions[:, None]
    out = torch.zeros((T, n_heads, head_dim), dtype=F64, device=h.device)
    for head in range(n_heads):
        kv = head // group
        scores = (q[:, head, :] @ k[:, kv, :].T) / math.sqrt(head_dim)
        scores = scores.masked_fill(~allowed, float("-inf"))
        p = torch.exp(scores - scores.max(dim=-1, keepdim=True).values)
        out[:, head, :] = (p / p.sum(dim=-1, keepdim=True)) @ v[:, kv, :]
    return out.reshape(T, n_heads * head_dim) @ w[prefix + "self_attn.out_proj.weight"].T


def shortconv_mixer(h, w, prefix, *, taps_len, has_bias):
    """B | C | x; u = B*x; y[t] = sum_k taps[k] * u[t-(L-1)+k] with zeros before the start;
    bias after the taps; out_proj(C * y) (plain_lfm2.shortconv_mixer)."""
    T, H = h.shape
    p = h @ w[prefix + "conv.in_proj.weight"].T
    B, C, xg = p[:, :H], p[:, H:2 * H], p[:, 2 * H:]
    bx = B * xg
    taps = w[prefix + "conv.conv.weight"].reshape(H, taps_len)
    padded = torch.cat([torch.zeros((taps_len - 1, H), dtype=F64, device=h.device), bx], dim=0)
    y = torch.zeros((T, H), dtype=F64, device=h.device)
    for k in range(taps_len):
        y = y + padded[k:k + T, :] * taps[:, k][None, :]
    if has_bias:
        y = y + w[prefix + "conv.conv.bias"][None, :]
    return (C * y) @ w[prefix + "conv.out_proj.weight"].T


def silu(x):
    """x * sigmoid(x) with the sign-split sigmoid (plain_lfm2.silu)."""
    pos = 1.0 / (1.0 + torch.exp(-x.abs()))
    return x * torch.where(x >= 0, pos, 1.0 - pos)


def swiglu(h, w, prefix):
    gate = h @ w[prefix + "feed_forward.w1.weight"].T
    up = h @ w[prefix + "feed_forward.w3.weight"].T
    return (silu(gate) * up) @ w[prefix + "feed_forward.w2.weight"].T


def block(x, w, layer, kind, cfg):
    """x += mixer(norm(x)); x += ffn(norm(x)) (plain_lfm2.block)."""
    prefix = f"model.layers.{layer}."
    eps = float(cfg.get("norm_eps", 1e-6) or 1e-6)
    h = rms_norm(x, w[prefix + "operator_norm.weight"], eps)
    if kind == "attention":
        n_heads = int(cfg["num_attention_heads"])
        delta = attention_mixer(h, w, prefix, n_heads=n_heads,
                                n_kv_heads=int(cfg["num_key_value_heads"]),
                                head_dim=int(cfg["hidden_size"]) // n_heads, eps=eps,
                                theta=float(cfg.get("rope_theta", 1e6) or 1e6))
    else:
        delta = shortconv_mixer(h, w, prefix, taps_len=int(cfg.get("conv_L_cache", 3)),
                                has_bias=bool(cfg.get("conv_bias", False)))
    x = x + delta
    return x + swiglu(rms_norm(x, w[prefix + "ffn_norm.weight"], eps), w, prefix)


def forward(cfg, w, tokens, rows=None) -> np.ndarray:
    """Logits of one whole sequence as a float64 numpy array: [T, V], or [len(rows), V] for the
    given positions only (the head is the largest product at a real vocabulary)."""
    device = w["model.embed_tokens.weight"].device
    tokens = torch.as_tensor(list(tokens), dtype=torch.int64, device=device)
    if int(tokens.min()) < 0 or int(tokens.max()) >= int(cfg["vocab_size"]):
        raise ValueError("token id out of range")
    x = w["model.embed_tokens.weight"][tokens]
    for layer, kind in enumerate(layer_kinds(cfg)):
        x = block(x, w, layer, kind, cfg)
    if rows is not None:
        x = x[torch.as_tensor(list(rows), dtype=torch.int64, device=device)]
    n = rms_norm(x, w["model.embedding_norm.weight"], float(cfg.get("norm_eps", 1e-6) or 1e-6))
    head = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return (n @ head.T).cpu().numpy()
