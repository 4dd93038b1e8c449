"""The reference arm of bench.py: the UNMODIFIED yairpatch/flyweight, installed offline into
``baseline/_ref`` (``pip install --no-index --no-build-isolation --no-deps --target baseline/_ref``
on a copy of its tree, with ``CXX=/usr/bin/g++`` so that CMake finds OpenMP), driven through its own public Python
API and stock code path for the same metric and configuration as the engine's own arm.

flyweight loads LFM2 from GGUF only, so this file writes one: the LFM2-1.2B geometry with
seeded random weights (bf16 matrices, f32 norm weights and conv taps, as its loader requires),
straight from the GGUF v3 container layout (magic, version, counts, key/values, tensor infos,
aligned payload).  Nothing of this repository's engine, models or kernels is on this path.

What is measured: ``V2Model(path).native_runtime(context_limit, parallel_sequences=B)`` with the
reference's defaults (f16 KV cache), B tasks queued with ``task_submit`` (greedy) over
uniform-random prompts of the benchmark's context length, ``engine_step`` pumped until every task
decodes, then K timed cycles.  A cycle yields one token per task (flyweight decodes LFM2 slots
one after another inside the cycle), so tokens/s = B * K / seconds.  The clock is the host's around
the public call -- the reference synchronises once per token itself -- so the same number stands
for ``value`` and for ``e2e``.
"""
from __future__ import annotations

import json
import os
import struct
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

GGUF_UINT32, GGUF_FLOAT32, GGUF_STRING, GGUF_ARRAY = 4, 6, 8, 9
GGML_F32, GGML_BF16 = 0, 30
ALIGNMENT = 32


def _s(text: str) -> bytes:
    raw = text.encode("utf-8")
    return struct.pack("<Q", len(raw)) + raw


def _kv(key: str, kind: int, payload: bytes) -> bytes:
    return _s(key) + struct.pack("<I", kind) + payload


def write_lfm2_gguf(path: str, config: dict, seed: int = 0) -> dict:
    """A dense-LFM2 GGUF with seeded N(0, 0.02) weights (norm weights 1 + N(0, 0.1))."""
    import torch
    H = config["hidden_size"]
    L = config["num_hidden_layers"]
    nh, nkv = config["num_attention_heads"], config["num_key_value_heads"]
    hd = H // nh
    V = config["vocab_size"]
    taps = config.get("conv_L_cache", 3)
    width = config["intermediate_size"]
    if config.get("block_auto_adjust_ff_dim"):
        width = int(2 * width / 3)
        multiple = config.get("block_multiple_of", 256)
        width = multiple * ((width + multiple - 1) // multiple)
    attention = set(config["full_attn_idxs"])
    gen = torch.Generator().manual_seed(seed)

    tensors = []          # (name, dims in GGUF order (innermost first), ggml type, torch tensor)

    def matrix(name, outputs, inputs):
        data = (torch.randn(outputs, inputs, generator=gen) * 0.02).to(torch.bfloat16)
        tensors.append((name, (inputs, outputs), GGML_BF16, data))

    def vector(name, size):
        tensors.append((name, (size,), GGML_F32, 1.0 + 0.1 * torch.randn(size, generator=gen)))

    matrix("token_embd.weight", V, H)
    vector("token_embd_norm.weight", H)
    for i in range(L):
        p = f"blk.{i}."
        vector(p + "attn_norm.weight", H)
        if i in attention:
            matrix(p + "attn_q.weight", nh * hd, H)
            matrix(p + "attn_k.weight", nkv * hd, H)
            matrix(p + "attn_v.weight", nkv * hd, H)
            matrix(p + "attn_output.weight", H, nh * hd)
            vector(p + "attn_q_norm.weight", hd)
            vector(p + "attn_k_norm.weight", hd)
        else:
            matrix(p + "shortconv.in_proj.weight", 3 * H, H)
            matrix(p + "shortconv.out_proj.weight", H, H)
            tensors.append((p + "shortconv.conv.weight", (taps, H), GGML_F32,
                            torch.randn(H, taps, generator=gen) * 0.02))
        vector(p + "ffn_norm.weight", H)
        matrix(p + "ffn_gate.weight", width, H)
        matrix(p + "ffn_up.weight", width, H)
        matrix(p + "ffn_down.weight", H, width)

    arch = "lfm2"
    kv_heads = [nkv if i in attention else 0 for i in range(L)]
    vocabulary = [f"<{i}>" for i in range(V)]
    u32 = lambda v: struct.pack("<I", v)
    u32_array = lambda values: struct.pack("<IQ", GGUF_UINT32, len(values)) + b"".join(u32(v) for v in values)
    str_array = lambda values: struct.pack("<IQ", GGUF_STRING, len(values)) + b"".join(_s(v) for v in values)
    metadata = [
        _kv("general.architecture", GGUF_STRING, _s(arch)),
        _kv("general.name", GGUF_STRING, _s("lfm2-random")),
        _kv(arch + ".block_count", GGUF_UINT32, u32(L)),
        _kv(arch + ".context_length", GGUF_UINT32, u32(config.get("max_position_embeddings", 128000))),
        _kv(arch + ".embedding_length", GGUF_UINT32, u32(H)),
        _kv(arch + ".feed_forward_length", GGUF_UINT32, u32(width)),
        _kv(arch + ".attention.head_count", GGUF_UINT32, u32(nh)),
        _kv(arch + ".attention.head_count_kv", GGUF_ARRAY, u32_array(kv_heads)),
        _kv(arch + ".rope.freq_base", GGUF_FLOAT32, struct.pack("<f", config.get("rope_theta", 1e6))),
        _kv(arch + ".attention.layer_norm_rms_epsilon", GGUF_FLOAT32, struct.pack("<f", config.get("norm_eps", 1e-5))),
        _kv(arch + ".vocab_size", GGUF_UINT32, u32(V)),
        _kv(arch + ".shortconv.l_cache", GGUF_UINT32, u32(taps)),
        _kv("tokenizer.ggml.model", GGUF_STRING, _s("gpt2")),
        _kv("tokenizer.ggml.pre", GGUF_STRING, _s("lfm2")),
        _kv("tokenizer.ggml.tokens", GGUF_ARRAY, str_array(vocabulary)),
        _kv("tokenizer.ggml.token_type", GGUF_ARRAY, u32_array([1] * V)),
        _kv("tokenizer.ggml.merges", GGUF_ARRAY, str_array([])),
        _kv("tokenizer.ggml.bos_token_id", GGUF_UINT32, u32(1)),
        _kv("tokenizer.ggml.eos_token_id", GGUF_UINT32, u32(2)),
        _kv("general.alignment", GGUF_UINT32, u32(ALIGNMENT)),
    ]
    infos = bytearray()
    offset = 0
    for name, dims, kind, data in tensors:
        infos += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", kind, offset)
        nbytes = data.numel() * data.element_size()
        offset += nbytes + ((-nbytes) % ALIGNMENT)
    header = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata))
    body = header + b"".join(metadata) + bytes(infos)
    body += b"\0" * ((-len(body)) % ALIGNMENT)
    with open(path, "wb") as handle:
        handle.write(body)
        for _, _, _, data in tensors:
            raw = data.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
            handle.write(raw)
            handle.write(b"\0" * ((-len(raw)) % ALIGNMENT))
    return {"tensors": len(tensors), "bytes": os.path.getsize(path), "ffn_dim": width}


def unavailable(reason: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": reason[:300].replace("\n", " ")}))
    return 0


def run(args, config: dict, batch: int, context: int, backend: str = "cuda") -> int:
    if not os.path.isdir(os.path.join(REF, "flyweight")):
        return unavailable("baseline/_ref holds no installed flyweight (offline install not done on this machine)")
    sys.path.insert(0, REF)
    try:
        import random
        from flyweight.v2 import V2Model
    except Exception as error:                                          # noqa: BLE001
        return unavailable(f"importing the installed reference failed: {type(error).__name__}: {error}")
    steps, warmup = args.steps, max(3, args.warmup)
    workdir = tempfile.mkdtemp(prefix="fwb200-ref-")
    path = os.path.join(workdir, "lfm2-random.gguf")
    try:
        try:
            selected = V2Model.select_backend(backend)
        except Exception as error:                                      # noqa: BLE001
            return unavailable(f"the reference found no usable {backend} backend: {error}")
        info = write_lfm2_gguf(path, config, seed=0)
        rng = random.Random(0)
        vocab = config["vocab_size"]
        limit = context + warmup + steps + 8
        model = V2Model(path)
        runtime = model.native_runtime(context_limit=limit, parallel_sequences=batch)
        runtime.prepare()
        tasks = []
        for _ in range(batch):
            prompt = [rng.randrange(vocab) for _ in range(context)]
            tasks.append(runtime.task_submit(prompt, warmup + steps + 4, ()))
        produced = {task: 0 for task in tasks}

        def cycle():
            count = 0
            for task, _token, kind in runtime.engine_step():
                if kind == 0:
                    produced[task] += 1
                    count += 1
                elif kind == 2:
                    raise RuntimeError(f"reference task {task} failed")
            return count

        deadline = time.time() + 1500
        while min(produced.values()) < 1:                                # prompts in (untimed)
            cycle()
            if time.time() > deadline:
                return unavailable("the reference did not finish ingesting the prompts in 25 minutes")
        for _ in range(warmup):
            cycle()
        begin = time.perf_counter()
        tokens = 0
        for _ in range(steps):
            tokens += cycle()
        seconds = time.perf_counter() - begin
        value = tokens / seconds
        line = {
            "impl": "reference", "metric": "decode tokens/s, LFM2-1.2B bf16, batch 8, context 4096",
            "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
            "ms_per_step": seconds * 1e3 / steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 weights, f32 activations, f16 KV (reference defaults)",
            "data": "synthetic: uniform-random token ids, seeded random weights N(0, 0.02)",
            "config": {"model": "LFM2-1.2B", "layers": config["num_hidden_layers"],
                       "layers_full": config["num_hidden_layers"],
                       "attention_layers": len(config["full_attn_idxs"]),
                       "hidden": config["hidden_size"], "heads": config["num_attention_heads"],
                       "kv_heads": config["num_key_value_heads"],
                       "head_dim": config["hidden_size"] // config["num_attention_heads"],
                       "ffn_dim": info["ffn_dim"], "conv_L_cache": config["conv_L_cache"], "vocab": vocab,
                       "global_batch": batch, "seq_len": context, "backend": selected,
                       "gguf_bytes": info["bytes"], "parallelism": "single GPU"},
            # per step the reference's runtime hands each sequence's last token id (4 bytes) to its
            # decode kernels and reads the new id and its event back (8 bytes); the prompt ids went
            # in with task_submit, before the timed region
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 4 * batch,
                    "d2h_bytes_per_step": 8 * batch},
            "tokens_timed": tokens,
        }
        print(json.dumps(line))
        try:
            runtime.close()
            model.close()
        except Exception:                                               # noqa: BLE001
            pass
        return 0
    except Exception as error:                                          # noqa: BLE001
        return unavailable(f"the reference failed on this workload: {type(error).__name__}: {error}")
    finally:
        try:
            os.remove(path)
            os.rmdir(workdir)
        except OSError:
            pass
