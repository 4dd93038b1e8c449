"""Safetensors container, binding by name and the random-weights mode (no GPU)."""
import json
import struct

import pytest
import torch

import flyweight_b200.models  # noqa: F401
from flyweight_b200.config import Lfm2Config
from flyweight_b200.models import Lfm2ForCausalLM
from flyweight_b200.parts import Precision
from flyweight_b200.weights import (SafetensorsError, TensorDecl, WeightError, bind, load_file,
                                    load_model_tensors, random_tensors, read_header, save_file)
from tiny_configs import TINY_A, TINY_B, make_model_dir


def cpu_model(raw):
    return Lfm2ForCausalLM(Lfm2Config.from_dict(raw), Precision("float32"), torch.device("cpu"))


def test_safetensors_round_trip_keeps_dtypes(tmp_path):
    tensors = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16),
               "c": torch.arange(6, dtype=torch.int32).reshape(2, 3), "d": torch.zeros(0, 4)}
    save_file(tensors, tmp_path / "x.safetensors", {"k": "v"})
    back = load_file(tmp_path / "x.safetensors")
    assert set(back) == set(tensors)
    for name in tensors:
        assert back[name].dtype == tensors[name].dtype
        assert torch.equal(back[name], tensors[name])


def test_safetensors_header_is_checked(tmp_path):
    path = tmp_path / "bad.safetensors"
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 12)
    with pytest.raises(SafetensorsError, match="needs 16"):
        read_header(path)
    header = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    path.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 8)
    with pytest.raises(SafetensorsError, match="outside the file"):
        read_header(path)
    path.write_bytes(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError, match="exceeds the file"):
        read_header(path)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    model = cpu_model(TINY_B)
    stored = random_tensors(model.declare(), 0, "unit", torch.float32)
    del stored["model.layers.1.conv.in_proj.weight"]
    del stored["lm_head.weight"]
    stored["model.layers.0.extra.weight"] = torch.zeros(2)
    stored["model.layers.2.self_attn.q_proj.weight"] = torch.zeros(5, 5)
    with pytest.raises(WeightError) as info:
        model.load(stored)
    err = info.value
    assert err.missing == ["lm_head.weight", "model.layers.1.conv.in_proj.weight"]
    assert err.unexpected == ["model.layers.0.extra.weight"]
    assert [w[0] for w in err.wrong_shape] == ["model.layers.2.self_attn.q_proj.weight"]
    text = str(err)
    for fragment in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (1)",
                     "stored [5, 5]", "model needs [96, 96]"):
        assert fragment in text


def test_conv_weight_is_accepted_in_conv1d_layout():
    model = cpu_model(TINY_A)
    stored = random_tensors(model.declare(), 0, "unit", torch.float32)
    name = "model.layers.0.conv.conv.weight"
    flat = stored[name].clone()
    stored[name] = flat.reshape(64, 1, 3)
    model.load(stored)
    assert torch.equal(model.layers[0].mixer.taps, flat)


def test_stored_dtypes_are_kept():
    decl = {"m": TensorDecl((2, 2)), "f": TensorDecl((2, 2)), "t": TensorDecl((3,), "table"),
            "h": TensorDecl((2,), "norm")}
    out = bind(decl, {"m": torch.zeros(2, 2, dtype=torch.bfloat16), "f": torch.zeros(2, 2),
                      "t": torch.arange(3), "h": torch.zeros(2, dtype=torch.float16)})
    assert out["m"].dtype == torch.bfloat16      # kept in bfloat16
    assert out["f"].dtype == torch.float32       # stored in 32-bit: stays so
    assert out["t"].dtype == torch.int32         # integer tables as int32
    assert out["h"].dtype == torch.float32
    bf = Precision("bfloat16")
    assert bf.matrix(out["m"], "cpu").dtype == torch.bfloat16
    assert bf.matrix(out["f"], "cpu").dtype == torch.float32
    assert Precision("float32").matrix(out["m"], "cpu").dtype == torch.float32


def test_random_mode_writes_a_loadable_folder_and_is_seeded(tmp_path):
    a = make_model_dir(tmp_path / "a", TINY_A, seed=5, dtype=torch.bfloat16)
    b = make_model_dir(tmp_path / "b", TINY_A, seed=5, dtype=torch.bfloat16)
    c = make_model_dir(tmp_path / "c", TINY_A, seed=6, dtype=torch.bfloat16)
    ta, tb, tc = (load_model_tensors(p) for p in (a, b, c))
    assert json.loads((a / "config.json").read_text())["hidden_size"] == 64
    assert set(ta) == set(cpu_model(TINY_A).declare())
    assert all(t.dtype == torch.bfloat16 for t in ta.values())
    assert all(torch.equal(ta[k], tb[k]) for k in ta)
    assert any(not torch.equal(ta[k], tc[k]) for k in ta)
    norm = ta["model.layers.0.operator_norm.weight"].float()
    assert abs(norm.mean().item() - 1.0) < 0.1
    model = cpu_model(TINY_A)
    model.load(ta)                               # binds without error
    assert model.head is model.embedding         # tied head shares the table


def test_baseline_preset_scales():
    model = cpu_model(TINY_B)
    t = random_tensors(model.declare(), 1, "baseline", torch.float32)
    assert abs(t["model.layers.1.conv.in_proj.weight"].std().item() - 0.02) < 0.002
    assert abs(t["model.embed_tokens.weight"].std().item() - 0.02) < 0.002
    assert abs(t["model.embedding_norm.weight"].mean().item() - 1.0) < 0.05


def test_without_a_gpu_the_entry_points_say_so_in_one_line(tmp_path):
    """No CPU path: where there is no CUDA device, opening a model says that (and the command line and
    the trace replay exit with 3) instead of failing somewhere inside the first CUDA call."""
    import subprocess
    import sys
    from pathlib import Path
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from flyweight_b200.engine.loading import NoGpu, load_model, random_model
    folder = make_model_dir(tmp_path / "m", TINY_A, seed=1)
    with pytest.raises(NoGpu, match="no CPU path"):
        load_model(folder, "float32")
    with pytest.raises(NoGpu, match="no CPU path"):
        random_model(TINY_A, seed=1)
    root = Path(__file__).resolve().parent.parent
    for command in ([sys.executable, "-m", "flyweight_b200", "generate", str(folder), "--prompt", "1,2", "--max-tokens", "2"],
                    [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                     "--out", str(tmp_path / "out"), "--max-tokens", "64"]):
        done = subprocess.run(command, cwd=root, capture_output=True, text=True, input="", timeout=120)
        assert done.returncode == 3, done.stderr[-500:]
        assert "no CPU path" in done.stderr and "Traceback" not in done.stderr
