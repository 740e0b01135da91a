"""The safetensors container, the by-name loader's errors and the random-weights mode."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from liyab_b200 import ErrorCode, LiyabError
from liyab_b200.config import parse_config
from liyab_b200.weights import (SafetensorsFile, load_parameters, normal_values, random_tensors, write_random_model,
                                write_safetensors)
from tiny_models import CONFIG_A, CONFIG_B


def test_container_round_trip_and_independent_reader(tmp_path):
    path = str(tmp_path / "t.safetensors")
    tensors = {"a": torch.arange(12, dtype=torch.float32).reshape(3, 4), "b": torch.randn(5).to(torch.bfloat16),
               "c": torch.tensor([1, 2, 3], dtype=torch.int64), "d": torch.zeros((0, 4))}
    write_safetensors(path, tensors, {"k": "v"})
    with SafetensorsFile(path) as f:
        assert f.metadata == {"k": "v"}
        for k, v in tensors.items():
            assert torch.equal(f.read(k), v)
    from safetensors.torch import load_file           # another implementation reads what we wrote
    other = load_file(path)
    assert all(torch.equal(other[k], v) for k, v in tensors.items())


def _raw_file(path, header: dict, data: bytes):
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + data)


def test_malformed_files_are_refused_with_the_tensor_named(tmp_path):
    p = str(tmp_path / "m.safetensors")
    _raw_file(p, {"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(LiyabError, match="'x'.*truncated"):
        SafetensorsFile(p)
    _raw_file(p, {"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}, b"\0" * 16)
    with pytest.raises(LiyabError, match="'x' has the wrong size"):
        SafetensorsFile(p)
    _raw_file(p, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                  "y": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 16)
    with pytest.raises(LiyabError, match="overlap"):
        SafetensorsFile(p)
    _raw_file(p, {"x": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(LiyabError, match="unsupported dtype"):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(struct.pack("<Q", 10) + b'{"x": 1, "x": 2}')
    with pytest.raises(LiyabError):
        SafetensorsFile(p)
    with open(p, "wb") as f:
        f.write(b"abc")
    with pytest.raises(LiyabError, match="too short"):
        SafetensorsFile(p)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    cfg = parse_config(CONFIG_B)
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=1, dtype="float32")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    params = load_parameters(folder, cfg, "float32", "cpu")
    assert params["layers.0.mixer.qkv.weight"].shape == (288, 96)        # [out, in] after the transpose
    assert params["layers.2.feed_forward.down.weight"].shape == (96, 320)
    with SafetensorsFile(os.path.join(folder, "model.safetensors")) as f:
        assert f.entries["h.0.attn.c_attn.weight"].shape == (96, 288)    # the file keeps GPT-2's [in, out]
        assert torch.equal(f.read("h.0.attn.c_attn.weight").t(), params["layers.0.mixer.qkv.weight"])
    # the init scheme: N(0, 0.02), projections back into the stream N(0, 0.02/sqrt(2 L)), gains 1 + N(0, 0.1)
    assert params["embedding.weight"].std().item() == pytest.approx(0.02, rel=0.05)
    assert params["layers.1.feed_forward.down.weight"].std().item() == pytest.approx(0.02 / 6 ** 0.5, rel=0.05)
    assert params["final_norm.weight"].mean().item() == pytest.approx(1.0, abs=0.05)
    # same seed, same values; another seed, other values; values depend on (seed, name, index) only
    again = random_tensors(cfg, 1)
    assert torch.equal(again["wte.weight"].t().t(), params["embedding.weight"])
    assert not torch.equal(random_tensors(cfg, 2)["wte.weight"], again["wte.weight"])
    assert np.array_equal(normal_values(1, "x", 10, 0, 1)[:5], normal_values(1, "x", 5, 0, 1))


def test_storage_types_per_mode(tmp_path):
    cfg = parse_config(CONFIG_A)
    f32 = write_random_model(str(tmp_path / "f32"), cfg, 0, "float32")
    b16 = write_random_model(str(tmp_path / "b16"), cfg, 0, "bfloat16")
    p = load_parameters(f32, cfg, "bfloat16", "cpu")
    assert p["embedding.weight"].dtype == torch.bfloat16 and p["layers.0.mixer.out.weight"].dtype == torch.bfloat16
    assert p["layers.0.mixer.out.bias"].dtype == torch.float32 and p["final_norm.weight"].dtype == torch.float32
    q = load_parameters(b16, cfg, "float32", "cpu")
    assert all(t.dtype == torch.float32 for t in q.values())
    with pytest.raises(LiyabError):
        load_parameters(f32, cfg, "float16", "cpu")


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    cfg = parse_config(CONFIG_A)
    tensors = random_tensors(cfg, 0)
    del tensors["h.1.ln_2.bias"]
    del tensors["wpe.weight"]
    tensors["h.0.attn.c_proj.weight"] = torch.zeros(64, 63)
    tensors["h.7.extra"] = torch.zeros(3)
    tensors["h.0.attn.bias"] = torch.ones(1, 1, 8, 8)          # GPT-2's mask buffer: ignored, not unexpected
    folder = tmp_path / "bad"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg.to_dict()))
    write_safetensors(str(folder / "model.safetensors"), tensors)
    with pytest.raises(LiyabError) as e:
        load_parameters(str(folder), cfg, "float32", "cpu")
    msg = e.value.message
    assert e.value.code == ErrorCode.INVALID_MODEL
    assert "missing tensor 'h.1.ln_2.bias'" in msg and "missing tensor 'wpe.weight'" in msg
    assert "unexpected tensor 'h.7.extra'" in msg and "h.0.attn.bias" not in msg
    assert "tensor 'h.0.attn.c_proj.weight' has shape [64, 63], expected [64, 64]" in msg


def test_names_with_the_transformer_prefix(tmp_path):
    cfg = parse_config(CONFIG_A)
    tensors = {"transformer." + k: v for k, v in random_tensors(cfg, 0).items()}
    tensors["lm_head.weight"] = tensors["transformer.wte.weight"]
    folder = tmp_path / "pref"
    folder.mkdir()
    write_safetensors(str(folder / "model.safetensors"), tensors)
    # lm_head.weight sits outside the prefix: a stored copy of the tied table, not an error
    assert load_parameters(str(folder), cfg, "float32", "cpu")["embedding.weight"].shape == (512, 64)
