"""The safetensors container, the by-name loader's errors and the random-weights mode."""
import json
import os
import struct

import numpy as np
import pytest

from liyab_b200 import ErrorCode, LiyabError
from liyab_b200.config import describe_config
from liyab_b200.weights import (bf16_to_f32, f32_to_bf16, load_parameters, normal_values, read_tensor, safetensors_describe,
                                write_random_model, write_safetensors)
from tiny_models import CONFIG_A, CONFIG_B


def file_tensors(folder):
    path = os.path.join(folder, "model.safetensors")
    info = safetensors_describe(path)["tensors"]
    return {name: read_tensor(path, name, i) for name, i in info.items()}


def test_container_round_trip_and_independent_reader(tmp_path):
    path = str(tmp_path / "t.safetensors")
    rng = np.random.default_rng(0)
    tensors = {"a": np.arange(12, dtype=np.float32).reshape(3, 4), "b": f32_to_bf16(rng.standard_normal(5).astype(np.float32)),
               "c": np.array([1, 2, 3], dtype=np.int64), "d": np.zeros((0, 4), dtype=np.float32)}
    write_safetensors(path, tensors, {"k": "v"}, tags={"b": "BF16"})
    d = safetensors_describe(path)
    assert d["metadata"] == {"k": "v"} and d["tensors"]["b"] == {"dtype": "BF16", "shape": [5], "bytes": 10}
    for k, v in tensors.items():
        assert np.array_equal(read_tensor(path, k), v)
    import torch
    from safetensors.torch import load_file           # another implementation reads what we wrote
    other = load_file(path)
    assert torch.equal(other["a"], torch.from_numpy(tensors["a"])) and other["b"].dtype == torch.bfloat16
    assert np.array_equal(other["b"].view(torch.int16).numpy().view(np.uint16), tensors["b"])
    assert torch.equal(other["c"], torch.from_numpy(tensors["c"])) and tuple(other["d"].shape) == (0, 4)


def _raw_file(path, header: dict, data: bytes):
    text = json.dumps(header).encode()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + data)


def test_malformed_files_are_refused_with_the_tensor_named(tmp_path):
    p = str(tmp_path / "m.safetensors")
    _raw_file(p, {"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8)
    with pytest.raises(LiyabError, match="'x'.*truncated"):
        safetensors_describe(p)
    _raw_file(p, {"x": {"dtype": "F32", "shape": [4], "data_offsets": [0, 12]}}, b"\0" * 16)
    with pytest.raises(LiyabError, match="'x' has the wrong size"):
        safetensors_describe(p)
    _raw_file(p, {"x": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]},
                  "y": {"dtype": "F32", "shape": [2], "data_offsets": [4, 12]}}, b"\0" * 16)
    with pytest.raises(LiyabError, match="overlap"):
        safetensors_describe(p)
    _raw_file(p, {"x": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8)
    with pytest.raises(LiyabError, match="unsupported dtype"):
        safetensors_describe(p)
    with open(p, "wb") as f:
        text = b'{"x": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}, "x": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}'
        f.write(struct.pack("<Q", len(text)) + text + b"\0" * 8)
    with pytest.raises(LiyabError, match="'x' appears twice") as e:
        safetensors_describe(p)
    assert e.value.code == ErrorCode.INVALID_MODEL
    with open(p, "wb") as f:
        f.write(b"abc")
    with pytest.raises(LiyabError, match="too short"):
        safetensors_describe(p)
    with pytest.raises(LiyabError) as e:
        safetensors_describe(str(tmp_path / "absent.safetensors"))
    assert e.value.code == ErrorCode.IO_ERROR


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), CONFIG_B, seed=1, dtype="float32")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    params = load_parameters(folder, "float32")
    assert params["layers.0.mixer.qkv.weight"].shape == (288, 96)        # [out, in] after the transpose
    assert params["layers.2.feed_forward.down.weight"].shape == (96, 320)
    stored = file_tensors(folder)
    assert stored["h.0.attn.c_attn.weight"].shape == (96, 288)           # the file keeps GPT-2's [in, out]
    assert np.array_equal(stored["h.0.attn.c_attn.weight"].T, params["layers.0.mixer.qkv.weight"])
    # the init scheme: N(0, 0.02), projections back into the stream N(0, 0.02/sqrt(2 L)), gains 1 + N(0, 0.1)
    assert params["embedding.weight"].std() == pytest.approx(0.02, rel=0.05)
    assert params["layers.1.feed_forward.down.weight"].std() == pytest.approx(0.02 / 6 ** 0.5, rel=0.05)
    assert params["final_norm.weight"].mean() == pytest.approx(1.0, abs=0.05)
    # same seed, same values; another seed, other values; values depend on (seed, name, index) only
    again = file_tensors(write_random_model(str(tmp_path / "m2"), CONFIG_B, seed=1, dtype="float32"))
    assert np.array_equal(again["wte.weight"], params["embedding.weight"])
    other = file_tensors(write_random_model(str(tmp_path / "m3"), CONFIG_B, seed=2, dtype="float32"))
    assert not np.array_equal(other["wte.weight"], again["wte.weight"])
    assert np.array_equal(normal_values(1, "x", 10, 0, 1)[:5], normal_values(1, "x", 5, 0, 1))
    assert np.array_equal(normal_values(1, "x", 10, 0, 1)[4:], normal_values(1, "x", 6, 0, 1, first=4))
    wte = normal_values(1, "wte.weight", 1000 * 96, 0.0, 0.02).astype(np.float32).reshape(1000, 96)
    assert np.array_equal(wte, again["wte.weight"])
    # the folder's config.json reads back to the same typed configuration
    assert describe_config(json.load(open(os.path.join(folder, "config.json"))))["config"] == describe_config(CONFIG_B)["config"]


def test_storage_types_per_mode(tmp_path):
    f32 = write_random_model(str(tmp_path / "f32"), CONFIG_A, 0, "float32")
    b16 = write_random_model(str(tmp_path / "b16"), CONFIG_A, 0, "bfloat16")
    p = load_parameters(f32, "bfloat16")
    assert p["embedding.weight"].dtype == np.uint16 and p["layers.0.mixer.out.weight"].dtype == np.uint16      # bfloat16 bits
    assert p["layers.0.mixer.out.bias"].dtype == np.float32 and p["final_norm.weight"].dtype == np.float32
    full = load_parameters(f32, "float32")
    assert np.array_equal(p["embedding.weight"], f32_to_bf16(full["embedding.weight"]))        # rounded to nearest even
    q = load_parameters(b16, "float32")
    assert all(t.dtype == np.float32 for t in q.values())
    assert np.array_equal(q["embedding.weight"], bf16_to_f32(f32_to_bf16(full["embedding.weight"])))
    with pytest.raises(LiyabError):
        load_parameters(f32, "float16")


def test_one_error_lists_missing_unexpected_and_misshapen(tmp_path):
    tensors = file_tensors(write_random_model(str(tmp_path / "good"), CONFIG_A, 0))
    del tensors["h.1.ln_2.bias"]
    del tensors["wpe.weight"]
    tensors["h.0.attn.c_proj.weight"] = np.zeros((64, 63), dtype=np.float32)
    tensors["h.7.extra"] = np.zeros(3, dtype=np.float32)
    tensors["h.0.attn.bias"] = np.ones((1, 1, 8, 8), dtype=np.float32)          # GPT-2's mask buffer: ignored, not unexpected
    folder = tmp_path / "bad"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(CONFIG_A))
    write_safetensors(str(folder / "model.safetensors"), tensors)
    with pytest.raises(LiyabError) as e:
        load_parameters(str(folder), "float32")
    msg = e.value.message
    assert e.value.code == ErrorCode.INVALID_MODEL
    assert "missing tensor 'h.1.ln_2.bias'" in msg and "missing tensor 'wpe.weight'" in msg
    assert "unexpected tensor 'h.7.extra'" in msg and "h.0.attn.bias" not in msg
    assert "tensor 'h.0.attn.c_proj.weight' has shape [64, 63], expected [64, 64]" in msg


def test_names_with_the_transformer_prefix_and_shards(tmp_path):
    tensors = {"transformer." + k: v for k, v in file_tensors(write_random_model(str(tmp_path / "good"), CONFIG_A, 0)).items()}
    tensors["lm_head.weight"] = tensors["transformer.wte.weight"]
    folder = tmp_path / "pref"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(CONFIG_A))
    write_safetensors(str(folder / "model.safetensors"), tensors)
    # lm_head.weight sits outside the prefix: a stored copy of the tied table, not an error
    whole = load_parameters(str(folder), "float32")
    assert whole["embedding.weight"].shape == (512, 64)
    # the same tensors spread over two files with an index
    shards = tmp_path / "shards"
    shards.mkdir()
    (shards / "config.json").write_text(json.dumps(CONFIG_A))
    names = list(tensors)
    parts = {"model-00001-of-00002.safetensors": names[:7], "model-00002-of-00002.safetensors": names[7:]}
    for fname, ns in parts.items():
        write_safetensors(str(shards / fname), {n: tensors[n] for n in ns})
    (shards / "model.safetensors.index.json").write_text(json.dumps({"weight_map": {n: f for f, ns in parts.items() for n in ns}}))
    spread = load_parameters(str(shards), "float32")
    assert spread.keys() == whole.keys() and all(np.array_equal(spread[k], whole[k]) for k in whole)


def test_parameters_joined_and_cut_from_several_file_tensors(tmp_path):
    """A checkpoint map may build one parameter from several tensors of the file (separate q, k, v matrices joined
    into the fused projection) or from a part of one (a half of a fused matrix)."""
    spec = describe_config(CONFIG_A)["spec"]
    d = describe_config({"model_type": "liyab_spec", "spec": spec})
    ck = d["checkpoint"]
    qkv = "layers.0.mixer.qkv.weight"
    ck[qkv] = {"sources": [{"name": f"blk0.{n}", "shape": [64, 64]} for n in "qkv"], "transform": "transpose", "concat_axis": 0, "kind": "matrix"}
    up = "layers.0.feed_forward.up.weight"
    ck[up] = {"sources": [{"name": "blk0.gate_up", "shape": [512, 64]}], "slice": {"axis": 0, "begin": 256, "end": 512}, "kind": "matrix"}
    folder = tmp_path / "joined"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps({"model_type": "liyab_spec", "spec": spec, "checkpoint": ck}))
    rng = np.random.default_rng(3)
    tensors = {}
    for dest, entry in ck.items():
        for s in entry["sources"]:
            tensors[s["name"]] = rng.standard_normal(s["shape"]).astype(np.float32)
    write_safetensors(str(folder / "model.safetensors"), tensors)
    p = load_parameters(str(folder), "float32")
    assert np.array_equal(p[qkv], np.concatenate([tensors[f"blk0.{n}"].T for n in "qkv"], axis=0))
    assert np.array_equal(p[up], tensors["blk0.gate_up"][256:512])
