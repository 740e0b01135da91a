"""Leveled diagnostics with a sink (the reference's logger: src/core/log.h:14-35, liyab_c_api.h:200-221)."""
import json

import numpy as np

from liyab_b200.engine import set_log
from liyab_b200.weights import load_parameters, read_tensor, safetensors_describe, write_random_model, write_safetensors
from tiny_models import CONFIG_A


def test_messages_reach_the_callback_at_or_above_the_level(tmp_path):
    folder = write_random_model(str(tmp_path / "m"), CONFIG_A, 0)
    path = str(tmp_path / "m" / "model.safetensors")
    tensors = {n: read_tensor(path, n, i) for n, i in safetensors_describe(path)["tensors"].items()}
    tensors["lm_head.weight"] = tensors["wte.weight"]            # a stored copy of the tied head: ignored, and said so at level info
    write_safetensors(path, tensors)
    seen = []
    try:
        set_log(1, lambda level, message: seen.append((level, message)))
        load_parameters(folder, "float32")
        assert any(level == 1 and "lm_head.weight" in message and "ignored" in message for level, message in seen)
        seen.clear()
        set_log(2, lambda level, message: seen.append((level, message)))
        load_parameters(folder, "float32")
        assert not seen                                           # below the level now
    finally:
        set_log(2, None)
