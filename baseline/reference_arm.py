"""The reference arm of bench.py: the unmodified reference, through its own tools, for the benchmark's metric.

liyab is a CMake C++ project without a Python package (pip finds neither setup.py nor pyproject.toml), so it is
configured and built with cmake into baseline/_ref/build, which is not part of the repository's history."""
from __future__ import annotations

import json


def run(args) -> int:
    print(json.dumps({"impl": "reference", "unavailable": "the reference arm is not set up in this checkout (baseline/_ref is absent)"}))
    return 0
