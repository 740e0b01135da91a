"""liyab_b200: a single-GPU inference engine for NVIDIA B200 in the manner of
andrei-borcea/liyab, built around one step function over a paged cache.

The engine is a C++ library with a C interface (include/liyab_b200.h); this package
is that interface seen from Python.

    from liyab_b200 import Engine, EngineConfig, SamplingParams
    engine = Engine(EngineConfig(model="/path/to/folder", dtype="bfloat16"))
    result = engine.generate_tokens([464, 3290], SamplingParams(temperature=0.0, max_tokens=16))
"""
from .status import ErrorCode, LiyabError, OutOfPages
from .sampling import SamplingParams

__version__ = "0.2.0"
__all__ = ["ErrorCode", "LiyabError", "OutOfPages", "SamplingParams", "Engine", "EngineConfig", "generate", "__version__"]


def __getattr__(name):
    if name in ("Engine", "EngineConfig", "generate", "GenerationResult", "GenerationStats"):
        from . import engine as _engine
        return getattr(_engine, name)
    raise AttributeError(name)
