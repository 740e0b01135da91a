"""liyab_b200: a single-GPU inference engine for NVIDIA B200 in the manner of
andrei-borcea/liyab, built around one step function over a paged cache."""
from .status import ErrorCode, LiyabError

__version__ = "0.1.0"
__all__ = ["ErrorCode", "LiyabError", "__version__"]
