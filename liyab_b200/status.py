"""Error codes and the one exception type the engine raises.

The codes and their numbers are the reference's (include/liyab/types.h:36-48,
mirrored by the C enum at include/liyab/liyab_c_api.h:41-53), so a caller that
already switches on liyab's status values keeps working.
"""
from __future__ import annotations

import enum


class ErrorCode(enum.IntEnum):
    OK = 0
    INVALID_ARGUMENT = 1
    IO_ERROR = 2
    INVALID_MODEL = 3
    UNSUPPORTED = 4
    OUT_OF_MEMORY = 5
    CONTEXT_FULL = 6
    CANCELLED = 7
    BACKEND_ERROR = 8
    BUSY = 9
    INTERNAL = 10


class LiyabError(Exception):
    """An engine failure with a reference status code and a message that names
    the key, tensor or request at fault."""

    def __init__(self, code: ErrorCode, message: str):
        super().__init__(f"{code.name}: {message}")
        self.code = code
        self.message = message


def invalid_argument(msg: str) -> LiyabError:
    return LiyabError(ErrorCode.INVALID_ARGUMENT, msg)


def invalid_model(msg: str) -> LiyabError:
    return LiyabError(ErrorCode.INVALID_MODEL, msg)


def unsupported(msg: str) -> LiyabError:
    return LiyabError(ErrorCode.UNSUPPORTED, msg)


def out_of_memory(msg: str) -> LiyabError:
    return LiyabError(ErrorCode.OUT_OF_MEMORY, msg)


def context_full(msg: str) -> LiyabError:
    return LiyabError(ErrorCode.CONTEXT_FULL, msg)


def backend_error(msg: str) -> LiyabError:
    return LiyabError(ErrorCode.BACKEND_ERROR, msg)


class OutOfPages(LiyabError):
    """A reservation that the free pages cannot cover; nothing was taken."""

