"""Typed failures.

Every refusal of the engine is a :class:`GessoError` carrying one code, so a
caller can tell a bad model folder from an exhausted cache from a numerical
failure.  The code names follow the reference's taxonomy
(src/errors.jl:39-56); only the codes this engine can actually raise are kept.
"""
from __future__ import annotations

import enum


class ErrorCode(enum.IntEnum):
    INTERNAL = 0                 # a bug in this engine
    INVALID_PLAN = 1             # malformed request / configuration, refused before any work
    COMPILE = 3                  # the CUDA library could not be built or loaded
    RESOURCE_LIMIT = 4           # pages, slots, context length or batch exhausted
    ALLOCATION = 5               # device allocation failure
    LAUNCH = 6                   # a kernel launch was refused (size the kernel does not take)
    RUNTIME = 7                  # failure while a request was running (callback, cancelled step)
    NUMERICAL_INSTABILITY = 10   # NaN / Inf where a token would be emitted


class GessoError(RuntimeError):
    """One failure: ``code`` (an :class:`ErrorCode`) and a diagnostic message."""

    def __init__(self, code: ErrorCode, message: str):
        super().__init__(f"[{ErrorCode(code).name}] {message}")
        self.code = ErrorCode(code)
        self.message = message


def invalid(message: str) -> GessoError:
    return GessoError(ErrorCode.INVALID_PLAN, message)


def resource(message: str) -> GessoError:
    return GessoError(ErrorCode.RESOURCE_LIMIT, message)
