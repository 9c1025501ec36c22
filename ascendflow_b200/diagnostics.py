"""Caller-actionable errors of the host side.

The reference raises one exception type, `CompileError` (a `ValueError`), for every violated
contract, tagged with a category (`src/diagnostics.py:6-35` of the reference); its tests and
callers match on the type and on the message. This module provides the same names so that code
written against the reference keeps working: `ErrorKind`, `CompileError`, `require`.
"""

import enum


class ErrorKind(str, enum.Enum):
    """Category of a failure; the values are the reference's strings."""

    INVALID = "invalid-input"
    UNSUPPORTED = "unsupported"
    RESOURCE = "resource-exhausted"
    ANALYSIS_LIMIT = "analysis-limit"

    def __str__(self):
        return self.value


def _render(message, phase, location, witness):
    """`message [phase, location]: witness; witness`, leaving out what is absent."""
    parts = [message]
    origin = ", ".join(str(value) for value in (phase, location) if value is not None)
    if origin:
        parts.append(f" [{origin}]")
    if witness:
        parts.append(": " + "; ".join(map(str, witness)))
    return "".join(parts)


class CompileError(ValueError):
    """A bad tensor, a bad size, a closed runtime, a missing or stale library."""

    def __init__(self, message, *, kind=ErrorKind.INVALID, phase=None, location=None, witness=()):
        self.message, self.kind = message, ErrorKind(kind)
        self.phase, self.location, self.witness = phase, location, tuple(witness)
        super().__init__(_render(message, phase, location, self.witness))


def require(condition, message, **context):
    """Raise `CompileError(message, **context)` unless `condition` holds."""
    if condition:
        return
    raise CompileError(message, **context)
