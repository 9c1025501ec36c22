"""Error type of the host runtime.

Mirrors the reference's `src/diagnostics.py:6-35`: contract violations raise
`CompileError` (a `ValueError`) through `require`, with a category.
"""

from enum import StrEnum


class ErrorKind(StrEnum):
    INVALID = "invalid-input"
    UNSUPPORTED = "unsupported"
    RESOURCE = "resource-exhausted"
    ANALYSIS_LIMIT = "analysis-limit"


class CompileError(ValueError):
    """A caller-actionable failure: bad tensor, bad size, closed runtime, missing library."""

    def __init__(self, message, *, kind=ErrorKind.INVALID, phase=None, location=None, witness=()):
        self.message = message
        self.kind = ErrorKind(kind)
        self.phase = phase
        self.location = location
        self.witness = tuple(witness)
        where = [str(item) for item in (phase, location) if item is not None]
        text = message + (" [" + ", ".join(where) + "]" if where else "")
        if self.witness:
            text += ": " + "; ".join(str(item) for item in self.witness)
        super().__init__(text)


def require(condition, message, **context):
    if not condition:
        raise CompileError(message, **context)
