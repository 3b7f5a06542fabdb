"""Error convention of the backend surface.

Same contract as the reference's ``CompilerError`` (src/megabake/diagnostics.py:6-32):
a ``ValueError`` carrying a structured diagnostic and a ``safe_for_fallback``
flag, rendered as ``stage: message; source operations: ...; regions: ...;
requirement: ...``.
"""

from __future__ import annotations

from typing import NamedTuple, Optional, Tuple


class CompilerDiagnostic(NamedTuple):
    stage: str
    message: str
    source_op_ids: Tuple[str, ...] = ()
    region_ids: Tuple[str, ...] = ()
    requirement: Optional[str] = None

    def render(self) -> str:
        text = [f"{self.stage}: {self.message}"]
        for label, items in (("source operations", self.source_op_ids), ("regions", self.region_ids)):
            if items:
                text.append(f"{label}: " + ", ".join(items))
        if self.requirement:
            text.append(f"requirement: {self.requirement}")
        return "; ".join(text)


class CompilerError(ValueError):
    """Raised before any device work when a graph or binding cannot run on the megakernel."""

    def __init__(self, diagnostic: CompilerDiagnostic, *, safe_for_fallback: bool = False):
        ValueError.__init__(self, diagnostic.message)
        self.diagnostic = diagnostic
        self.safe_for_fallback = bool(safe_for_fallback)

    def __str__(self) -> str:
        return self.diagnostic.render()
