"""Records and the pattern protocol of the patch framework.

The field names, defaults and method names are the interface of src/zmlx/patch/_types.py:7-51, which callers of
``patch()`` and writers of patterns rely on; everything else here is this package's own.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Protocol, runtime_checkable


@dataclasses.dataclass(frozen=True)
class PatchConfig:
    """What ``patch()`` hands to every pattern's ``apply``."""

    compute_dtype: str = "float32"
    threadgroup: int | str = 256  # kept for signature compatibility: CUDA launch shapes are chosen by the library
    verbose: bool = False
    moe_fused_swiglu_max_tokens: int | None = None


@dataclasses.dataclass
class PatchResult:
    """What ``patch()`` did: modules rewritten in total and per pattern, modules a pattern gave up on."""

    patched_count: int = 0
    pattern_counts: dict[str, int] = dataclasses.field(default_factory=dict)
    skipped: list[str] = dataclasses.field(default_factory=list)
    benchmarks: dict[str, float] = dataclasses.field(default_factory=dict)  # pattern -> measured speed-up, if any

    def summary(self) -> str:
        """Human-readable report, one line per pattern in alphabetical order."""

        def line(pattern: str) -> str:
            text = f"  {pattern}: {self.pattern_counts[pattern]}"
            if pattern in self.benchmarks:
                text += f" ({self.benchmarks[pattern]:.3f}x)"
            return text

        report = [f"Patched {self.patched_count} modules:", *map(line, sorted(self.pattern_counts))]
        if self.skipped:
            report.append(f"  Skipped: {len(self.skipped)}")
        return "\n".join(report)


@runtime_checkable
class PatchPattern(Protocol):
    """A pattern names itself, says whether a module is its business, and rewrites it in place."""

    @property
    def name(self) -> str: ...

    def matches(self, module: Any, name: str, parent: Any | None = None) -> bool: ...

    def apply(self, module: Any, config: PatchConfig) -> Any: ...
