"""Pattern registry (src/zmlx/patch/_registry.py:8-49)."""

from __future__ import annotations

from ._types import PatchPattern

_PATTERNS: dict[str, PatchPattern] = {}


def register(pattern: PatchPattern) -> PatchPattern:
    _PATTERNS[pattern.name] = pattern
    return pattern


def get_pattern(name: str) -> PatchPattern:
    _ensure_loaded()
    if name not in _PATTERNS:
        raise KeyError(f"Unknown patch pattern: {name!r}. Available: {list_patterns()}")
    return _PATTERNS[name]


def list_patterns() -> list[str]:
    _ensure_loaded()
    return sorted(_PATTERNS.keys())


def get_all_patterns() -> dict[str, PatchPattern]:
    _ensure_loaded()
    return dict(_PATTERNS)


_LOADED = False


def _ensure_loaded() -> None:
    global _LOADED
    if _LOADED:
        return
    _LOADED = True
    from .patterns import deepseek_router, moe_mlp, swiglu_mlp  # noqa: F401
