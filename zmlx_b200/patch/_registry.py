"""Name -> pattern table of the patch framework.

The function names (``register``, ``get_pattern``, ``list_patterns``, ``get_all_patterns``) and the wording of the
unknown-name error are the interface of src/zmlx/patch/_registry.py:8-49; third-party patterns register themselves
through them.
"""

from __future__ import annotations

import importlib

from ._types import PatchPattern

# modules whose import registers this package's own patterns
_BUILTIN_MODULES = ("deepseek_router", "moe_mlp", "swiglu_mlp")


class _Table:
    """The registry proper: patterns by name; the built-in ones are imported on first use."""

    def __init__(self) -> None:
        self.by_name: dict[str, PatchPattern] = {}
        self.builtins_imported = False

    def import_builtins(self) -> None:
        if self.builtins_imported:
            return
        self.builtins_imported = True  # set first: the imported modules call register(), which must not recurse
        for mod in _BUILTIN_MODULES:
            importlib.import_module(f"{__package__}.patterns.{mod}")


_TABLE = _Table()


def _ensure_loaded() -> None:
    _TABLE.import_builtins()


def register(pattern: PatchPattern) -> PatchPattern:
    """Adds (or replaces) a pattern under its own name; returns it, so it can be used as a decorator target."""
    _TABLE.by_name[pattern.name] = pattern
    return pattern


def list_patterns() -> list[str]:
    _ensure_loaded()
    return sorted(_TABLE.by_name)


def get_all_patterns() -> dict[str, PatchPattern]:
    _ensure_loaded()
    return dict(_TABLE.by_name)


def get_pattern(name: str) -> PatchPattern:
    _ensure_loaded()
    found = _TABLE.by_name.get(name)
    if found is None:
        raise KeyError(f"Unknown patch pattern: {name!r}. Available: {list_patterns()}")
    return found
