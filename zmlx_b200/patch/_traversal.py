"""Depth-first walk of a torch module tree that applies matching patterns (src/zmlx/patch/_traversal.py:10-81)."""

from __future__ import annotations

from typing import Any

import torch.nn as nn

from ._types import PatchConfig, PatchPattern, PatchResult


def _walk_modules(module: Any, patterns: list[PatchPattern], config: PatchConfig, result: PatchResult,
                  path: str = "") -> None:
    children = dict(module.named_children()) if isinstance(module, nn.Module) else {}
    for child_name, child in children.items():
        child_path = f"{path}.{child_name}" if path else child_name
        _walk_modules(child, patterns, config, result, child_path)
    for child_name, child in children.items():
        child_path = f"{path}.{child_name}" if path else child_name
        for pattern in patterns:
            if pattern.matches(child, child_name, parent=module):
                try:
                    replacement = pattern.apply(child, config)
                    if replacement is not child:
                        setattr(module, child_name, replacement)
                    result.patched_count += 1
                    result.pattern_counts[pattern.name] = result.pattern_counts.get(pattern.name, 0) + 1
                    if config.verbose:
                        print(f"  [zmlx.patch] {child_path}: {pattern.name}")
                except Exception as e:  # the reference records and moves on
                    result.skipped.append(f"{child_path}: {e}")
                break


def apply_patterns(model: Any, patterns: list[PatchPattern], config: PatchConfig) -> PatchResult:
    result = PatchResult()
    _walk_modules(model, patterns, config, result)
    return result
