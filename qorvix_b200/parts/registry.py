"""Registries of part builders.  A part kind ('attention', 'swiglu', 'rmsnorm', 'rotary',
'pre_norm', or one a user adds) maps to a callable `build(spec, source, rt)` that returns
the part.  Adding a mixer, feed-forward, norm, position encoding or block arrangement is one
`register_part` call; nothing else in the package changes.
"""
from __future__ import annotations

from typing import Callable, Dict

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block")
_PARTS: Dict[str, Dict[str, Callable]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, builder: Callable, *, replace: bool = False) -> None:
    if category not in _PARTS:
        raise ValueError(f"unknown part category '{category}' (known: {', '.join(CATEGORIES)})")
    if kind in _PARTS[category] and not replace:
        raise ValueError(f"{category} '{kind}' is already registered")
    _PARTS[category][kind] = builder


def unregister_part(category: str, kind: str) -> None:
    _PARTS[category].pop(kind, None)


def build_part(category: str, spec, source, rt):
    """Builds the part that `spec.kind` names (None stays None)."""
    if spec is None:
        return None
    kind = getattr(spec, "kind", None)
    table = _PARTS[category]
    if kind not in table:
        raise KeyError(f"no {category} of kind '{kind}' is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[kind](spec, source, rt)


def registered_parts(category: str) -> list:
    return sorted(_PARTS[category])
