"""Which class builds which part: one table per category, keyed by a spec's `kind`.

Categories: "mixer", "feed_forward", "norm", "position", "block", "embedding", "head". A new
part registers its class under a new kind; a configuration that names that kind in its
ModelSpec gets it built, with no change to the engine. The interface each class must have is
in `kapel_b200.parts.base`.
"""
from __future__ import annotations

from typing import Dict, Tuple

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_PARTS: Dict[Tuple[str, str], type] = {}


def register_part(category: str, kind: str, cls: type) -> None:
    if category not in CATEGORIES:
        raise ValueError(f"unknown part category {category!r}; one of {CATEGORIES}")
    key = (category, kind)
    if key in _PARTS and _PARTS[key] is not cls:
        raise ValueError(f"{category} kind {kind!r} is already registered")
    _PARTS[key] = cls


def unregister_part(category: str, kind: str) -> None:
    _PARTS.pop((category, kind), None)


def part_class(category: str, kind: str) -> type:
    try:
        return _PARTS[(category, kind)]
    except KeyError:
        known = sorted(k for c, k in _PARTS if c == category)
        raise KeyError(f"no {category} of kind {kind!r} is registered (known: {known})") from None


def build_part(category: str, spec, ctx):
    return part_class(category, spec.kind)(spec, ctx)


def register_mixer(kind, cls): register_part("mixer", kind, cls)
def register_feed_forward(kind, cls): register_part("feed_forward", kind, cls)
def register_norm(kind, cls): register_part("norm", kind, cls)
def register_position(kind, cls): register_part("position", kind, cls)
def register_block(kind, cls): register_part("block", kind, cls)
