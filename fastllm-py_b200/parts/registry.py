"""Registries of parts: kind name -> class, one table per category.

A ModelPlan names parts by (category, kind); the decoder looks the class up
here.  Registering a new mixer, feed-forward, norm, position encoding, block
arrangement, embedding or head is one call of `register_part` and needs no
change anywhere else; tests do exactly that with toy parts.
"""
from __future__ import annotations

CATEGORIES = ("mixer", "feed_forward", "norm", "position", "block", "embedding", "head")
_PARTS: dict = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str, cls=None):
    """`register_part("mixer", "my_mixer", MyMixer)` or as a class decorator."""
    if category not in _PARTS:
        raise ValueError(f"unknown part category {category!r} (one of {CATEGORIES})")

    def put(c):
        _PARTS[category][kind] = c
        return c

    return put if cls is None else put(cls)


def part_class(category: str, kind: str):
    try:
        return _PARTS[category][kind]
    except KeyError:
        raise ValueError(f"no {category} part of kind {kind!r} is registered "
                         f"(known: {sorted(_PARTS.get(category, {}))})") from None


def build_part(category: str, spec, ctx):
    return part_class(category, spec.kind)(spec, ctx)
