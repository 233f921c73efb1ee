"""Parts by kind and name, so that a configuration can choose them layer by layer.

Kinds: "mixer" (attention and whatever else mixes tokens), "feed_forward", "norm", "position",
"block" (the arrangement of the others around the residual stream).  Registering a class under a new
name is all it takes to make it choosable; nothing else in the framework lists the parts.
"""
from __future__ import annotations

KINDS = ("mixer", "feed_forward", "norm", "position", "block")
_PARTS: dict[str, dict[str, type]] = {k: {} for k in KINDS}


def register_part(kind: str, name: str, cls: type | None = None, *, replace: bool = False):
    """`register_part("mixer", "toy", Toy)` or as a decorator `@register_part("mixer", "toy")`."""
    if kind not in _PARTS:
        raise ValueError(f"unknown kind of part '{kind}'; kinds: {', '.join(KINDS)}")

    def _do(c: type) -> type:
        if name in _PARTS[kind] and not replace:
            raise ValueError(f"{kind} '{name}' is already registered")
        _PARTS[kind][name] = c
        return c

    return _do if cls is None else _do(cls)


def unregister_part(kind: str, name: str) -> None:
    _PARTS[kind].pop(name, None)


def get_part(kind: str, name: str) -> type:
    try:
        return _PARTS[kind][name]
    except KeyError:
        known = ", ".join(sorted(_PARTS.get(kind, {}))) or "(none)"
        raise KeyError(f"no {kind} registered under '{name}'; registered: {known}") from None


def part_names(kind: str) -> list[str]:
    return sorted(_PARTS[kind])
