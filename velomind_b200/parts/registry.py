"""Registries of part kinds.  A part is looked up by (role, kind) when a model is built from its plan.

Roles: "norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head".
Registering a new kind needs no change to this package: call `register_part(role, kind, factory)`
and name the kind in a `PartSpec`.
"""
from __future__ import annotations

from typing import Callable, Dict, Tuple

from .spec import PartSpec

ROLES = ("norm", "position", "mixer", "feed_forward", "arrangement", "embedding", "head")
_PARTS: Dict[Tuple[str, str], Callable] = {}


def register_part(role: str, kind: str, factory: Callable) -> None:
    """`factory(**spec.args)` returns the part.  Re-registering a kind replaces it."""
    if role not in ROLES:
        raise ValueError(f"unknown role {role!r}; roles: {', '.join(ROLES)}")
    _PARTS[(role, kind)] = factory


def unregister_part(role: str, kind: str) -> None:
    _PARTS.pop((role, kind), None)


def registered_parts(role: str):
    return sorted(k for r, k in _PARTS if r == role)


def build_part(role: str, spec: PartSpec):
    try:
        factory = _PARTS[(role, spec.kind)]
    except KeyError:
        raise ValueError(f"no {role} of kind {spec.kind!r} is registered; registered: "
                         f"{', '.join(registered_parts(role)) or '(none)'}") from None
    return factory(**spec.args)
