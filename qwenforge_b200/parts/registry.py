"""Registries from a part's kind (the name in a `PartSpec`) to its class, one per role.
A new part is one class and one `register_*` call; specs can name it from then on."""
from __future__ import annotations

from ..config.spec import PartSpec

_ROLES = ("norm", "mixer", "feed_forward", "position", "block", "embedding", "head")
_REGISTRY: dict[str, dict[str, type]] = {role: {} for role in _ROLES}


def register_part(role: str, kind: str, cls: type) -> None:
    if role not in _REGISTRY:
        raise ValueError(f"unknown part role {role!r}; roles: {', '.join(_ROLES)}")
    _REGISTRY[role][kind] = cls
    cls.kind = kind


def build_part(role: str, spec: PartSpec):
    kinds = _REGISTRY[role]
    if spec.kind not in kinds:
        raise ValueError(f"no {role} part of kind {spec.kind!r} is registered; known: {', '.join(sorted(kinds)) or 'none'}")
    return kinds[spec.kind](spec)


def registered_parts(role: str) -> list[str]:
    return sorted(_REGISTRY[role])


def build_block(layer_spec):
    """The arrangement named by `layer_spec.block`, built over the layer's named part specs."""
    kinds = _REGISTRY["block"]
    if layer_spec.block not in kinds:
        raise ValueError(f"no block of kind {layer_spec.block!r} is registered; known: {', '.join(sorted(kinds)) or 'none'}")
    return kinds[layer_spec.block](layer_spec)
