"""Helpers for nested containers of tensors (lists, tuples, namedtuples, dicts).

Flattening order is a state-format contract: dictionaries are traversed in sorted-key order
(reference: hivemind/utils/nested.py:32-43), because optimizer state is shipped as a flat tensor list plus
``nested_flatten``-ordered metadata (hivemind/optim/state_averager.py:719-740).
"""
from __future__ import annotations

from typing import Any, Iterator


def is_namedtuple(x: Any) -> bool:
    return isinstance(x, tuple) and hasattr(type(x), "_fields") and all(isinstance(f, str) for f in type(x)._fields)


def nested_flatten(t: Any) -> Iterator[Any]:
    """Yield the leaves of ``t`` depth-first; dict values come in sorted-key order."""
    if isinstance(t, (list, tuple)):
        for item in t:
            yield from nested_flatten(item)
    elif isinstance(t, dict):
        for key in sorted(t.keys()):
            yield from nested_flatten(t[key])
    else:
        yield t


def _pack(it: Iterator[Any], structure: Any) -> Any:
    if is_namedtuple(structure):
        return type(structure)(*[_pack(it, s) for s in structure])
    if isinstance(structure, (list, tuple)):
        return type(structure)(_pack(it, s) for s in structure)
    if isinstance(structure, dict):
        return {key: _pack(it, structure[key]) for key in sorted(structure.keys())}
    return next(it)


def nested_pack(flat: Any, structure: Any) -> Any:
    """Inverse of :func:`nested_flatten`: arrange the items of ``flat`` in the shape of ``structure``."""
    return _pack(iter(flat), structure)


def nested_compare(t: Any, u: Any) -> bool:
    """True if ``t`` and ``u`` have the same nesting structure (container kinds, lengths, dict keys)."""
    if isinstance(t, (list, tuple)):
        if not isinstance(u, type(t)) or len(t) != len(u):
            return False
        return all(nested_compare(a, b) for a, b in zip(t, u))
    if isinstance(t, dict):
        if not isinstance(u, dict) or set(t.keys()) != set(u.keys()):
            return False
        return all(nested_compare(t[k], u[k]) for k in t)
    return not isinstance(u, (list, tuple, dict))


def nested_map(fn, *t: Any) -> Any:
    """Apply ``fn`` to the corresponding leaves of one or more identically nested structures."""
    if not t:
        raise ValueError("nested_map needs at least one structure")
    for other in t[1:]:
        if not nested_compare(t[0], other):
            raise ValueError("nested structures do not match")
    flat = [list(nested_flatten(x)) for x in t]
    return nested_pack([fn(*leaves) for leaves in zip(*flat)], t[0])
