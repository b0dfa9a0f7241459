"""Kernel plugin registry: maps ``(op_name, backend)`` to a kernel class.

Mirrors the four public functions of the reference registry
(ezops/registry.py:4-54): ``register_kernel`` stamps ``op_name`` / ``backend``
on the class and refuses duplicates with ``ValueError``; ``get_kernel`` raises
``KeyError`` naming the backends that do exist.  The reference wraps
``__call__`` in a TileLang cache-naming scope (registry.py:19-29); this package
has no TileLang backend, so classes are stored unwrapped.
"""

from __future__ import annotations

_REGISTRY: dict[tuple[str, str], type] = {}


def register_kernel(op_name: str, backend: str):
    """Class decorator: make ``cls`` the ``backend`` implementation of ``op_name``."""

    def decorator(cls):
        key = (op_name, backend)
        prior = _REGISTRY.get(key)
        if prior is not None:
            raise ValueError(f"Kernel already registered for ({op_name!r}, {backend!r}): {prior.__name__}")
        cls.op_name = op_name
        cls.backend = backend
        _REGISTRY[key] = cls
        return cls

    return decorator


def get_kernel(op_name: str, backend: str) -> type:
    try:
        return _REGISTRY[(op_name, backend)]
    except KeyError:
        have = list_backends(op_name)
        raise KeyError(
            f"No kernel registered for ({op_name!r}, {backend!r}). Available backends for {op_name!r}: {have!r}"
        ) from None


def list_backends(op_name: str) -> list[str]:
    return [b for (name, b) in _REGISTRY if name == op_name]


def list_ops() -> list[str]:
    return sorted({name for (name, _) in _REGISTRY})
