"""Named operations for ``loop-explore --op-name`` (the reference keeps such a
registry in ``artifacts/operations.py:8-70``, filled from its benchmark tables).

Only the operations this backend's own benchmark configurations use are
registered here; ``register_operation`` adds more.
"""

from __future__ import annotations

_REGISTRY: dict[str, dict[str, dict]] = {}


def register_operation(operator: str, name: str, dims: dict[str, int]) -> None:
    _REGISTRY.setdefault(operator, {})[name.lower()] = {"name": name, "dims": dict(dims)}


def get_operation(operator: str, name: str) -> dict:
    try:
        return _REGISTRY[operator][name.lower()]
    except KeyError:
        raise ValueError(f"operation {name!r} is not registered for operator {operator!r}") from None


def has_operation(operator: str, name: str) -> bool:
    return name.lower() in _REGISTRY.get(operator, {})


def list_operations(operator: str = "") -> list[tuple[str, str]]:
    ops = [operator] if operator else sorted(_REGISTRY)
    return [(o, e["name"]) for o in ops for e in _REGISTRY.get(o, {}).values()]


register_operation("matmul", "c1", {"i": 512, "j": 256, "k": 1024})
register_operation("matmul_relu", "c2", {"i": 4096, "j": 4096, "k": 4096})
register_operation("matmul", "c4_gemm", {"i": 8192, "j": 1024, "k": 8192})
register_operation("matmul", "c5_shard8", {"i": 8192, "j": 8192, "k": 8192})
register_operation("conv2d", "c3_conv", {"n": 32, "h": 56, "w": 56, "f": 64, "r": 3, "s": 3, "c": 64,
                                         "SH": 1, "SW": 1})
