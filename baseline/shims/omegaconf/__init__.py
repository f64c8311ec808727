"""Minimal stand-in for ``omegaconf`` (not installed on this image, not in the offline wheelhouse).

The reference's configuration loader (``galvatron/core/arguments.py:125-154``) uses exactly one call of this
package: ``OmegaConf.to_container(cfg, resolve=True)``.  The configuration object handed in is the one produced
by the ``hydra`` stand-in next to this file: a ``DictConfig`` wrapping a plain nested dict, with ``${a.b.c}``
interpolations left as strings until ``resolve=True`` substitutes them.  Nothing here touches a GPU path.
"""
from __future__ import annotations

import copy
import re
from typing import Any

_REF = re.compile(r"\$\{([^${}]+)\}")


class DictConfig:
    """A nested-dict configuration as loaded from YAML (interpolations unresolved)."""

    def __init__(self, content: dict):
        self._content = content


def _lookup(root: dict, dotted: str) -> Any:
    node: Any = root
    for part in dotted.strip().split("."):
        if isinstance(node, list):
            node = node[int(part)]
        else:
            if part not in node:
                raise KeyError("interpolation key '%s' not found" % dotted)
            node = node[part]
    return node


def _resolve_value(value: Any, root: dict, depth: int = 0) -> Any:
    if depth > 32:
        raise ValueError("interpolation cycle")
    if isinstance(value, str):
        whole = _REF.fullmatch(value)
        if whole:  # a value that is exactly one reference keeps the referenced type
            return _resolve_value(_lookup(root, whole.group(1)), root, depth + 1)
        if _REF.search(value):
            return _REF.sub(lambda m: str(_resolve_value(_lookup(root, m.group(1)), root, depth + 1)), value)
        return value
    if isinstance(value, dict):
        return {k: _resolve_value(v, root, depth) for k, v in value.items()}
    if isinstance(value, list):
        return [_resolve_value(v, root, depth) for v in value]
    return value


class OmegaConf:
    @staticmethod
    def create(content: Any = None) -> DictConfig:
        return DictConfig(copy.deepcopy(content or {}))

    @staticmethod
    def to_container(cfg: Any, resolve: bool = False, **_: Any) -> Any:
        content = cfg._content if isinstance(cfg, DictConfig) else cfg
        content = copy.deepcopy(content)
        return _resolve_value(content, content) if resolve else content
