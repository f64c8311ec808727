"""Minimal stand-in for ``hydra`` (not installed on this image, not in the offline wheelhouse).

The reference's configuration loader (``galvatron/core/arguments.py:125-154``) uses two calls:
``initialize_config_dir(config_dir=..., version_base=None)`` as a context manager and
``compose(config_name=<file>.yaml, overrides=[...])``.  This module does what those two do for the reference's
YAML files, which have no ``defaults`` list: read one YAML file from the directory and apply the override grammar
``key.path=value``, ``+key.path=value`` (add), ``++key.path=value`` (add or replace), ``~key.path`` (delete);
values are parsed as YAML scalars, so ``true``, ``null``, ``1e-4`` and ``[1,2]`` keep their types.  The result is
an ``omegaconf.DictConfig`` of the sibling stand-in.  It is a configuration reader only; no GPU code is involved.
"""
from __future__ import annotations

import contextlib
import os
from typing import Any, List, Optional

import yaml
from omegaconf import DictConfig

_CONFIG_DIR: List[str] = []


class _Loader(yaml.SafeLoader):
    pass


# YAML 1.1 does not read "6.0e-4" style floats without a sign in the exponent as floats in every case; Hydra
# (through OmegaConf) does, so the resolver is widened the way OmegaConf's loader widens it.
import re as _re
_Loader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    _re.compile(r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
                    |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
                    |\.[0-9_]+(?:[eE][-+]?[0-9]+)?
                    |[-+]?\.(?:inf|Inf|INF)|\.(?:nan|NaN|NAN))$""", _re.X),
    list("-+0123456789."))


def _parse_scalar(text: str) -> Any:
    if text == "":
        return ""
    return yaml.load(text, Loader=_Loader)


@contextlib.contextmanager
def initialize_config_dir(config_dir: str, version_base: Optional[str] = None, job_name: str = "app"):
    _CONFIG_DIR.append(os.path.abspath(config_dir))
    try:
        yield
    finally:
        _CONFIG_DIR.pop()


def _set(root: dict, dotted: str, value: Any, must_exist: bool, may_exist: bool) -> None:
    parts = dotted.split(".")
    node = root
    for p in parts[:-1]:
        if p not in node or node[p] is None:
            if must_exist:
                raise KeyError("override '%s': key '%s' is not in the config (use +%s=... to add it)" % (dotted, p, dotted))
            node[p] = {}
        node = node[p]
    leaf = parts[-1]
    if must_exist and leaf not in node:
        raise KeyError("override '%s': key is not in the config (use +%s=... to add it)" % (dotted, dotted))
    if not may_exist and leaf in node:
        raise KeyError("override '+%s': key already exists (use ++ to replace it)" % dotted)
    node[leaf] = value


def compose(config_name: str, overrides: Optional[List[str]] = None, **_: Any) -> DictConfig:
    if not _CONFIG_DIR:
        raise RuntimeError("compose() outside initialize_config_dir()")
    path = os.path.join(_CONFIG_DIR[-1], config_name)
    if not os.path.exists(path) and os.path.exists(path + ".yaml"):
        path += ".yaml"
    with open(path) as f:
        content = yaml.load(f, Loader=_Loader) or {}
    if "defaults" in content:
        raise NotImplementedError("config groups ('defaults') are not supported by this stand-in")
    for ov in overrides or []:
        if ov.startswith("~"):
            parts = ov[1:].split("=")[0].split(".")
            node = content
            for p in parts[:-1]:
                node = node[p]
            node.pop(parts[-1], None)
            continue
        if "=" not in ov:
            raise ValueError("override '%s' is not of the form key=value" % ov)
        key, raw = ov.split("=", 1)
        if key.startswith("++"):
            _set(content, key[2:], _parse_scalar(raw), must_exist=False, may_exist=True)
        elif key.startswith("+"):
            _set(content, key[1:], _parse_scalar(raw), must_exist=False, may_exist=False)
        else:
            _set(content, key, _parse_scalar(raw), must_exist=True, may_exist=True)
    return DictConfig(content)
