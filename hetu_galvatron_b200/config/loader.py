"""YAML + dotted-override loader (the Hydra syntax subset the entry points use).

``load_config(path, overrides, mode)`` reads one YAML file, applies ``a.b.c=value`` overrides
(``+a.b=v`` / ``++a.b=v`` add or force keys, ``~a.b`` deletes), resolves ``${x.y}`` interpolations and
``${oc.env:NAME[,default]}``, validates the whole tree with :class:`CoreArgs` and returns the section
that belongs to ``mode``: ``train_dist -> runtime``, ``search -> search_engine``, ``model_profiler``,
``profiler_hardware``.  Same contract as the reference's ``load_with_hydra``
(galvatron/core/arguments.py:125-154) without depending on hydra / omegaconf.

The legacy ``--flag value`` spelling is translated into overrides by :func:`legacy_cli_to_overrides`
(galvatron/core/arguments.py:33-85).
"""
from __future__ import annotations

import os
import re
from typing import Any, Dict, Iterable, List, Optional

import yaml

from .schema import MODE_TO_SECTION, CoreArgs

_INTERP = re.compile(r"\$\{([^${}]+)\}")


class ConfigError(ValueError):
    pass


class _Loader(yaml.SafeLoader):
    pass


# YAML 1.1 does not read "6.0e-4" style floats without a sign in the exponent consistently: accept them.
_Loader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    re.compile(r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
                   |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
                   |\.[0-9_]+(?:[eE][-+]?[0-9]+)?
                   |[-+]?\.(?:inf|Inf|INF)|\.(?:nan|NaN|NAN))$""", re.X),
    list("-+0123456789."))


def parse_value(text: str) -> Any:
    """Parse the right-hand side of an override with YAML scalar / flow rules (``[1,2]``, ``null``, ``1e-5``)."""
    if text == "":
        return ""
    try:
        return yaml.load(text, Loader=_Loader)
    except yaml.YAMLError:
        return text


def _set(tree: Dict, dotted: str, value: Any, must_exist: bool, force: bool):
    keys = dotted.split(".")
    node = tree
    for k in keys[:-1]:
        if not isinstance(node, dict):
            raise ConfigError("cannot descend into %r while setting %s" % (k, dotted))
        if k not in node or node[k] is None:
            if must_exist and not force:
                raise ConfigError("override %s: key %r does not exist (use +%s=... to add)" % (dotted, k, dotted))
            node[k] = {}
        node = node[k]
    last = keys[-1]
    if must_exist and not force and last not in node:
        raise ConfigError("override %s: key does not exist (use +%s=... to add)" % (dotted, dotted))
    node[last] = value


def _delete(tree: Dict, dotted: str):
    keys = dotted.split(".")
    node = tree
    for k in keys[:-1]:
        node = node.get(k, {}) if isinstance(node, dict) else {}
    if isinstance(node, dict):
        node.pop(keys[-1], None)


def apply_overrides(tree: Dict, overrides: Iterable[str], strict: bool = False) -> Dict:
    for ov in overrides or []:
        ov = ov.strip()
        if not ov:
            continue
        if ov.startswith("~"):
            _delete(tree, ov[1:].split("=")[0])
            continue
        if "=" not in ov:
            raise ConfigError("override %r is not of the form key=value" % ov)
        key, _, val = ov.partition("=")
        force = key.startswith("++")
        add = key.startswith("+") and not force
        key = key.lstrip("+")
        _set(tree, key, parse_value(val), must_exist=strict and not add, force=force)
    return tree


def _lookup(root: Dict, dotted: str):
    node: Any = root
    for k in dotted.split("."):
        if isinstance(node, dict) and k in node:
            node = node[k]
        elif isinstance(node, list) and k.isdigit() and int(k) < len(node):
            node = node[int(k)]
        else:
            raise ConfigError("interpolation ${%s}: no such key" % dotted)
    return node


def _resolve_str(root: Dict, s: str, depth: int = 0):
    if depth > 16:
        raise ConfigError("interpolation cycle in %r" % s)
    m = _INTERP.fullmatch(s)

    def one(expr: str):
        expr = expr.strip()
        if expr.startswith("oc.env:") or expr.startswith("env:"):
            body = expr.split(":", 1)[1]
            name, _, default = body.partition(",")
            if name in os.environ:
                return parse_value(os.environ[name])
            if default == "" and "," not in body:
                raise ConfigError("environment variable %s is not set" % name)
            return parse_value(default.strip())
        val = _lookup(root, expr)
        if isinstance(val, str) and _INTERP.search(val):
            val = _resolve_str(root, val, depth + 1)
        return val

    if m:  # whole string is one interpolation: keep the referenced type
        return one(m.group(1))
    return _INTERP.sub(lambda mm: str(one(mm.group(1))), s)


def resolve(tree: Any, root: Optional[Dict] = None) -> Any:
    root = tree if root is None else root
    if isinstance(tree, dict):
        return {k: resolve(v, root) for k, v in tree.items()}
    if isinstance(tree, list):
        return [resolve(v, root) for v in tree]
    if isinstance(tree, str) and "${" in tree:
        return _resolve_str(root, tree)
    return tree


def read_yaml(path: str) -> Dict:
    with open(path, "r") as f:
        data = yaml.load(f, Loader=_Loader)
    return data or {}


def compose(path: str, overrides: Optional[List[str]] = None) -> Dict:
    """YAML file + overrides + interpolation -> plain dict (no validation)."""
    tree = read_yaml(path)
    apply_overrides(tree, overrides or [])
    return resolve(tree)


def load_config(path: str, overrides: Optional[List[str]] = None, mode: str = "train_dist"):
    """Validated arguments of one entry point; see the module docstring."""
    if mode not in MODE_TO_SECTION:
        raise ConfigError("unknown mode %r (expected one of %s)" % (mode, sorted(MODE_TO_SECTION)))
    tree = compose(path, overrides)
    known = {k: v for k, v in tree.items() if k in CoreArgs.model_fields}
    args = CoreArgs(**known)
    section = getattr(args, MODE_TO_SECTION[mode])
    if section is None:
        raise ConfigError("%s has no %r section" % (path, MODE_TO_SECTION[mode]))
    return section


# name kept for users of the reference API
load_with_hydra = load_config

_LEGACY_SECTIONS = ("parallel", "model", "profile", "train", "data", "ckpt", "logging")
# flags of the argparse era whose field was renamed in the YAML schema
_LEGACY_ALIASES = {"global_train_batch_size": "global_batch_size", "epochs": "train_iters", "adam_weight_decay": "weight_decay",
                   "dropout_prob": "hidden_dropout", "set_model_config_manually": "set_model_config_manually",
                   "galvatron_config_path": "galvatron_config_path", "default_dp_type": "default_dp_type"}


def legacy_cli_to_overrides(argv: List[str], section_of: Optional[Dict[str, str]] = None) -> List[str]:
    """``--lr 1e-4 --pp_deg 2 --use-flash-attn`` -> ``++runtime.train.lr=1e-4 ++runtime.parallel.pp_deg=2 ...``.

    A flag's section is found in the runtime schema; flags without a value become ``true``."""
    from .schema import GalvatronRuntimeArgs

    if section_of is None:
        section_of = {}
        for sec in _LEGACY_SECTIONS:
            for name in GalvatronRuntimeArgs.model_fields[sec].annotation.model_fields:
                section_of.setdefault(name, sec)
    out: List[str] = []
    i = 0
    while i < len(argv):
        tok = argv[i]
        if not tok.startswith("--"):
            out.append(tok)  # already an override
            i += 1
            continue
        name = tok[2:].replace("-", "_")
        if "=" in name:
            name, _, val = name.partition("=")
        elif i + 1 < len(argv) and not argv[i + 1].startswith("--"):
            vals = []
            while i + 1 < len(argv) and not argv[i + 1].startswith("--"):
                vals.append(argv[i + 1])
                i += 1
            val = vals[0] if len(vals) == 1 else "[" + ",".join(vals) + "]"
        else:
            val = "true"
        name = _LEGACY_ALIASES.get(name, name)
        sec = section_of.get(name)
        prefix = "runtime.%s." % sec if sec else "runtime."
        out.append("++%s%s=%s" % (prefix, name, val))
        i += 1
    return out
