"""Strategy value types of the planner and their JSON encoding.

A strategy is the tuple ``(pp, tp, sp, cp, dp, dp_type[, checkpoint])`` of one layer (or of the
embedding / LM-head pair).  Strategies are hashable, totally ordered by that tuple (``dp_type`` by its
string value: ``ddp < zero2 < zero3``) and print as ``"{pp}-{tp|sp}{*}-{dp}{f}{-c}{-sp}"``, e.g.
``1-4*-2f-c``: pp 1, tp 4, dp 2 with ZeRO-3, checkpointed.

JSON side (the artifact the runtime consumes): ``strategy_list2config`` / ``strategies_from_config``
and the plain ``config2strategy`` tuple reader used by the runtime.

Capability parity: galvatron/utils/strategy_utils.py:14-30 (DPType), :36-116 (base strategy),
:118-193 (attention / FFN / layer), :195-245 (MoE FFN), :247-306 (legacy list form), :308-353 (JSON);
galvatron/utils/config_utils.py:8-46.
"""
from __future__ import annotations

import enum
import functools
import json
import os
import warnings
from dataclasses import dataclass, fields, replace
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

BYTES_PER_MB = 1024 * 1024
MODEL_STATES_PER_PARAM = 4  # params + grads + two Adam moments, in units of the parameter size


def is_power_of_two(n: int) -> bool:
    return n > 0 and n & (n - 1) == 0


@functools.total_ordering
class DPType(enum.Enum):
    DDP = "ddp"
    ZERO2 = "zero2"
    ZERO3 = "zero3"

    def __lt__(self, other):
        if not isinstance(other, DPType):
            return NotImplemented
        return self.value < other.value

    @classmethod
    def parse(cls, v) -> "DPType":
        return v if isinstance(v, DPType) else cls(v)


class _Ordered:
    """Field-tuple equality / ordering / hashing shared by the strategy dataclasses."""

    def _key(self) -> Tuple:
        return tuple(getattr(self, f.name) for f in fields(self))

    def __eq__(self, other):
        return type(other) is type(self) and self._key() == other._key()

    def __lt__(self, other):
        if type(other) is not type(self):
            return NotImplemented
        return self._key() < other._key()

    def __hash__(self):
        return hash(self._key())

    def __str__(self):
        body = ", ".join("%s=%s" % (f.name, getattr(self, f.name)) for f in fields(self))
        return "[%s](%s)" % (type(self).__name__, body)

    to_string = __str__


@dataclass(eq=False)
class EmbeddingLMHeadStrategy(_Ordered):
    pp_size: int = 1
    tp_size: int = 1
    sp_size: int = 1
    cp_size: int = 1
    dp_size: int = 1
    dp_type: DPType = DPType.ZERO2

    def __post_init__(self):
        if self.tp_size > 1 and self.sp_size > 1:
            raise AssertionError("tensor parallelism and Ulysses sequence parallelism are exclusive per layer "
                                 "(tp=%d, sp=%d)" % (self.tp_size, self.sp_size))
        if self.sdp_size == 1 and self.dp_type != DPType.DDP:
            # nothing to shard over: normalise so that equal strategies compare equal
            self.dp_type = DPType.DDP

    @property
    def world_size(self) -> int:
        return self.pp_size * self.tp_size * self.sp_size * self.cp_size * self.dp_size

    @property
    def sdp_size(self) -> int:
        return self.dp_size * self.sp_size * self.cp_size

    @property
    def tp_sp_size(self) -> int:
        return max(self.tp_size, self.sp_size)

    def to_simple_string(self) -> str:
        w = self.tp_sp_size
        s = "%d-%d%s-%d%s" % (self.pp_size, w, "*" if w != 1 else "", self.dp_size,
                              "f" if self.dp_type == DPType.ZERO3 else "")
        if getattr(self, "checkpoint", False):
            s += "-c"
        if self.sp_size > 1:
            s += "-sp"
        return s

    def to_embedding_lmhead_strategy(self) -> "EmbeddingLMHeadStrategy":
        return EmbeddingLMHeadStrategy(self.pp_size, self.tp_size, self.sp_size, self.cp_size, self.dp_size,
                                       self.dp_type)


@dataclass(eq=False)
class LayerStrategy(EmbeddingLMHeadStrategy):
    checkpoint: bool = False

    def _as(self, cls):
        return cls(self.pp_size, self.tp_size, self.sp_size, self.cp_size, self.dp_size, self.dp_type, self.checkpoint)

    def to_layer_strategy(self):
        return self._as(LayerStrategy)

    def to_ffn_strategy(self):
        return self._as(FFNStrategy)

    def to_attention_strategy(self):
        return self._as(AttentionStrategy)


@dataclass(eq=False)
class AttentionStrategy(LayerStrategy):
    pass


@dataclass(eq=False)
class FFNStrategy(LayerStrategy):
    pass


@dataclass(eq=False)
class MoEFFNStrategy(_Ordered):
    pp_size: int = 1
    ep_size: int = 1
    tp_size: int = 1
    dp_size: int = 1
    dp_type: DPType = DPType.ZERO2
    checkpoint: bool = False

    def __post_init__(self):
        if self.dp_size == 1 and self.dp_type != DPType.DDP:
            self.dp_type = DPType.DDP

    @property
    def world_size(self) -> int:
        return self.pp_size * self.tp_size * self.dp_size * self.ep_size

    @property
    def sdp_size(self) -> int:
        return self.dp_size


# ---- legacy list form  [pp, tp, dp, {"fsdp":0/1, "tp":1, "sp":0/1, "cpt":1}] -----------------------------
def legacy_to_strategy(item: Sequence, default_dp_type: str) -> LayerStrategy:
    pp, width, dp, info = item[0], item[1], item[2], item[-1]
    ulysses = info.get("sp", 0) == 1
    tp, sp = (1, width) if ulysses else (width, 1)
    if dp == 1:
        dpt = DPType.DDP
    elif info.get("fsdp", 0) == 1:
        dpt = DPType.ZERO3
    else:
        dpt = DPType.DDP if default_dp_type == "ddp" else DPType.ZERO2
    return LayerStrategy(pp, tp, sp, 1, dp, dpt, info.get("cpt", 0) == 1)


def strategy_to_legacy(s: LayerStrategy) -> list:
    info: Dict[str, int] = {}
    if s.dp_size > 1:
        info["fsdp"] = 1 if s.dp_type == DPType.ZERO3 else 0
    if s.tp_sp_size > 1:
        info["tp"] = 1
        info["sp"] = 1 if s.sp_size > 1 else 0
    if getattr(s, "checkpoint", False):
        info["cpt"] = 1
    return [s.pp_size, s.tp_sp_size, s.dp_size, info]


old_version_strategy_to_new_version_strategy = legacy_to_strategy
new_version_strategy_to_old_version_strategy = strategy_to_legacy


def format_strategy_list(strategies: Optional[Iterable]) -> str:
    return "" if strategies is None else ", ".join(s.to_simple_string() for s in strategies)


def print_strategy_list(strategies, logger=None):
    if strategies is None:
        return
    text = format_strategy_list(strategies)
    (logger.info if logger is not None else print)(text)


# ---- JSON encoding -------------------------------------------------------------------------------------
def str2array(s) -> List[int]:
    if isinstance(s, (list, tuple)):
        return [int(x) for x in s]
    return [int(x) for x in str(s).split(",")]


def array2str(a: Iterable) -> str:
    return ",".join(str(x) for x in a)


def read_json_config(path: str) -> Dict[str, Any]:
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def write_json_config(config: Dict[str, Any], path: str):
    d = os.path.dirname(path)
    if d:
        os.makedirs(d, exist_ok=True)
    with open(path, "w") as f:
        json.dump(config, f, indent=4)


def strategy_list2config(strategies: Sequence[LayerStrategy]) -> Dict[str, Any]:
    """Per-layer strategies -> the ``*_enc`` strings of the strategy JSON."""
    if not strategies:
        return {}
    return {
        "pp_deg": strategies[0].pp_size,
        "tp_sizes_enc": array2str(s.tp_sp_size for s in strategies),
        "tp_consecutive_flags": array2str(1 for _ in strategies),
        "dp_types_enc": array2str(1 if s.dp_type == DPType.ZERO3 else 0 for s in strategies),
        "use_sp": array2str(1 if s.sp_size > 1 else 0 for s in strategies),
        "checkpoint": array2str(1 if s.checkpoint else 0 for s in strategies),
        "world_size": strategies[0].world_size,
    }


def strategies_from_config(config: Dict[str, Any], default_dp_type: str = "zero2") -> List[LayerStrategy]:
    """Inverse of :func:`strategy_list2config` (needs ``world_size`` in the dict)."""
    pp = config["pp_deg"]
    widths = str2array(config["tp_sizes_enc"])
    zero3 = str2array(config["dp_types_enc"])
    ckpt = str2array(config["checkpoint"])
    use_sp = str2array(config["use_sp"])
    cps = str2array(config["cp_sizes_enc"]) if "cp_sizes_enc" in config else [1] * len(widths)
    world = config["world_size"]
    out = []
    for w, z, c, u, cp in zip(widths, zero3, ckpt, use_sp, cps):
        dp = world // pp // w // cp
        tp, sp = (1, w) if u else (w, 1)
        if dp * sp * cp == 1:
            dpt = DPType.DDP
        elif z == 1 and default_dp_type == "zero2":
            dpt = DPType.ZERO3
        elif z == 1:
            dpt = DPType.ZERO3
        else:
            dpt = DPType.ZERO2 if default_dp_type != "ddp" else DPType.DDP
        out.append(LayerStrategy(pp, tp, sp, cp, dp, dpt, bool(c)))
    return out


def config2strategy(config: Dict[str, Any]):
    """Runtime-side reader: ``(pp_deg, tp_sizes, cp_sizes, tp_consecutive, dp_types, use_sp, vtp, vsp, vcp)``."""
    widths = str2array(config["tp_sizes_enc"])
    n = len(widths)
    return (config["pp_deg"], widths,
            str2array(config["cp_sizes_enc"]) if "cp_sizes_enc" in config else [1] * n,
            str2array(config["tp_consecutive_flags"]) if "tp_consecutive_flags" in config else [1] * n,
            str2array(config["dp_types_enc"]),
            str2array(config["use_sp"]) if "use_sp" in config else [0] * n,
            config.get("vtp", 1), config.get("vsp", 0), config.get("vcp", 1))
