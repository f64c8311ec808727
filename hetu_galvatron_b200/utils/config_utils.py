"""JSON / key-format helpers shared by profilers, search engine and runtime
(galvatron/utils/config_utils.py:8-46, :48-88, :90-101, :108-184)."""
from __future__ import annotations

import json
import os
from typing import Dict, Sequence, Tuple

import numpy as np


def str2array(s: str):
    return list(map(int, s.split(",")))


def array2str(a) -> str:
    return ",".join(str(int(x)) for x in a)


def read_json_config(path: str) -> Dict:
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def write_json_config(config: Dict, path: str):
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w", encoding="utf-8") as f:
        json.dump(config, f, indent=4)


def num2str(num, name: str) -> str:
    if isinstance(num, Sequence) and not isinstance(num, (str, bytes)):
        return name + "_".join(str(v) for v in num)
    return "%s%s" % (name, num)


def read_allreduce_bandwidth_config(config, gpu_num: int) -> Tuple[Dict, Dict]:
    """``allreduce_size_{n}_consec_{c}`` (MB/ms) -> (bandwidth dict, 1/bandwidth dict) keyed ``"{n}_{c}"`` with a
    ``"1"`` entry for the trivial group."""
    cfg = read_json_config(config) if isinstance(config, str) else config
    bw, coe = {}, {}
    n = gpu_num
    while n > 1:
        for c in (1, 0):
            key = "allreduce_size_%d_consec_%d" % (n, c)
            if key in cfg:
                bw["%d_%d" % (n, c)] = cfg[key]
                coe["%d_%d" % (n, c)] = 1.0 / cfg[key]
        n //= 2
    top = "%d_1" % gpu_num
    if top in bw:
        bw["%d" % gpu_num], coe["%d" % gpu_num] = bw[top], coe[top]
    coe["1"] = 0
    return bw, coe


def read_p2p_bandwidth_config(config) -> Tuple[Dict, Dict]:
    cfg = read_json_config(config) if isinstance(config, str) else config
    bw, coe = {}, {}
    for k, v in cfg.items():
        if "pp_size_" in k:
            p = int(k.split("_")[-1])
            bw[p], coe[p] = v, 1.0 / v
    return bw, coe


def remap_config(config: Dict, op: str) -> Dict:
    """``{op}_size_{n}_{s}MB_time`` entries -> ``{n: {bytes: ms, "popt": [slope, intercept]}}`` with a linear fit
    of time over message size; all-reduce times are halved (an all-gather or reduce-scatter is half of one)."""
    out: Dict[int, Dict] = {}
    for key, val in config.items():
        if not key.startswith(op):
            continue
        parts = key.split("_")
        n, mb = int(parts[-3]), int(parts[-2][:-2])
        out.setdefault(n, {})[mb * 1024 * 1024] = val / 2 if op == "allreduce" else val
    for n, table in out.items():
        xs = np.asarray(sorted(table), dtype=np.float64)
        ys = np.asarray([table[int(x)] for x in xs], dtype=np.float64)
        if len(xs) >= 2:
            slope, icpt = np.polyfit(xs, ys, 1)
        else:
            slope, icpt = (ys[0] / xs[0] if len(xs) else 0.0), 0.0
        table["popt"] = [float(slope), float(icpt)]
    return out
