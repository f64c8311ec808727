"""Hardware profiler: collective / p2p / all-to-all / overlap measurements that feed the search engine.

Two ways to use it, both producing the reference's files under ``<path>/hardware_configs/``:

* ``HardwareProfiler.profile_bandwidth() / profile_sp_bandwidth()`` write shell scripts
  (``scripts/profile_{allreduce,p2p,allreduce_sp,all2all_sp}.sh``) whose single ``torchrun`` line runs this module
  with the sweep on its command line, and ``profile_overlap()`` launches the overlap measurement
  (galvatron/core/profiler/hardware_profiler.py:39-96, :99-154, :180-190);
* ``python -m hetu_galvatron_b200.profiler.hardware <allreduce|p2p|all2all|overlap|all> ...`` under torchrun runs the
  sweep in-process (profile_hardware/profile_allreduce.py:84-160, profile_p2p.py:59-147, profile_all2all.py:34-90,
  profile_overlap.py:10-186).

Files and keys::

    allreduce_bandwidth_{N}nodes_{G}gpus_per_node.json   allreduce_size_{n}_consec_{0|1}   bus MB/ms = 2(n-1)/n * MB / ms
    p2p_bandwidth_{N}nodes_{G}gpus_per_node.json         pp_size_{P}                      MB/ms along the pipeline chain
    sp_time_{N}nodes_{G}gpus_per_node.json               allreduce_size_{n}_{s}MB_time, all2all_size_{n}_{s}MB_time   ms
    overlap_coefficient.json                             overlap_coe                      >= 1

Method: a bf16 tensor ``[bs, 512, 1024]`` (= ``bs`` MiB); 5 warm-ups, then 20 measurements of 10 back-to-back
operations bracketed by CUDA events after a group barrier; sorted, 2 trimmed at each end, mean; averaged over the
group.  On CPU ranks (gloo; used by the tests) the same loop is timed with ``perf_counter``.  The overlap
coefficient runs a 4096^3 GEMM stream and an all-reduce stream alone and together and reports the larger slow-down,
measured with CUDA events on each stream (the reference parses a profiler table instead).
"""
from __future__ import annotations

import argparse
import datetime
import os
import sys
import time
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils.config_utils import read_json_config, write_json_config
from ..utils.training_utils import gen_profiling_groups
from .runtime import BaseProfiler

WARMUP, MEASUREMENTS, OPS_PER_MEASUREMENT, TRIM = 5, 20, 10, 2
SEQ, HIDDEN = 512, 1024


# ---- sweeps ------------------------------------------------------------------------------------------------------
def halving_degrees(world_size: int, max_deg: int) -> List[int]:
    out, s = [], min(world_size, max_deg)
    while s > 1:
        out.append(s)
        s //= 2
    return out


def halving_batch_sizes(start: int = 1024) -> List[int]:
    out, b = [], start
    while b >= 1:
        out.append(b)
        b //= 2
    return out


def pp_degree_sweep(world_size: int, max_pp_deg: int) -> List[int]:
    out, p = [], 2
    while p <= world_size and p <= max_pp_deg:
        out.append(p)
        p *= 2
    return out


def bandwidth_jobs(world_size: int, tp_degrees: List[int]):
    """(tp, consecutive) pairs: each degree consecutive then strided; the full-world strided case is the same group
    as the consecutive one and is skipped."""
    jobs = []
    for tp in tp_degrees:
        jobs.append((tp, 1))
        if tp != world_size:
            jobs.append((tp, 0))
    return jobs


# ---- script generation -----------------------------------------------------------------------------------------------
class HardwareProfiler(BaseProfiler):
    def __init__(self, args):
        super().__init__()
        self.args = args
        self.path: Optional[str] = None

    def set_path(self, path: str):
        self.path = path

    def get_env(self) -> str:
        a = self.args
        env = {"NUM_NODES": a.num_nodes, "NUM_GPUS_PER_NODE": a.num_gpus_per_node, "MASTER_ADDR": a.master_addr,
               "MASTER_PORT": a.master_port, "NODE_RANK": a.node_rank}
        return "\n".join(a.envs) + "\n" + "\n".join("export %s=%s" % kv for kv in env.items()) + "\n"

    _LAUNCH = ("torchrun \\\n    --nnodes=$NUM_NODES \\\n    --nproc_per_node=$NUM_GPUS_PER_NODE \\\n"
               "    --master_addr=$MASTER_ADDR \\\n    --master_port=$MASTER_PORT \\\n    --node_rank=$NODE_RANK \\\n"
               "    -m hetu_galvatron_b200.profiler.hardware")

    def _write_script(self, name: str, log_dir: str, body: str):
        d = os.path.join(self.path, "scripts")
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, name), "w") as f:
            f.write(self.get_env())
            f.write("mkdir -p %s\n" % log_dir)
            f.write(body)
        return os.path.join(d, name)

    def generate_script(self, num_nodes: int, num_gpus_per_node: int):
        world = num_nodes * num_gpus_per_node
        ints = lambda xs: " ".join(str(x) for x in xs)  # noqa: E731
        out = ["--output_dir %s" % os.path.join(self.path, "hardware_configs")]
        a = self._write_script("profile_allreduce.sh", "logs/allreduce",
                               "%s allreduce \\\n    --global_tp_deg %s \\\n    --profile_time 0 %s \\\n    2>&1 | tee logs/allreduce/allreduce_bandwidth_tp_time0.log\n"
                               % (self._LAUNCH, ints(halving_degrees(world, world)), out[0]))
        b = self._write_script("profile_p2p.sh", "logs/p2p",
                               "%s p2p \\\n    --pp_deg %s %s \\\n    2>&1 | tee logs/p2p/p2p_pp.log\n"
                               % (self._LAUNCH, ints(pp_degree_sweep(world, self.args.max_pp_deg)), out[0]))
        return a, b

    def generate_sp_script(self, num_nodes: int, num_gpus_per_node: int):
        world = num_nodes * num_gpus_per_node
        ints = lambda xs: " ".join(str(x) for x in xs)  # noqa: E731
        tp = ints(halving_degrees(world, self.args.max_tp_size))
        bs = ints(halving_batch_sizes(1024))
        out = "--output_dir %s" % os.path.join(self.path, "hardware_configs")
        a = self._write_script("profile_allreduce_sp.sh", "logs/allreduce_sp",
                               "%s allreduce \\\n    --global_tp_deg %s \\\n    --local_batch_size %s \\\n    --profile_time 1 %s \\\n    2>&1 | tee logs/allreduce_sp/allreduce_sp_time1.log\n"
                               % (self._LAUNCH, tp, bs, out))
        b = self._write_script("profile_all2all_sp.sh", "logs/all2all_sp",
                               "%s all2all \\\n    --global_tp_deg %s \\\n    --local_batch_size %s %s \\\n    2>&1 | tee logs/all2all_sp/all2all_sp.log\n"
                               % (self._LAUNCH, tp, bs, out))
        return a, b

    def profile_bandwidth(self):
        return self.generate_script(self.args.num_nodes, self.args.num_gpus_per_node)

    def profile_sp_bandwidth(self):
        return self.generate_sp_script(self.args.num_nodes, self.args.num_gpus_per_node)

    def write_config(self, hardware_config_path: str, key: str, value: float):
        cfg = read_json_config(hardware_config_path) if os.path.exists(hardware_config_path) else {}
        cfg[key] = value
        write_json_config(cfg, hardware_config_path)

    def overlap_command(self) -> str:
        a = self.args
        return ("OVERLAP_TIME_MULTIPLY=%d torchrun --nnodes=1 --nproc_per_node=%d --master_addr=127.0.0.1 "
                "--master_port=%s -m hetu_galvatron_b200.profiler.hardware overlap --overlap_time_multiply %d --output_dir %s"
                % (a.overlap_time_multiply, a.num_gpus_per_node, str(a.master_port).replace("$MASTER_PORT", "29511"),
                   a.overlap_time_multiply, os.path.join(self.path, "hardware_configs")))

    def profile_overlap(self, run: Callable[[str], int] = os.system):
        return run(self.overlap_command())


# ---- in-process measurements -------------------------------------------------------------------------------------
class _Clock:
    """CUDA events on the current stream on a GPU, ``perf_counter`` on CPU ranks."""

    def __init__(self, device):
        self.cuda = device.type == "cuda"
        if self.cuda:
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def start(self):
        if self.cuda:
            torch.cuda.synchronize()
            self.a.record()
        else:
            self.t0 = time.perf_counter()

    def stop_ms(self) -> float:
        if self.cuda:
            self.b.record()
            torch.cuda.synchronize()
            return self.a.elapsed_time(self.b)
        return (time.perf_counter() - self.t0) * 1e3


def _trimmed_mean(xs: List[float]) -> float:
    xs = sorted(xs)
    core = xs[TRIM:-TRIM] if len(xs) > 2 * TRIM else xs
    return sum(core) / len(core)


def _measure(op: Callable[[torch.Tensor], None], make: Callable[[], torch.Tensor], device, barrier: Callable[[], None],
             measurements: int = MEASUREMENTS, per: int = OPS_PER_MEASUREMENT) -> float:
    clock = _Clock(device)
    for _ in range(WARMUP):
        op(make())
    ts = []
    for _ in range(measurements):
        x = make()
        barrier()
        clock.start()
        for _ in range(per):
            op(x)
        ts.append(clock.stop_ms() / per)
    return _trimmed_mean(ts)


def _device():
    if torch.cuda.is_available():
        return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    return torch.device("cpu")


def _tensor(bs: int, device, seq=SEQ, hidden=HIDDEN):
    dt = torch.bfloat16 if device.type == "cuda" else torch.float32
    return torch.randn(bs, seq, hidden, dtype=dt, device=device)


def _mb(bs: int, seq=SEQ, hidden=HIDDEN) -> float:
    return bs * seq * hidden * 2 / (1024 * 1024)


def _group_mean(value: float, group, size: int, device) -> float:
    t = torch.tensor([value], dtype=torch.float64 if device.type == "cpu" else torch.float32, device=device)
    dist.all_reduce(t, group=group)
    return float(t.item()) / size


def _save(output_dir: str, template: str, nodes: int, gpus: int, key: str, value: float) -> str:
    path = os.path.join(output_dir, template % (nodes, gpus))
    cfg = read_json_config(path) if os.path.exists(path) else {}
    cfg[key] = value
    write_json_config(cfg, path)
    return path


def profile_allreduce(tp_degrees: List[int], batch_sizes: List[int], profile_time: int, output_dir: str, nodes: int,
                      gpus_per_node: int, measurements: int = MEASUREMENTS, seq=SEQ, hidden=HIDDEN) -> Dict[str, float]:
    """Bandwidth mode (``profile_time=0``): one message size, every (tp, consecutive) layout.  Time mode: every
    (tp, message size) on consecutive groups."""
    device, world, rank = _device(), dist.get_world_size(), dist.get_rank()
    out: Dict[str, float] = {}
    jobs = bandwidth_jobs(world, tp_degrees) if profile_time == 0 else [(tp, 1) for tp in tp_degrees]
    groups = {}
    for tp, consec in jobs:
        groups[(tp, consec)] = gen_profiling_groups(tp, bool(consec))
    for tp, consec in jobs:
        g = groups[(tp, consec)]
        for bs in batch_sizes:
            ms = _measure(lambda x: dist.all_reduce(x, group=g), lambda: _tensor(bs, device, seq, hidden), device,
                          lambda: dist.barrier(group=g), measurements)
            ms = _group_mean(ms, g, tp, device)
            if profile_time == 0:
                key, val = "allreduce_size_%d_consec_%d" % (tp, consec), 2 * (tp - 1) / tp * _mb(bs, seq, hidden) / ms
                tmpl = "allreduce_bandwidth_%dnodes_%dgpus_per_node.json"
            else:
                key, val = "allreduce_size_%d_%dMB_time" % (tp, bs), ms
                tmpl = "sp_time_%dnodes_%dgpus_per_node.json"
            out[key] = val
            if rank == 0:
                _save(output_dir, tmpl, nodes, gpus_per_node, key, val)
                print("%s: %.4f" % (key, val))
        dist.barrier()
    return out


def profile_all2all(tp_degrees: List[int], batch_sizes: List[int], output_dir: str, nodes: int, gpus_per_node: int,
                    measurements: int = MEASUREMENTS, seq=SEQ, hidden=HIDDEN) -> Dict[str, float]:
    device, rank = _device(), dist.get_rank()
    out: Dict[str, float] = {}
    groups = {tp: gen_profiling_groups(tp, True) for tp in tp_degrees}
    for tp in tp_degrees:
        g = groups[tp]
        ranks = dist.get_process_group_ranks(g)
        me = ranks.index(rank)

        def a2a(x, g=g, ranks=ranks, me=me, tp=tp):
            y = torch.empty_like(x)
            if device.type == "cuda":
                dist.all_to_all_single(y, x, group=g)
                return
            xs, ys = x.view(tp, -1), y.view(tp, -1)  # gloo has no all-to-all: pairwise exchange
            ys[me].copy_(xs[me])
            ops = []
            for j, r in enumerate(ranks):
                if j != me:
                    ops.append(dist.isend(xs[j].contiguous(), dst=r, group=g))
                    ops.append(dist.irecv(ys[j], src=r, group=g))
            for o in ops:
                o.wait()

        for bs in batch_sizes:
            ms = _measure(a2a, lambda: _tensor(bs, device, seq, hidden), device, lambda: dist.barrier(group=g), measurements)
            ms = _group_mean(ms, g, tp, device)
            key = "all2all_size_%d_%dMB_time" % (tp, bs)
            out[key] = ms
            if rank == 0:
                _save(output_dir, "sp_time_%dnodes_%dgpus_per_node.json", nodes, gpus_per_node, key, ms)
                print("%s: %.4f" % (key, ms))
        dist.barrier()
    return out


def profile_p2p(pp_degrees: List[int], output_dir: str, nodes: int, gpus_per_node: int, batch_size: int = 32,
                measurements: int = MEASUREMENTS, seq=SEQ, hidden=HIDDEN) -> Dict[str, float]:
    """Every rank forwards the tensor along its pipeline chain (stage ``s`` = ``rank // (world/pp)``), all hops
    posted together; MB/ms of one hop."""
    device, world, rank = _device(), dist.get_world_size(), dist.get_rank()
    out: Dict[str, float] = {}
    for pp in pp_degrees:
        if world % pp:
            raise SystemExit("pp_deg %d must divide world size %d" % (pp, world))
        stride = world // pp
        stage = rank // stride
        prev_rank = rank - stride if stage > 0 else None
        next_rank = rank + stride if stage < pp - 1 else None
        recv_buf = _tensor(batch_size, device, seq, hidden)

        def hop(x):
            ops = []
            if prev_rank is not None:
                ops.append(dist.P2POp(dist.irecv, recv_buf, prev_rank))
            if next_rank is not None:
                ops.append(dist.P2POp(dist.isend, x, next_rank))
            if device.type == "cuda":
                for r in dist.batch_isend_irecv(ops):
                    r.wait()
            else:
                for r in [o.op(o.tensor, o.peer) for o in ops]:
                    r.wait()

        ms = _measure(hop, lambda: _tensor(batch_size, device, seq, hidden), device, dist.barrier, measurements)
        ms = _group_mean(ms, None, world, device)
        key, val = "pp_size_%d" % pp, _mb(batch_size, seq, hidden) / ms
        out[key] = val
        if rank == 0:
            _save(output_dir, "p2p_bandwidth_%dnodes_%dgpus_per_node.json", nodes, gpus_per_node, key, val)
            print("%s: %.4f MB/ms" % (key, val))
        dist.barrier()
    return out


def profile_overlap(output_dir: str, multiply: int = 4, n: int = 4096, iters: int = 20) -> float:
    """Slow-down of a GEMM stream and an all-reduce stream when they run together.  ``multiply`` all-reduces are
    issued per GEMM group so that both streams stay busy for a comparable time."""
    device, rank = _device(), dist.get_rank()
    dt = torch.bfloat16 if device.type == "cuda" else torch.float32
    a = torch.randn(n, n, dtype=dt, device=device)
    b = torch.randn(n, n, dtype=dt, device=device)
    m = torch.randn(n, n, dtype=dt, device=device)
    if device.type == "cuda":
        from .. import ops

        mm = lambda: ops.gemm(a, b)  # noqa: E731
    else:
        mm = lambda: torch.matmul(a, b)  # noqa: E731
    if device.type != "cuda":
        # no concurrent streams on CPU ranks: the coefficient is 1 by definition
        coe = 1.0
    else:
        s_comp, s_comm = torch.cuda.Stream(), torch.cuda.Stream()

        def run(compute: bool, comm: bool):
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            dist.barrier()
            torch.cuda.synchronize()
            if compute:
                with torch.cuda.stream(s_comp):
                    ev[0].record()
                    for _ in range(iters * multiply):
                        mm()
                    ev[1].record()
            if comm:
                with torch.cuda.stream(s_comm):
                    ev[2].record()
                    for _ in range(iters):
                        dist.all_reduce(m)
                    ev[3].record()
            torch.cuda.synchronize()
            return (ev[0].elapsed_time(ev[1]) if compute else 0.0), (ev[2].elapsed_time(ev[3]) if comm else 0.0)

        for _ in range(2):
            run(True, True)
        comp_alone, _ = run(True, False)
        _, comm_alone = run(False, True)
        comp_both, comm_both = run(True, True)
        coe = max(comp_both / comp_alone, comm_both / comm_alone, 1.0)
    coe = _group_mean(coe, None, dist.get_world_size(), device)
    if rank == 0:
        path = os.path.join(output_dir, "overlap_coefficient.json")
        cfg = read_json_config(path) if os.path.exists(path) else {}
        cfg["overlap_coe"] = max(coe, 1.0)
        write_json_config(cfg, path)
        print("overlap_coe: %.4f" % coe)
    return coe


def profile_fused_tp(tp_degrees: List[int], output_dir: str, nodes: int, gpus_per_node: int, slab_tokens: int = 8192,
                     hidden: int = 4096, ffn: int = 11008) -> Dict[str, float]:
    """The fused tensor-parallel kernels (all-gather -> GEMM, GEMM -> reduce-scatter over peer memory) against "NCCL
    collective + the same GEMM" on consecutive groups of every degree, on the two GEMM shapes of a decoder layer
    (QKV-like ``hidden -> 3*hidden/t`` and fc2-like ``ffn/t -> hidden``; ``slab_tokens`` rows in total).

    Written to ``fused_tp_time_<nodes>nodes_<gpus>gpus_per_node.json``: the raw times per degree, and
    ``fused_comm_hidden_fraction_tp<t>`` = the share of the collective's exposed time that the fused kernel hides,
    ``1 - (fused - gemm_only) / (nccl_path - gemm_only)`` averaged over the two ops (clamped to [0, 1]).  The same
    fractions are copied into ``b200_refit.json``, where the search's cost model reads them (CUDA only)."""
    from ..parallel.groups import CommGroup
    from .fused_tp_bench import fused_vs_nccl

    device, rank = _device(), dist.get_rank()
    out: Dict[str, float] = {}
    if device.type != "cuda":
        return out
    for tp in tp_degrees:
        if tp < 2:
            continue
        g = gen_profiling_groups(tp, True)
        ranks = dist.get_process_group_ranks(g)
        grp = CommGroup(list(ranks), g, ranks.index(rank))
        slab = max(256, slab_tokens // tp // 256 * 256)
        ag = fused_vs_nccl(grp, slab, hidden, 3 * hidden // tp // 8 * 8, iters=6)
        rs = fused_vs_nccl(grp, slab, ffn // tp // 8 * 8, hidden, iters=6)
        hid = []
        for res, op in ((ag, "ag"), (rs, "rs")):
            exposed = res["%s_nccl_ms" % op] - res["gemm_only_ms"]
            left = res["%s_fused_ms" % op] - res["gemm_only_ms"]
            hid.append(min(1.0, max(0.0, 1.0 - left / exposed)) if exposed > 1e-6 else 0.0)
        frac = sum(hid) / len(hid)
        frac = _group_mean(frac, None, dist.get_world_size(), device)
        entry = {"fused_tp_size_%d_ag_fused_ms" % tp: ag["ag_fused_ms"], "fused_tp_size_%d_ag_nccl_ms" % tp: ag["ag_nccl_ms"],
                 "fused_tp_size_%d_rs_fused_ms" % tp: rs["rs_fused_ms"], "fused_tp_size_%d_rs_nccl_ms" % tp: rs["rs_nccl_ms"],
                 "fused_tp_size_%d_ag_frac_of_roofline" % tp: ag["ag_frac_of_roofline"],
                 "fused_tp_size_%d_rs_frac_of_roofline" % tp: rs["rs_frac_of_roofline"],
                 "fused_comm_hidden_fraction_tp%d" % tp: frac}
        out.update(entry)
        if rank == 0:
            for k, v in entry.items():
                _save(output_dir, "fused_tp_time_%dnodes_%dgpus_per_node.json", nodes, gpus_per_node, k, v)
                print("%s: %.4f" % (k, v))
            refit = os.path.join(output_dir, "b200_refit.json")
            cfg = read_json_config(refit) if os.path.exists(refit) else {}
            cfg["fused_comm_hidden_fraction_tp%d" % tp] = frac
            write_json_config(cfg, refit)
        dist.barrier()
    return out


# ---- command line -----------------------------------------------------------------------------------------------------
def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("what", choices=["allreduce", "p2p", "all2all", "overlap", "fused", "all"])
    ap.add_argument("--global_tp_deg", type=int, nargs="+", default=None)
    ap.add_argument("--pp_deg", type=int, nargs="+", default=None)
    ap.add_argument("--local_batch_size", type=int, nargs="+", default=[32])
    ap.add_argument("--profile_time", type=int, default=0)
    ap.add_argument("--overlap_time_multiply", type=int, default=4)
    ap.add_argument("--max_pp_deg", type=int, default=8)
    ap.add_argument("--output_dir", default="./hardware_configs")
    ap.add_argument("--measurements", type=int, default=MEASUREMENTS)
    a = ap.parse_args(argv)
    dev = _device()
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    if not dist.is_initialized():
        kw = dict(timeout=datetime.timedelta(minutes=10))
        if dev.type == "cuda":
            kw["device_id"] = dev
        dist.init_process_group("nccl" if dev.type == "cuda" else "gloo", **kw)
    world = dist.get_world_size()
    gpn = int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("NUM_GPUS_PER_NODE", world)))
    nodes = max(1, world // gpn)
    tp = a.global_tp_deg or halving_degrees(world, world)
    res = {}
    if a.what in ("allreduce", "all"):
        res.update(profile_allreduce(tp, a.local_batch_size if a.what == "allreduce" else [32], a.profile_time if a.what == "allreduce" else 0,
                                     a.output_dir, nodes, gpn, a.measurements))
    if a.what == "all":
        res.update(profile_allreduce(tp, halving_batch_sizes(1024), 1, a.output_dir, nodes, gpn, a.measurements))
    if a.what in ("all2all", "all"):
        res.update(profile_all2all(tp, a.local_batch_size if a.what == "all2all" else halving_batch_sizes(1024), a.output_dir,
                                   nodes, gpn, a.measurements))
    if a.what in ("p2p", "all"):
        res.update(profile_p2p(a.pp_deg or pp_degree_sweep(world, a.max_pp_deg), a.output_dir, nodes, gpn,
                               measurements=a.measurements))
    if a.what in ("overlap", "all"):
        res["overlap_coe"] = profile_overlap(a.output_dir, a.overlap_time_multiply)
    if a.what in ("fused", "all"):
        res.update(profile_fused_tp(tp, a.output_dir, nodes, gpn))
    dist.barrier()
    return res


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
