"""Spawn ``world_size`` CPU ranks (gloo) of a test file as subprocesses and collect their JSON results.

Same idea as the reference's ``run_distributed`` fixture (tests/conftest.py:80-191 there) but on the
gloo backend, so every parallelism path is exercised without GPUs."""
import json
import os
import socket
import subprocess
import sys
import tempfile
import time


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_distributed(script, func, world_size, payload, timeout=300, extra_env=None):
    port = free_port()
    outdir = tempfile.mkdtemp(prefix="hgdist_")
    procs = []
    for r in range(world_size):
        env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(r), LOCAL_RANK=str(r),
                   WORLD_SIZE=str(world_size), HG_QUIET="1", OMP_NUM_THREADS="1", HG_OUT=os.path.join(outdir, "%d.json" % r))
        if extra_env:
            env.update(extra_env)
        procs.append(subprocess.Popen([sys.executable, script, "_worker", func, json.dumps(payload)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                      start_new_session=True))
    deadline = time.time() + timeout
    outs = [None] * world_size
    failed = None
    while any(o is None for o in outs):
        for i, p in enumerate(procs):
            if outs[i] is None and p.poll() is not None:
                outs[i] = p.stdout.read()
                if p.returncode != 0 and failed is None:
                    failed = i
        if failed is not None or time.time() > deadline:
            for p in procs:
                if p.poll() is None:
                    try:
                        os.killpg(p.pid, 9)
                    except Exception:
                        p.kill()
            for i, p in enumerate(procs):
                if outs[i] is None:
                    try:
                        outs[i] = p.communicate(timeout=5)[0]
                    except Exception:
                        outs[i] = ""
            break
        time.sleep(0.05)
    if failed is not None or any(p.returncode != 0 for p in procs):
        msg = "\n".join("---- rank %d (rc=%s) ----\n%s" % (i, procs[i].returncode, (outs[i] or "")[-3000:])
                        for i in range(world_size))
        raise AssertionError("distributed run failed (timeout=%s)\n%s" % (time.time() > deadline, msg))
    results = []
    for r in range(world_size):
        with open(os.path.join(outdir, "%d.json" % r)) as f:
            results.append(json.load(f))
    return results


def worker_main(registry):
    """``python test_x.py _worker <func> <json>`` entry: init gloo, call, dump the result."""
    import datetime

    import torch.distributed as dist

    func, payload = sys.argv[2], json.loads(sys.argv[3])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    try:
        out = registry[func](payload)
    finally:
        pass
    with open(os.environ["HG_OUT"], "w") as f:
        json.dump(out, f)
    dist.barrier()
    dist.destroy_process_group()
