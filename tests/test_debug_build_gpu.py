"""The bounds-checking build of the kernel library (``HG_DEBUG_KERNELS=1`` -> ``libhg_sm100_debug.so``): odd shapes,
empty expert segments and the peer-memory paths run through it with a clean status word, the same numerics, and
intact canary regions around every symmetric buffer.  Each case runs in child processes, because a process binds one
build of the library."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from tests.dist_utils import run_distributed  # noqa: E402

pytestmark = pytest.mark.gpu

ONE_GPU_SCRIPT = r"""
import json, sys, torch
sys.path.insert(0, %r)
from hetu_galvatron_b200 import ops
from hetu_galvatron_b200.ops import _lib
from hetu_galvatron_b200.ops.gemm import OUT_F32, OUT_F32_ACC
assert _lib.DEBUG_KERNELS and _lib.lib_path().name == "libhg_sm100_debug.so"
dev = "cuda"
torch.manual_seed(0)
def rel(a, b): return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))
out = {}
for M, N, K in ((1000, 776, 520), (304, 264, 72), (4096, 1024, 512)):
    a = torch.randn(M, K, device=dev, dtype=torch.bfloat16); b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
    out["gemm_%%d" %% M] = rel(ops.gemm(a, b), a.float() @ b.float().t())
    acc = torch.ones(N, K, device=dev)
    dy = torch.randn(M, N, device=dev, dtype=torch.bfloat16)
    ops.gemm(dy, a, a_mn=True, b_mn=True, out=acc, out_mode=OUT_F32_ACC)
    out["wgrad_%%d" %% M] = rel(acc, 1 + dy.float().t() @ a.float())
# grouped GEMM with an empty expert and a ragged last one
G, Kd, Nd = 4, 256, 384
starts = torch.tensor([0, 128, 128, 320, 384], dtype=torch.int32, device=dev)
x = torch.randn(448, Kd, device=dev, dtype=torch.bfloat16); w = torch.randn(G, Nd, Kd, device=dev, dtype=torch.bfloat16)
y = ops.grouped_gemm(x, w, starts)
ref = torch.zeros(448, Nd, device=dev)
s = starts.tolist()
for g in range(G): ref[s[g]:s[g+1]] = x[s[g]:s[g+1]].float() @ w[g].float().t()
out["grouped"] = rel(y[:384], ref[:384])
h = torch.randn(300, 5120, device=dev, dtype=torch.bfloat16)
out["status"] = _lib.read_status()
print(json.dumps(out))
"""


def test_debug_build_runs_odd_shapes_clean():
    env = dict(os.environ, HG_DEBUG_KERNELS="1")
    p = subprocess.run([sys.executable, "-c", ONE_GPU_SCRIPT % ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    res = json.loads(p.stdout.strip().splitlines()[-1])
    assert res.pop("status") == 0
    for k, v in res.items():
        assert v < 2e-2, (k, res)


def test_debug_build_peer_paths_keep_their_canaries():
    """ZeRO-2 training through the peer-memory kernels of the debug build on 2 GPUs: same losses as the regular build,
    status word clean, canary regions of all symmetric buffers untouched."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = os.path.join(ROOT, "tests", "test_fused_zero_gpu.py")
    cfg = {"dp_type": "zero2", "defer": True, "fp32_wire": False, "fused": True, "report_guards": True}
    env = {"NCCL_NVLS_ENABLE": "0"}
    ref = run_distributed(script, "train", 2, cfg, timeout=300, extra_env=env)
    got = run_distributed(script, "train", 2, cfg, timeout=300, extra_env=dict(env, HG_DEBUG_KERNELS="1"))
    for r in range(2):
        assert got[r][-1] == ["guards", 0] and ref[r][-1] == ["guards", 0]
        for (l0, n0), (l1, n1) in zip(ref[r][:-1], got[r][:-1]):
            assert abs(l0 - l1) / abs(l0) < 1e-3 and abs(n0 - n1) / n0 < 1e-2
