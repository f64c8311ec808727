"""The fp16 build of the kernel library (``mixed_precision: fp16`` -> ``libhg_sm100_fp16.so``, the same sources compiled
with IEEE half as the 16-bit type): every kernel family against fp32 PyTorch, and a small model trained in fp16 on the
GPU against the same model trained in fp16 by the plain PyTorch path on the CPU (the counterpart of the reference's
tests/core/test_mixed_precision.py:158-182).  Runs in a child process: a process binds one build of the library."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu

SCRIPT = r"""
import json, math, sys, torch
sys.path.insert(0, %r)
from hetu_galvatron_b200 import ops
from hetu_galvatron_b200.ops import _lib
from hetu_galvatron_b200.ops.gemm import OUT_F32_ACC
assert _lib.lp_dtype() == torch.float16 and _lib.lib_path().name == "libhg_sm100_fp16.so"
dev, H16 = "cuda", torch.float16
torch.manual_seed(0)
def rel(a, b): return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))
out = {}
# GEMM: forward, dgrad and wgrad layouts, both kernels
for M, N, K in ((1000, 776, 520), (4096, 1024, 512)):
    a = torch.randn(M, K, device=dev, dtype=H16); b = torch.randn(N, K, device=dev, dtype=H16) * 0.1
    out["gemm_%%d" %% M] = rel(ops.gemm(a, b), a.float() @ b.float().t())
    out["gemm1_%%d" %% M] = rel(ops.gemm(a, b, pair=False), a.float() @ b.float().t())
    dy = torch.randn(M, N, device=dev, dtype=H16) * 0.1
    out["dgrad_%%d" %% M] = rel(ops.gemm(dy, b, b_mn=True), dy.float() @ b.float())
    acc = torch.ones(N, K, device=dev)
    ops.gemm(dy, a, a_mn=True, b_mn=True, out=acc, out_mode=OUT_F32_ACC)
    out["wgrad_%%d" %% M] = rel(acc, 1 + dy.float().t() @ a.float())
# norm (RMS) with residual, forward and backward through autograd
x = torch.randn(512, 1024, device=dev, dtype=H16, requires_grad=True); w = torch.nn.Parameter(torch.ones(1024, device=dev, dtype=H16))
y = ops.norm(x, w, None, 1e-5, rms=True)
y = y[0] if isinstance(y, tuple) else y
g = torch.randn_like(y); y.backward(g)
xr = x.detach().float().requires_grad_(); yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5); yr.backward(g.float())
out["norm_fwd"] = rel(y, yr); out["norm_bwd"] = rel(x.grad, xr.grad)
# SwiGLU
z = torch.randn(256, 2 * 768, device=dev, dtype=H16, requires_grad=True)
a = ops.activation(z, "swiglu"); ga = torch.randn_like(a); a.backward(ga)
zr = z.detach().float().requires_grad_(); ar = torch.nn.functional.silu(zr[:, :768]) * zr[:, 768:]; ar.backward(ga.float())
out["glu_fwd"] = rel(a, ar); out["glu_bwd"] = rel(z.grad, zr.grad)
# flash attention forward + backward (GQA)
S, B, nh, ng, hd = 512, 2, 4, 2, 128
q = torch.randn(S, B, nh, hd, device=dev, dtype=H16, requires_grad=True)
k = torch.randn(S, B, ng, hd, device=dev, dtype=H16, requires_grad=True)
v = torch.randn(S, B, ng, hd, device=dev, dtype=H16, requires_grad=True)
o = ops.flash_attention(q, k, v, causal=True); go = torch.randn_like(o); o.backward(go)
qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
orf, _ = ops.attention_reference(qr, kr, vr, True); orf.backward(go.float())
out["attn_fwd"] = rel(o, orf); out["attn_dq"] = rel(q.grad, qr.grad); out["attn_dk"] = rel(k.grad, kr.grad); out["attn_dv"] = rel(v.grad, vr.grad)
# AdamW with a half working copy
p32 = torch.randn(4096, device=dev); gr = torch.randn(4096, device=dev, dtype=H16); m = torch.zeros(4096, device=dev); vv = torch.zeros(4096, device=dev)
lp = torch.empty(4096, device=dev, dtype=H16); ref = p32.clone()
ops.adamw_step(p32, gr, m, vv, lp, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, step=1)
gf = gr.float(); mr = 0.1 * gf; vr2 = 0.05 * gf * gf
ref = ref - 1e-2 * (mr / 0.1) / ((vr2 / 0.05).sqrt() + 1e-8)
out["adam"] = rel(p32, ref); out["adam_lp"] = rel(lp, ref)
out["status"] = _lib.read_status()
# a small model, three steps, against the CPU fp16 oracle path
from hetu_galvatron_b200.config.schema import GalvatronRuntimeArgs
from hetu_galvatron_b200.runtime.engine import build_model
from hetu_galvatron_b200.runtime.optimizer import ShardedAdamW
def train(device):
    torch.manual_seed(0)
    args = GalvatronRuntimeArgs(parallel=dict(mixed_precision="fp16"),
        model=dict(model_size="llama-test", hidden_size=256, num_layers=2, num_attention_heads=4, ffn_hidden_size=768, vocab_size=1024,
                   make_vocab_size_divisible_by=8, normalization="RMSNorm", activation_func="torch.nn.functional.silu", gated_linear_unit=True),
        train=dict(seq_length=128, global_batch_size=4, chunks=1, lr=1e-3))
    mdl = build_model(args, device=torch.device(device), full_init=True)
    opt = ShardedAdamW(mdl.sharded_units, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.01, clip_grad=1.0, device=torch.device(device))
    tok = torch.randint(0, 1024, (4, 129), generator=torch.Generator().manual_seed(3)).to(device)
    ls = []
    for it in range(3):
        opt.zero_grad(); loss = mdl.forward_backward(tok[:, :-1], it, labels=tok[:, 1:]); opt.step(); ls.append(float(loss))
    return ls
out["train_gpu"] = train("cuda:0"); out["train_cpu"] = train("cpu")
out["status2"] = _lib.read_status()
print(json.dumps(out))
"""


def test_fp16_kernels_and_training():
    env = dict(os.environ, HG_KERNEL_DTYPE="fp16", HG_QUIET="1")
    p = subprocess.run([sys.executable, "-c", SCRIPT % ROOT], env=env, capture_output=True, text=True, timeout=900)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    res = json.loads(p.stdout.strip().splitlines()[-1])
    assert res.pop("status") == 0 and res.pop("status2") == 0
    gpu, cpu = res.pop("train_gpu"), res.pop("train_cpu")
    for a, b in zip(gpu, cpu):
        assert abs(a - b) / abs(b) < 2e-2, (gpu, cpu)
    assert gpu[-1] < gpu[0]
    for k, v in res.items():
        assert v < 3e-2, (k, res)
