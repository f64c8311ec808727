"""Single-kernel micro-benchmarks (CUDA-event timed, L2 flushed between iterations).

    python -m hetu_galvatron_b200.profiler.kernel_bench gemm --m 8192 --n 4096 --k 4096 [--variant fwd|dgrad|wgrad]
    python -m hetu_galvatron_b200.profiler.kernel_bench attn --s 4096 --b 1 --heads 32 --kv-heads 32 --hd 128 [--bwd]
    python -m hetu_galvatron_b200.profiler.kernel_bench norm|glu|xent|adam --rows 8192 --cols 4096

Prints one JSON line with the achieved rate and its fraction of the measured peaks (``MEASURED_PEAKS.json``
at the repository root when present, else 6650 GB/s and 1590 TFLOP/s, marked "of fallback").  The same
command line is what the committed ncu summaries under ``profiles/`` were captured from (small ``--iters``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def peaks():
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


def timed(fn, iters, warmup, flush):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def sustained(fn, secs):
    """Launch ``fn`` back to back for ``secs`` seconds; returns (ms per call, median SM MHz, median watts) of the
    second half, when the 1 kW power cap has settled the clocks.  Clocks and power are read (never set) via NVML."""
    import threading
    import time

    import pynvml

    pynvml.nvmlInit()
    h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
    samples, stop = [], []

    def sample():
        while not stop:
            samples.append((pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM),
                            pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0))
            time.sleep(0.05)

    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    th = threading.Thread(target=sample)
    th.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n, t0 = 0, time.time()
    e0.record()
    while time.time() - t0 < secs:
        for _ in range(50):
            fn()
        n += 50
        torch.cuda.synchronize()
    e1.record()
    torch.cuda.synchronize()
    stop.append(1)
    th.join()
    half = samples[len(samples) // 2:] or [(0, 0.0)]
    mhz = sorted(c for c, _ in half)[len(half) // 2]
    watts = sorted(w for _, w in half)[len(half) // 2]
    return e0.elapsed_time(e1) / n, mhz, watts


def main(argv=None):
    from hetu_galvatron_b200 import ops
    from hetu_galvatron_b200.ops import _lib
    from hetu_galvatron_b200.ops.gemm import OUT_F32_ACC

    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "attn", "norm", "norm_bwd", "glu", "glu_bwd", "rope", "xent", "adam", "sumsq"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--variant", default="fwd", choices=["fwd", "dgrad", "wgrad", "wgrad_bf16", "a_mn", "b_mn"],
                    help="operand layouts / epilogue: fwd (both K-major), dgrad (B N-major), wgrad (A M-major, B N-major, "
                         "fp32 C += acc), wgrad_bf16 (the same layouts with the plain bf16 store), a_mn (only A "
                         "M-major), b_mn (only B N-major; dgrad's layout on the wgrad shape)")
    ap.add_argument("--s", type=int, default=4096)
    ap.add_argument("--b", type=int, default=1)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=32)
    ap.add_argument("--hd", type=int, default=128)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--fwd-variant", type=int, default=0,
                    help="attn, head dim 128: 0 = forward with two query tiles per CTA and P in tensor memory, 1 = one "
                         "tile per CTA, P staged in shared memory")
    ap.add_argument("--dkv-variant", type=int, default=0,
                    help="attn --bwd, head dim 128: 0 = dK/dV kernel with 128-query steps and P^T / dS^T in tensor "
                         "memory, 1 = the 64-query kernel that stages them in shared memory")
    ap.add_argument("--rows", type=int, default=8192)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--sustain", type=float, default=0.0,
                    help="gemm only: also run back to back for this many seconds (ours and torch.matmul) and report "
                         "the power-capped rate with the clocks and watts seen")
    a = ap.parse_args(argv)
    dev = "cuda"
    hbm, tf, tag = peaks()
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    out = {"kernel": a.kernel}
    if a.kernel == "gemm":
        M, N, K = a.m, a.n, a.k
        x = torch.randn(M, K, device=dev, dtype=bf)
        w = torch.randn(N, K, device=dev, dtype=bf)
        dy = torch.randn(M, N, device=dev, dtype=bf)
        mg = torch.zeros(N, K, device=dev, dtype=torch.float32)
        # layout probes on the weight-gradient shape: C[N, K] = A[N, M-tokens] B[M-tokens, K] with one or both operands
        # stored transposed (same arithmetic, the operand values do not matter for the rate)
        dy_t = torch.randn(N, M, device=dev, dtype=bf) if a.variant == "b_mn" else None
        x_t = torch.randn(K, M, device=dev, dtype=bf) if a.variant == "a_mn" else None
        fn = {"fwd": lambda: ops.gemm(x, w), "dgrad": lambda: ops.gemm(dy, w, b_mn=True),
              "wgrad": lambda: ops.gemm(dy, x, a_mn=True, b_mn=True, out=mg, out_mode=OUT_F32_ACC),
              "wgrad_bf16": lambda: ops.gemm(dy, x, a_mn=True, b_mn=True),
              "a_mn": lambda: ops.gemm(dy, x_t, a_mn=True),
              "b_mn": lambda: ops.gemm(dy_t, x, b_mn=True)}[a.variant]
        ms = timed(fn, a.iters, a.warmup, flush)
        rate = 2.0 * M * N * K / ms / 1e9
        out.update(shape=[M, N, K], variant=a.variant, ms=ms, tflops=rate, frac=rate / tf, frac_of=tag)
        if a.sustain > 0:
            lib_fn = {"fwd": lambda: torch.matmul(x, w.t()), "dgrad": lambda: torch.matmul(dy, w),
                      "wgrad": lambda: torch.matmul(dy.t(), x), "wgrad_bf16": lambda: torch.matmul(dy.t(), x),
                      "a_mn": lambda: torch.matmul(dy.t(), x_t.t()), "b_mn": lambda: torch.matmul(dy_t, x)}[a.variant]
            for name, f in (("sustained", fn), ("sustained_cublas", lib_fn)):
                ms_s, mhz, watts = sustained(f, a.sustain)
                out[name] = {"tflops": 2.0 * M * N * K / ms_s / 1e9, "sm_mhz": mhz, "watts": watts}
    elif a.kernel == "attn":
        S, B, nh, ng, hd = a.s, a.b, a.heads, a.kv_heads, a.hd
        q = torch.randn(S, B, nh, hd, device=dev, dtype=bf, requires_grad=True)
        k = torch.randn(S, B, ng, hd, device=dev, dtype=bf, requires_grad=True)
        v = torch.randn(S, B, ng, hd, device=dev, dtype=bf, requires_grad=True)
        fl = 4.0 * S * S * B * nh * hd / 2
        _lib.load().hg_attn_set_fwd_variant(a.fwd_variant)
        out["fwd_variant"] = a.fwd_variant
        if a.bwd:
            _lib.load().hg_attn_set_dkv_variant(a.dkv_variant)
            out["dkv_variant"] = a.dkv_variant
            o, lse = ops.flash_attention(q, k, v, return_lse=True)
            g = torch.randn_like(o)
            fn = lambda: ops.flash_backward(q.detach(), k.detach(), v.detach(), o.detach(), g, lse, True,
                                            1.0 / hd ** 0.5)
            fl *= 2.5
        else:
            fn = lambda: ops.flash_attention(q.detach(), k.detach(), v.detach())
        ms = timed(fn, a.iters, a.warmup, flush)
        rate = fl / ms / 1e9
        out.update(shape=[S, B, nh, ng, hd], bwd=a.bwd, ms=ms, tflops=rate, frac=rate / tf, frac_of=tag)
    else:
        R, C = a.rows, a.cols
        if a.kernel == "norm":
            x = torch.randn(R, C, device=dev, dtype=bf)
            r = torch.randn_like(x)
            w = torch.ones(C, device=dev, dtype=bf)
            fn = lambda: ops.norm(x, w, None, 1e-5, True, residual=r)
            nbytes = 4 * R * C * 2
        elif a.kernel == "norm_bwd":
            x = torch.randn(R, C, device=dev, dtype=bf, requires_grad=True)
            r = torch.randn(R, C, device=dev, dtype=bf)
            w = torch.ones(C, device=dev, dtype=bf, requires_grad=True)
            y, hres = ops.norm(x, w, None, 1e-5, True, residual=r)
            gy, gh = torch.randn_like(y), torch.randn_like(hres)
            fn = lambda: torch.autograd.grad([y, hres], [x, w], [gy, gh], retain_graph=True)
            nbytes = 4 * R * C * 2        # dy, h, dres read; dx written
        elif a.kernel == "glu":
            y = torch.randn(R, 2 * C, device=dev, dtype=bf)
            fn = lambda: ops.activation(y, "swiglu")
            nbytes = 3 * R * C * 2
        elif a.kernel == "glu_bwd":
            y = torch.randn(R, 2 * C, device=dev, dtype=bf, requires_grad=True)
            o = ops.activation(y, "swiglu")
            g = torch.randn_like(o)
            fn = lambda: torch.autograd.grad(o, y, g, retain_graph=True)
            nbytes = 5 * R * C * 2
        elif a.kernel == "rope":
            hd = a.hd
            slots = C // hd                       # C = width of the packed projection; the first two thirds rotate
            rot = torch.arange(slots * 2 // 3, device=dev, dtype=torch.int32)
            qkv = torch.randn(R, C, device=dev, dtype=bf)
            cos, sin = ops.rope_tables(R, hd, 10000.0, dev)
            fn = lambda: ops.rope_packed(qkv, rot, hd, cos, sin, 1)
            nbytes = 2 * R * int(rot.numel()) * hd * 2
        elif a.kernel == "sumsq":
            x = torch.randn(R * C, device=dev)
            acc = torch.zeros(1, device=dev)
            fn = lambda: ops.sumsq(x, acc)
            nbytes = R * C * 4
        elif a.kernel == "xent":
            lg = torch.randn(R, C, device=dev, dtype=bf)
            tg = torch.randint(0, C, (R,), device=dev)
            fn = lambda: ops.cross_entropy(lg, tg)
            nbytes = R * C * 2
        else:
            n = R * C
            p = torch.randn(n, device=dev)
            g = torch.randn(n, device=dev)
            m, v = torch.zeros_like(p), torch.zeros_like(p)
            lp = torch.empty(n, device=dev, dtype=bf)
            fn = lambda: ops.adamw_step(p, g, m, v, lp, lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                        step=1)
            nbytes = n * 30
        ms = timed(fn, a.iters, a.warmup, flush)
        rate = nbytes / ms / 1e6
        out.update(shape=[R, C], ms=ms, gbs=rate, frac=rate / hbm, frac_of=tag)
    out["status"] = _lib.read_status()
    if os.environ.get("HG_ATTN_TIMING"):
        # a library built with -DHG_ATTN_TIMING leaves per-role cycle counts of one CTA in words 16..31 of the
        # device status buffer (see HG_DKV_REPORT in csrc/sm100/attention.cu)
        import ctypes

        words = (ctypes.c_int * 64)()
        lib = _lib.load()
        lib.hg_status_address.restype = ctypes.c_void_p
        torch.cuda.synchronize()
        ctypes.CDLL("libcudart.so.12").cudaMemcpy(words, ctypes.c_void_p(lib.hg_status_address()), 256, 2)
        out["role_cycles"] = {"softmax": list(words[16:21]), "mma": list(words[24:29]),
                              "dq_softmax": list(words[40:45]), "dq_mma": list(words[48:53])}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
