"""ctypes binding of ``libhg_sm100.so`` (the hand-written sm_100a kernel library).

The library is built in-tree by ``hetu_galvatron_b200/csrc/build.py``.  On a machine with a GPU the
ops of this package *require* it: a missing library raises instead of silently falling back to
PyTorch, so that a GPU run never measures the wrong code path.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB = None
# HG_DEBUG_KERNELS=1 selects the bounds-checking build of the same kernels (csrc/build.py::build_cuda(debug=True))
DEBUG_KERNELS = os.environ.get("HG_DEBUG_KERNELS", "0") == "1"
# 16-bit storage type of the kernels: "bf16" (libhg_sm100.so) or "fp16" (libhg_sm100_fp16.so, the same sources built
# with IEEE half).  A process binds one build: HG_KERNEL_DTYPE or select_precision() before the first kernel call.
_PRECISION = os.environ.get("HG_KERNEL_DTYPE", "bf16")
_LIB_DIR = Path(__file__).resolve().parent.parent / "_lib"


def _path_for(precision: str) -> Path:
    if precision == "fp16":
        if DEBUG_KERNELS:
            raise RuntimeError("the bounds-checking debug build exists for the bf16 kernels only")
        return _LIB_DIR / "libhg_sm100_fp16.so"
    return _LIB_DIR / ("libhg_sm100_debug.so" if DEBUG_KERNELS else "libhg_sm100.so")


_LIB_PATH = _path_for(_PRECISION)


def select_precision(precision: str):
    """Bind this process to the bf16 or the fp16 build of the kernel library (called by ``build_model`` from
    ``mixed_precision``).  Fails if kernels of the other build have already been loaded."""
    global _PRECISION, _LIB_PATH
    if precision not in ("bf16", "fp16"):
        raise ValueError("kernel precision must be bf16 or fp16, not %r" % (precision,))
    if precision == _PRECISION:
        return
    if _LIB is not None:
        raise RuntimeError("the %s kernel library is already loaded; a process trains in one 16-bit precision"
                           % _PRECISION)
    _PRECISION, _LIB_PATH = precision, _path_for(precision)


def lp_dtype() -> torch.dtype:
    """The 16-bit tensor dtype the loaded (or selected) kernel build works on."""
    return torch.float16 if _PRECISION == "fp16" else torch.bfloat16

c_void_p, c_int, c_float, c_ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class AttnTensor(ctypes.Structure):
    """Mirror of ``HgAttnTensor`` in csrc/sm100/attention.cu."""

    _fields_ = [("ptr", c_void_p), ("ss", c_ll), ("sb", c_ll), ("slots", c_int), ("gs", c_int), ("hs", c_int),
                ("off", c_int)]


_SIGNATURES = {
    "hg_gemm_bf16": [c_void_p] * 4 + [c_int] * 10 + [c_void_p],
    "hg_gemm2_bf16": [c_void_p] * 4 + [c_int] * 10 + [c_void_p],
    "hg_grouped_gemm_bf16": [c_void_p] * 4 + [c_int] * 9 + [c_void_p],
    "hg_grouped_wgrad_bf16": [c_void_p] * 4 + [c_int] * 8 + [c_void_p],
    "hg_norm_fwd": [c_void_p] * 8 + [c_int, c_int, c_float, c_int, c_void_p],
    "hg_norm_bwd": [c_void_p] * 10 + [c_int] * 5 + [c_void_p],
    "hg_peer_gather_bf16": [c_void_p, c_int, c_ll, c_ll, c_ll, c_ll, c_void_p, c_ll, c_ll, c_void_p],
    "hg_peer_gather_rows_bf16": [c_void_p, c_int, c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_void_p, c_void_p, c_void_p],
    "hg_peer_gather_bf16_rv": [c_void_p, c_int, c_ll, c_ll, c_ll, c_ll, c_void_p, c_ll, c_ll, c_void_p, c_int, c_int, c_void_p],
    "hg_peer_gather_rows_bf16_rv": [c_void_p, c_int, c_void_p, c_void_p, c_ll, c_int, c_ll, c_ll, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_void_p],
    "hg_router_topk_fwd": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float] + [c_void_p] * 5,
    "hg_router_topk_bwd": [c_void_p] * 5 + [c_int, c_int, c_int, c_int, c_float, c_void_p, c_void_p],
    "hg_zero_reduce_scatter": [c_void_p, c_int, c_int, c_ll, c_void_p, c_void_p],
    "hg_zero_reduce_scatter_capped": [c_void_p, c_int, c_int, c_ll, c_void_p, c_int, c_void_p],
    "hg_zero_reduce_scatter_bf16wire": [c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p, c_int, c_int, c_void_p, c_int,
                                        c_void_p],
    "hg_add_inplace_f32": [c_void_p, c_void_p, c_ll, c_void_p],
    "hg_zero_adamw_allgather": [c_void_p] * 5 + [c_int, c_ll, c_ll] + [ctypes.c_float] * 5 + [c_int, c_void_p, c_void_p, c_void_p],
    "hg_rope": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                c_void_p],
    "hg_glu_fwd": [c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p],
    "hg_glu_bwd": [c_void_p, c_void_p, c_void_p, c_ll, c_int, c_int, c_void_p],
    "hg_embedding_fwd": [c_void_p] * 4 + [c_int] * 6 + [c_void_p],
    "hg_embedding_bwd": [c_void_p] * 4 + [c_int] * 6 + [c_void_p],
    "hg_cast_f32_bf16": [c_void_p, c_void_p, c_ll, c_void_p],
    "hg_add_bf16": [c_void_p, c_void_p, c_void_p, c_ll, c_void_p],
    "hg_attn_set_dkv_variant": [c_int],
    "hg_attn_set_fwd_variant": [c_int],
    "hg_attn_merge": [c_void_p, c_void_p, c_ll, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "hg_xent_stats": [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "hg_xent_bwd": [c_void_p, c_ll, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "hg_adamw": [c_void_p] * 5 + [c_ll, c_int, c_float, c_float, c_float, c_float, c_float, c_int, c_void_p,
                                  c_void_p, c_void_p],
    "hg_sumsq": [c_void_p, c_ll, c_int, c_void_p, c_void_p, c_int, c_float, c_void_p],
    "hg_clip_coef": [c_void_p, c_float, c_void_p, c_void_p, c_void_p],
    "hg_scale": [c_void_p, c_ll, c_int, c_void_p, c_float, c_void_p],
    "hg_flash_fwd": [ctypes.POINTER(AttnTensor)] * 4 + [c_void_p] + [c_int] * 9 + [c_float, c_void_p],
    "hg_flash_bwd": [ctypes.POINTER(AttnTensor)] * 5 + [c_void_p, c_void_p] + [ctypes.POINTER(AttnTensor)] * 3 +
                    [c_int] * 9 + [c_float, c_void_p],
    "hg_ag_gemm_bf16": [c_void_p] * 7 + [c_int] * 10 + [c_void_p],
    "hg_gemm_rs_bf16": [c_void_p] * 5 + [c_int] * 10 + [c_void_p],
    "hg_ag_gemm2_bf16": [c_void_p] * 7 + [c_int] * 10 + [c_void_p],
    "hg_gemm_rs2_bf16": [c_void_p] * 5 + [c_int] * 10 + [c_void_p],
    "hg_debug_set_gather_row_limit": [c_ll],
    "hg_read_status": [c_int],
    "hg_gemm_gated_selftest": [c_void_p],
    "hg_library_version": [],
}


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load():
    """Load (once) and return the kernel library.  Raises if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not _LIB_PATH.exists():
        if os.environ.get("HG_AUTOBUILD", "1") == "1":
            from ..csrc import build as _build

            _build.build_cuda(debug=DEBUG_KERNELS and _PRECISION != "fp16", half=_PRECISION == "fp16")
    if not _LIB_PATH.exists():
        raise RuntimeError(
            "libhg_sm100.so is missing: run `python -m hetu_galvatron_b200.csrc.build` (nvcc, sm_100a) first")
    lib = ctypes.CDLL(str(_LIB_PATH))
    for name, argtypes in _SIGNATURES.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = argtypes
        fn.restype = c_int
    if hasattr(lib, "hg_status_address"):
        lib.hg_status_address.restype = c_void_p
        lib.hg_status_address.argtypes = []
    _LIB = lib
    return lib


class KernelError(RuntimeError):
    pass


def check(rc: int, what: str):
    if rc != 0:
        raise KernelError("%s failed with code %d" % (what, rc))


def ptr(t):
    return 0 if t is None else t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


_STATUS_NAMES = {0: "ok", 1: "timeout: smem stage never filled", 2: "timeout: smem stage never freed",
                 3: "timeout: accumulator never ready", 4: "timeout: accumulator never drained",
                 5: "timeout: peer flag never set", 6: "bad argument", 7: "timeout: other"}


def read_status(clear: bool = True) -> int:
    """Synchronise and return the device status word (0 == healthy).

    Every wait inside the kernels is bounded; a wait that runs out records a code here and the kernel
    unwinds instead of hanging the GPU."""
    return int(load().hg_read_status(1 if clear else 0))


def assert_healthy():
    code = read_status(clear=True)
    if code != 0:
        raise KernelError("device status word = %d (%s)" % (code, _STATUS_NAMES.get(code, "?")))


_launch_count = 0


def count_launch(n: int = 1):
    global _launch_count
    _launch_count += n


def launches() -> int:
    return _launch_count


def reset_launches():
    global _launch_count
    _launch_count = 0
