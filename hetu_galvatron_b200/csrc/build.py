"""In-tree build of the native code.

Two artefacts are produced under ``hetu_galvatron_b200/_lib``:

* ``libhg_sm100.so``  -- every ``csrc/sm100/*.cu`` kernel, compiled by ``nvcc`` for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``) and loaded from Python through ``ctypes``.
* ``hg_dp_core*.so`` / ``hg_dataset_helpers*.so`` -- the host-side C++ modules (pybind11): the
  strategy-search dynamic program and the dataset index builders.

Objects are rebuilt only when a source or header is newer than the object.  ``nvcc`` cross-compiles
without a GPU, so the build also serves as the "does it compile" check on a CPU-only machine.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PKG = CSRC.parent
LIB_DIR = PKG / "_lib"
OBJ_DIR = CSRC / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr", "--expt-extended-lambda",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _newer(src_paths, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in src_paths)


def _run(cmd, log: Path | None = None):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if log is not None:
        log.write_text(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), proc.stdout, proc.stderr))
    return proc


def build_cuda(verbose: bool = False, jobs: int | None = None, debug: bool = False, half: bool = False) -> Path:
    """The kernel library, or one of its variants built from the same sources:

    * ``debug=True``  ``libhg_sm100_debug.so`` (``-DHG_DEBUG_BOUNDS``: index checks that record a status code instead of
      touching memory; see ``HG_BOUNDS_OK`` in sm100_common.cuh), loaded when ``HG_DEBUG_KERNELS=1``;
    * ``half=True``   ``libhg_sm100_fp16.so`` (``-DHG_HALF``: IEEE half as the 16-bit storage type instead of bfloat16;
      see ``hg_lp_t`` in sm100_common.cuh), loaded for ``mixed_precision: fp16`` models."""
    if debug and half:
        raise ValueError("one variant at a time")
    if debug:
        return _build_cuda_variant(OBJ_DIR / "debug", "libhg_sm100_debug.so", ["-DHG_DEBUG_BOUNDS=1"], verbose, jobs)
    if half:
        return _build_cuda_variant(OBJ_DIR / "fp16", "libhg_sm100_fp16.so", ["-DHG_HALF=1"], verbose, jobs)
    return _build_cuda_variant(OBJ_DIR, "libhg_sm100.so", [], verbose, jobs)


def _build_cuda_variant(obj_dir: Path, lib_name: str, extra_flags, verbose: bool, jobs) -> Path:
    src_dir = CSRC / "sm100"
    sources = sorted(src_dir.glob("*.cu"))
    headers = sorted(src_dir.glob("*.cuh")) + sorted(src_dir.glob("*.h"))
    OBJ_DIR.mkdir(exist_ok=True)
    obj_dir.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    todo = []
    objs = []
    for s in sources:
        o = obj_dir / (s.stem + ".o")
        objs.append(o)
        if _newer([s, *headers], o):
            todo.append((s, o))

    def compile_one(pair):
        s, o = pair
        _run([nvcc, *NVCC_FLAGS, *extra_flags, "-I", str(src_dir), "-c", str(s), "-o", str(o)],
             log=obj_dir / (s.stem + ".log"))
        if verbose:
            print("[build] nvcc", s.name)

    with ThreadPoolExecutor(max_workers=jobs or os.cpu_count() or 4) as ex:
        list(ex.map(compile_one, todo))
    lib = LIB_DIR / lib_name
    if todo or _newer(objs, lib):
        _run([nvcc, "-shared", "-o", str(lib), *map(str, objs), "-lcudart"])
        if verbose:
            print("[build] link", lib.name)
    return lib


def build_host(verbose: bool = False):
    import pybind11

    LIB_DIR.mkdir(exist_ok=True)
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    out = []
    for name, src in (("hg_dp_core", "dp_core.cpp"), ("hg_dataset_helpers", "dataset_helpers.cpp")):
        s = CSRC / "host" / src
        if not s.exists():
            continue
        target = LIB_DIR / (name + ext)
        if _newer([s], target):
            _run(["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-pthread", *inc, str(s), "-o", str(target)])
            if verbose:
                print("[build] g++", src)
        out.append(target)
    return out


def build_all(verbose: bool = False, variants: bool = True):
    host = build_host(verbose)
    cuda = build_cuda(verbose)
    out = [cuda, *host]
    if variants:
        out.append(build_cuda(verbose, debug=True))
        out.append(build_cuda(verbose, half=True))
    return out


def ptxas_report() -> str:
    """Registers / spills / shared memory per kernel, as printed by ``-Xptxas -v`` at build time."""
    parts = []
    for log in sorted(OBJ_DIR.glob("*.log")):
        parts.append("== %s ==\n%s" % (log.stem, log.read_text()))
    return "\n".join(parts)


if __name__ == "__main__":
    built = build_all(verbose=True)
    for b in built:
        print(b)
    if "--report" in sys.argv:
        print(ptxas_report())
