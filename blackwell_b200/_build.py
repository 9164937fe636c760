"""In-tree build of libblackwell_kernels for sm_100a.

``python -m blackwell_b200._build`` compiles every ``csrc/*.cu`` with nvcc
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``), one object per source in
parallel, and links them into ``blackwell_b200/lib/libblackwell_kernels.so`` and
the static ``libblackwell_kernels.a`` the reference's consumers link against, and builds the JSON-lines daemon
``blackwell_b200/lib/inference_server_w4a8`` from ``daemon/``.
No GPU is needed to build.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
SO = os.path.join(LIBDIR, "libblackwell_kernels.so")
AR = os.path.join(LIBDIR, "libblackwell_kernels.a")
DAEMON_SRC = os.path.join(HERE, "daemon", "inference_server_w4a8.cpp")
DAEMON = os.path.join(LIBDIR, "inference_server_w4a8")

# IEEE division and square root are requested explicitly: the quantizers must
# round exactly like the reference's (v / sc, roundf).
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-prec-div=true", "-prec-sqrt=true",
]


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps_mtime():
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h")) + glob.glob(
        os.path.join(HERE, "..", "include", "*.h*"))
    return max(os.path.getmtime(h) for h in hdrs) if hdrs else 0.0


def _compile(src: str, verbose: bool, extra: list[str]) -> str:
    obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
    newest = max(os.path.getmtime(src), _deps_mtime())
    if os.path.exists(obj) and os.path.getmtime(obj) >= newest:
        return obj
    cmd = ["nvcc", *NVCC_FLAGS, *extra, "-c", src, "-o", obj]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)
    return obj


def build(verbose: bool = False, force: bool = False, extra: list[str] | None = None) -> str:
    """Build (if stale) and return the path of the shared library.  Extra nvcc flags can be given in the environment
    variable BW_NVCC_EXTRA (with -f), e.g. ``-DBW_GEMV_TIMELINE`` for the phase-timeline build of ``bench.py --timeline``."""
    os.makedirs(OBJDIR, exist_ok=True)
    extra = (extra or []) + os.environ.get("BW_NVCC_EXTRA", "").split()
    srcs = _sources()
    if force:
        for f in glob.glob(os.path.join(OBJDIR, "*.o")):
            os.remove(f)
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, extra), srcs))
    newest_obj = max(os.path.getmtime(o) for o in objs)
    if not os.path.exists(SO) or os.path.getmtime(SO) < newest_obj:
        cmd = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "shared", "-o", SO, *objs]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    if not os.path.exists(AR) or os.path.getmtime(AR) < newest_obj:
        if os.path.exists(AR):
            os.remove(AR)
        subprocess.check_call(["ar", "rcs", AR, *objs])
    # the JSON-lines daemon on the decode-step driver: host C++ above the C ABI, linked against the shared library
    if not os.path.exists(DAEMON) or os.path.getmtime(DAEMON) < max(os.path.getmtime(DAEMON_SRC), os.path.getmtime(SO)):
        cmd = ["nvcc", "-std=c++17", "-O2", "-Wno-deprecated-gpu-targets", "-o", DAEMON, DAEMON_SRC, "-L" + LIBDIR, "-lblackwell_kernels", "-cudart",
               "shared", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return SO


if __name__ == "__main__":
    print(build(verbose="-v" in sys.argv, force="-f" in sys.argv))
