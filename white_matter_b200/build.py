"""Build libwm_b200.so (sm_100a) in-tree with nvcc.

``python -m white_matter_b200.build`` compiles every ``csrc/*.cu`` to an object
file (in parallel) and links them into ``white_matter_b200/libwm_b200.so``.
Objects are rebuilt only when their source or a header is newer.  ``--trace``
adds the pipeline event trace of the tcgen05 kernels (a developer build; rebuild
without the flag and with ``-f`` afterwards).
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
INCLUDE = PACKAGE_DIR.parent / "include"
BUILD_DIR = CSRC / "build"
LIBRARY = PACKAGE_DIR / "libwm_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
    f"-I{INCLUDE}",
    f"-I{CSRC}",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: libwm_b200.so cannot be built on this machine")
    return found


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False, trace: bool = False) -> Path:
    """Compile and link; returns the library path.  ``trace`` builds the pipeline event trace in (see wm_debug_trace)."""
    force = force or trace
    nvcc = _nvcc()
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_time = _newest_header()
    jobs = []
    for src in sources:
        obj = BUILD_DIR / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time)
        if stale:
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            if trace:
                cmd[1:1] = ["-DWM_B200_TRACE"]
            jobs.append(cmd)

    def run(cmd):
        result = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, result

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as pool:
            for cmd, result in pool.map(run, jobs):
                if verbose or result.returncode:
                    sys.stderr.write(" ".join(cmd) + "\n" + result.stdout + result.stderr)
                if result.returncode:
                    raise RuntimeError(f"nvcc failed for {cmd[-3]}")
    objects = [str(BUILD_DIR / (src.stem + ".o")) for src in sources]
    newest_obj = max(os.path.getmtime(o) for o in objects)
    if force or jobs or not LIBRARY.exists() or LIBRARY.stat().st_mtime < newest_obj:
        link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIBRARY), *objects]
        result = subprocess.run(link, capture_output=True, text=True)
        if result.returncode:
            sys.stderr.write(result.stdout + result.stderr)
            raise RuntimeError("linking libwm_b200.so failed")
    return LIBRARY


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv, trace="--trace" in sys.argv)
    print(path)
