"""In-tree build of the CUDA library (sm_100a only) with plain nvcc.

``python -m jointqk_b200.build`` compiles every ``csrc/*.cu`` into
``jointqk_b200/libjointqk_b200.so``.  The build is skipped when the library is newer than
all sources.  There is no other backend and no fallback: importing the kernels without the
library raises.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libjointqk_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def sources() -> list[Path]:
    return sorted(SRC_DIR.glob("*.cu"))


def is_stale() -> bool:
    if not LIB_PATH.exists():
        return True
    deps = list(SRC_DIR.glob("*.cu")) + list(SRC_DIR.glob("*.cuh")) + [PKG_DIR.parent / "include" / "jointqk_b200.h"]
    newest = max(p.stat().st_mtime for p in deps if p.exists())
    return LIB_PATH.stat().st_mtime < newest


def build(force: bool = False, verbose: bool = False, defines: tuple[str, ...] = ()) -> Path:
    """Compile the library if needed and return its path.  ``defines`` adds -D flags (development
    builds, e.g. the phase counters of the decode kernel)."""
    if not force and not is_stale():
        return LIB_PATH
    obj_dir = PKG_DIR / "build"
    obj_dir.mkdir(exist_ok=True)
    # one builder at a time: several ranks importing the package on a stale tree must not compile
    # into the same object files at once
    import fcntl

    with open(obj_dir / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and not is_stale():
            return LIB_PATH
        return _build_locked(obj_dir, verbose, defines)


def _build_locked(obj_dir: Path, verbose: bool, defines: tuple[str, ...]) -> Path:
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    for src, p in procs:
        out, _ = p.communicate()
        if verbose and out:
            print(out)
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{out}")
    tmp = LIB_PATH.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-o", str(tmp), *objs, "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC", "--cudart", "shared"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}")
    tmp.replace(LIB_PATH)          # readers never see a half-written library
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv or any(a.startswith("-D") for a in sys.argv), verbose="-v" in sys.argv,
                 defines=tuple(a[2:] for a in sys.argv if a.startswith("-D")))
    print(path)
