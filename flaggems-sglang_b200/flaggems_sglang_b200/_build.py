"""In-tree build of the CUDA extension (one shared object, nvcc, sm_100a only)."""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR.parent / "csrc"
LIB_PATH = PKG_DIR / "libb200moe.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
    "-Xcompiler", "-fPIC",
]
OBJ_DIR = PKG_DIR.parent / "build"          # per-source objects (git-ignored)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return list(CSRC.glob("*.cuh")) + [PKG_DIR.parent.parent / "include" / "b200moe.h"]


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + _headers()
    return any(p.exists() and p.stat().st_mtime > t for p in deps)


def build(force: bool = False, verbose: bool = False, extra_flags=(), out: Path | None = None) -> Path:
    """Compile csrc/*.cu (one object per source, in parallel, only what changed) and link
    libb200moe.so next to this file.  ``extra_flags`` / ``out`` build a variant elsewhere
    (development: -D switches), always from scratch."""
    variant = bool(extra_flags) or out is not None
    target = Path(out) if out is not None else LIB_PATH
    if not force and not variant and not needs_build():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libb200moe.so")
    obj_dir = OBJ_DIR / (target.stem if variant else "default")
    obj_dir.mkdir(parents=True, exist_ok=True)
    newest_header = max((h.stat().st_mtime for h in _headers() if h.exists()), default=0.0)
    flags = [*NVCC_FLAGS, *extra_flags] + (["-Xptxas=-v"] if verbose else [])
    jobs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        stale = force or variant or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, newest_header)
        if stale:
            jobs.append((src, obj, subprocess.Popen([nvcc, *flags, "-c", "-o", str(obj), str(src)],
                                                    stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    log = []
    failed = False
    for src, obj, proc in jobs:
        text, _ = proc.communicate()
        log.append(f"== {src.name}\n{text}")
        failed |= proc.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed:\n" + "\n".join(log))
    tmp = target.with_suffix(".so.tmp")
    objs = [str(obj_dir / (src.stem + ".o")) for src in sources()]
    res = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(tmp), *objs],
                         capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("link failed:\n" + res.stdout + res.stderr)
    os.replace(tmp, target)
    if verbose:
        print("\n".join(log))
    return target


if __name__ == "__main__":
    print(build(force=True, verbose=True))
