"""In-tree build of the sm_100a extension ``miles_b200/_C.so``.

Kernels are plain CUDA translation units compiled by nvcc without the PyTorch headers (seconds per
file); only ``bindings.cpp`` sees ``torch/extension.h``.  Objects are cached under ``csrc/build`` and
rebuilt when a source or header is newer.  ``python -m miles_b200._build`` builds everything.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
TARGET = PKG / "_C.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand


def _cuda_home() -> Path:
    return Path(_nvcc()).resolve().parent.parent


def _newest_header() -> float:
    hs = list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def sources() -> tuple[list[Path], list[Path]]:
    cu = sorted(p for p in CSRC.rglob("*.cu") if "build" not in p.parts)
    cpp = sorted(p for p in CSRC.rglob("*.cpp") if "build" not in p.parts and "native" not in p.parts)
    return cu, cpp


# ---------------------------------------------------------------------------------------------- host-only module
NATIVE_DIR = CSRC / "native"
NATIVE_TARGET = PKG / "_native.so"


def native_needs_build() -> bool:
    if not NATIVE_TARGET.exists():
        return True
    t = NATIVE_TARGET.stat().st_mtime
    return any(s.stat().st_mtime > t for s in NATIVE_DIR.glob("*.cpp"))


def build_native(verbose: bool = False, force: bool = False) -> Path:
    """`miles_b200/_native.so`: scheduler / page pool, quorum store, router table. Plain C++17 + pybind11."""
    if not force and not native_needs_build():
        return NATIVE_TARGET
    import pybind11

    srcs = sorted(NATIVE_DIR.glob("*.cpp"))
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-isystem", pybind11.get_include(),
           "-isystem", sysconfig.get_paths()["include"], *map(str, srcs), "-o", str(NATIVE_TARGET)]
    if verbose:
        print(f"[miles_b200] building {NATIVE_TARGET.name} from {len(srcs)} files", file=sys.stderr)
    _run(cmd)
    return NATIVE_TARGET


def needs_build() -> bool:
    if not TARGET.exists():
        return True
    t = TARGET.stat().st_mtime
    cu, cpp = sources()
    return any(s.stat().st_mtime > t for s in cu + cpp) or _newest_header() > t


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def _obj_for(src: Path) -> Path:
    rel = src.relative_to(CSRC)
    return OBJ / ("_".join(rel.parts) + ".o")


def build(verbose: bool = False, force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    OBJ.mkdir(parents=True, exist_ok=True)
    import fcntl

    # ranks of one job may all find the library stale at once: one compiles, the others wait and then find it fresh
    lock = open(OBJ / ".build.lock", "w")
    fcntl.flock(lock, fcntl.LOCK_EX)
    try:
        return _build_locked(verbose, force)
    finally:
        fcntl.flock(lock, fcntl.LOCK_UN)
        lock.close()


def _build_locked(verbose: bool, force: bool) -> Path:
    import torch
    from torch.utils import cpp_extension

    cu, cpp = sources()
    hdr_t = _newest_header()
    jobs: list[list[str]] = []
    objs: list[Path] = []
    for s in cu:
        o = _obj_for(s)
        objs.append(o)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_t):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(s), "-o", str(o)])
    inc = cpp_extension.include_paths(device_type="cpu") + [str(_cuda_home() / "include"), str(CSRC),
                                                            sysconfig.get_paths()["include"]]
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
                 f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}", "-Wno-deprecated-declarations"]
    for s in cpp:
        o = _obj_for(s)
        objs.append(o)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_t):
            cmd = ["g++", *cxx_flags]
            for i in inc:
                cmd += ["-isystem", i]
            jobs.append(cmd + ["-c", str(s), "-o", str(o)])
    if verbose:
        print(f"[miles_b200] compiling {len(jobs)} translation units", file=sys.stderr)
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as ex:
        list(ex.map(_run, jobs))
    if jobs or not TARGET.exists() or force:
        torch_lib = Path(torch.__file__).parent / "lib"
        link = ["g++", "-shared", "-o", str(TARGET), *map(str, objs), f"-L{torch_lib}", "-lc10", "-ltorch_cpu",
                "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
                f"-L{_cuda_home() / 'lib64'}", "-lcudart", f"-Wl,-rpath,{torch_lib}",
                f"-Wl,-rpath,{_cuda_home() / 'lib64'}"]
        _run(link)
    build_native(verbose=verbose, force=force)
    return TARGET


if __name__ == "__main__":
    print(build(verbose=True, force="--force" in sys.argv))
