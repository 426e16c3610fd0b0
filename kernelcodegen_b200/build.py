"""Build recipe for the native library: nvcc, sm_100a only, in-tree output.

`python -m kernelcodegen_b200.build` compiles every `.cu` under `csrc/` into
`kernelcodegen_b200/libkcg_b200.so`.  nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libkcg_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put the CUDA toolkit on PATH")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


BOUNDS_LIB_PATH = PKG_DIR / "libkcg_b200_bounds.so"


def needs_build(lib: Path = LIB_PATH) -> bool:
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG_DIR.parent / "include" / "kcg_capi.h"]
    return any(p.stat().st_mtime > t for p in deps if p.exists())


def build_bounds(force: bool = False) -> Path:
    """The same sources with -DKCG_DEBUG_BOUNDS (every result store and scratch access checked
    against its buffer's extent, see include/kcg_capi.h) -> libkcg_b200_bounds.so; selected at load
    time by KCG_DEBUG_BOUNDS=1 in the environment."""
    return build(force=force, lib=BOUNDS_LIB_PATH, defines=["-DKCG_DEBUG_BOUNDS"], obj_subdir="build_bounds")


def build(force: bool = False, verbose: bool = False, lib: Path = LIB_PATH, defines: list[str] | None = None,
          obj_subdir: str = "build") -> Path:
    """Compile the library if it is missing or older than its sources."""
    if not force and not needs_build(lib):
        return lib
    nvcc = _nvcc()
    obj_dir = PKG_DIR / obj_subdir
    obj_dir.mkdir(exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *(defines or []), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode != 0:
            sys.stderr.write(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
    tmp = lib.with_suffix(".so.tmp")
    link = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("link failed")
    os.replace(tmp, lib)
    return lib


HOST_LIB_PATH = PKG_DIR / "libkcg_runtime.so"
ROOT = PKG_DIR.parent


def shared_libstdcxx(cxx: str) -> list[str]:
    """Extra link inputs that make `cxx` link the C++ runtime dynamically.

    Some toolchain installs ship a libstdc++.so link that points nowhere next to a libstdc++.a;
    the linker then silently takes the archive, and every shared library built that way carries
    (and exports) its own copy of the C++ runtime -- two such libraries in one process corrupt
    each other's iostream state.  When the compiler's own libstdc++.so does not resolve, the
    system's libstdc++.so.6 is named explicitly so that the archive is never consulted."""
    try:
        found = subprocess.run([cxx, "-print-file-name=libstdc++.so"], stdout=subprocess.PIPE, text=True).stdout.strip()
    except OSError:
        found = ""
    if found and os.path.isabs(found) and os.path.exists(found):
        return []
    for cand in ("/usr/lib/x86_64-linux-gnu/libstdc++.so.6", "/lib/x86_64-linux-gnu/libstdc++.so.6",
                 "/usr/lib64/libstdc++.so.6", "/usr/lib/aarch64-linux-gnu/libstdc++.so.6"):
        if os.path.exists(cand):
            return [cand]
    return []


def host_sources() -> list[Path]:
    return sorted((ROOT / "src").rglob("*.cc"))


def build_host(force: bool = False) -> Path:
    """Compile the C++ operator API (include/, src/) into libkcg_runtime.so, linked against the
    kernel library.  Plain g++; no CUDA headers are needed on this side of the C-ABI."""
    build(force=False)
    deps = host_sources() + list((ROOT / "include").rglob("*.h"))
    if not force and HOST_LIB_PATH.exists():
        t = HOST_LIB_PATH.stat().st_mtime
        if all(p.stat().st_mtime <= t for p in deps) and LIB_PATH.stat().st_mtime <= t:
            return HOST_LIB_PATH
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    tmp = HOST_LIB_PATH.with_suffix(".so.tmp")
    cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-I", str(ROOT / "include"),
           *map(str, host_sources()), "-o", str(tmp), "-L", str(PKG_DIR), "-lkcg_b200",
           "-Wl,-rpath,$ORIGIN", *shared_libstdcxx(cxx)]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("building libkcg_runtime.so failed")
    os.replace(tmp, HOST_LIB_PATH)
    return HOST_LIB_PATH


def compile_program(source: Path, output: Path, extra: list[str] | None = None) -> Path:
    """Compile a user program against the operator API (used by the C++ tests/examples)."""
    build_host()
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    cmd = [cxx, "-std=c++17", "-O1", "-I", str(ROOT / "include"), str(source), "-o", str(output),
           "-L", str(PKG_DIR), "-lkcg_runtime", "-lkcg_b200", f"-Wl,-rpath,{PKG_DIR}", *shared_libstdcxx(cxx),
           *(extra or [])]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"compiling {source} failed:\n{res.stdout}")
    return output


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    print(build_bounds(force="--force" in sys.argv))
    print(build_host(force="--force" in sys.argv))
