"""In-tree build of the native parts: the sm_100a kernel library, the C++ plan compiler /
oracle / runtime library, and the command-line tools.

Everything is compiled with explicit ``nvcc`` / ``g++`` commands (no JIT cache), objects land in
``build/`` and the products in ``cai_b200/lib`` and ``bin/`` so that they travel with the source
tree. A target is rebuilt when any of its sources or headers is newer than it.

Run as ``python -m cai_b200._build`` or call :func:`build_all`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
LIBDIR = ROOT / "cai_b200" / "lib"
BINDIR = ROOT / "bin"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
# The system g++ links libstdc++ dynamically; a toolchain that links it statically (some images set
# CXX to one) puts a second copy of the C++ runtime next to the one PyTorch loads, which crashes.
CXX = os.environ.get("CAI_CXX") or ("/usr/bin/g++" if os.path.exists("/usr/bin/g++") else shutil.which("g++") or "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-I", str(CSRC / "kernels"), "-I", str(CSRC),
]
CXX_FLAGS = ["-std=c++17", "-O2", "-g", "-fPIC", "-Wall", "-Wextra", "-I", str(CSRC), "-I", str(CSRC / "plan")]


def _newer(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(str(c) for c in cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose and (r.stdout.strip() or r.stderr.strip()):
        print(r.stdout, r.stderr, flush=True)
    return r


def kernel_sources():
    return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu")) + sorted(
        (CSRC / "runtime").glob("*.cu"))


def host_lib_sources():
    return sorted((CSRC / "plan").glob("*.cc")) + sorted((CSRC / "ref").glob("*.cc"))


def build_kernels(verbose=False, ptxas_info=False) -> Path:
    """Compile every .cu for sm_100a and link libcai_kernels.so."""
    objdir = BUILD / "kernels"
    objdir.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    headers = list((CSRC / "kernels").glob("*.h")) + list((CSRC / "kernels").glob("*.cuh")) + list(
        (CSRC / "comm").glob("*.h")) + list((CSRC / "comm").glob("*.cuh")) + list((CSRC / "runtime").glob("*.h"))
    srcs = kernel_sources()
    jobs = []
    objs = []
    for s in srcs:
        o = objdir / (s.parent.name + "_" + s.stem + ".o")
        objs.append(o)
        if _newer(o, [s] + headers):
            cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", s, "-o", o]
            jobs.append(cmd)
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        results = list(ex.map(lambda c: _run(c, verbose), jobs))
    if ptxas_info:
        for r in results:
            print(r.stderr)
    lib = LIBDIR / "libcai_kernels.so"
    if jobs or _newer(lib, objs):
        _run([NVCC, "-shared", "-o", lib] + objs + ["-cudart", "static", "-ldl", "-lpthread"], verbose)
    # stand-alone CUDA tools (measurement programs that need no Python): bin/<name>
    BINDIR.mkdir(parents=True, exist_ok=True)
    for t in sorted((CSRC / "tools").glob("*.cu")):
        exe = BINDIR / t.stem
        if _newer(exe, [t] + headers):
            _run([NVCC] + NVCC_FLAGS + [t, "-o", exe, "-cudart", "static", "-lcuda"], verbose)
    return lib


def build_host(verbose=False) -> Path:
    """Compile the GPU-free C++ library (plan compiler, analytic runtime, fp64 oracle) and tools."""
    objdir = BUILD / "host"
    objdir.mkdir(parents=True, exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    BINDIR.mkdir(parents=True, exist_ok=True)
    headers = list((CSRC / "plan").glob("*.h")) + list((CSRC / "ref").glob("*.h"))
    srcs = host_lib_sources()
    jobs, objs = [], []
    for s in srcs:
        o = objdir / (s.parent.name + "_" + s.stem + ".o")
        objs.append(o)
        if _newer(o, [s] + headers):
            jobs.append([CXX] + CXX_FLAGS + ["-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    lib = LIBDIR / "libcai_host.so"
    if jobs or _newer(lib, objs):
        _run([CXX, "-shared", "-o", lib] + objs + ["-lm", "-lpthread", "-ldl"], verbose)
    tool_jobs = []
    for t in sorted((CSRC / "tools").glob("*.cc")):
        exe = BINDIR / t.stem
        if _newer(exe, [t, lib] + headers):
            tool_jobs.append([CXX] + CXX_FLAGS + [t, "-o", exe, "-L", LIBDIR, "-lcai_host",
                                                 "-Wl,-rpath,$ORIGIN/../cai_b200/lib", "-lm", "-lpthread"])
    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(lambda c: _run(c, verbose), tool_jobs))
    return lib


def build_sanitized_selftest(verbose=False) -> Path:
    """The GPU-free C++ code (plan compiler, verifier, analytic runtime, oracle) and its self-test compiled as
    one executable under AddressSanitizer + UndefinedBehaviorSanitizer."""
    out = BUILD / "asan" / "cai_selftest_asan"
    out.parent.mkdir(parents=True, exist_ok=True)
    srcs = host_lib_sources() + [CSRC / "tools" / "cai_selftest.cc"]
    headers = list((CSRC / "plan").glob("*.h")) + list((CSRC / "ref").glob("*.h"))
    if _newer(out, srcs + headers):
        _run([CXX, "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-omit-frame-pointer", "-fno-sanitize-recover=undefined",
              "-I", CSRC, "-I", CSRC / "plan"] + srcs + ["-o", out, "-lm", "-lpthread", "-ldl"], verbose)
    return out


# the reference's source tree: next to this repository unless CAI_REFERENCE_SRC says otherwise
REFERENCE_SRC = Path(os.environ.get("CAI_REFERENCE_SRC", ROOT.parent / "reference"))
REFERENCE_OUT = ROOT / "baseline" / "_ref"


def build_reference(verbose=False):
    """Build the UNMODIFIED reference project (its own Makefile, ``make CUDA=1 NCCL=1``) from a scratch copy of its
    source tree and keep its executables under ``baseline/_ref/bin`` for the reference arm of ``bench.py``.

    Nothing of the reference's source is edited: its Makefile as shipped lacks ``-Isrc/cuda`` for
    ``tools/gpu_trainer.c`` and a library path for ``-lcudart``, both of which the Makefile lets the environment
    supply (``CFLAGS ?=``, ``LDLIBS +=``); ``NVCCFLAGS ?=`` gets an sm_100 code object so the box does not have
    to JIT the default PTX. Returns the path of ``gpu_trainer`` or None (with the reason in
    ``baseline/_ref/BUILD_LOG.txt``) when the source tree or the toolchain is missing."""
    out_bin = REFERENCE_OUT / "bin"
    exe = out_bin / "gpu_trainer"
    log = REFERENCE_OUT / "BUILD_LOG.txt"
    if exe.exists():
        return exe
    REFERENCE_OUT.mkdir(parents=True, exist_ok=True)
    if not (REFERENCE_SRC / "Makefile").exists():
        log.write_text(f"reference source tree not found at {REFERENCE_SRC}\n")
        return None
    import tempfile
    with tempfile.TemporaryDirectory(prefix="cai_ref_build_") as tmp:
        work = Path(tmp) / "cai"
        shutil.copytree(REFERENCE_SRC, work)
        cuda_home = Path(NVCC).resolve().parent.parent
        env = dict(os.environ)
        env["PATH"] = f"{cuda_home / 'bin'}:{env.get('PATH', '')}"
        env["CFLAGS"] = "-std=c11 -O2 -g -Isrc/cuda"
        env["LDLIBS"] = f"-L{cuda_home / 'lib64'}"
        env["NVCCFLAGS"] = "-O2 -std=c++14 -Iinclude -Isrc -gencode arch=compute_100,code=sm_100"
        r = subprocess.run(["make", "-C", str(work), "CUDA=1", "NCCL=1", "bin/gpu_trainer", "bin/trainer",
                            "bin/plan_compiler"], env=env, capture_output=True, text=True)
        log.write_text(f"$ make CUDA=1 NCCL=1 (CFLAGS/LDLIBS/NVCCFLAGS from the environment, source untouched)\n"
                       f"exit {r.returncode}\n{r.stdout[-4000:]}\n{r.stderr[-4000:]}\n")
        if verbose:
            print(log.read_text())
        if r.returncode != 0 or not (work / "bin" / "gpu_trainer").exists():
            return None
        out_bin.mkdir(parents=True, exist_ok=True)
        for name in ("gpu_trainer", "trainer", "plan_compiler"):
            if (work / "bin" / name).exists():
                shutil.copy2(work / "bin" / name, out_bin / name)
    return exe


def build_all(verbose=False):
    host = build_host(verbose)
    kern = build_kernels(verbose)
    try:
        build_reference(verbose)   # the comparison arm of bench.py; its absence never fails the product build
    except Exception as e:  # noqa: BLE001
        REFERENCE_OUT.mkdir(parents=True, exist_ok=True)
        (REFERENCE_OUT / "BUILD_LOG.txt").write_text(f"reference build raised: {e}\n")
    return host, kern


if __name__ == "__main__":
    v = "-v" in sys.argv
    if "--ptxas" in sys.argv:
        for o in (BUILD / "kernels").glob("*.o"):
            o.unlink()
        build_kernels(verbose=v, ptxas_info=True)
    else:
        build_all(verbose=v)
    print("build ok")
