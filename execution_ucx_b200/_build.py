"""In-tree native build for the package.

Everything native is compiled by explicit ``nvcc`` / ``g++`` command lines into
shared objects that live next to the Python sources (so that a copy of the
source tree carries the binaries with it):

* ``execution_ucx_b200/_lib/libeux_kernels.so`` -- the sm_100a CUDA kernels
  (tensor transfer, MoE dispatch/combine, tcgen05 GEMM) behind a C ABI.
* ``execution_ucx_b200/_lib/libeux_runtime.so`` -- the host runtime (executor,
  active-message context, rpc core, axon worker, storage) behind C++ headers.
* ``execution_ucx_b200/axon/_axon*.so`` -- the pybind11 module.
* ``execution_ucx_b200/_lib/eux_*`` -- C++ unit-test and perf binaries.

A target is rebuilt when any of its inputs is newer than its output.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = ROOT / "csrc"
LIB = PKG / "_lib"
OBJ = ROOT / "build" / "obj"

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
CXX = os.environ.get("CXX", "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
    "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden", "-I", str(CSRC),
]
CXX_FLAGS = [
    "-std=c++23", "-O2", "-g1", "-fPIC", "-Wall", "-Wno-unused-function",
    "-Wno-interference-size", "-pthread", "-I", str(CSRC), "-I", str(CUDA_HOME / "include"),
]


def _stdcxx_link_flags():
    """Link against the system's shared libstdc++ and export nothing from static archives.

    Some toolchain wrappers find only a static libstdc++.a: the runtime libraries would then carry
    their own copy of the C++ runtime *and export it*, and a process that loads them before another
    C++ library (PyTorch, say) would have that library's calls bound to the wrong copy."""
    flags = ["-Wl,--exclude-libs,ALL"]
    for cand in ("/usr/lib/x86_64-linux-gnu/libstdc++.so.6", "/lib/x86_64-linux-gnu/libstdc++.so.6", "/usr/lib64/libstdc++.so.6"):
        if Path(cand).exists():
            flags.append(cand)
            break
    return flags


STDCXX = _stdcxx_link_flags()


def _newer(inputs, output: Path) -> bool:
    if not output.exists():
        return True
    t = output.stat().st_mtime
    return any(Path(i).stat().st_mtime > t for i in inputs)


def _run(cmd, verbose):
    if verbose:
        print("[build]", " ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError("native build failed: " + " ".join(str(c) for c in cmd[:4]) + " ...")
    if verbose and (r.stdout.strip() or r.stderr.strip()):
        print(r.stdout + r.stderr, flush=True)


def _headers(*dirs):
    out = []
    for d in dirs:
        for ext in ("*.h", "*.hpp", "*.cuh"):
            out += list(Path(d).rglob(ext))
    return out


def _obj_path(src: Path, tag: str) -> Path:
    h = hashlib.sha1(str(src.relative_to(ROOT)).encode()).hexdigest()[:8]
    return OBJ / f"{src.stem}.{tag}.{h}.o"


def _compile_objects(sources, compile_cmd, tag, deps, verbose, jobs=8):
    OBJ.mkdir(parents=True, exist_ok=True)
    objs, todo = [], []
    for s in sources:
        o = _obj_path(s, tag)
        objs.append(o)
        if _newer([s, *deps], o):
            todo.append((s, o))
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        list(ex.map(lambda so: _run(compile_cmd(so[0], so[1]), verbose), todo))
    return objs, bool(todo)


def build_kernels(verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every ``csrc/kernels/*.cu`` for sm_100a into libeux_kernels.so."""
    LIB.mkdir(exist_ok=True)
    out = LIB / "libeux_kernels.so"
    srcs = sorted((CSRC / "kernels").glob("*.cu"))
    deps = _headers(CSRC / "kernels")
    extra = ["-Xptxas", "-v"] if ptxas_info else []

    def cc(s, o):
        return [NVCC, *NVCC_FLAGS, *extra, "-c", s, "-o", o]

    objs, changed = _compile_objects(srcs, cc, "cu", deps, verbose or ptxas_info)
    if changed or not out.exists():
        _run([NVCC, "-shared", "-o", out, *objs, "-Xlinker", "-rpath=" + str(CUDA_HOME / "lib64")], verbose)
    return out


def _runtime_sources():
    srcs = []
    for sub in ("eux/ucxx", "eux/rpc", "eux/axon", "eux/exec"):
        srcs += sorted((CSRC / sub).rglob("*.cpp"))
    return srcs


def build_runtime(verbose: bool = False) -> Path:
    """Compile the host runtime (C++23) into libeux_runtime.so."""
    LIB.mkdir(exist_ok=True)
    out = LIB / "libeux_runtime.so"
    srcs = _runtime_sources()
    if not srcs:
        return out
    deps = _headers(CSRC / "eux", CSRC / "kernels")

    def cc(s, o):
        return [CXX, *CXX_FLAGS, "-c", s, "-o", o]

    objs, changed = _compile_objects(srcs, cc, "rt", deps, verbose)
    if changed or not out.exists():
        _run([CXX, "-shared", "-o", out, *objs, *STDCXX, "-L", LIB, "-leux_kernels",
              "-L", CUDA_HOME / "lib64", "-lcudart", "-ldl", "-lrt", "-pthread",
              "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + str(CUDA_HOME / "lib64")], verbose)
    return out


def build_binaries(verbose: bool = False):
    """C++ unit tests (csrc/tests/*.cpp) and perf tools (csrc/perf/*.cpp)."""
    outs = []
    deps = _headers(CSRC / "eux", CSRC / "tests")
    rt = LIB / "libeux_runtime.so"
    srcs = sorted((CSRC / "tests").glob("*.cpp")) + sorted((CSRC / "perf").glob("*.cpp"))

    def one(s):
        out = LIB / ("eux_" + s.stem)
        if _newer([s, *deps] + ([rt] if rt.exists() else []), out):
            _run([CXX, *CXX_FLAGS, s, "-o", out, *STDCXX, "-L", LIB, "-leux_runtime", "-leux_kernels",
                  "-L", CUDA_HOME / "lib64", "-lcudart", "-ldl", "-lrt",
                  "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + str(CUDA_HOME / "lib64")], verbose)
        return out

    with ThreadPoolExecutor(max_workers=8) as ex:
        outs = list(ex.map(one, srcs))
    return outs


def build_python_module(verbose: bool = False) -> Path:
    """pybind11 module ``execution_ucx_b200.axon._axon``."""
    import pybind11

    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    out = PKG / "axon" / ("_axon" + suffix)
    srcs = sorted((CSRC / "eux" / "python").glob("*.cpp"))
    if not srcs:
        return out
    deps = _headers(CSRC / "eux")
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]

    def cc(s, o):
        return [CXX, *CXX_FLAGS, "-fvisibility=hidden", *inc, "-c", s, "-o", o]

    objs, changed = _compile_objects(srcs, cc, "py", deps, verbose)
    rt = LIB / "libeux_runtime.so"
    if changed or _newer([rt], out):
        _run([CXX, "-shared", "-o", out, *objs, *STDCXX, "-L", LIB, "-leux_runtime", "-leux_kernels",
              "-L", CUDA_HOME / "lib64", "-lcudart", "-Wl,-rpath,$ORIGIN/../_lib",
              "-Wl,-rpath," + str(CUDA_HOME / "lib64")], verbose)
    return out


def build_sanitized(kind: str = "thread", verbose: bool = False):
    """Host runtime and C++ tests under a sanitizer (``thread``, ``address`` or ``undefined``), for
    CPU-only runs: ``python -m execution_ucx_b200._build --sanitize thread`` builds
    ``build/sanitize-<kind>/eux_*_test``. The CUDA kernels are not instrumented (device code is
    checked by its numerics tests and by the bounded waits)."""
    if kind not in ("thread", "address", "undefined"):
        raise ValueError("sanitizer must be thread, address or undefined")
    out_dir = ROOT / "build" / f"sanitize-{kind}"
    out_dir.mkdir(parents=True, exist_ok=True)
    build_kernels(verbose)
    flags = [f for f in CXX_FLAGS if f != "-O2"] + ["-O1", "-g", f"-fsanitize={kind}", "-fno-omit-frame-pointer"]
    deps = _headers(CSRC / "eux", CSRC / "kernels")
    # the sanitizer runtimes ship with the distribution's compiler
    san_cxx = os.environ.get("EUX_SANITIZE_CXX", "/usr/bin/g++" if Path("/usr/bin/g++").exists() else CXX)

    def cc(s, o):
        return [san_cxx, *flags, "-c", s, "-o", o]

    objs, _ = _compile_objects(_runtime_sources(), cc, f"rt-{kind}", deps, verbose)
    outs = []

    def one(s):
        out = out_dir / ("eux_" + s.stem)
        if _newer([s, *deps, *objs], out):
            _run([san_cxx, *flags, s, *objs, "-o", out, "-L", LIB, "-leux_kernels", "-L", CUDA_HOME / "lib64", "-lcudart",
                  "-ldl", "-lrt", "-Wl,-rpath," + str(LIB), "-Wl,-rpath," + str(CUDA_HOME / "lib64")], verbose)
        return out

    with ThreadPoolExecutor(max_workers=8) as ex:
        outs = list(ex.map(one, sorted((CSRC / "tests").glob("*.cpp"))))
    return outs


def build_all(verbose: bool = False) -> None:
    if shutil.which(NVCC) is None and not Path(NVCC).exists():
        raise RuntimeError(f"nvcc not found at {NVCC}")
    build_kernels(verbose)
    build_runtime(verbose)
    build_python_module(verbose)
    build_binaries(verbose)


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        kind = sys.argv[sys.argv.index("--sanitize") + 1]
        for b in build_sanitized(kind, verbose="-q" not in sys.argv):
            print(b)
    else:
        build_all(verbose="-q" not in sys.argv)
        print("build ok")
