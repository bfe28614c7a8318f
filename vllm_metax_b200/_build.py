"""In-tree build of the native extensions for sm_100a.

Two shared objects are produced next to this file:

* ``_b200_C.so``            - CUDA kernels + ``torch.ops.b200`` bindings
* ``cumem_allocator.so``    - sleep-mode VMM allocator (CPython module, driver API)

Every ``.cu`` is compiled with ``-gencode arch=compute_100a,code=sm_100a`` by a
direct ``nvcc`` call (cross-compiles without a GPU); objects are rebuilt only
when their source or a header is newer.  ``python -m vllm_metax_b200._build``
builds from the command line.

Parity: the reference drives CMake from setup.py (setup.py:82-262) for the three
targets of CMakeLists.txt:181-686; a plain incremental nvcc driver is enough here.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig
from pathlib import Path
from typing import Optional

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "_obj"
LIB = ROOT / "_b200_C.so"
CUMEM_LIB = ROOT / "cumem_allocator.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O3", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-DNDEBUG",
]


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _newer(src_paths, target: Path) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(p).stat().st_mtime > t for p in src_paths)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout + r.stderr)


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(verbose: bool = False, force: bool = False) -> Optional[Path]:
    """Compile ``csrc/*.cu`` for sm_100a and link ``_b200_C.so`` in-tree.  ``B200_TARGET_DEVICE=empty`` skips the
    native build (a CPU-only checkout that runs the PyTorch reference ops; the reference's ``VLLM_TARGET_DEVICE``)."""
    if os.environ.get("B200_TARGET_DEVICE", "cuda").lower() in ("empty", "cpu"):
        return None
    import torch
    from torch.utils.cpp_extension import include_paths, library_paths

    OBJ.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    jobs = []
    objs = []
    for src in sources():
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _newer([src, *headers], obj):
            jobs.append([nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)])
    bind_src = CSRC / "bindings.cpp"
    bind_obj = OBJ / "bindings.o"
    objs.append(bind_obj)
    inc = []
    for p in include_paths(device_type="cuda") if "device_type" in include_paths.__code__.co_varnames else include_paths(cuda=True):
        inc += ["-I", p]
    inc += ["-I", os.path.join(_cuda_home(), "include"), "-I", sysconfig.get_paths()["include"]]
    cxx_abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    if force or _newer([bind_src, *headers], bind_obj):
        jobs.append(["g++", "-std=c++17", "-O2", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={cxx_abi}",
                     "-DTORCH_EXTENSION_NAME=_b200_C", *inc, "-I", str(CSRC), "-c", str(bind_src), "-o", str(bind_obj)])
    if jobs:
        workers = int(os.environ.get("MAX_JOBS", "0")) or min(8, os.cpu_count() or 4)
        import json
        import time

        def timed(job):
            t0 = time.perf_counter()
            _run(job)
            return os.path.basename(job[-1]), time.perf_counter() - t0

        times_file = OBJ / "build_times.json"
        try:
            times = json.loads(times_file.read_text())
        except (OSError, ValueError):
            times = {}
        with cf.ThreadPoolExecutor(workers) as ex:
            for fut in [ex.submit(timed, j) for j in jobs]:
                unit, dt = fut.result()
                times[unit] = round(dt, 2)
        times_file.write_text(json.dumps(times, indent=1, sort_keys=True))
        if verbose:
            print(f"[b200 build] compiled {len(jobs)} translation units")
    if force or jobs or not LIB.exists():
        libdirs = []
        for p in library_paths(device_type="cuda") if "device_type" in library_paths.__code__.co_varnames else library_paths(cuda=True):
            libdirs += ["-L", p, f"-Wl,-rpath,{p}"]
        _run(["g++", "-shared", "-o", str(LIB), *map(str, objs), *libdirs, "-L", os.path.join(_cuda_home(), "lib64"),
              "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"])
    build_cumem(verbose=verbose, force=force)
    return LIB


def build_cumem(verbose: bool = False, force: bool = False) -> Path | None:
    src = CSRC / "cumem_allocator.cpp"
    if not src.exists():
        return None
    if force or _newer([src], CUMEM_LIB):
        inc = ["-I", os.path.join(_cuda_home(), "include"), "-I", sysconfig.get_paths()["include"]]
        # the driver is dlopen'ed at first use: no link-time dependency on libcuda
        _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", *inc, str(src), "-o", str(CUMEM_LIB), "-ldl"])
        if verbose:
            print("[b200 build] built cumem_allocator")
    return CUMEM_LIB


def report_build_times() -> str:
    """Seconds each translation unit took the last time it was compiled, slowest first (what to split or to look
    at when the build gets slow; the reference's tools/report_build_time_ninja.py for its ninja logs)."""
    import json

    try:
        times = json.loads((OBJ / "build_times.json").read_text())
    except (OSError, ValueError):
        return "no build recorded yet: run python -m vllm_metax_b200._build --force"
    rows = sorted(times.items(), key=lambda kv: -kv[1])
    width = max(len(k) for k in times)
    total = sum(times.values())
    lines = [f"{'unit':<{width}}  seconds  share"] + [f"{k:<{width}}  {v:7.2f}  {v / total:5.1%}" for k, v in rows]
    return "\n".join(lines + [f"{'total (cpu-seconds over all workers)':<{width}}  {total:7.2f}"])


if __name__ == "__main__":
    if "--report" in sys.argv:
        print(report_build_times())
    else:
        build(verbose=True, force="--force" in sys.argv)
        print(LIB)
