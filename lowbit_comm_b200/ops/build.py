"""In-tree build of the sm_100a extension `_lbc_cuda`.

The kernels are compiled with plain `nvcc -gencode arch=compute_100a,code=sm_100a`
(no torch headers, seconds per file); only the bindings see torch.  The shared
object is written next to this file so that it travels with the source tree.

Role parity: ccdl_comm/build/extension.py:33-76 (extension spec) and
ccdl_comm/build/codegen.py (not needed: kernels take runtime parameters instead
of being generated per combination).

Run `python -m lowbit_comm_b200.ops.build` to (re)build.
"""

from __future__ import annotations

import hashlib
import json
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
EXT_NAME = "_lbc_cuda"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wno-attributes"]


def extension_path() -> Path:
    return HERE / f"{EXT_NAME}.so"


def cuda_sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


HOST_SOURCE = "host_codec.cpp"       # plain C++ (no torch, no CUDA): its own small library
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-pthread", "-ffp-contract=off", "-fno-fast-math"]


def cxx_sources() -> list[Path]:
    return sorted(p for p in CSRC.glob("*.cpp") if p.name != HOST_SOURCE)


def host_library_path() -> Path:
    return HERE / "_lbc_host.so"


def build_host_library(*, force: bool = False, verbose: bool = False) -> Path:
    """Compile the CPU implementation of the wire format (`csrc/host_codec.cpp`) with g++."""

    src, target = CSRC / HOST_SOURCE, host_library_path()
    obj_dir = HERE / "build"
    obj_dir.mkdir(exist_ok=True)
    stamp = obj_dir / "host_fingerprint.json"
    h = hashlib.sha256(src.read_bytes())
    h.update(" ".join(HOST_FLAGS).encode())
    fp = h.hexdigest()
    if not force and target.exists() and stamp.exists() and json.loads(stamp.read_text()).get("fp") == fp:
        return target
    _run(["g++", *HOST_FLAGS, str(src), "-o", str(target)], verbose)
    stamp.write_text(json.dumps({"fp": fp}))
    return target


def _cuda_home() -> Path:
    for key in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(key):
            return Path(os.environ[key])
    return Path("/usr/local/cuda")


def _fingerprint(files: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for f in sorted(files + sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed ({proc.returncode}): {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose and proc.stderr.strip():
        print(proc.stderr, file=sys.stderr)


def build_extension(*, force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every `.cu`/`.cpp` under csrc/ for sm_100a and link `_lbc_cuda.so`."""

    from torch.utils import cpp_extension

    cuda = _cuda_home()
    nvcc = str(cuda / "bin" / "nvcc")
    obj_dir = HERE / "build"
    obj_dir.mkdir(exist_ok=True)
    target = extension_path()
    stamp = obj_dir / "fingerprint.json"
    fp = _fingerprint(cuda_sources() + cxx_sources(), ARCH_FLAGS + NVCC_FLAGS + CXX_FLAGS)
    if not force and target.exists() and stamp.exists() and json.loads(stamp.read_text()).get("fp") == fp:
        return target

    torch_includes = [f"-I{p}" for p in cpp_extension.include_paths(device_type="cuda")]
    py_include = f"-I{sysconfig.get_paths()['include']}"
    cuda_include = f"-I{cuda / 'include'}"
    jobs = []
    for src in cuda_sources():
        obj = obj_dir / (src.stem + ".cu.o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, f"-I{CSRC}", "-c", str(src), "-o", str(obj)]
        if ptxas_info:
            cmd += ["-Xptxas", "-v"]
        jobs.append((cmd, obj))
    for src in cxx_sources():
        obj = obj_dir / (src.stem + ".cpp.o")
        cmd = ["g++", *CXX_FLAGS, f"-DTORCH_EXTENSION_NAME={EXT_NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
               "-D_GLIBCXX_USE_CXX11_ABI=1", f"-I{CSRC}", *torch_includes, py_include, cuda_include,
               "-c", str(src), "-o", str(obj)]
        jobs.append((cmd, obj))
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        list(pool.map(lambda job: _run(job[0], verbose or ptxas_info), jobs))
    lib_dirs = cpp_extension.library_paths(device_type="cuda")
    link = ["g++", "-shared", "-o", str(target), *[str(obj) for _, obj in jobs],
            *[f"-L{d}" for d in lib_dirs], f"-L{cuda / 'lib64'}",
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart",
            *[f"-Wl,-rpath,{d}" for d in lib_dirs]]
    _run(link, verbose)
    stamp.write_text(json.dumps({"fp": fp}))
    return target


if __name__ == "__main__":
    out = build_extension(force="--force" in sys.argv, verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(out)
    print(build_host_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
