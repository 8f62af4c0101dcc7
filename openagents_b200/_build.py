"""In-tree native build: host C++ library, sm_100a CUDA library and the node CLI.

Everything is compiled with plain ``g++`` / ``nvcc`` into ``openagents_b200/_lib`` so the built
objects sit beside the package.  A content hash of sources, headers and flags decides whether a
target is stale; timestamps are ignored because a copied tree does not keep them.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "_lib"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--use_fast_math", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=default", "--expt-relaxed-constexpr"]
# measurement builds: B200_NVCC_DEFINES="QGEMM_STAMPS" compiles the in-kernel cycle counters (part of the flag digest, so
# switching it on or off rebuilds)
NVCC_FLAGS += ["-D" + d for d in os.environ.get("B200_NVCC_DEFINES", "").replace(",", " ").split()]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fopenmp", "-Wall", "-Wno-unused-function", "-ffp-contract=off"]


def _sources(sub: str, exts: tuple[str, ...]) -> list[Path]:
    root = CSRC / sub
    return sorted(p for p in root.rglob("*") if p.suffix in exts)


def host_sources() -> list[Path]:
    out = []
    for sub in ("gguf", "kv", "data", "oracle", "host"):
        if (CSRC / sub).is_dir():
            out += _sources(sub, (".cpp",))
    return out


def cuda_sources() -> list[Path]:
    out = []
    for sub in ("kernels", "comm", "engine"):
        if (CSRC / sub).is_dir():
            out += _sources(sub, (".cu",))
    return out


def node_sources() -> list[Path]:
    return _sources("node", (".cpp",)) if (CSRC / "node").is_dir() else []


def _headers() -> list[Path]:
    return sorted(p for p in CSRC.rglob("*") if p.suffix in (".h", ".cuh", ".hpp"))


def _digest(paths: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(str(p.relative_to(PKG)).encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.stderr.strip() and os.environ.get("B200_BUILD_VERBOSE"):
        sys.stderr.write(r.stderr)


def _compile_objects(srcs: list[Path], compiler: list[str], flags: list[str], tag: str) -> list[Path]:
    """Compile each source to an object, skipping those whose stamp matches."""
    objdir = LIB / "obj"
    objdir.mkdir(parents=True, exist_ok=True)
    hdrs = _headers()
    jobs, objs = [], []
    for s in srcs:
        obj = objdir / (tag + "_" + "_".join(s.relative_to(CSRC).with_suffix("").parts) + ".o")
        stamp = obj.with_suffix(".stamp")
        want = _digest([s] + hdrs, compiler + flags)
        objs.append(obj)
        if obj.exists() and stamp.exists() and stamp.read_text() == want:
            continue
        jobs.append((s, obj, stamp, want))
    def one(job):
        s, obj, stamp, want = job
        _run(compiler + flags + ["-I", str(CSRC), "-c", str(s), "-o", str(obj)])
        stamp.write_text(want)
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            list(ex.map(one, jobs))
    return objs


def _link(objs: list[Path], out: Path, linker: list[str], extra: list[str]) -> None:
    stamp = out.with_suffix(out.suffix + ".stamp")
    want = _digest(objs, linker + extra)
    if out.exists() and stamp.exists() and stamp.read_text() == want:
        return
    _run(linker + [str(o) for o in objs] + ["-o", str(out)] + extra)
    stamp.write_text(want)


def host_lib_path() -> Path:
    return LIB / "libb200_host.so"


def cuda_lib_path() -> Path:
    return LIB / "libb200_cuda.so"


def node_cli_path() -> Path:
    return LIB / "b200-node"


def build_host() -> Path:
    objs = _compile_objects(host_sources(), ["g++"], CXX_FLAGS, "host")
    _link(objs, host_lib_path(), ["g++", "-shared", "-fopenmp"], [])
    return host_lib_path()


def build_cuda() -> Path:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    objs = _compile_objects(cuda_sources(), [nvcc], NVCC_ARCH + NVCC_FLAGS, "cuda")
    _link(objs, cuda_lib_path(), [nvcc, "-shared"] + NVCC_ARCH, ["-lcudart_static", "-ldl", "-lrt", "-lpthread"])
    return cuda_lib_path()


def build_node() -> Path | None:
    srcs = node_sources()
    if not srcs:
        return None
    objs = _compile_objects(srcs, ["g++"], CXX_FLAGS, "node")
    _link(objs, node_cli_path(), ["g++", "-fopenmp"], [])
    return node_cli_path()


def build_all(verbose: bool = False) -> dict[str, str]:
    LIB.mkdir(exist_ok=True)
    out = {"host": str(build_host())}
    if cuda_sources():
        out["cuda"] = str(build_cuda())
    n = build_node()
    if n:
        out["node"] = str(n)
    if verbose:
        for k, v in out.items():
            print(f"built {k}: {v}")
    return out


def is_stale(kind: str) -> bool:
    """True when the library of that kind is missing or older than its sources."""
    try:
        if kind == "host":
            srcs, comp, flags, out = host_sources(), ["g++"], CXX_FLAGS, host_lib_path()
        else:
            nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
            srcs, comp, flags, out = cuda_sources(), [nvcc], NVCC_ARCH + NVCC_FLAGS, cuda_lib_path()
        if not out.exists():
            return True
        hdrs = _headers()
        for s in srcs:
            obj = LIB / "obj" / (kind + "_" + "_".join(s.relative_to(CSRC).with_suffix("").parts) + ".o")
            stamp = obj.with_suffix(".stamp")
            if not stamp.exists() or stamp.read_text() != _digest([s] + hdrs, comp + flags):
                return True
        return False
    except Exception:
        return True


if __name__ == "__main__":
    build_all(verbose=True)
