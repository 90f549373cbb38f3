"""In-tree native build: compiles the C++ host core and the sm_100a kernels.

The reference builds one shared library out of per-directory static libraries with
CMake (reference: CMakeLists.txt:19-117, src/CMakeLists.txt:15-82).  Here the same
sources are also buildable without CMake, so that `build()` in the repo root's
entry file and the test-suite can produce the libraries with nothing but nvcc
and g++.  Outputs land in `nccl_plugin_gpudirecttcpx_b200/_lib/`:

  libtcpxb_kernels.so   device kernels behind a C ABI (needs nvcc)
  libnccl-net.so        the NCCL net plugin: host core + kernels + engine (needs nvcc)
  libtcpxb_host.so      host core + engine with no CUDA: device calls go to a stand-in
                        device in host memory (g++ only; used by CPU tests)
  tcpxb_loopback        stand-alone driver of the ncclNet table (g++ only)
  tcpxb_rxdm            rx buffer manager daemon (host pools; g++ only)
  tcpxb_rxdm_gpu        the same daemon linked against the CUDA build: can own device pools

Objects are rebuilt only when a source or header is newer than the object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OUT = PKG / "_lib"
OBJ = OUT / "obj"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-Wextra", "-I", str(CSRC / "include")]
CXX_FLAGS = ["-O2", "-g", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-pthread", "-I", str(CSRC / "include")]


def _nvcc() -> str | None:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    return None


def _headers_mtime() -> float:
    return max((p.stat().st_mtime for p in CSRC.rglob("*.h")), default=0.0)


def _stale(out: Path, srcs: list[Path], hdr_mtime: float) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(s.stat().st_mtime > t for s in srcs) or hdr_mtime > t


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"native build failed: {cmd[0]} {cmd[-1]}")


def _sources(sub: str, ext: str) -> list[Path]:
    return sorted((CSRC / sub).glob(f"*{ext}"))


def _compile(srcs: list[Path], tag: str, compiler: list[str], flags: list[str], hdr: float,
             verbose: bool) -> list[Path]:
    OBJ.mkdir(parents=True, exist_ok=True)
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / f"{tag}_{s.parent.name}_{s.stem}.o"
        objs.append(o)
        if _stale(o, [s], hdr):
            jobs.append(compiler + flags + ["-c", str(s), "-o", str(o)])
    if jobs:
        if verbose:
            print(f"[build] compiling {len(jobs)} file(s) for {tag}", flush=True)
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            list(ex.map(_run, jobs))
    return objs


def build_host(verbose: bool = False, sanitize: str | None = None) -> Path:
    """Host core without CUDA + the loopback driver.  `sanitize` = 'address' / 'thread'."""
    hdr = _headers_mtime()
    tag = "host" if not sanitize else f"host_{sanitize}"
    flags = CXX_FLAGS + ["-DTCPXB_NO_CUDA=1"]
    if sanitize:
        flags = flags + [f"-fsanitize={sanitize}", "-fno-omit-frame-pointer", "-O1"]
    # kernels/*.cc is the CPU statement of the kernel ABI for the stand-in device
    srcs = _sources("core", ".cc") + _sources("plugin", ".cc") + _sources("engine", ".cc") + _sources("kernels", ".cc")
    objs = _compile(srcs, tag, ["g++"], flags, hdr, verbose)
    suffix = "" if not sanitize else f"_{sanitize}"
    lib = OUT / f"libtcpxb_host{suffix}.so"
    if _stale(lib, objs, 0.0):
        link = ["g++", "-shared", "-o", str(lib)] + [str(o) for o in objs] + ["-pthread", "-ldl"]
        if sanitize:
            link.append(f"-fsanitize={sanitize}")
        _run(link)
    tool_srcs = _sources("tools", ".cc")
    for t in tool_srcs:
        exe = OUT / f"tcpxb_{t.stem}{suffix}"
        if _stale(exe, [t, lib], hdr):
            cmd = ["g++"] + flags + [str(t), "-o", str(exe), "-L", str(OUT), f"-l:{lib.name}",
                                     "-Wl,-rpath,$ORIGIN", "-ldl", "-pthread"]
            if sanitize:
                cmd.append(f"-fsanitize={sanitize}")
            _run(cmd)
    return lib


def build_cuda(verbose: bool = False) -> list[Path]:
    """Kernels library and the full plugin (host core + kernels + engine), for sm_100a."""
    nvcc = _nvcc()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build the sm_100a kernels")
    hdr = _headers_mtime()
    nv = [nvcc] + NVCC_ARCH
    kobjs = _compile(_sources("kernels", ".cu"), "cu", nv, NVCC_FLAGS, hdr, verbose)
    klib = OUT / "libtcpxb_kernels.so"
    if _stale(klib, kobjs, 0.0):
        _run([nvcc, "-shared", "-o", str(klib)] + [str(o) for o in kobjs] + ["-cudart", "static"])
    outs = [klib]
    core = _sources("core", ".cc") + _sources("plugin", ".cc") + _sources("engine", ".cc")
    if core:
        cobjs = _compile(core, "full", ["g++"], CXX_FLAGS + ["-I", _cuda_include(nvcc)], hdr, verbose)
        eobjs = _compile(_sources("engine", ".cu") + _sources("core", ".cu"), "cu", nv, NVCC_FLAGS, hdr, verbose)
        plug = OUT / "libnccl-net.so"
        if _stale(plug, cobjs + eobjs + kobjs, 0.0):
            _run([nvcc, "-shared", "-o", str(plug)] + [str(o) for o in cobjs + eobjs + kobjs] +
                 ["-cudart", "static", "-Xlinker", "--no-undefined", "-lpthread", "-ldl", "-lrt"])
        outs.append(plug)
        # the buffer-manager daemon against the CUDA build: the one that can own device pools
        daemon = OUT / "tcpxb_rxdm_gpu"
        src = CSRC / "tools" / "rxdm.cc"
        if _stale(daemon, [src, plug], hdr):
            _run(["g++"] + CXX_FLAGS + ["-I", _cuda_include(nvcc), str(src), "-o", str(daemon), "-L", str(OUT),
                                        f"-l:{plug.name}", "-Wl,-rpath,$ORIGIN", "-ldl", "-pthread"])
        outs.append(daemon)
    return outs


def _cuda_include(nvcc: str) -> str:
    return str(Path(nvcc).resolve().parent.parent / "include")


def build_all(verbose: bool = False) -> None:
    OUT.mkdir(parents=True, exist_ok=True)
    if _sources("core", ".cc"):
        build_host(verbose)
    build_cuda(verbose)


if __name__ == "__main__":
    build_all(verbose=True)
    for p in sorted(OUT.glob("*")):
        if p.is_file():
            print(p)
