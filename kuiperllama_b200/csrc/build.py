"""Compiling the CUDA sources of this folder for sm_100a, one shared library per source.

A library is built the first time something needs it (so a run compiles only what its
model and dtype use) and is kept beside the sources in ``_build/``; a record of the source
hash and flags decides whether it is still current.  ``build_all()`` compiles everything.
While nvcc runs, a line is printed to stderr every few seconds.

There is no fallback: if nvcc is missing or a source does not compile, ``ExtensionError``
is raised with the compiler's output.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, List, Optional

CSRC = os.path.dirname(os.path.abspath(__file__))

# module name -> source file.  Headers every module depends on are listed in HEADERS.
SOURCES: Dict[str, str] = {
    "rowwise": "rowwise.cu",
    "rope_kv": "rope_kv.cu",
    "attention_simt": "attention_simt.cu",
    "attention_decode": "attention_decode.cu",
    "attention_mma": "attention_mma.cu",
    "attention_tcgen05": "attention_tcgen05.cu",
    "gemm_simt": "gemm_simt.cu",
    "gemm_tcgen05": "gemm_tcgen05.cu",
    "sampling": "sampling.cu",
}
HEADERS: List[str] = ["common.cuh", "tcgen05.cuh", "tma_host.cuh", "attention_decode_noalloc.h"]

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared", "--expt-relaxed-constexpr", "--extended-lambda"]
# Extra flags for experiments (for instance -DNAME to switch a variant on); they are part of the
# record that decides whether a built library is current.
NVCC_FLAGS += os.environ.get("KL_NVCC_FLAGS", "").split()


class ExtensionError(RuntimeError):
    """The CUDA extension is missing and cannot be built, or failed to load."""


def find_nvcc() -> str:
    cands = [os.environ.get("KL_NVCC"),
             os.path.join(os.environ.get("CUDA_HOME", ""), "bin", "nvcc") if os.environ.get("CUDA_HOME") else None,
             "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")]
    for c in cands:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise ExtensionError("nvcc was not found (looked at $KL_NVCC, $CUDA_HOME/bin, /usr/local/cuda/bin and PATH); "
                         "the kernels of kuiperllama_b200 cannot be built and there is no fallback")


def _say(msg: str) -> None:
    print(f"[kuiperllama_b200] {msg}", file=sys.stderr, flush=True)


def _source_hash(name: str) -> str:
    h = hashlib.sha256()
    for f in [SOURCES[name]] + HEADERS:
        with open(os.path.join(CSRC, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _build_dirs() -> List[str]:
    """Where built libraries may live, in order of preference: beside the sources, else a
    per-user folder under the temporary directory (a read-only checkout)."""
    return [os.path.join(CSRC, "_build"),
            os.path.join(tempfile.gettempdir(), f"kuiperllama_b200-build-{os.getuid()}")]


def _writable_dir() -> str:
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".probe-{os.getpid()}-{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise ExtensionError(f"no writable folder for built kernels among {_build_dirs()}")


def _current(path: str, digest: str) -> bool:
    try:
        with open(path + ".hash") as f:
            return f.read().strip() == digest and os.path.isfile(path)
    except OSError:
        return False


def ensure_built(name: str, quiet: bool = False) -> str:
    """Path of the current shared library of module ``name``, compiling it if needed."""
    if name not in SOURCES:
        raise ExtensionError(f"unknown kernel module {name!r}")
    digest = _source_hash(name)
    for d in _build_dirs():
        p = os.path.join(d, f"{name}.so")
        if _current(p, digest):
            return p
    nvcc = find_nvcc()
    out_dir = _writable_dir()
    out = os.path.join(out_dir, f"{name}.so")
    tmp = os.path.join(out_dir, f".{name}.{os.getpid()}.{threading.get_ident()}.so")
    cmd = [nvcc] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, os.path.join(CSRC, SOURCES[name])]
    if not quiet:
        _say(f"compiling {SOURCES[name]} for sm_100a (first use) ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(5.0):
            if not quiet:
                _say(f"  still compiling {SOURCES[name]} ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    output, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise ExtensionError(f"nvcc failed on {SOURCES[name]} (exit {proc.returncode}):\n{' '.join(cmd)}\n{output}")
    os.replace(tmp, out)
    with open(out + ".hash.tmp", "w") as f:
        f.write(digest)
    os.replace(out + ".hash.tmp", out + ".hash")
    if not quiet:
        _say(f"  built {name}.so in {time.time() - t0:.1f} s")
    return out


def build_all(quiet: bool = False, jobs: Optional[int] = None) -> Dict[str, str]:
    """Compile every module (in parallel) and return name -> library path."""
    jobs = jobs or min(len(SOURCES), os.cpu_count() or 2)
    with ThreadPoolExecutor(max_workers=jobs) as pool:
        paths = list(pool.map(lambda n: ensure_built(n, quiet), SOURCES))
    return dict(zip(SOURCES, paths))


if __name__ == "__main__":
    for n, p in build_all().items():
        print(n, p)
