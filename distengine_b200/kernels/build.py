"""Compiles the CUDA sources under ``csrc/`` for sm_100a into shared libraries, in the tree.

One library per source file, named ``<module>-<hash>.so`` where the hash covers the source, the
shared header, the definitions and the compiler flags: a stale library is never loaded.  A module
is compiled at its first use, so a run compiles what its model and dtype need; meanwhile a line is
printed every few seconds.  Libraries go to ``csrc/_build`` inside the package (they are loaded
from there, and they travel with the tree); if that folder cannot be written they go to a
per-user folder under the temporary directory.

nvcc cross-compiles without a GPU, so ``build_all`` also serves as the "does it build" check.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

# module -> (source file, libraries to link)
MODULES: dict[str, tuple[str, tuple[str, ...]]] = {
    "core": ("core.cu", ()),
    "gemm_f32": ("gemm_f32.cu", ()),
    "attention_simt": ("attention_simt.cu", ()),
    "linear_small": ("linear_small.cu", ()),
    "gemm_tcgen05": ("gemm_tcgen05.cu", ()),
    "attention_mma": ("attention_mma.cu", ()),          # built per head size: HEAD_DIM=<d>
    "attention_decode": ("attention_decode.cu", ()),    # built per head size: HEAD_DIM=<d>
    "linear_mid": ("linear_mid.cu", ("cuda",)),
    "attention_tcgen05": ("attention_tcgen05.cu", ()),  # built per head size: HEAD_DIM=64|128
}


class BuildError(RuntimeError):
    pass


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.isfile(candidate):
            return candidate
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the "
                     "CUDA kernels of distengine_b200 cannot be compiled")


def _build_dir() -> str:
    primary = os.path.join(CSRC, "_build")
    try:
        os.makedirs(primary, exist_ok=True)
        probe = os.path.join(primary, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return primary
    except OSError:
        fallback = os.path.join(tempfile.gettempdir(), f"distengine_b200-build-{os.getuid()}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def _digest(source: str, defines: tuple[str, ...], libs: tuple[str, ...]) -> str:
    h = hashlib.sha256()
    # the source and every header beside it (a change of a shared header rebuilds all modules)
    headers = sorted(name for name in os.listdir(CSRC) if name.endswith((".cuh", ".h")))
    for path in [os.path.join(CSRC, source)] + [os.path.join(CSRC, name) for name in headers]:
        with open(path, "rb") as handle:
            h.update(handle.read())
    h.update(repr((NVCC_FLAGS, defines, libs)).encode())
    return h.hexdigest()[:12]


def library_path(module: str, defines: tuple[str, ...] = ()) -> tuple[str, str, list[str]]:
    """(path of the library, label, nvcc command that makes it)."""
    if module not in MODULES:
        raise BuildError(f"unknown kernel module '{module}'")
    source, libs = MODULES[module]
    # extra definitions for experiments, e.g. DISTENGINE_B200_DEFINES="PDL_TRIGGER_LATE"
    defines = tuple(defines) + tuple(d for d in os.environ.get("DISTENGINE_B200_DEFINES",
                                                               "").split() if d)
    tag = "".join("_" + d.replace("=", "").replace("-D", "") for d in defines)
    name = f"{module}{tag}-{_digest(source, defines, libs)}.so"
    path = os.path.join(_build_dir(), name)
    command = [find_nvcc(), *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-I", CSRC,
               os.path.join(CSRC, source), *[f"-l{lib}" for lib in libs]]
    return path, f"{source}{tag}", command


def build_many(requests: list[tuple[str, tuple[str, ...]]], verbose: bool = True) -> list[str]:
    """Compile the requested (module, defines) side by side; returns the libraries' paths."""
    paths: list[str] = []
    running: list[tuple[subprocess.Popen, str, str, str, str]] = []
    for module, defines in requests:
        path, label, command = library_path(module, defines)
        paths.append(path)
        if os.path.isfile(path) or any(path == r[1] for r in running):
            continue
        tmp = f"{path}.{os.getpid()}.tmp"
        log = tmp + ".log"
        if verbose:
            print(f"[distengine_b200] compiling {label} for sm_100a ...", file=sys.stderr,
                  flush=True)
        with open(log, "w") as sink:
            proc = subprocess.Popen([*command, "-o", tmp], stdout=sink, stderr=subprocess.STDOUT)
        running.append((proc, path, tmp, log, label))
    started = last = time.time()
    while running:
        time.sleep(0.2)
        for entry in list(running):
            proc, path, tmp, log, label = entry
            if proc.poll() is None:
                continue
            running.remove(entry)
            with open(log) as handle:
                output = handle.read()
            os.remove(log)
            if proc.returncode != 0 or not os.path.isfile(tmp):
                if os.path.isfile(tmp):
                    os.remove(tmp)
                raise BuildError(f"nvcc failed on {label} (exit {proc.returncode}):\n{output}")
            os.replace(tmp, path)
            if verbose:
                print(f"[distengine_b200] compiled {label} in {time.time() - started:.0f} s",
                      file=sys.stderr, flush=True)
        if running and verbose and time.time() - last >= 5.0:
            last = time.time()
            names = ", ".join(r[4] for r in running)
            print(f"[distengine_b200] still compiling {names} ({last - started:.0f} s)",
                  file=sys.stderr, flush=True)
    return paths


def build(module: str, defines: tuple[str, ...] = (), verbose: bool = True) -> str:
    return build_many([(module, defines)], verbose)[0]


def build_all(verbose: bool = True) -> list[str]:
    """Every module in its default form (the build check)."""
    from .library import default_build_requests
    return build_many(default_build_requests(), verbose)
