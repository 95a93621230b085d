"""Compiles the CUDA sources of `holon_b200/csrc` into one shared library for sm_100a.

The library is plain C (`csrc/api.h`), built with nvcc alone: no Python headers, no torch headers, so a first build
takes seconds per file. It lands beside the sources in `csrc/_build/`, named by a hash of the sources, the flags
and the compiler's version, so a stale library is never loaded; where that folder cannot be written it goes to the
system's temporary folder. The reference builds its native plugins ahead of time in the same spirit, keyed by
sources, flags and SM (plugins/holon_plugins/kernels/cpu_task/extension.py:60-69).

A part that brings CUDA of its own does not edit this library: `extension_path(name, sources)` compiles its files the
same way (same flags, the headers of `csrc` on the include path, a name hashed from all of it) into a library of their
own, which the kernel table loads beside this one (`CudaKernels.extension`).
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import pathlib
import shutil
import subprocess
import sys
import tempfile
import time

CSRC = pathlib.Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ("-gencode", "arch=compute_100a,code=sm_100a")
FLAGS = (*ARCH_FLAGS, "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC")
LINK_LIBS = ("-lcuda",)


class BuildError(RuntimeError):
    pass


def nvcc_path() -> str:
    candidates = [os.environ.get("HOLON_B200_NVCC"), shutil.which("nvcc")]
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root:
            candidates.append(os.path.join(root, "bin", "nvcc"))
    for c in candidates:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (looked at HOLON_B200_NVCC, PATH, CUDA_HOME, /usr/local/cuda): the CUDA "
                     "kernels cannot be compiled, and this engine has no other path")


def sources() -> list[pathlib.Path]:
    return sorted(CSRC.glob("*.cu"))


def _key(nvcc: str, extra: tuple[pathlib.Path, ...] | None = None) -> str:
    """Hash of what a library is made from: the sources (`extra`: an extension's own files, beside the headers of
    csrc that they may include; None: all of csrc), the flags and the compiler's version."""
    h = hashlib.sha256()
    own = [*CSRC.glob("*.cuh"), *CSRC.glob("*.h")] + ([*CSRC.glob("*.cu")] if extra is None else [])
    for path in [*sorted(own), *(extra or ())]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    h.update(" ".join(FLAGS + LINK_LIBS).encode())
    version = subprocess.run([nvcc, "--version"], capture_output=True, text=True).stdout
    h.update(version.encode())
    return h.hexdigest()[:16]


def _folders(first: pathlib.Path) -> tuple[pathlib.Path, pathlib.Path]:
    return first, pathlib.Path(tempfile.gettempdir()) / f"holon_b200_build_{os.getuid()}"


def _build_dir(first: pathlib.Path = CSRC / "_build") -> pathlib.Path:
    for folder in _folders(first):
        try:
            folder.mkdir(parents=True, exist_ok=True)
            probe = folder / f".probe{os.getpid()}"
            probe.write_bytes(b"")
            probe.unlink()
            return folder
        except OSError:
            continue
    raise BuildError("no writable folder for the compiled kernels (tried csrc/_build and the temporary folder)")


def library_path(create: bool = True, verbose: bool = True) -> pathlib.Path:
    """The compiled library's path; compiles it first if it is not there (`create`)."""
    nvcc = nvcc_path()
    name = f"libholon_b200_{_key(nvcc)}.so"
    for folder in _folders(CSRC / "_build"):
        if (folder / name).is_file():
            return folder / name
    if not create:
        raise BuildError(f"{name} is not built")
    return _compile(nvcc, _build_dir(), name, verbose, sources(), "libholon_b200_*.so")


def extension_path(name: str, srcs, build_dir=None, verbose: bool = True) -> pathlib.Path:
    """The library of a part's own CUDA files `srcs` (compiled on first use): `build_dir`, else `_build/` beside the
    first file, else the temporary folder. The files may include the headers of csrc (`common.cuh` for the storage
    types, the reductions and HB_REFUSE / HB_CUDA / HB_LAUNCH_CHECK, whose texts the main library's hb_last_error
    hands out; `tcgen05.cuh` for the bounded waits); every exported function is `extern "C"`, returns an int (0: done)
    and takes the stream as its last argument, like the functions of api.h."""
    if not name.isidentifier():
        raise BuildError(f"an extension's name must be an identifier, not {name!r}")
    srcs = tuple(pathlib.Path(s).resolve() for s in srcs)
    missing = [str(s) for s in srcs if not s.is_file()]
    if not srcs or missing:
        raise BuildError(f"extension {name}: no sources" if not srcs else f"extension {name}: no such file: {missing}")
    nvcc = nvcc_path()
    lib = f"libholon_b200x_{name}_{_key(nvcc, srcs)}.so"
    first = pathlib.Path(build_dir) if build_dir is not None else srcs[0].parent / "_build"
    for folder in _folders(first):
        if (folder / lib).is_file():
            return folder / lib
    return _compile(nvcc, _build_dir(first), lib, verbose, list(srcs), f"libholon_b200x_{name}_*.so")


def _say(verbose: bool, text: str) -> None:
    if verbose:
        print(f"holon_b200: {text}", file=sys.stderr, flush=True)


def _compile(nvcc: str, folder: pathlib.Path, name: str, verbose: bool, srcs: list[pathlib.Path],
             older: str) -> pathlib.Path:
    """Compiles `srcs` into `folder/name` and removes the libraries of earlier sources (`older`, a glob)."""
    work = folder / f"obj_{name[:-3]}"
    work.mkdir(parents=True, exist_ok=True)
    _say(verbose, f"compiling {len(srcs)} CUDA files for sm_100a into {folder} (first call only)")
    began = time.time()

    def one(src: pathlib.Path) -> pathlib.Path:
        obj = work / (src.stem + ".o")
        cmd = [nvcc, *FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        while True:
            try:
                out, _ = proc.communicate(timeout=20)
                break
            except subprocess.TimeoutExpired:
                _say(verbose, f"  still compiling {src.name} ({time.time() - began:.0f} s)")
        if proc.returncode:
            raise BuildError(f"nvcc failed on {src.name}:\n{out}")
        _say(verbose, f"  compiled {src.name} ({time.time() - began:.0f} s)")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
        objs = list(pool.map(one, srcs))
    tmp = folder / f".{name}.{os.getpid()}"
    link = subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs), *LINK_LIBS],
                          capture_output=True, text=True)
    if link.returncode:
        raise BuildError(f"linking {name} failed:\n{link.stdout}{link.stderr}")
    os.replace(tmp, folder / name)                      # another process may have built it meanwhile: same bytes
    for old in folder.glob(older):                      # libraries of earlier sources are never loaded again
        if old.name != name:
            try:
                old.unlink()
            except OSError:
                pass
    shutil.rmtree(work, ignore_errors=True)
    _say(verbose, f"built {name} in {time.time() - began:.0f} s")
    return folder / name
