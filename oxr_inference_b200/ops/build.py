"""Compiles the CUDA sources under ``csrc/`` for sm_100a with nvcc and loads them with ctypes.

Two kinds of library: ``core`` (everything whose code does not depend on a model size) and ``attn_d<D>``
(the attention kernels, compiled for one head size). A library is compiled at its first use, so a model folder
costs only what that model needs; ``build_all`` compiles a given list up front. Objects are compiled in
parallel, a progress line goes to stderr every few seconds, and the result is kept beside the sources
(``csrc/_build``) when that folder can be written, else in a per-user folder under the system's temp
directory. A hash of the sources and flags decides whether a built library is still current.

There is no fallback: if nvcc is missing or a compile fails, :class:`BuildError` is raised.
"""

from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

CORE_SOURCES = ["elementwise.cu", "qk_norm_rope.cu", "gemm_f32.cu", "gemm_skinny.cu", "gemm_stream.cu", "gemm_tcgen05.cu", "gemm_tcgen05_pair.cu", "gemm_tcgen05_few_rows.cu", "sampling.cu"]
ATTENTION_SOURCES = ["attention.cu"]
HEADERS = ["common.cuh", "tma.cuh", "umma.cuh", "sampling_static.h"]


TIMELINE = os.environ.get("OXR_B200_TIMELINE") == "1"
"""Build (as libraries of their own, ``*_tl``) with the kernels' optional timeline stamps compiled in: every block of a decode
step's kernels then records when it was released and when it ended (``csrc/common.cuh``; read by
``python -m oxr_inference_b200.ops.microbench timeline``). Not for serving: the stamps cost a little time."""


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[oxr_inference_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("OXR_B200_NVCC"), shutil.which("nvcc")]
    for home in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            candidates.append(str(Path(home) / "bin" / "nvcc"))
    for c in candidates:
        if c and Path(c).is_file() and os.access(c, os.X_OK):
            return c
    raise BuildError("nvcc was not found (looked at OXR_B200_NVCC, PATH, CUDA_HOME, /usr/local/cuda); "
                     "the engine has no path that runs without its CUDA kernels")


def build_dir() -> Path:
    """Where built libraries live: $OXR_B200_BUILD_DIR, else csrc/_build, else a per-user temp folder."""
    override = os.environ.get("OXR_B200_BUILD_DIR")
    choices = [Path(override)] if override else []
    choices.append(CSRC / "_build")
    choices.append(Path(tempfile.gettempdir()) / f"oxr_inference_b200_build_{os.getuid()}")
    for d in choices:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".write_probe_{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return d
        except OSError:
            continue
    raise BuildError(f"no writable build folder among {[str(c) for c in choices]}")


def _existing(names: list[str]) -> list[str]:
    return [n for n in names if (CSRC / n).is_file()]


def _digest(sources: list[str], defines: list[str]) -> str:
    h = hashlib.sha256()
    for name in sorted(set(sources) | set(HEADERS)):
        h.update(name.encode())
        h.update((CSRC / name).read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + defines).encode())
    return h.hexdigest()


def _compile(lib_name: str, sources: list[str], defines: list[str]) -> Path:
    out_dir = build_dir()
    lib = out_dir / f"liboxr_b200_{lib_name}.so"
    stamp = out_dir / f"liboxr_b200_{lib_name}.hash"
    digest = _digest(sources, defines)
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
        return lib

    lock_path = out_dir / f".{lib_name}.lock"
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
                return lib  # another process built it while we waited
            nvcc = find_nvcc()
            started = time.monotonic()
            _say(f"compiling {lib_name} ({len(sources)} CUDA file(s)) for sm_100a into {out_dir}")
            work = Path(tempfile.mkdtemp(prefix=f"{lib_name}_", dir=out_dir))
            try:
                jobs = []
                for src in sources:
                    obj = work / (Path(src).stem + ".o")
                    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, *defines, "-I", str(CSRC), "-c", str(CSRC / src), "-o", str(obj)]
                    log = open(work / (Path(src).stem + ".log"), "w+")
                    jobs.append((src, obj, log, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT)))
                last = time.monotonic()
                while any(p.poll() is None for *_, p in jobs):
                    time.sleep(0.2)
                    if time.monotonic() - last >= 5.0:
                        left = [s for s, _, _, p in jobs if p.poll() is None]
                        _say(f"  still compiling {', '.join(left)} ({time.monotonic() - started:.0f} s)")
                        last = time.monotonic()
                failed = []
                for src, _, log, p in jobs:
                    log.seek(0)
                    text = log.read()
                    log.close()
                    if p.returncode != 0:
                        failed.append(f"--- {src} (exit {p.returncode}) ---\n{text}")
                if failed:
                    raise BuildError("nvcc failed:\n" + "\n".join(failed))
                tmp_lib = work / lib.name
                link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp_lib), *[str(o) for _, o, _, _ in jobs]]
                res = subprocess.run(link, capture_output=True, text=True)
                if res.returncode != 0:
                    raise BuildError(f"link of {lib.name} failed:\n{res.stdout}\n{res.stderr}")
                os.replace(tmp_lib, lib)
                stamp.write_text(digest)
            finally:
                shutil.rmtree(work, ignore_errors=True)
            _say(f"built {lib.name} in {time.monotonic() - started:.1f} s")
            return lib
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


_LOADED: dict[str, ctypes.CDLL] = {}


def _load(lib_name: str, sources: list[str], defines: list[str]) -> ctypes.CDLL:
    if lib_name not in _LOADED:
        path = _compile(lib_name, sources, defines)
        try:
            _LOADED[lib_name] = ctypes.CDLL(str(path))
        except OSError as exc:
            raise BuildError(f"could not load {path}: {exc}") from exc
    return _LOADED[lib_name]


def _variant(name: str, defines: list[str]) -> tuple[str, list[str]]:
    return (name + "_tl", defines + ["-DOXR_TIMELINE"]) if TIMELINE else (name, defines)


def core_library() -> ctypes.CDLL:
    name, defines = _variant("core", [])
    return _load(name, _existing(CORE_SOURCES), defines)


def check_head_dim(head_dim: int) -> None:
    if head_dim % 16 != 0 or not 16 <= head_dim <= 256:
        raise ValueError(f"attention kernels take head sizes that are multiples of 16 from 16 to 256, got {head_dim}")


def attention_library(head_dim: int) -> ctypes.CDLL:
    check_head_dim(head_dim)
    name, defines = _variant(f"attn_d{head_dim}", [f"-DHEAD_DIM={head_dim}"])
    return _load(name, _existing(ATTENTION_SOURCES), defines)


def build_all(head_dims: tuple[int, ...] = (16, 32, 64, 128)) -> list[Path]:
    """Compile the core library and the attention library of each head size; returns the library paths."""
    out = [_compile("core", _existing(CORE_SOURCES), [])]
    for d in head_dims:
        check_head_dim(d)
        out.append(_compile(f"attn_d{d}", _existing(ATTENTION_SOURCES), [f"-DHEAD_DIM={d}"]))
    return out
