"""Compile the CUDA sources under ``csrc/`` for sm_100a and load them with ctypes.

Each ``csrc/<group>.cu`` becomes one shared library ``<group>-<hash>.so``; a model
loads only the groups its parts use, and a group is compiled the first time it is
needed (a few seconds each with nvcc; nothing else is required).  Libraries are kept
in ``csrc/_build/`` inside the package when that folder can be written, else under
the system's temporary folder, so a fresh checkout run by any user works without a
home directory.  The hash covers the source, the shared header and the flags, so an
edited kernel is rebuilt and a stale library is never loaded.
"""

from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "csrc"

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-shared",
]

# extra link flags per group
EXTRA_FLAGS: dict[str, list[str]] = {
    "gemm_tcgen05": ["-lcuda"],
}


class KernelBuildError(RuntimeError):
    pass


def all_groups() -> list[str]:
    return sorted(p.stem for p in CSRC.glob("*.cu"))


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise KernelBuildError(
        "nvcc was not found (set NVCC or put it on PATH); the CUDA kernels of this engine "
        "are compiled from source at first use and there is no other code path"
    )


def _writable(path: Path) -> bool:
    try:
        path.mkdir(parents=True, exist_ok=True)
        probe = path / f".probe-{os.getpid()}-{threading.get_ident()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


_build_dir: Path | None = None


def build_dir() -> Path:
    global _build_dir
    if _build_dir is None:
        cands = []
        if os.environ.get("QWEN3_RUNTIME_B200_BUILD_DIR"):
            cands.append(Path(os.environ["QWEN3_RUNTIME_B200_BUILD_DIR"]))
        cands.append(CSRC / "_build")
        cands.append(Path(tempfile.gettempdir()) / f"qwen3_runtime_b200_build_{os.getuid()}")
        for cand in cands:
            if _writable(cand):
                _build_dir = cand
                break
        else:
            raise KernelBuildError(f"no writable folder for compiled kernels among {cands}")
    return _build_dir


def _digest(group: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + EXTRA_FLAGS.get(group, [])).encode())
    for path in [CSRC / f"{group}.cu", *sorted(CSRC.glob("*.cuh")), *sorted(CSRC.glob("*.h"))]:
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()[:16]


def library_path(group: str, variant: str = "", defines: tuple[str, ...] = ()) -> Path:
    tag = hashlib.sha256((_digest(group) + " ".join(defines)).encode()).hexdigest()[:16] if defines else _digest(group)
    return build_dir() / f"{group}{variant}-{tag}.so"


def compile_group(group: str, *, verbose: bool = True, variant: str = "", defines: tuple[str, ...] = ()) -> Path:
    """Compile one group if its library is missing; return the library path.  ``variant`` and
    ``defines`` (``-D`` flags) build the same source a second time under another name (a test
    build with other limits); the ordinary library is not touched."""
    src = CSRC / f"{group}.cu"
    if not src.is_file():
        raise KernelBuildError(f"no kernel source {src}")
    out = library_path(group, variant, defines)
    if out.is_file():
        return out
    nvcc = find_nvcc()
    tmp = out.with_name(f".{out.name}.{os.getpid()}.{threading.get_ident()}.tmp")
    cmd = [nvcc, *NVCC_FLAGS, *defines, str(src), "-o", str(tmp), *EXTRA_FLAGS.get(group, [])]
    start = time.time()
    if verbose:
        print(f"[qwen3_runtime_b200] compiling {group}.cu for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=str(CSRC))
    while True:
        try:
            log, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[qwen3_runtime_b200] still compiling {group}.cu ({time.time() - start:.0f} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise KernelBuildError(f"nvcc failed for {group}.cu:\n{log}")
    os.replace(tmp, out)
    for old in out.parent.glob(f"{group}{variant}-*.so"):
        if old != out:
            try:
                old.unlink()
            except OSError:
                pass
    if verbose:
        print(f"[qwen3_runtime_b200] compiled {group}.cu in {time.time() - start:.1f} s", file=sys.stderr, flush=True)
    return out


def compile_groups(groups: list[str], *, verbose: bool = True) -> dict[str, Path]:
    """Compile several groups in parallel (one nvcc each)."""
    results: dict[str, Path] = {}
    errors: list[BaseException] = []
    build_dir()  # settle the folder before the threads start

    def work(g: str) -> None:
        try:
            results[g] = compile_group(g, verbose=verbose)
        except BaseException as exc:  # noqa: BLE001 - re-raised below
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(g,)) for g in groups]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return results


_loaded: dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def load_group(group: str) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(group)
        if lib is None:
            lib = ctypes.CDLL(str(compile_group(group)))
            _loaded[group] = lib
        return lib
