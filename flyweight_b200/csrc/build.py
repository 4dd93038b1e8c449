"""Compile the CUDA sources of this folder into one shared library for sm_100a.

The library has a plain C interface (no torch headers), so a source file compiles
in seconds.  It is built in-tree (``flyweight_b200/_native/``) at the first call
that needs it and again whenever a source changed; if the tree is read-only the
build goes to a per-user folder under the temporary directory instead.  Progress
lines go to stderr so a first call that compiles is not mistaken for a hang.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from pathlib import Path

SOURCE_DIR = Path(__file__).resolve().parent
PACKAGE_DIR = SOURCE_DIR.parent
LIB_NAME = "libflyweight_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _log(message: str) -> None:
    print(f"[flyweight_b200 build] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for candidate in (
        os.environ.get("FLYWEIGHT_B200_NVCC"),
        shutil.which("nvcc"),
        os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
        "/usr/local/cuda/bin/nvcc",
    ):
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise RuntimeError(
        "flyweight_b200 needs nvcc to compile its CUDA kernels (looked on PATH, in $CUDA_HOME "
        "and in /usr/local/cuda); there is no CPU fallback")


def sources() -> list[Path]:
    return sorted(SOURCE_DIR.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(list(SOURCE_DIR.glob("*.cuh")) + list(SOURCE_DIR.glob("*.h")))


def source_digest() -> str:
    digest = hashlib.sha256()
    for path in sources() + _headers():
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()[:16]


def _writable(directory: Path) -> bool:
    try:
        directory.mkdir(parents=True, exist_ok=True)
        probe = directory / f".probe-{os.getpid()}"
        probe.write_bytes(b"")
        probe.unlink()
        return True
    except OSError:
        return False


def output_dir() -> Path:
    in_tree = PACKAGE_DIR / "_native"
    if _writable(in_tree):
        return in_tree
    fallback = Path(tempfile.gettempdir()) / f"flyweight_b200-{os.getuid()}" / "_native"
    if _writable(fallback):
        return fallback
    raise RuntimeError(f"cannot write the compiled kernels to {in_tree} or {fallback}")


def library_path(build_if_needed: bool = True) -> Path:
    """Path of an up-to-date library, compiling it first when needed."""
    out = output_dir()
    lib = out / LIB_NAME
    stamp = out / "source.digest"
    digest = source_digest()
    if lib.is_file() and stamp.is_file() and stamp.read_text().strip() == digest:
        return lib
    if not build_if_needed:
        raise RuntimeError(f"{lib} is missing or stale")
    build(out, digest)
    return lib


def _compile_one(nvcc: str, src: Path, obj: Path, extra: list[str]) -> tuple[str, float, str]:
    start = time.time()
    cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(SOURCE_DIR), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return src.name, time.time() - start, proc.stderr


def build(out: Path | None = None, digest: str | None = None, verbose_ptxas: bool = False) -> Path:
    """Compile every ``*.cu`` here and link them into one shared library."""
    nvcc = find_nvcc()
    out = out or output_dir()
    digest = digest or source_digest()
    objects_dir = out / "_build"
    objects_dir.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    extra = ["-Xptxas", "-v"] if verbose_ptxas else []
    _log(f"compiling {len(srcs)} CUDA sources for sm_100a into {out} (first call only) ...")
    started = time.time()
    objects: list[Path] = []
    jobs = min(len(srcs), max(1, (os.cpu_count() or 2)))
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        futures = []
        for src in srcs:
            obj = objects_dir / (src.stem + ".o")
            objects.append(obj)
            futures.append(pool.submit(_compile_one, nvcc, src, obj, extra))
        pending = set(futures)
        while pending:
            done, pending = concurrent.futures.wait(pending, timeout=10.0,
                                                    return_when=concurrent.futures.FIRST_COMPLETED)
            for future in done:
                name, seconds, stderr = future.result()
                _log(f"  {name}: {seconds:.1f} s")
                if verbose_ptxas and stderr:
                    print(stderr, file=sys.stderr)
            if pending and not done:
                _log(f"  still compiling ({len(pending)} left, {time.time() - started:.0f} s) ...")
    tmp_lib = out / f".{LIB_NAME}.{os.getpid()}.tmp"
    link = [nvcc, "-shared", "-o", str(tmp_lib), *[str(o) for o in objects],
            "-gencode", "arch=compute_100a,code=sm_100a"]
    proc = subprocess.run(link, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp_lib, out / LIB_NAME)
    (out / "source.digest").write_text(digest + "\n")
    _log(f"built {LIB_NAME} in {time.time() - started:.1f} s")
    return out / LIB_NAME


if __name__ == "__main__":
    build(verbose_ptxas="-v" in sys.argv)
