"""Compiling the CUDA sources into one shared library, and finding it again.

The library is built with nvcc for sm_100a only, at the first call that needs it, and kept beside
the package (``zephyr_b200/_native/``) when that folder can be written, else under the system's
temporary folder.  A stamp made of the sources' contents and the compiler flags tells whether a
library found there still matches the sources.  No home directory, network or Python build
machinery is needed: nvcc and a C++ compiler are.
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
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent.parent
SOURCE_DIR = PACKAGE_DIR / "csrc"
LIBRARY_NAME = "libzephyr_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--threads", "2"]


class BuildError(RuntimeError):
    pass


def sources() -> list[Path]:
    return sorted(SOURCE_DIR.glob("*.cu"))


def find_nvcc() -> str:
    for candidate in (os.environ.get("ZEPHYR_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise BuildError("nvcc was not found (looked at $ZEPHYR_B200_NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of zephyr_b200 cannot be built")


def source_stamp() -> str:
    digest = hashlib.sha256()
    digest.update(" ".join(NVCC_FLAGS).encode())
    for path in sources() + sorted(SOURCE_DIR.glob("*.cuh")) + sorted(SOURCE_DIR.glob("*.h")):
        digest.update(path.name.encode())
        digest.update(path.read_bytes())
    return digest.hexdigest()


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dirs() -> list[Path]:
    """Where a built library may live, in order of preference."""
    dirs = []
    if os.environ.get("ZEPHYR_B200_BUILD_DIR"):
        dirs.append(Path(os.environ["ZEPHYR_B200_BUILD_DIR"]))
    dirs.append(PACKAGE_DIR / "_native")
    dirs.append(Path(tempfile.gettempdir()) / f"zephyr_b200-{os.getuid()}")
    return dirs


def _log(message: str) -> None:
    print(f"[zephyr_b200] {message}", file=sys.stderr, flush=True)


def _compile_one(nvcc: str, src: Path, obj: Path) -> None:
    command = [nvcc, *NVCC_FLAGS, "-I", str(SOURCE_DIR), "-c", str(src), "-o", str(obj)]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{' '.join(command)}\n{result.stdout}\n{result.stderr}")


def build_library(force: bool = False, verbose: bool = True) -> Path:
    """Return the path of an up-to-date library, compiling it if there is none."""
    stamp = source_stamp()
    if not force:
        for folder in build_dirs():
            library, mark = folder / LIBRARY_NAME, folder / "stamp.txt"
            if library.is_file() and mark.is_file() and mark.read_text().strip() == stamp:
                return library
    nvcc = find_nvcc()
    target = next((folder for folder in build_dirs() if _writable(folder)), None)
    if target is None:
        raise BuildError("no writable folder for the compiled kernels: tried " +
                         ", ".join(str(d) for d in build_dirs()))
    files = sources()
    if not files:
        raise BuildError(f"no CUDA sources under {SOURCE_DIR}")
    work = Path(tempfile.mkdtemp(prefix="zephyr_b200_build_", dir=str(target)))
    started = time.time()
    if verbose:
        _log(f"compiling {len(files)} CUDA sources for sm_100a into {target} (first call only)")
    done = threading.Event()

    def heartbeat() -> None:
        while not done.wait(15.0):
            _log(f"still compiling ... {time.time() - started:.0f} s")

    beat = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        beat.start()
    try:
        objects = [work / (src.stem + ".o") for src in files]
        with ThreadPoolExecutor(max_workers=min(len(files), max(1, (os.cpu_count() or 2) // 2))) as pool:
            futures = [pool.submit(_compile_one, nvcc, src, obj) for src, obj in zip(files, objects)]
            for index, (src, future) in enumerate(zip(files, futures), 1):
                future.result()
                if verbose:
                    _log(f"compiled {src.name} ({index}/{len(files)})")
        staged = work / LIBRARY_NAME
        link = [nvcc, "-shared", "-cudart", "shared", "-o", str(staged), *map(str, objects)]
        result = subprocess.run(link, capture_output=True, text=True)
        if result.returncode != 0:
            raise BuildError(f"linking the kernels failed:\n{' '.join(link)}\n{result.stdout}\n{result.stderr}")
        os.replace(staged, target / LIBRARY_NAME)          # atomic: a concurrent reader sees old or new
        (target / "stamp.txt").write_text(stamp + "\n")
    finally:
        done.set()
        shutil.rmtree(work, ignore_errors=True)
    if verbose:
        _log(f"kernels ready after {time.time() - started:.0f} s")
    return target / LIBRARY_NAME
