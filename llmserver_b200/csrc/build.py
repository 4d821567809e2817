"""Builds the sm_100a kernel library from the ``.cu`` files beside this module.

The sources include no PyTorch header, so a file compiles in seconds with plain ``nvcc``; the
result is one shared library with a C interface that ``llmserver_b200.ops`` loads with ctypes.
Objects are cached under ``_build/`` in the source tree, keyed by a hash of the source, the
shared headers and the flags; only what changed is compiled again.  When the tree cannot be
written the build goes to a per-user folder under the system's temporary directory.

The first call in a fresh checkout compiles everything and prints a progress line per file to
standard error; later calls return at once.
"""
from __future__ import annotations

import concurrent.futures
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time

SOURCE_DIR = os.path.dirname(os.path.abspath(__file__))
LIBRARY_NAME = "libllmserver_b200_kernels.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH_FLAGS + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
                           "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


class KernelBuildError(RuntimeError):
    """The kernel library could not be built; the engine has no other way to run."""


def _say(message: str) -> None:
    print(f"[llmserver_b200] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = [os.environ.get("LLMSERVER_B200_NVCC"), shutil.which("nvcc")]
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root:
            candidates.append(os.path.join(root, "bin", "nvcc"))
    for candidate in candidates:
        if candidate and os.path.isfile(candidate) and os.access(candidate, os.X_OK):
            return candidate
    raise KernelBuildError("nvcc was not found (looked at LLMSERVER_B200_NVCC, PATH, CUDA_HOME and /usr/local/cuda); "
                           "the engine's kernels are CUDA sources that have to be compiled for sm_100a")


def sources() -> list:
    return sorted(name for name in os.listdir(SOURCE_DIR) if name.endswith(".cu"))


def _headers_digest() -> str:
    digest = hashlib.sha256()
    for name in sorted(os.listdir(SOURCE_DIR)):
        if name.endswith((".cuh", ".h")):
            with open(os.path.join(SOURCE_DIR, name), "rb") as handle:
                digest.update(name.encode() + b"\0" + handle.read())
    digest.update(" ".join(NVCC_FLAGS).encode())
    return digest.hexdigest()


def _object_name(source: str, headers_digest: str) -> str:
    with open(os.path.join(SOURCE_DIR, source), "rb") as handle:
        key = hashlib.sha256(handle.read() + headers_digest.encode()).hexdigest()[:16]
    return f"{os.path.splitext(source)[0]}.{key}.o"


def _writable_build_dir() -> str:
    in_tree = os.path.join(SOURCE_DIR, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        tag = hashlib.sha256(SOURCE_DIR.encode()).hexdigest()[:12]
        fallback = os.path.join(tempfile.gettempdir(), f"llmserver_b200-build-{os.getuid()}-{tag}")
        os.makedirs(fallback, exist_ok=True)
        return fallback


def _compile(nvcc: str, source: str, target: str, verbose_ptxas: bool) -> str:
    command = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else []) + \
        ["-I", SOURCE_DIR, "-c", os.path.join(SOURCE_DIR, source), "-o", target + ".tmp"]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise KernelBuildError(f"nvcc failed on {source}:\n{result.stdout}\n{result.stderr}")
    os.replace(target + ".tmp", target)
    return result.stderr


def ensure_built(verbose_ptxas: bool = False, force: bool = False) -> str:
    """Returns the path of an up-to-date kernel library, compiling what is missing."""
    build_dir = _writable_build_dir()
    library = os.path.join(build_dir, LIBRARY_NAME)
    headers_digest = _headers_digest()
    names = sources()
    objects = {source: os.path.join(build_dir, _object_name(source, headers_digest)) for source in names}
    manifest = os.path.join(build_dir, "manifest.txt")
    wanted_manifest = "\n".join(os.path.basename(objects[source]) for source in names)

    def up_to_date() -> bool:
        if force or not os.path.isfile(library) or not os.path.isfile(manifest):
            return False
        with open(manifest) as handle:
            return handle.read() == wanted_manifest

    if up_to_date():
        return library
    with open(os.path.join(build_dir, ".lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if up_to_date():  # another process built it while this one waited
            return library
        nvcc = find_nvcc()
        missing = [source for source in names if force or not os.path.isfile(objects[source])]
        started = time.time()
        if missing:
            _say(f"compiling {len(missing)} CUDA source file(s) for sm_100a into {build_dir} (first use only)")
        done = 0
        logs = {}
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
            futures = {pool.submit(_compile, nvcc, source, objects[source], verbose_ptxas): source for source in missing}
            for future in concurrent.futures.as_completed(futures):
                source = futures[future]
                logs[source] = future.result()
                done += 1
                _say(f"  [{done}/{len(missing)}] {source} ({time.time() - started:.0f} s)")
        if verbose_ptxas:
            for source in sorted(logs):
                sys.stderr.write(logs[source])
        link = [nvcc, "-shared"] + ARCH_FLAGS + ["-o", library + ".tmp"] + [objects[source] for source in names]
        result = subprocess.run(link, capture_output=True, text=True)
        if result.returncode != 0:
            raise KernelBuildError(f"linking the kernel library failed:\n{result.stdout}\n{result.stderr}")
        os.replace(library + ".tmp", library)
        with open(manifest, "w") as handle:
            handle.write(wanted_manifest)
        keep = {os.path.basename(path) for path in objects.values()}
        for name in os.listdir(build_dir):  # objects of older source versions
            if name.endswith(".o") and name not in keep:
                try:
                    os.remove(os.path.join(build_dir, name))
                except OSError:
                    pass
        if missing:
            _say(f"kernel library ready after {time.time() - started:.0f} s")
    return library


if __name__ == "__main__":
    print(ensure_built(verbose_ptxas="-v" in sys.argv, force="--force" in sys.argv))
