"""Builds the CUDA library of this package for sm_100a with nvcc, once, and finds it again; and the
small host library (`host/*.cpp`: the cache manager's bookkeeping) with the C++ compiler alone.

`ensure_built()` returns the path of `libkapel_b200.so`. It compiles every `.cu` file of this
folder in parallel when the library is missing or older than its sources (a stamp beside it
holds a hash of sources and flags), printing a line as each file finishes and one every few
seconds meanwhile, so a first call in a fresh checkout shows that it is alive. The library
lands in `_build/` beside the sources; if that folder cannot be written, in a per-user folder
under the system's temporary directory (or `$KAPEL_B200_BUILD_DIR`).

The kernels have plain C launchers (pointers, sizes, a stream), so nothing here needs torch's
headers and a file compiles in seconds.
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
from concurrent.futures import ThreadPoolExecutor, as_completed
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_NAME = "libkapel_b200.so"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC"]      # no fast-math: the 32-bit path is exact arithmetic
# KAPEL_B200_TIMELINE=1: the library with time stamps compiled into the decoding kernels (timeline.cuh),
# in a folder of its own beside the ordinary one. A measuring build: nothing else uses it.
TIMELINE = os.environ.get("KAPEL_B200_TIMELINE") == "1"
if TIMELINE:
    NVCC_FLAGS = NVCC_FLAGS + ["-DKB_TIMELINE"]
BUILD_FOLDER = "_build_timeline" if TIMELINE else "_build"


def sources():
    return sorted(HERE.glob("*.cu"))


def _headers():
    return sorted(HERE.glob("*.cuh")) + sorted(HERE.glob("*.h"))


def _nvcc() -> str:
    for root in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if root and (Path(root) / "bin" / "nvcc").is_file():
            return str(Path(root) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise RuntimeError("kapel_b200: nvcc was not found (CUDA_HOME, /usr/local/cuda, PATH); the kernels cannot be built")


def _stamp() -> str:
    h = hashlib.sha256()
    for f in sources() + _headers():
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    return h.hexdigest()


def _writable(folder: Path) -> bool:
    try:
        folder.mkdir(parents=True, exist_ok=True)
        probe = folder / f".probe-{os.getpid()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("KAPEL_B200_BUILD_DIR")
    if env and _writable(Path(env)):
        return Path(env)
    local = HERE / BUILD_FOLDER
    if _writable(local):
        return local
    fallback = Path(tempfile.gettempdir()) / f"kapel_b200-{BUILD_FOLDER.strip('_')}-{os.getuid()}"
    if _writable(fallback):
        return fallback
    raise RuntimeError(f"kapel_b200: no folder to build in ({local} and {fallback} cannot be written)")


def _say(msg: str, verbose: bool) -> None:
    if verbose:
        print(f"[kapel_b200 build] {msg}", file=sys.stderr, flush=True)


def ensure_built(verbose: bool = True, force: bool = False) -> Path:
    stamp = _stamp()
    # A library that an earlier call built anywhere it could is good if its stamp matches.
    candidates = [HERE / BUILD_FOLDER]
    if os.environ.get("KAPEL_B200_BUILD_DIR"):
        candidates.insert(0, Path(os.environ["KAPEL_B200_BUILD_DIR"]))
    candidates.append(Path(tempfile.gettempdir()) / f"kapel_b200-{BUILD_FOLDER.strip('_')}-{os.getuid()}")
    if not force:
        for d in candidates:
            lib, st = d / LIB_NAME, d / "stamp"
            try:
                if lib.is_file() and st.is_file() and st.read_text().strip() == stamp:
                    return lib
            except OSError:
                continue
    out = build_dir()
    nvcc = _nvcc()
    srcs = sources()
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out} (first call only)", verbose)
    t0 = time.time()
    done = threading.Event()

    def ticker():
        while not done.wait(8.0):
            _say(f"still compiling ... {time.time() - t0:.0f} s", verbose)

    threading.Thread(target=ticker, daemon=True).start()

    def compile_one(src: Path):
        obj = out / (src.stem + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(HERE), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, obj, r

    try:
        objs = []
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
            futures = [pool.submit(compile_one, s) for s in srcs]
            for fut in as_completed(futures):
                src, obj, r = fut.result()
                if r.returncode != 0:
                    raise RuntimeError(f"kapel_b200: nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
                objs.append(obj)
                _say(f"compiled {src.name} ({time.time() - t0:.0f} s)", verbose)
        tmp = out / (LIB_NAME + f".tmp{os.getpid()}")
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for o in sorted(objs)]]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"kapel_b200: linking failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, out / LIB_NAME)
        (out / "stamp").write_text(stamp)
    finally:
        done.set()
    _say(f"built {out / LIB_NAME} in {time.time() - t0:.0f} s", verbose)
    return out / LIB_NAME


# ---------------------------------------------------------------------------------------
# The host library: no CUDA in it, so it builds (in a second or two) and is tested where there is
# neither a GPU nor nvcc.
HOST_LIB_NAME = "libkapel_b200_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-pthread"]


def host_sources():
    return sorted((HERE / "host").glob("*.cpp"))


def _cxx() -> str:
    for name in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        if name and shutil.which(name):
            return shutil.which(name)
    raise RuntimeError("kapel_b200: no C++ compiler was found (CXX, g++, c++, clang++); the cache manager cannot be built")


def _host_stamp() -> str:
    h = hashlib.sha256()
    for f in host_sources():
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(HOST_FLAGS).encode())
    return h.hexdigest()


def ensure_host_built(verbose: bool = True, force: bool = False) -> Path:
    stamp = _host_stamp()
    candidates = [HERE / BUILD_FOLDER]
    if os.environ.get("KAPEL_B200_BUILD_DIR"):
        candidates.insert(0, Path(os.environ["KAPEL_B200_BUILD_DIR"]))
    candidates.append(Path(tempfile.gettempdir()) / f"kapel_b200-{BUILD_FOLDER.strip('_')}-{os.getuid()}")
    if not force:
        for d in candidates:
            lib, st = d / HOST_LIB_NAME, d / "stamp_host"
            try:
                if lib.is_file() and st.is_file() and st.read_text().strip() == stamp:
                    return lib
            except OSError:
                continue
    out = build_dir()
    t0 = time.time()
    tmp = out / (HOST_LIB_NAME + f".tmp{os.getpid()}")
    cmd = [_cxx(), *HOST_FLAGS, *[str(s) for s in host_sources()], "-o", str(tmp)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"kapel_b200: the host library did not compile:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, out / HOST_LIB_NAME)
    (out / "stamp_host").write_text(stamp)
    _say(f"built {out / HOST_LIB_NAME} in {time.time() - t0:.0f} s", verbose)
    return out / HOST_LIB_NAME


if __name__ == "__main__":
    print(ensure_host_built(force="--force" in sys.argv))
    print(ensure_built(force="--force" in sys.argv))
