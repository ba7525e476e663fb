"""In-tree build of the CUDA library (sm_100a only).

``build()`` compiles ``csrc/*.cu`` with nvcc into ``deepshift_b200/_lib/libdeepshift_b200.so``.
The file is git-ignored but travels with the source tree, so a machine without nvcc can use
a library built elsewhere from the same sources.
"""
import concurrent.futures
import glob
import hashlib
import os
import shutil
import subprocess

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "_lib")
LIB_PATH = os.path.join(LIB_DIR, "libdeepshift_b200.so")
STAMP = os.path.join(LIB_DIR, "sources.sha256")
# The checked flavour: every global access of the linear / convolution kernels tests its address
# first (see "Checked build" in include/deepshift_b200.h).  Slower; for tests and for debugging.
CHECKED_LIB_PATH = os.path.join(LIB_DIR, "libdeepshift_b200_checked.so")
CHECKED_STAMP = os.path.join(LIB_DIR, "sources_checked.sha256")
CHECKED_FLAGS = ("-DDS_BOUNDS_CHECK",)
# The timing flavour: the warp-specialised kernel counts, per warp of one CTA, the cycles spent
# waiting at the hand-shake, staging and in the epilogue, and prints them (a diagnostic).
TIMING_LIB_PATH = os.path.join(LIB_DIR, "libdeepshift_b200_timing.so")
TIMING_STAMP = os.path.join(LIB_DIR, "sources_timing.sha256")
TIMING_FLAGS = ("-DDS_WS_TIMING",)

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]  # precise math throughout: never add --use_fast_math, the kernels rely on IEEE rounding


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _digest():
    h = hashlib.sha256()
    files = _sources() + sorted(glob.glob(os.path.join(CSRC, "*.cuh")))
    files.append(os.path.join(os.path.dirname(PKG), "include", "deepshift_b200.h"))
    for f in files:
        h.update(os.path.basename(f).encode())
        with open(f, "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _flavour(checked, timing):
    if checked:
        return CHECKED_LIB_PATH, CHECKED_STAMP, CHECKED_FLAGS, "obj_checked"
    if timing:
        return TIMING_LIB_PATH, TIMING_STAMP, TIMING_FLAGS, "obj_timing"
    return LIB_PATH, STAMP, (), "obj"


def is_current(checked=False, timing=False):
    lib, stamp = _flavour(checked, timing)[:2]
    try:
        with open(stamp) as fh:
            return os.path.exists(lib) and fh.read().strip() == _digest()
    except OSError:
        return False


def nvcc_path():
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def build(force=False, verbose=False, extra_flags=(), checked=False, timing=False):
    """Compile the library if the sources changed.  Returns the library path.

    Every ``.cu`` file is compiled to an object file by its own nvcc process (they run side by
    side), then the objects are linked into the shared library.  ``checked=True`` builds the
    bounds-checking flavour beside the normal one, ``timing=True`` the cycle-counting one."""
    lib_path, stamp, flavour_flags, obj_name = _flavour(checked, timing)
    extra_flags = tuple(extra_flags) + tuple(flavour_flags)
    if not force and is_current(checked, timing):
        return lib_path
    # One builder at a time: the ranks of a multi-process job may all find the library stale at
    # once.  The others wait here and then find it current.
    import fcntl
    os.makedirs(LIB_DIR, exist_ok=True)
    with open(os.path.join(LIB_DIR, ".build.lock"), "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and is_current(checked, timing):
            return lib_path
        return _build_locked(verbose, extra_flags, obj_name, lib_path, stamp)


def _build_locked(verbose, extra_flags, obj_name, lib_path, stamp):
    nvcc = nvcc_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found and %s is missing or stale" % lib_path)
    os.makedirs(LIB_DIR, exist_ok=True)
    obj_dir = os.path.join(LIB_DIR, obj_name)
    os.makedirs(obj_dir, exist_ok=True)
    env = dict(os.environ)
    env.pop("CC", None)
    env.pop("CXX", None)
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"] + list(extra_flags) + ["-ccbin", "g++"]

    def compile_one(src):
        obj = os.path.join(obj_dir, os.path.splitext(os.path.basename(src))[0] + ".o")
        cmd = [nvcc] + compile_flags + ["-c", "-o", obj, src]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        return obj, res.returncode, res.stdout

    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        results = list(pool.map(compile_one, _sources()))
    for _, rc, out in results:
        if verbose or rc:
            print(out, end="")
    bad = [obj for obj, rc, _ in results if rc]
    if bad:
        raise RuntimeError("nvcc failed for: " + ", ".join(os.path.basename(b) for b in bad))
    cmd = [nvcc, "-shared", "-ccbin", "g++", "-o", lib_path] + [obj for obj, _, _ in results]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.run(cmd, check=True, env=env)
    shutil.rmtree(obj_dir, ignore_errors=True)
    with open(stamp, "w") as fh:
        fh.write(_digest())
    return lib_path


if __name__ == "__main__":
    import sys
    flags = [a for a in sys.argv[1:] if a not in ("--checked", "--timing")]
    print(build(force=True, verbose=True, extra_flags=flags, checked="--checked" in sys.argv,
                timing="--timing" in sys.argv))
