"""Compile the reference's own CPU shift kernel, unmodified, into oracle/_ref/.

Test infrastructure only.  The single source file
``pytorch/deepshift/kernels/cpu/shift_cpu.cpp`` is compiled where it lies in the reference
checkout with the flags of the reference's ``kernels/cpu/setup.py:9`` (``-O3 -fopenmp``),
by one direct g++ command (no reference build system is run, no source is copied).  The
result is the pybind module ``deepshift_cpu`` exporting ``linear_kernel`` and
``convolution_kernel`` (shift_cpu.cpp:376-379).  It is used to pin oracle/ds_oracle.c, to
generate tests/golden/*.npz and as the timed "reference" CPU baseline.

Usage: python oracle/build_ref.py path-to-reference-checkout   (or DEEPSHIFT_REFERENCE in the environment)
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
SRC_REL = os.path.join("pytorch", "deepshift", "kernels", "cpu", "shift_cpu.cpp")


def ref_module_path():
    return os.path.join(OUT_DIR, "deepshift_cpu" + sysconfig.get_config_var("EXT_SUFFIX"))


def build(reference_root=None, force=False):
    """Returns the path of the built module, or None when the reference is not mounted."""
    reference_root = reference_root or os.environ.get("DEEPSHIFT_REFERENCE")
    out = ref_module_path()
    src = os.path.join(reference_root, SRC_REL) if reference_root else None
    if src is None or not os.path.exists(src):
        return out if os.path.exists(out) else None
    if os.path.exists(out) and not force and os.path.getmtime(out) >= os.path.getmtime(src):
        return out
    from torch.utils import cpp_extension as ce
    import torch

    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["g++", "-O3", "-fopenmp", "-shared", "-fPIC", "-std=c++17",
           "-DTORCH_EXTENSION_NAME=deepshift_cpu", "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in ce.include_paths() + [sysconfig.get_paths()["include"]]:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", out]
    for lib in ce.library_paths():
        cmd += ["-L" + lib, "-Wl,-rpath," + lib]
    cmd += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python"]
    subprocess.run(cmd, check=True)
    return out


if __name__ == "__main__":
    p = build(sys.argv[1] if len(sys.argv) > 1 else None, force=True)
    print(p if p else "reference checkout not found; nothing built")
