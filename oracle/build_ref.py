"""Compile the reference's own CPU kernels into ``oracle/_ref/`` (test infrastructure).

The reference's native CPU path is one C++ file, ``src/qste/kernels/cpu.cpp``, a
pybind11/ATen extension.  This script compiles it where it lies, with g++ directly
(the reference's own loader is not run), into ``oracle/_ref/qste_cpu.so``.  No
reference source is copied into this repository.

Flags follow the reference's loader (``src/qste/kernels/loader.py:45-50``) with its
``QSTE_NATIVE_ARCH=0`` setting: ``-O3 -std=c++17`` and no ``-march=native``, so the
compiler cannot contract ``a*b+c`` into an FMA and the integer outputs depend only
on IEEE fp32 arithmetic.  Like the loader's build, there is no ``-fopenmp``: the
hand-written loops run on the calling thread and only ``at::mm`` is threaded.

Where the reference checkout is: the argument, else the environment variable
QSTE_REFERENCE, else a directory named ``reference`` beside this repository.

Usage:  python oracle/build_ref.py [path/to/reference]
"""

from __future__ import annotations

import importlib.util
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref" / "qste_cpu.so"


def reference_root() -> Path:
    """The reference checkout: $QSTE_REFERENCE, else ``reference`` beside this repository."""

    named = os.environ.get("QSTE_REFERENCE")
    return Path(named) if named else HERE.parent.parent / "reference"


def build(reference: Path | None = None, force: bool = False) -> Path | None:
    source = (reference or reference_root()) / "src" / "qste" / "kernels" / "cpu.cpp"
    if not source.exists():
        return OUT if OUT.exists() else None
    if OUT.exists() and not force and OUT.stat().st_mtime >= source.stat().st_mtime:
        return OUT
    import torch
    from torch.utils import cpp_extension

    OUT.parent.mkdir(parents=True, exist_ok=True)
    includes = cpp_extension.include_paths() + [sysconfig.get_paths()["include"]]
    lib_dir = str(Path(torch.__file__).parent / "lib")
    command = [
        "/usr/bin/g++", "-O3", "-std=c++17", "-fPIC", "-shared",
        "-DTORCH_EXTENSION_NAME=qste_cpu", "-DTORCH_API_INCLUDE_EXTENSION_H",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        *[f"-isystem{path}" for path in includes],
        str(source), "-o", str(OUT),
        f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}",
        "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
    ]
    subprocess.run(command, check=True)
    return OUT


def load():
    """Import the compiled reference module, or return None when it was never built."""

    if not OUT.exists():
        return None
    import torch  # noqa: F401  (the extension links against libtorch)

    spec = importlib.util.spec_from_file_location("qste_cpu", OUT)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    target = build(Path(sys.argv[1]) if len(sys.argv) > 1 else None, force=True)
    print(target if target else "reference not present; nothing built")
