"""Builds the stand-in UCX of ``tests/fake_ucx`` into a prefix that ``UCX_HOME`` can point at."""
from __future__ import annotations

import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent / "fake_ucx"


def install(prefix: Path) -> Path:
    """``prefix/include`` (the stand-in headers) and ``prefix/lib/libucp.so``, ``libucs.so``."""
    cxx = shutil.which("c++") or shutil.which("g++")
    if cxx is None:
        raise RuntimeError("no C++ compiler")
    (prefix / "lib").mkdir(parents=True, exist_ok=True)
    if not (prefix / "include").exists():
        shutil.copytree(HERE / "include", prefix / "include")
    subprocess.run([cxx, "-std=c++17", "-O1", "-g", "-fPIC", "-shared", f"-I{prefix / 'include'}",
                    str(HERE / "fake_ucp.cpp"), "-o", str(prefix / "lib" / "libucp.so")], check=True)
    empty = prefix / "lib" / "ucs.cpp"
    empty.write_text("extern \"C\" int fake_ucs_is_here(void) { return 1; }\n")
    subprocess.run([cxx, "-fPIC", "-shared", str(empty), "-o", str(prefix / "lib" / "libucs.so")], check=True)
    return prefix
