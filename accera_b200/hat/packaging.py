"""Turns a HAT package whose link target is an object file into a static or dynamic package.

The reference builds `P.o` first and then calls the third-party hatlib for the last step
(accera/python/accera/Package.py:766-784):

    hat.create_static_package(header_path, lib_hat_path)     ->  P_lib.hat + a static library
    hat.create_dynamic_package(header_path, dyn_hat_path)    ->  P_dyn.hat + a shared library

and afterwards records the library name under `dependencies.auxiliary["static" | "dynamic"]` and moves the
new `.hat` over the original.  These two functions do that last step with the host toolchain (`ar`, `g++`):
the new `.hat` is a copy of the input whose `link_target` names the library written beside it.  Object files
of accera_b200 packages hold only the thin stubs; the shared library is linked against libaccera_b200.so
(the C-ABI library with the kernels), a static library must be linked with it by the client.

Not checked against hatlib 0.0.39 itself (not installable here): signatures and effects follow the call sites.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from typing import List, Optional

from .hat_file import HATFile, LibraryReference

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CORE_LIBRARY = "libaccera_b200.so"


def _run(cmd: List[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)} failed:\n{r.stdout}\n{r.stderr}")


def _object_of(hat: HATFile, hat_path: str) -> str:
    obj = hat.link_target_path
    if not obj or not obj.endswith((".o", ".obj")):
        raise ValueError(f"{hat_path}: link_target {hat.dependencies.link_target!r} is not an object file")
    if not os.path.exists(obj):
        raise FileNotFoundError(obj)
    return obj


def create_static_package(src_hat_path, dst_hat_path, additional_link_targets: Optional[List[str]] = None) -> HATFile:
    """Archives the object file of `src_hat_path` (and of `additional_link_targets`) into `<dst stem>.a` next to
    `dst_hat_path` and writes `dst_hat_path` pointing at it."""
    src_hat_path, dst_hat_path = str(src_hat_path), str(dst_hat_path)
    hat = HATFile.Deserialize(src_hat_path)
    objs = [_object_of(hat, src_hat_path)] + [str(x) for x in (additional_link_targets or [])]
    stem = os.path.splitext(os.path.basename(dst_hat_path))[0]
    lib_path = os.path.join(os.path.dirname(os.path.abspath(dst_hat_path)), stem + ".a")
    if os.path.exists(lib_path):
        os.remove(lib_path)
    ar = shutil.which("ar")
    if ar is None:
        raise RuntimeError("`ar` is required to create a static package")
    _run([ar, "rcs", lib_path] + objs)
    hat.dependencies.link_target = os.path.basename(lib_path)
    hat.Serialize(dst_hat_path)
    return hat


def create_dynamic_package(src_hat_path, dst_hat_path, additional_link_targets: Optional[List[str]] = None) -> HATFile:
    """Links the object file of `src_hat_path` into `<dst stem>.so` next to `dst_hat_path` (against the libraries
    listed under `dependencies.dynamic`; libaccera_b200.so is found in the accera_b200 package directory, and
    both that directory and the library's own are recorded as run paths) and writes `dst_hat_path` pointing at it."""
    src_hat_path, dst_hat_path = str(src_hat_path), str(dst_hat_path)
    hat = HATFile.Deserialize(src_hat_path)
    objs = [_object_of(hat, src_hat_path)] + [str(x) for x in (additional_link_targets or [])]
    stem = os.path.splitext(os.path.basename(dst_hat_path))[0]
    lib_path = os.path.join(os.path.dirname(os.path.abspath(dst_hat_path)), stem + ".so")
    cxx = shutil.which("g++") or shutil.which("c++")
    if cxx is None:
        raise RuntimeError("a host C++ compiler (g++) is required to create a dynamic package")
    cmd = [cxx, "-shared", "-o", lib_path] + objs + ["-Wl,-rpath,$ORIGIN"]
    for dep in hat.dependencies.dynamic:
        target = dep.get("target_file", "") if isinstance(dep, dict) else ""
        if os.path.basename(target) == CORE_LIBRARY:
            core_dir = os.path.dirname(target) if os.path.isabs(target) and os.path.exists(target) else _PKG_DIR
            cmd += [f"-L{core_dir}", "-laccera_b200", f"-Wl,-rpath,{core_dir}"]
        elif target and os.path.isabs(target) and os.path.exists(target):
            cmd.append(target)
    _run(cmd)
    hat.dependencies.link_target = os.path.basename(lib_path)
    hat.Serialize(dst_hat_path)
    return hat


__all__ = ["create_static_package", "create_dynamic_package", "LibraryReference", "CORE_LIBRARY"]
