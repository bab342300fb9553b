"""The `.hat` descriptor: a C header with an embedded TOML document.

Layout and key names follow the reference's emitter
(accera/hat/include/HATEmitter.h:21-75 guards, :95-165 enumerations, :309-410
argument tables, :459-480 function tables, :1197-1265 section order) and the
Python post-processing in accera/python/accera/Package.py:672-784.  Every line the
C preprocessor sees outside `#ifdef TOML` is a `#` comment to a TOML parser and the
header text sits inside a TOML multi-line literal string, so the same file is
both a valid header and a valid TOML document.
"""
from __future__ import annotations

import dataclasses
import os
import re
from typing import Any, Dict, List, Optional

try:                                    # Python >= 3.11
    import tomllib as _toml_reader
except ModuleNotFoundError:             # pragma: no cover
    import tomli as _toml_reader

LOGICAL_TYPES = ("affine_array", "runtime_array", "element", "void")
USAGES = ("input", "output", "input_output")
CALLING_CONVENTIONS = ("stdcall", "cdecl", "fastcall", "vectorcall", "device")


@dataclasses.dataclass
class Parameter:
    """One function argument (or the return slot)."""
    name: str = ""
    description: str = ""
    logical_type: str = "affine_array"
    declared_type: str = "float*"
    element_type: str = "float"
    usage: str = "input"
    shape: Optional[List[int]] = None            # affine_array
    affine_map: Optional[List[int]] = None       # affine_array: strides in elements
    affine_offset: Optional[int] = None          # affine_array
    size: Optional[str] = None                   # runtime_array: product of dimension-argument names

    def to_table(self) -> Dict[str, Any]:
        t: Dict[str, Any] = {
            "name": self.name, "description": self.description, "logical_type": self.logical_type,
            "declared_type": self.declared_type, "element_type": self.element_type, "usage": self.usage,
        }
        if self.logical_type == "affine_array":
            t["shape"] = list(self.shape or [])
            t["affine_map"] = list(self.affine_map or [])
            t["affine_offset"] = int(self.affine_offset or 0)
        elif self.logical_type == "runtime_array":
            t["size"] = self.size or ""
        return t

    @staticmethod
    def from_table(t: Dict[str, Any]) -> "Parameter":
        if t.get("logical_type") not in LOGICAL_TYPES:
            raise ValueError(f"unknown logical_type {t.get('logical_type')!r}")
        if t.get("usage") not in USAGES:
            raise ValueError(f"unknown usage {t.get('usage')!r}")
        return Parameter(
            name=t.get("name", ""), description=t.get("description", ""), logical_type=t["logical_type"],
            declared_type=t["declared_type"], element_type=t["element_type"], usage=t["usage"],
            shape=list(t["shape"]) if "shape" in t else None,
            affine_map=list(t["affine_map"]) if "affine_map" in t else None,
            affine_offset=t.get("affine_offset"), size=t.get("size"))


VOID_RETURN = Parameter(name="", description="", logical_type="void", declared_type="void", element_type="void",
                        usage="output")


@dataclasses.dataclass
class Function:
    name: str
    description: str = ""
    calling_convention: str = "cdecl"
    arguments: List[Parameter] = dataclasses.field(default_factory=list)
    return_info: Parameter = dataclasses.field(default_factory=lambda: dataclasses.replace(VOID_RETURN))
    auxiliary: Dict[str, Any] = dataclasses.field(default_factory=dict)
    # GPU bookkeeping the reference adds for CUDA/ROCm packages (Package.py:726-743)
    launches: Optional[str] = None
    launch_parameters: Optional[List[int]] = None
    dynamic_shared_mem_bytes: Optional[int] = None
    provider: Optional[str] = None
    runtime: Optional[str] = None

    def c_declaration(self) -> str:
        """`void name(T*, T*, ...);` - prototypes carry no parameter names (TranslateToHeader.cpp:402-453)."""
        args = ", ".join(a.declared_type for a in self.arguments)
        return f"{self.return_info.declared_type} {self.name}({args});"

    def c_alias(self, base_name: str) -> str:
        """Guarded fixed-name alias (TranslateToHeader.cpp:455-506)."""
        args = ", ".join(a.declared_type for a in self.arguments)
        return (f"#ifndef __{base_name}_DEFINED__\n#define __{base_name}_DEFINED__\n"
                f"{self.return_info.declared_type} (*{base_name})({args}) = {self.name};\n#endif\n")


@dataclasses.dataclass
class HATFile:
    name: str
    description: Dict[str, Any] = dataclasses.field(default_factory=lambda: {
        "comment": "", "author": "", "version": "", "license_url": ""})
    functions: List[Function] = dataclasses.field(default_factory=list)
    device_functions: List[Function] = dataclasses.field(default_factory=list)
    target: Dict[str, Any] = dataclasses.field(default_factory=dict)
    dependencies: Dict[str, Any] = dataclasses.field(default_factory=lambda: {
        "link_target": "", "deploy_files": [], "dynamic": []})
    compiled_with: Dict[str, Any] = dataclasses.field(default_factory=lambda: {
        "compiler": "", "flags": "", "crt": "", "libraries": []})
    declaration_code: str = ""
    path: Optional[str] = None

    # -- lookup ------------------------------------------------------------
    @property
    def function_map(self) -> Dict[str, Function]:
        return {f.name: f for f in self.functions}

    @property
    def link_target_path(self) -> Optional[str]:
        lt = self.dependencies.get("link_target", "")
        if not lt:
            return None
        base = os.path.dirname(self.path) if self.path else "."
        return os.path.join(base, lt)

    # -- serialisation -----------------------------------------------------
    def serialize(self) -> str:
        out: List[str] = []
        out.append(f"\n#ifndef __{self.name}__\n#define __{self.name}__\n")
        out.append("\n#ifdef TOML\n")
        out.append(_table("description", self.description) + "\n")
        for group, funcs in (("functions", self.functions), ("device_functions", self.device_functions)):
            if not funcs and group == "device_functions":
                continue
            if not funcs:
                out.append(f"[{group}]\n")
            for f in funcs:
                out.append(_function_table(group, f))
            out.append("\n")
        out.append(_table("target", self.target) + "\n")
        out.append(_table("dependencies", self.dependencies) + "\n")
        out.append(_table("compiled_with", self.compiled_with) + "\n")
        if "'''" in self.declaration_code:
            raise ValueError("declaration code must not contain ''' (it is stored in a TOML literal string)")
        out.append("[declaration]\ncode = '''\n#endif // TOML\n" + self.declaration_code + "\n#ifdef TOML\n'''\n")
        out.append("\n#endif // TOML\n")
        out.append(f"\n#endif // __{self.name}__\n")
        return "".join(out)

    def write(self, path: str) -> None:
        with open(path, "w") as f:
            f.write(self.serialize())
        self.path = path

    # the method names of the third-party library the reference calls
    # (accera/python/accera/Package.py:678-764)
    def Serialize(self, path: str) -> None:      # noqa: N802
        self.write(path)

    @staticmethod
    def Deserialize(path: str) -> "HATFile":     # noqa: N802
        return HATFile.read(path)

    @staticmethod
    def read(path: str) -> "HATFile":
        with open(path, "rb") as f:
            doc = _toml_reader.load(f)
        text = open(path).read()
        m = re.search(r"#ifndef __(\w+)__", text)
        name = m.group(1) if m else os.path.splitext(os.path.basename(path))[0]
        hf = HATFile(name=name, path=path)
        hf.description = dict(doc.get("description", {}))
        for group, dest in (("functions", hf.functions), ("device_functions", hf.device_functions)):
            for fname, ft in doc.get(group, {}).items():
                fn = Function(
                    name=ft.get("name", fname), description=ft.get("description", ""),
                    calling_convention=ft.get("calling_convention", "cdecl"),
                    arguments=[Parameter.from_table(a) for a in ft.get("arguments", [])],
                    return_info=Parameter.from_table(ft["return"]) if "return" in ft else dataclasses.replace(VOID_RETURN),
                    auxiliary=dict(ft.get("auxiliary", {})),
                    launches=ft.get("launches"), launch_parameters=ft.get("launch_parameters"),
                    dynamic_shared_mem_bytes=ft.get("dynamic_shared_mem_bytes"), provider=ft.get("provider"),
                    runtime=ft.get("runtime"))
                if fn.calling_convention not in CALLING_CONVENTIONS:
                    raise ValueError(f"{fname}: unknown calling_convention {fn.calling_convention!r}")
                dest.append(fn)
        hf.target = dict(doc.get("target", {}))
        hf.dependencies = dict(doc.get("dependencies", {}))
        hf.compiled_with = dict(doc.get("compiled_with", {}))
        code = doc.get("declaration", {}).get("code", "")
        code = re.sub(r"^\s*#endif // TOML\n", "", code)
        code = re.sub(r"\n#ifdef TOML\s*$", "", code)
        hf.declaration_code = code
        return hf


# ---------------------------------------------------------------------------
# a small TOML writer for exactly the shapes above (inline tables inside arrays,
# nested tables as dotted headers) - tomli_w cannot emit inline tables
# ---------------------------------------------------------------------------

def _scalar(v: Any) -> str:
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, int):
        return str(v)
    if isinstance(v, float):
        return repr(v)
    if isinstance(v, str):
        if "'" not in v and "\n" not in v:
            return f"'{v}'"
        return '"' + v.replace("\\", "\\\\").replace('"', '\\"').replace("\n", "\\n") + '"'
    if isinstance(v, (list, tuple)):
        return "[ " + ", ".join(_scalar(x) for x in v) + " ]" if v else "[]"
    if isinstance(v, dict):
        return "{ " + ", ".join(f"{_key(k)} = {_scalar(x)}" for k, x in v.items()) + " }" if v else "{}"
    raise TypeError(f"cannot serialise {type(v).__name__} into a .hat file")


def _key(k: str) -> str:
    return k if re.fullmatch(r"[A-Za-z0-9_-]+", k) else '"' + k.replace('"', '\\"') + '"'


def _table(header: str, table: Dict[str, Any]) -> str:
    """`[header]` with scalar / array / empty-table keys first, then non-empty nested tables as `[header.sub]`.
    A table that holds nothing but nested tables gets no header of its own (TOML creates it implicitly)."""
    lines = []
    nested = []
    for k, v in table.items():
        if isinstance(v, dict) and v:
            nested.append((k, v))
        else:
            lines.append(f"{_key(k)} = {_scalar(v)}")
    text = ""
    if lines or not nested:
        text = "\n".join([f"[{header}]"] + lines) + "\n"
    for k, v in nested:
        text += ("\n" if text else "") + _table(f"{header}.{_key(k)}", v)
    return text


def _function_table(group: str, f: Function) -> str:
    h = f"{group}.{_key(f.name)}"
    lines = [f"[{h}]", f"name = {_scalar(f.name)}", f"description = {_scalar(f.description)}",
             f'calling_convention = "{f.calling_convention}"']
    if f.arguments:
        lines.append("arguments = [")
        lines.append(",\n".join("    " + _scalar(a.to_table()) for a in f.arguments))
        lines.append("]")
    else:
        lines.append("arguments = []")
    lines.append(f"return = {_scalar(f.return_info.to_table())}")
    for key in ("launches", "launch_parameters", "dynamic_shared_mem_bytes", "provider", "runtime"):
        v = getattr(f, key)
        if v is not None:
            lines.append(f"{key} = {_scalar(v)}")
    text = "\n".join(lines) + "\n"
    if f.auxiliary:
        text += "\n" + _table(f"{h}.auxiliary", f.auxiliary)
    return text + "\n"


# ---------------------------------------------------------------------------
# header text (TranslateToHeader.cpp:165-201)
# ---------------------------------------------------------------------------

def header_prologue(library_name: str) -> str:
    return (
        f"//\n// Header for Accera library {library_name}\n//\n\n"
        "#if defined(__cplusplus)\n#include <cstdint>\n#else\n#include <stdint.h>\n#include <stdbool.h>\n"
        "#endif // defined(__cplusplus)\n"
        "#if !defined(ACCERA_FLOAT)\n#define ACCERA_FLOAT 1\ntypedef uint16_t float16_t;\ntypedef uint16_t bfloat16_t;\n"
        "#endif // !defined(ACCERA_FLOAT)\n"
        "#if defined(__cplusplus)\nextern \"C\"\n{\n#endif // defined(__cplusplus)\n\n"
        "//\n// Functions\n//\n\n")


def header_epilogue() -> str:
    return "#if defined(__cplusplus)\n} // extern \"C\"\n#endif // defined(__cplusplus)\n"
