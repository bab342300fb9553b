"""The `.hat` descriptor: a C header with an embedded TOML document, and the object model the reference
drives it through.

Layout and key names follow the reference's emitter
(accera/hat/include/HATEmitter.h:21-75 guards, :95-165 enumerations, :309-410
argument tables, :459-480 function tables, :1197-1265 section order) and the
Python post-processing in accera/python/accera/Package.py:672-784.  Every line the
C preprocessor sees outside `#ifdef TOML` is a `#` comment to a TOML parser and the
header text sits inside a TOML multi-line literal string, so the same file is
both a valid header and a valid TOML document.

The reference never parses a `.hat` itself: it goes through the third-party hatlib
(hatlib==0.0.39, not part of the reference tree and not installable here), as
attribute accesses on a HATFile:

    hat_file = HATFile.Deserialize(path)                         Package.py:678
    hat_file.dependencies.link_target = "P.so"                   :681
    hat_file.dependencies.dynamic = [LibraryReference(target_file=...)]   :693, 701
    hat_file.declaration.code                                    :696, 700, 702
    hat_file.function_map.get(name).auxiliary = {...}            :708-712
    hat_file.target.required.gpu.runtime = "CUDA"                :726-728
    hat_file.device_function_map[name] = Function(..., calling_convention=CallingConventionType.Device, ...)  :733-743
    hat_file.target.required.os = OperatingSystem.Linux          :745-751
    hat_file.target.required.cpu.architecture / .extensions      :752-756
    hat_file.description.author / .version / .license_url / .auxiliary     :758-762
    hat_file.Serialize(path)                                     :764
    create_static_package / create_dynamic_package               :766-784   (accera_b200/hat/packaging.py)

This module offers exactly those spellings (written from the call sites above and the `.hat` schema, not from
hatlib's code; not checked against hatlib 0.0.39 itself: it cannot be installed here).  Every table is at the
same time a plain dict with the TOML key names, so `hat_file.dependencies["link_target"]` and
`hat_file.target["required"]["GPU"]` read the same data.
"""
from __future__ import annotations

import dataclasses
import enum
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


class CallingConventionType(str, enum.Enum):
    """calling_convention of a function table (HATEmitter.h:142-165; "device" is added by Package.py:736)."""
    StdCall = "stdcall"
    CDecl = "cdecl"
    FastCall = "fastcall"
    VectorCall = "vectorcall"
    Device = "device"

    def __str__(self) -> str:
        return self.value


class OperatingSystem(str, enum.Enum):
    """[target.required] os (HATEmitter.h:632-650)."""
    Windows = "windows"
    MacOS = "macos"
    Linux = "linux"

    def __str__(self) -> str:
        return self.value

    @staticmethod
    def host() -> "OperatingSystem":
        import platform
        return {"Windows": OperatingSystem.Windows, "Darwin": OperatingSystem.MacOS}.get(platform.system(), OperatingSystem.Linux)


class UsageType(str, enum.Enum):
    Input = "input"
    Output = "output"
    InputOutput = "input_output"

    def __str__(self) -> str:
        return self.value


class ParameterType(str, enum.Enum):
    AffineArray = "affine_array"
    RuntimeArray = "runtime_array"
    Element = "element"
    Void = "void"

    def __str__(self) -> str:
        return self.value


class AttrTable(dict):
    """A TOML table whose keys can also be read and written as attributes.

    `_ALIASES` maps an attribute spelling to the key the file uses (hatlib says `.cpu` / `.gpu`, the file says
    `CPU` / `GPU`); `_TABLES` names the nested tables that exist by schema: reading one that the file does not
    have yet creates it empty, so that `target.required.gpu.runtime = "CUDA"` works on a CPU-only file.  Tables
    created that way and never filled are left out when the file is written.
    """
    _ALIASES: Dict[str, str] = {}
    _TABLES: Dict[str, type] = {}

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        key = type(self)._ALIASES.get(name, name)
        if key in self:
            return self[key]
        cls = type(self)._TABLES.get(key)
        if cls is not None:
            t = cls()
            object.__setattr__(t, "_auto", True)
            self[key] = t
            return t
        raise AttributeError(f"{type(self).__name__} has no entry {name!r}")

    def __setattr__(self, name: str, value) -> None:
        self[type(self)._ALIASES.get(name, name)] = value

    def __delattr__(self, name: str) -> None:
        del self[type(self)._ALIASES.get(name, name)]

    def prune(self) -> None:
        """Drops the nested tables that were created by looking at them and never received an entry."""
        for k, v in list(self.items()):
            if isinstance(v, AttrTable):
                v.prune()
                if not v and getattr(v, "_auto", False):
                    del self[k]

    @classmethod
    def wrap(cls, d: Optional[dict]) -> "AttrTable":
        """A table of this class holding `d`'s entries, nested dicts wrapped by schema."""
        t = cls()
        for k, v in (d or {}).items():
            if isinstance(v, dict) and not isinstance(v, AttrTable):
                v = cls._TABLES.get(k, AttrTable).wrap(v)
            t[k] = v
        return t


class Description(AttrTable):
    """[description]: comment, author, version, license_url, auxiliary (HATEmitter.h:523-535)."""
    _TABLES = {"auxiliary": AttrTable}

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        for k in ("comment", "author", "version", "license_url"):
            self.setdefault(k, "")


class LibraryReference(AttrTable):
    """One entry of [dependencies] dynamic: {name, version, target_file} (HATEmitter.h:1000-1020)."""

    def __init__(self, name: str = "", version: str = "", target_file: str = "", **kw):
        super().__init__(name=name, version=version, target_file=target_file, **kw)


class Dependencies(AttrTable):
    """[dependencies]: link_target, deploy_files, dynamic, auxiliary (HATEmitter.h:1061-1080)."""
    _TABLES = {"auxiliary": AttrTable}

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.setdefault("link_target", "")
        self.setdefault("deploy_files", [])
        self.setdefault("dynamic", [])

    @classmethod
    def wrap(cls, d):
        t = super().wrap(d)
        t["dynamic"] = [x if isinstance(x, LibraryReference) else LibraryReference(**x) for x in t.get("dynamic", [])]
        return t


class CPU(AttrTable):
    """[target.required.CPU]: architecture, extensions (HATEmitter.h:652-662)."""


class GPU(AttrTable):
    """[target.required.GPU]: runtime, model, instruction_set_version, min_threads, min_*_memory_KB (:664-683)."""


class Required(AttrTable):
    _ALIASES = {"cpu": "CPU", "gpu": "GPU"}
    _TABLES = {"CPU": CPU, "GPU": GPU}


class OptimizedFor(AttrTable):
    _ALIASES = {"cpu": "CPU", "gpu": "GPU"}
    _TABLES = {"CPU": CPU, "GPU": GPU}


class Target(AttrTable):
    """[target]: required, optimized_for (HATEmitter.h:632-936)."""
    _TABLES = {"required": Required, "optimized_for": OptimizedFor}


class CompiledWith(AttrTable):
    """[compiled_with]: compiler, flags, crt, libraries (HATEmitter.h:1120-1138)."""

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        for k, v in (("compiler", ""), ("flags", ""), ("crt", ""), ("libraries", [])):
            self.setdefault(k, v)


class CodeString(str):
    """The header text of [declaration] code.  `_new` builds another value of the same kind, which is how the
    reference appends the declarations of supporting packages (Package.py:700-702)."""

    def _new(self, text) -> "CodeString":
        return CodeString(str(text))


class Declaration:
    """[declaration]: code."""

    def __init__(self, code: str = ""):
        self._code = CodeString(code)

    @property
    def code(self) -> CodeString:
        return self._code

    @code.setter
    def code(self, value) -> None:
        self._code = CodeString(str(value))

    def __eq__(self, other) -> bool:
        return isinstance(other, Declaration) and str(self._code) == str(other._code)


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
    calling_convention: str = "cdecl"           # a CALLING_CONVENTIONS string or a CallingConventionType
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


class FunctionTable:
    """Holds the functions of one group (host functions, or device functions), by name, in file order."""

    def __init__(self):
        self.function_map: Dict[str, Function] = {}


class HATFile:
    """One `.hat` file.  Tables are reached as attributes (see the module docstring) or as dicts."""

    def __init__(self, name: str = "", description=None, functions: Optional[List[Function]] = None,
                 device_functions: Optional[List[Function]] = None, target=None, dependencies=None, compiled_with=None,
                 declaration_code: str = "", path: Optional[str] = None):
        self.name = name
        self.description = description
        self._function_table = FunctionTable()
        self._device_function_table = FunctionTable()
        for f in functions or []:
            self._function_table.function_map[f.name] = f
        for f in device_functions or []:
            self._device_function_table.function_map[f.name] = f
        self.target = target
        self.dependencies = dependencies
        self.compiled_with = compiled_with
        self.declaration = Declaration(declaration_code)
        self.path = path

    # -- tables: whatever is assigned (a plain dict, another table) is kept as the schema's table class ------
    description = property(lambda self: self._description,
                           lambda self, v: setattr(self, "_description", v if isinstance(v, Description) else Description.wrap(v)))
    target = property(lambda self: self._target,
                      lambda self, v: setattr(self, "_target", v if isinstance(v, Target) else Target.wrap(v)))
    dependencies = property(lambda self: self._dependencies,
                            lambda self, v: setattr(self, "_dependencies", v if isinstance(v, Dependencies) else Dependencies.wrap(v)))
    compiled_with = property(lambda self: self._compiled_with,
                             lambda self, v: setattr(self, "_compiled_with", v if isinstance(v, CompiledWith) else CompiledWith.wrap(v)))

    # -- functions -----------------------------------------------------------
    @property
    def function_map(self) -> Dict[str, Function]:
        """name -> Function, the live table (assigning into it adds a function)."""
        return self._function_table.function_map

    @property
    def device_function_map(self) -> Dict[str, Function]:
        return self._device_function_table.function_map

    @property
    def functions(self) -> List[Function]:
        return list(self._function_table.function_map.values())

    @property
    def device_functions(self) -> List[Function]:
        return list(self._device_function_table.function_map.values())

    @property
    def declaration_code(self) -> str:
        return str(self.declaration.code)

    @declaration_code.setter
    def declaration_code(self, value: str) -> None:
        self.declaration.code = value

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
        for t in (self.description, self.target, self.dependencies, self.compiled_with):
            t.prune()
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
        code = self.declaration_code
        if "'''" in code:
            raise ValueError("declaration code must not contain ''' (it is stored in a TOML literal string)")
        out.append("[declaration]\ncode = '''\n#endif // TOML\n" + code + "\n#ifdef TOML\n'''\n")
        out.append("\n#endif // TOML\n")
        out.append(f"\n#endif // __{self.name}__\n")
        return "".join(out)

    def write(self, path: Optional[str] = None) -> None:
        path = path or self.path
        if not path:
            raise ValueError("no path to write the .hat file to")
        with open(path, "w") as f:
            f.write(self.serialize())
        self.path = str(path)

    def Serialize(self, path: Optional[str] = None) -> None:      # noqa: N802  (Package.py:764, 773, 783)
        self.write(path)

    @staticmethod
    def Deserialize(path) -> "HATFile":     # noqa: N802  (Package.py:678; also called on an instance, :772)
        return HATFile.read(str(path))

    @staticmethod
    def read(path: str) -> "HATFile":
        path = str(path)
        with open(path, "rb") as f:
            doc = _toml_reader.load(f)
        text = open(path).read()
        m = re.search(r"#ifndef __(\w+)__", text)
        name = m.group(1) if m else os.path.splitext(os.path.basename(path))[0]
        hf = HATFile(name=name, path=path)
        hf.description = doc.get("description", {})
        for group, dest in (("functions", hf.function_map), ("device_functions", hf.device_function_map)):
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
                dest[fn.name] = fn
        hf.target = doc.get("target", {})
        hf.dependencies = doc.get("dependencies", {})
        hf.compiled_with = doc.get("compiled_with", {})
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
    if isinstance(v, enum.Enum):
        v = v.value
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


def _enum_value(v):
    return v.value if isinstance(v, enum.Enum) else v


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
             f'calling_convention = "{_enum_value(f.calling_convention)}"']
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
