"""HAT package support: the `.hat` descriptor and its object model (hat_file), the last packaging step
(packaging), and a loader / benchmarker with hatlib's call shape (loader)."""
from .hat_file import (CallingConventionType, Declaration, Dependencies, Description, Function, HATFile, LibraryReference,
                       OperatingSystem, Parameter, ParameterType, Target, UsageType)
from .loader import BenchmarkResult, FunctionMap, HATFunction, HATPackage, generate_arg_values, load, run_benchmark
from .packaging import create_dynamic_package, create_static_package

__all__ = ["BenchmarkResult", "CallingConventionType", "Declaration", "Dependencies", "Description", "Function", "FunctionMap",
           "HATFile", "HATFunction", "HATPackage", "LibraryReference", "OperatingSystem", "Parameter", "ParameterType", "Target",
           "UsageType", "create_dynamic_package", "create_static_package", "generate_arg_values", "load", "run_benchmark"]
