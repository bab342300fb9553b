"""HAT package support: the `.hat` descriptor (hat_file) and a loader / benchmarker with hatlib's call shape (loader)."""
from .hat_file import Function, HATFile, Parameter
from .loader import BenchmarkResult, FunctionMap, HATFunction, HATPackage, generate_arg_values, load, run_benchmark

__all__ = ["BenchmarkResult", "Function", "FunctionMap", "HATFile", "HATFunction", "HATPackage", "Parameter",
           "generate_arg_values", "load", "run_benchmark"]
