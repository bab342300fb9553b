"""accera_b200: the HAT-exported GEMM(+ReLU) / reduce_mean / gather / range functions of Accera, re-implemented
as hand-written sm_100a kernels behind the unchanged HAT surface.

    import accera_b200 as acc          # describes functions with the Accera DSL subset in accera_b200.lang
    package = acc.Package(); package.add(...); package.build("name", format=acc.Package.Format.HAT_DYNAMIC)
    from accera_b200 import hat        # hat.load("name.hat"), hat.run_benchmark("name.hat")
"""
from .lang import (AUTO, Array, CacheStrategy, Dimension, Layout, MMAFragmentOp, MMASchedulingPolicy, MMAShape, Nest, Plan,
                   Role, Scalar, ScalarType, Schedule, Target, _cast, _MemorySpace, abs, cast, ceil, create_dimensions, floor, fuse,
                   inf, max, min)
from .package import Package
from .patterns import UnsupportedNestError

__version__ = "0.1.0"

__all__ = ["AUTO", "Array", "CacheStrategy", "Dimension", "Layout", "MMAFragmentOp", "MMASchedulingPolicy", "MMAShape", "Nest",
           "Package", "Plan", "Role", "Scalar", "ScalarType", "Schedule", "Target", "UnsupportedNestError", "abs", "cast",
           "ceil", "create_dimensions", "floor", "fuse", "inf", "max", "min"]
