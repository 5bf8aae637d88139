"""gemmkernels_b200 — the GemmKernels.jl API surface over a Blackwell-native GEMM engine.

Names follow the Julia package (`!` becomes a trailing underscore):

    import gemmkernels_b200 as GemmKernels
    GemmKernels.mul_(C, A, B)                       # GemmKernels.mul!
    GemmKernels.matmatmul_(C, 'N', 'T', A, B, 2, 3) # GemmKernels.matmatmul!
    conf = GemmKernels.get_config(gemm_shape=(M, N, K), operator=GemmKernels.Operator.TCGen05Operator[...], ...)
    GemmKernels.matmul(conf, a, b, c, d; epilogue=GemmKernels.Epilogue.Bias(bias))

Every call ends in libgemmkernels_b200.so (hand-written sm_100a kernels); importing fails when
the library has not been built.
"""
from . import _lib
from . import arrays
from . import cta_swizzle as CTASwizzle
from . import epilogue as Epilogue
from . import kernel as Kernel
from . import layout as Layout
from . import multigpu
from . import operator as Operator
from . import transform as Transform
from .arrays import cuarray, to_cuarray, to_numpy
from .contract import BoundContraction, bind_contract, contract_, contract_query
from .config import Config, ConfigError, DimensionMismatch, get_config, heuristic_block_shape
from .eltypes import (BFloat16, ComplexF16, ComplexF32, Float16, Float32, Float64, Int16, Int32, Int64)
from .matmul import (BoundMatmul, DeviceTimeout, GemmKernelsError, bind, create_config, handle, lower, matmatmul_,
                     matmul, matmul_batched, matmul_host, mul_, poll_status, query)

__all__ = [
    "CTASwizzle", "Epilogue", "Kernel", "Layout", "Operator", "Transform",
    "Config", "ConfigError", "DimensionMismatch", "get_config", "heuristic_block_shape",
    "contract_", "contract_query", "bind_contract", "BoundContraction", "matmul", "matmul_batched", "bind", "BoundMatmul", "matmul_host", "matmatmul_", "mul_", "query", "lower", "create_config", "handle", "poll_status",
    "cuarray", "to_cuarray", "to_numpy",
    "Float16", "BFloat16", "Float32", "Float64", "Int16", "Int32", "Int64", "ComplexF16", "ComplexF32",
    "GemmKernelsError", "DeviceTimeout",
]
