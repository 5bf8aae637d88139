# GemmKernels with the Blackwell engine underneath: same module and export names as the reference's
# src/GemmKernels.jl; device code replaced by libgemmkernels_b200 (C ABI: include/gemmkernels_b200.h).
# Not executed in this repository's environment (no Julia).
module GemmKernels

include("vocabulary.jl")
include("config.jl")
include("matmul.jl")
include("blas.jl")

export Layout, Operator, Transform, Epilogue, Kernel, CTASwizzle
export Config, ConfigError, get_config, matmul, matmatmul!, mul!, contract!

end
