"""gemmkernels_b200 — host-side mirror of the GemmKernels.jl API over libgemmkernels_b200.so."""
