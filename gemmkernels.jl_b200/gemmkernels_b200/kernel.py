"""Kernel tags (src/kernel.jl).  The three reference kernels differ in how they stage data through
shared memory; the tcgen05 engine always runs a multi-stage TMA pipeline, so the tags only keep
their validity rules (src/matmul.jl:34-36)."""


class KernelTag:
    def __init__(self, name, needs_two_k_steps):
        self.name = name
        self.needs_two_k_steps = needs_two_k_steps

    def __repr__(self):
        return f"Kernel.{self.name}"


matmul_singlestage = KernelTag("matmul_singlestage", False)     # src/kernel.jl:10-129
matmul_pipelined = KernelTag("matmul_pipelined", True)          # src/kernel.jl:147-350
matmul_pipelined_ng = KernelTag("matmul_pipelined_ng", False)   # src/kernel.jl:368-574
