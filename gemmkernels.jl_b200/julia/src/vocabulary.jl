# Type vocabulary of GemmKernels.jl kept as tags (no device code): the kernels live behind the C ABI.
# Not executed in this repository's environment (no Julia); mirrors gemmkernels_b200/*.py.

module Layout
    abstract type LayoutBase{T} end
    abstract type Zero{T} <: LayoutBase{T} end                      # src/layout.jl:82-89
    abstract type ColMajor{T} <: LayoutBase{T} end                  # 111-144
    abstract type RowMajor{T} <: LayoutBase{T} end                  # 150-184
    abstract type UnsafeAlignedColMajor{T} <: LayoutBase{T} end     # 192-219
    abstract type UnsafeAlignedRowMajor{T} <: LayoutBase{T} end     # 244-270
    abstract type Diagonal{T} <: LayoutBase{T} end                  # 225-236
    abstract type InterleavedColMajor{T} <: LayoutBase{T} end       # 276-303
    abstract type InterleavedRowMajor{T} <: LayoutBase{T} end       # 305-334
    abstract type SplitColMajor{T} <: LayoutBase{T} end             # 340-373
    abstract type SplitRowMajor{T} <: LayoutBase{T} end             # 379-411
    abstract type Padded{L, P} end                                  # 95-105: a no-op hint here (swizzle replaces padding)

    eltype(::Type{<:LayoutBase{T}}) where {T} = T
    eltype(::Type{<:Padded{L, P}}) where {L, P} = eltype(L)
    base(::Type{L}) where {L <: LayoutBase} = L
    base(::Type{<:Padded{L, P}}) where {L, P} = base(L)

    col_major(::Type{L}) where {L} = !(base(L) <: Union{RowMajor, UnsafeAlignedRowMajor, InterleavedRowMajor, SplitRowMajor})
    is_zero(::Type{L}) where {L} = base(L) <: Zero
    is_diagonal(::Type{L}) where {L} = base(L) <: Diagonal
    is_split(::Type{L}) where {L} = base(L) <: Union{SplitColMajor, SplitRowMajor}
    is_interleaved(::Type{L}) where {L} = base(L) <: Union{InterleavedColMajor, InterleavedRowMajor}

    physical_size(::Type{<:LayoutBase}, s::NamedTuple) = Tuple(s)
    physical_size(::Type{<:Union{SplitColMajor, SplitRowMajor}}, s::NamedTuple) = (Tuple(s)..., 2)
    function physical_size(::Type{Padded{L, P}}, s::NamedTuple) where {L, P}
        t = Tuple(s)
        col_major(L) ? (t[1] + P, Base.tail(t)...) : (t[2] + P, t[1])
    end
end

module Operator
    struct TF32 end                                                 # compute-type marker: FP32 storage, TF32 multiply
    abstract type GeneralFPUOp{M, N, K, mb, nb, kb, CT, AT} end     # src/operator.jl:35-153
    abstract type FPUOp{M, N, K, mb, nb, kb, CT, AT} <: GeneralFPUOp{M, N, K, mb, nb, kb, CT, AT} end
    abstract type TropicalFPUOp{M, N, K, mb, nb, kb, CT, AT} <: GeneralFPUOp{M, N, K, mb, nb, kb, CT, AT} end
    abstract type WMMAOp{M, N, K, CT, AT} end                       # 163-245: runs on the tcgen05 kernel
    abstract type WMMAComplexOp{M, N, K, CT, AT} end                # 251-314
    abstract type WMMADualOp{M, N, K, CT, AT} end                   # 320-372
    abstract type TCGen05Operator{CT, AT} end                       # new: tcgen05.mma, TMEM accumulators

    shape(::Type{<:GeneralFPUOp{M, N, K}}) where {M, N, K} = (M = M, N = N, K = K)
    base_shape(::Type{<:GeneralFPUOp{M, N, K, mb, nb, kb}}) where {M, N, K, mb, nb, kb} =
        (M = M, N = N, K = K, mb = mb, nb = nb, kb = kb)
    shape(::Type{<:Union{WMMAOp{M, N, K}, WMMAComplexOp{M, N, K}, WMMADualOp{M, N, K}}}) where {M, N, K} = (M = M, N = N, K = K)
    shape(::Type{<:TCGen05Operator{CT}}) where {CT} = (M = 16, N = 16, K = CT === TF32 ? 8 : 32 ÷ sizeof(CT))

    # gk_number: 0 real, 1 complex, 2 dual
    number(::Type) = Int32(0)
    number(::Type{<:WMMAComplexOp}) = Int32(1)
    number(::Type{<:WMMADualOp}) = Int32(2)
end

module Transform
    # The closed set of functors the kernels fuse (src/transform.jl:19-30 accepts any functor; a functor
    # cannot cross the C ABI).  Anything else makes `matmul` throw.
    struct Scale{T}; factor::T; end
    struct ReLU end
    struct GELU end
    struct Cast{T} end
    struct Elementwise{F}; func::F; end
    Elementwise() = Elementwise(identity)
end

module Epilogue
    using CUDA: CuPtr
    struct Default end                                              # src/epilogue.jl:14-34
    struct Bias{B}                                                  # src/epilogue.jl:40-73 (per column); axis = :row is new
        bias_pointer::B
        axis::Symbol
    end
    Bias(ptr) = Bias(ptr, :col)
end

module Kernel                                                       # tags only: one persistent TMA pipeline serves all three
    function matmul_singlestage end
    function matmul_pipelined end
    function matmul_pipelined_ng end
end

module CTASwizzle
    struct Identity end
    struct HorizontallyTiled{T} end
    struct VerticallyTiled{T} end
    struct LebesgueCurve end
    number_of_blocks(::Type, block_shape, matmul_shape) =
        (cld(matmul_shape.M, block_shape.M), cld(matmul_shape.N, block_shape.N))
end
