# BLAS-like front end (src/matmul.jl:47-215) and the contraction entry point.
# Not executed in this repository's environment (no Julia).

const configs = Dict{Any, Any}()
const configs_lock = ReentrantLock()
function get_config_cached(args...)
    lock(configs_lock) do
        get!(() -> create_config(args...), configs, args)
    end
end

const tensor_types = [(Float16, Float16, Float16), (Float16, Float16, Float32),
                      (Core.BFloat16, Core.BFloat16, Core.BFloat16), (Core.BFloat16, Core.BFloat16, Float32)]

function create_config(A::Type, sizeA::Dims, stridesA::Dims, transA::Bool,
                       B::Type, sizeB::Dims, stridesB::Dims, transB::Bool,
                       C::Type, sizeC::Dims, stridesC::Dims,
                       alpha::Type, zeroAlpha::Bool, beta::Type, zeroBeta::Bool, wmma::Union{Bool, Nothing})
    m = sizeA[transA ? 2 : 1]; k = sizeA[transA ? 1 : 2]; n = sizeB[transB ? 1 : 2]
    if m != sizeC[1] || n != sizeC[2] || k != sizeB[transB ? 2 : 1]
        throw(DimensionMismatch("Dimensions do not match"))
    end
    a_base = transA ? Layout.RowMajor : Layout.ColMajor
    b_base = transB ? Layout.RowMajor : Layout.ColMajor
    a_al = transA ? Layout.UnsafeAlignedRowMajor : Layout.UnsafeAlignedColMajor
    b_al = transB ? Layout.UnsafeAlignedRowMajor : Layout.UnsafeAlignedColMajor
    compute_type = promote_type(eltype(A), eltype(B))
    use_tensor = something(wmma, (compute_type, compute_type, eltype(C)) in tensor_types)
    shared_a_layout = Layout.Padded{a_al{use_tensor ? compute_type : eltype(A)}, 8}
    shared_b_layout = Layout.Padded{b_al{use_tensor ? compute_type : eltype(B)}, 8}
    shared_c_layout = zeroBeta ? Layout.Zero{eltype(C)} : Layout.UnsafeAlignedColMajor{eltype(C)}
    shared_d_layout = Layout.UnsafeAlignedColMajor{eltype(C)}
    block_shape = use_tensor ? heuristic_block_shape(shared_a_layout, shared_b_layout, shared_c_layout, shared_d_layout) :
                               (M = 128, N = 128, K = 32)
    a_aligned = (stridesA[2] * sizeof(eltype(A))) % 16 == 0
    b_aligned = (stridesB[2] * sizeof(eltype(B))) % 16 == 0
    c_aligned = (stridesC[2] * sizeof(eltype(C))) % 16 == 0
    if zeroAlpha
        global_a_layout = Layout.Zero{eltype(A)}; global_b_layout = Layout.Zero{eltype(B)}
    else
        global_a_layout = (a_aligned && m % block_shape.M == 0 && k % block_shape.K == 0) ? a_al{eltype(A)} : a_base{eltype(A)}
        global_b_layout = (b_aligned && k % block_shape.K == 0 && n % block_shape.N == 0) ? b_al{eltype(B)} : b_base{eltype(B)}
    end
    cd_ok = c_aligned && m % block_shape.M == 0 && n % block_shape.N == 0
    global_c_layout = zeroBeta ? Layout.Zero{eltype(C)} : (cd_ok ? Layout.UnsafeAlignedColMajor{eltype(C)} : Layout.ColMajor{eltype(C)})
    global_d_layout = cd_ok ? Layout.UnsafeAlignedColMajor{eltype(C)} : Layout.ColMajor{eltype(C)}
    operator = use_tensor ?
        Operator.TCGen05Operator{compute_type === Float32 ? Operator.TF32 : compute_type, eltype(C)} :
        Operator.FPUOp{8, 8, 1, 4, 8, 1, compute_type, eltype(C)}
    conf = get_config(; gemm_shape = (M = m, N = n, K = k), block_shape, operator,
                      global_a_layout, global_b_layout, global_c_layout, global_d_layout,
                      shared_a_layout, shared_b_layout, shared_c_layout, shared_d_layout,
                      is_a_col_major = !transA, is_b_col_major = !transB)
    aligned(l) = Layout.base(l) <: Union{Layout.UnsafeAlignedColMajor, Layout.UnsafeAlignedRowMajor}
    kern = (aligned(global_a_layout) && aligned(global_b_layout)) ? Kernel.matmul_pipelined : Kernel.matmul_singlestage
    return conf, compute_type, kern
end

function matmatmul!(C::CuArray, transA::Char, transB::Char, A::CuArray, B::CuArray, alpha::Number, beta::Number;
                    wmma::Union{Bool, Nothing} = nothing)
    conf, compute_type, kernel = get_config_cached(
        typeof(A), size(A), strides(A), transA == 'T', typeof(B), size(B), strides(B), transB == 'T',
        typeof(C), size(C), strides(C), typeof(alpha), iszero(alpha), typeof(beta), iszero(beta), wmma)
    # named functors instead of closures: a closure cannot cross the C ABI
    matmul(conf, A, B, C, C;
           transform_shared_to_regs_a = Transform.Elementwise(Transform.Scale(alpha)),
           transform_shared_to_regs_c = Transform.Elementwise(Transform.Scale(beta)),
           kernel)
    C
end

function mul!(C::CuArray,
              A::Union{CuArray, Adjoint{<:Any, <:CuArray}, Transpose{<:Any, <:CuArray}},
              B::Union{CuArray, Adjoint{<:Any, <:CuArray}, Transpose{<:Any, <:CuArray}},
              alpha = true, beta = false)
    transA = A isa Adjoint || A isa Transpose
    transB = B isa Adjoint || B isa Transpose
    matmatmul!(C, transA ? 'T' : 'N', transB ? 'T' : 'N', parent(A), parent(B), alpha, beta)
end

# ---- tensor contraction: D[modes_d] = alpha * sum A[modes_a] * B[modes_b] + beta * C -----------------
struct GkContractDesc
    struct_size::UInt32; rank_a::Int32; rank_b::Int32; rank_c::Int32
    modes_a::NTuple{8, Int32}; modes_b::NTuple{8, Int32}; modes_c::NTuple{8, Int32}
    extents_a::NTuple{8, Int64}; extents_b::NTuple{8, Int64}; extents_c::NTuple{8, Int64}
    strides_a::NTuple{8, Int64}; strides_b::NTuple{8, Int64}; strides_c::NTuple{8, Int64}; strides_d::NTuple{8, Int64}
    dtype_a::Int32; dtype_b::Int32; dtype_c::Int32; dtype_d::Int32
    compute::Int32; force_gather::Int32
    alpha::Float64; beta::Float64
    tile_n::Int32; cta_group::Int32; stages::Int32; debug::Int32; reserved::NTuple{2, Int32}
end

pad8(xs, T) = ntuple(i -> i <= length(xs) ? T(xs[i]) : zero(T), 8)

function contract!(D::CuArray, modes_d::AbstractString, A::CuArray, modes_a::AbstractString,
                   B::CuArray, modes_b::AbstractString; alpha = true, beta = false, C::CuArray = D, workspace = nothing)
    desc = GkContractDesc(sizeof(GkContractDesc), ndims(A), ndims(B), ndims(D),
                          pad8(Int32.(collect(modes_a)), Int32), pad8(Int32.(collect(modes_b)), Int32), pad8(Int32.(collect(modes_d)), Int32),
                          pad8(size(A), Int64), pad8(size(B), Int64), pad8(size(D), Int64),
                          pad8(strides(A), Int64), pad8(strides(B), Int64), pad8(strides(C), Int64), pad8(strides(D), Int64),
                          gk_dtype(eltype(A)), gk_dtype(eltype(B)), gk_dtype(eltype(C)), gk_dtype(eltype(D)),
                          gk_dtype(eltype(A) === Float32 ? Float32 : eltype(A)), 0, alpha, beta, 0, 0, 0, 0, (0, 0))
    if workspace === nothing
        plan = Ref{GkGemmPlan}()
        gk_check(ccall((:gk_contract_query, libgk), Cint, (Ptr{Cvoid}, Ref{GkContractDesc}, Ref{GkGemmPlan}), gk_handle(), desc, plan))
        plan[].workspace_bytes > 0 && (workspace = lent_workspace(plan[].workspace_bytes))
    end
    ws = workspace === nothing ? CU_NULL : reinterpret(CuPtr{Cvoid}, pointer(workspace))
    gk_check(ccall((:gk_contract, libgk), Cint,
                   (Ptr{Cvoid}, Ref{GkContractDesc}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, Int64, Ptr{Cvoid}),
                   gk_handle(), desc, pointer(A), pointer(B), pointer(C), pointer(D), ws,
                   workspace === nothing ? 0 : sizeof(workspace), CUDA.stream().handle))
    D
end


# ---- column-sharded GEMM over the GPUs of one box: one Julia process (or task) per GPU ---------------------
# The 128-byte id made on one rank reaches the others by any transport (Distributed.jl, MPI.jl, a file).
mgpu_unique_id() = (id = Vector{UInt8}(undef, 128); gk_check(ccall((:gk_mgpu_unique_id, libgk), Cint, (Ptr{UInt8},), id)); id)
mgpu_init(rank::Integer, world::Integer, id::Vector{UInt8}) =
    gk_check(ccall((:gk_mgpu_init, libgk), Cint, (Ptr{Cvoid}, Int32, Int32, Ptr{UInt8}), gk_handle(), rank, world, id))
mgpu_destroy() = gk_check(ccall((:gk_mgpu_destroy, libgk), Cint, (Ptr{Cvoid},), gk_handle()))

"""
    matmul_colshard(conf, a, b_block, c_block, d_block; a_mode = :resident, root = 0, k_panels = 0, ...)

This rank's column block of D = A * B (`conf` describes the block).  `a_mode = :broadcast` sends A from
rank `root` into every rank's `a` in panels that overlap the product (collective).
"""
function matmul_colshard(desc::GkGemmDesc, epi::GkEpilogueDesc, a, b, c, d; a_mode = :resident, root = 0, k_panels = 0)
    gk_check(ccall((:gk_mgpu_gemm_colshard, libgk), Cint,
                   (Ptr{Cvoid}, Ref{GkGemmDesc}, CuPtr{Cvoid}, Int32, Int32, Int32, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid},
                    Ref{GkEpilogueDesc}, CuPtr{Cvoid}, Int64, Ptr{Cvoid}),
                   gk_handle(), desc, pointer(a), a_mode === :broadcast ? 1 : 0, root, k_panels, pointer(b),
                   c === nothing ? CU_NULL : pointer(c), pointer(d), epi, CU_NULL, 0, CUDA.stream().handle))
end
