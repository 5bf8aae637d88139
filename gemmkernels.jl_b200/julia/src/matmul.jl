# matmul / matmatmul! / mul! / contract! over the C ABI (replacement for src/matmul.jl).
# Not executed in this repository's environment (no Julia); the executable mirror is
# gemmkernels_b200/matmul.py and contract.py, which lower to the same descriptors.

using CUDA
using LinearAlgebra: Adjoint, Transpose

const libgk = get(ENV, "GEMMKERNELS_B200_LIB", "libgemmkernels_b200")

# include/gemmkernels_b200.h, field for field
struct GkGemmDesc
    struct_size::UInt32; number::Int32
    m::Int64; n::Int64; k::Int64
    trans_a::Int32; trans_b::Int32
    dtype_a::Int32; dtype_b::Int32; dtype_c::Int32; dtype_d::Int32
    compute::Int32; op::Int32
    lda::Int64; ldb::Int64; ldc::Int64; ldd::Int64
    plane_a::Int64; plane_b::Int64; plane_c::Int64; plane_d::Int64
    layout_a::Int32; layout_b::Int32; layout_c::Int32; raster::Int32
    alpha::Float64; beta::Float64
    tile_n::Int32; cta_group::Int32; stages::Int32; raster_group::Int32; max_ctas::Int32
    debug::Int32; host_chunk_mib::Int32; a_resident::Int32
    batch::Int32; k_blocks_per_stage::Int32
    batch_stride_a::Int64; batch_stride_b::Int64; batch_stride_c::Int64; batch_stride_d::Int64
end
struct GkEpilogueDesc
    struct_size::UInt32; bias_axis::Int32
    bias::CuPtr{Float32}
    activation::Int32; reserved::NTuple{3, Int32}
end
struct GkGemmPlan
    kernel::Int32; grid::Int32; block::Int32; cluster::Int32
    smem_bytes::Int32; tmem_columns::Int32
    tile_m::Int32; tile_n::Int32; tile_k::Int32; stages::Int32
    workspace_bytes::Int64
end

gk_error() = unsafe_string(ccall((:gk_last_error_message, libgk), Cstring, ()))
function gk_check(st)
    st == 0 && return
    msg = gk_error()
    st == 1 && throw(ConfigError(msg))
    st == 3 && throw(DimensionMismatch(msg))
    error("gemmkernels_b200 status $st: $msg")
end

const gk_handles = Dict{CuDevice, Ptr{Cvoid}}()
const gk_handles_lock = ReentrantLock()
function gk_handle()
    lock(gk_handles_lock) do
        get!(gk_handles, device()) do
            h = Ref{Ptr{Cvoid}}(C_NULL)
            gk_check(ccall((:gk_create, libgk), Cint, (Ptr{Ptr{Cvoid}},), h))
            h[]
        end
    end
end

gk_dtype(::Type{Float16}) = Int32(0); gk_dtype(::Type{Core.BFloat16}) = Int32(1)
gk_dtype(::Type{Float32}) = Int32(2); gk_dtype(::Type{Float64}) = Int32(3)
gk_dtype(::Type{Int16}) = Int32(4); gk_dtype(::Type{Int32}) = Int32(5); gk_dtype(::Type{Int64}) = Int32(6)
gk_dtype(::Type{Complex{T}}) where {T} = gk_dtype(T)
gk_dtype(::Type{Operator.TF32}) = Int32(7)

# operator -> (gk_operator, compute type)
op_kind(::Type{<:Operator.TCGen05Operator{CT}}) where {CT} = (Int32(1), gk_dtype(CT === Float32 ? Operator.TF32 : CT))
op_kind(::Type{<:Union{Operator.WMMAOp{M, N, K, CT}, Operator.WMMAComplexOp{M, N, K, CT},
                        Operator.WMMADualOp{M, N, K, CT}}}) where {M, N, K, CT} = (Int32(1), gk_dtype(CT))
op_kind(::Type{<:Operator.TropicalFPUOp{M, N, K, mb, nb, kb, CT, AT}}) where {M, N, K, mb, nb, kb, CT, AT} = (Int32(3), gk_dtype(AT))
op_kind(::Type{<:Operator.FPUOp{M, N, K, mb, nb, kb, CT, AT}}) where {M, N, K, mb, nb, kb, CT, AT} = (Int32(2), gk_dtype(AT))

layout_kind(l) = Layout.is_zero(l) ? Int32(1) : Layout.is_diagonal(l) ? Int32(2) : Int32(0)
raster(::Type{CTASwizzle.HorizontallyTiled{T}}) where {T} = (Int32(2), Int32(T))
raster(::Type{CTASwizzle.VerticallyTiled{T}}) where {T} = (Int32(3), Int32(T))
raster(::Type{CTASwizzle.LebesgueCurve}) = (Int32(4), Int32(0))
raster(::Type) = (Int32(0), Int32(0))     # Identity: the persistent scheduler keeps its own band raster

# Folding of the eight hooks (src/matmul.jl:8-15) into alpha, beta and an activation.  Net math of the
# reference: D = g_d( r_d( sum s_a(g_a(A)) s_b(g_b(B)) + s_c(g_c(C)) ) + bias ).
unwrap(t::Transform.Elementwise) = t.func
function fold_transforms(ga, gb, gc, gd, sa, sb, sc, rd, has_bias)
    alpha = 1.0; beta = 1.0; act = Int32(0)
    for f in unwrap.((ga, sa, gb, sb))
        f isa Transform.Scale ? (alpha *= f.factor) :
        (f === identity || f isa Transform.Cast) ? nothing :
        throw(ArgumentError("transform $f on A/B: only identity, Cast and Scale are fused (no CPU fallback)"))
    end
    for f in unwrap.((gc, sc))
        f isa Transform.Scale ? (beta *= f.factor) :
        (f === identity || f isa Transform.Cast) ? nothing : throw(ArgumentError("transform $f on C is not fused"))
    end
    f = unwrap(rd)
    if f isa Transform.Scale
        alpha *= f.factor; beta *= f.factor
    elseif f isa Union{Transform.ReLU, Transform.GELU}
        has_bias && throw(ArgumentError("an activation in regs_to_shared_d runs before the bias; use shared_to_global_d"))
        act = f isa Transform.ReLU ? Int32(1) : Int32(2)
    elseif !(f === identity || f isa Transform.Cast)
        throw(ArgumentError("transform_regs_to_shared_d = $f is not fused"))
    end
    f = unwrap(gd)
    if f isa Transform.Scale
        (has_bias || act != 0) && throw(ArgumentError("Scale after a bias or activation is not fused"))
        alpha *= f.factor; beta *= f.factor
    elseif f isa Union{Transform.ReLU, Transform.GELU}
        act != 0 && throw(ArgumentError("two activations requested"))
        act = f isa Transform.ReLU ? Int32(1) : Int32(2)
    elseif !(f === identity || f isa Transform.Cast)
        throw(ArgumentError("transform_shared_to_global_d = $f is not fused"))
    end
    alpha, beta, act
end

ld(x, l) = Layout.is_zero(l) ? Int64(1) : Int64(max(stride(x, 2), size(x, 1), 1))
plane(x, l) = Layout.is_split(l) ? Int64(stride(x, 3)) : Int64(0)    # 0 = interleaved pairs / real
devptr(x, l) = Layout.is_zero(l) ? CU_NULL : reinterpret(CuPtr{Cvoid}, pointer(x))

function matmul(conf::Config, a, b, c, d;
                transform_global_to_shared_a = Transform.Elementwise(), transform_global_to_shared_b = Transform.Elementwise(),
                transform_global_to_shared_c = Transform.Elementwise(), transform_shared_to_global_d = Transform.Elementwise(),
                transform_shared_to_regs_a = Transform.Elementwise(), transform_shared_to_regs_b = Transform.Elementwise(),
                transform_shared_to_regs_c = Transform.Elementwise(), transform_regs_to_shared_d = Transform.Elementwise(),
                epilogue = Epilogue.Default(), kernel = Kernel.matmul_singlestage, workspace = nothing)
    kernel === Kernel.matmul_pipelined && conf.block_shape.K < 2 * conf.compute_op_shape.K &&
        throw(ConfigError("Need at least two stages to use a pipelined kernel, i.e. BLOCK_K ≥ 2 * OPERATOR_K"))
    has_bias = epilogue isa Epilogue.Bias
    alpha, beta, act = fold_transforms(transform_global_to_shared_a, transform_global_to_shared_b,
                                       transform_global_to_shared_c, transform_shared_to_global_d,
                                       transform_shared_to_regs_a, transform_shared_to_regs_b,
                                       transform_shared_to_regs_c, transform_regs_to_shared_d, has_bias)
    la, lb, lc, ldl = conf.global_a_layout, conf.global_b_layout, conf.global_c_layout, conf.global_d_layout
    op, compute = op_kind(conf.operator)
    rk, rg = raster(conf.cta_swizzle)
    Layout.is_zero(lc) && (beta = 0.0)
    desc = GkGemmDesc(sizeof(GkGemmDesc), Operator.number(conf.operator),
                      conf.matmul_shape.M, conf.matmul_shape.N, conf.matmul_shape.K,
                      !Layout.col_major(la), !Layout.col_major(lb),
                      gk_dtype(Layout.eltype(la)), gk_dtype(Layout.eltype(lb)), gk_dtype(Layout.eltype(lc)), gk_dtype(Layout.eltype(ldl)),
                      compute, op, ld(a, la), ld(b, lb), ld(c, lc), ld(d, ldl),
                      plane(a, la), plane(b, lb), plane(c, lc), plane(d, ldl),
                      layout_kind(la), layout_kind(lb), layout_kind(lc), rk, alpha, beta,
                      conf.tile_n, conf.cta_group, conf.stages, rg == 0 ? conf.raster_group : rg, 0,
                      0, 0, 0, 0, 0, 0, 0, 0, 0)
    epi = GkEpilogueDesc(sizeof(GkEpilogueDesc), has_bias ? (epilogue.axis === :row ? 1 : 2) : 0,
                         has_bias ? reinterpret(CuPtr{Float32}, epilogue.bias_pointer) : CuPtr{Float32}(0), act, (0, 0, 0))
    # Interleaved complex / dual operands need a workspace (they are split into planes first); real products
    # with few output tiles and a long K can use one (split-K).  gk_gemm_query reports the size.
    # The FFMA kernel cuts the tiles of a partly filled last round, or of a grid too small for the GPU, along K.
    ffma = desc.op == 2 && desc.dtype_d == 2
    wants = Operator.number(conf.operator) != 0 ? (desc.plane_a == 0 || desc.plane_b == 0) :
            ffma ? (desc.m * desc.n <= 148 * 128 * 128 ? desc.k >= 256 : (desc.m * desc.n >= 1 << 22 && desc.k >= 1024)) :
            (desc.m * desc.n <= 1 << 22 && desc.k >= 2048)
    if workspace === nothing && wants
        plan = Ref(GkGemmPlan(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0))
        gk_check(ccall((:gk_gemm_query, libgk), Cint, (Ptr{Cvoid}, Ref{GkGemmDesc}, Ref{GkEpilogueDesc}, Ref{GkGemmPlan}),
                       gk_handle(), desc, epi, plan))
        plan[].workspace_bytes > 0 && (workspace = lent_workspace(plan[].workspace_bytes))
    end
    ws = workspace === nothing ? CU_NULL : reinterpret(CuPtr{Cvoid}, pointer(workspace))
    gk_check(ccall((:gk_gemm, libgk), Cint,
                   (Ptr{Cvoid}, Ref{GkGemmDesc}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid}, CuPtr{Cvoid},
                    Ref{GkEpilogueDesc}, CuPtr{Cvoid}, Int64, Ptr{Cvoid}),
                   gk_handle(), desc, devptr(a, la), devptr(b, lb), devptr(c, lc), devptr(d, ldl), epi, ws,
                   workspace === nothing ? 0 : sizeof(workspace), CUDA.stream().handle))
    return
end

# Scratch the package lends to the library when the caller passes none: one buffer per (device, stream),
# allocated on first need and replaced only by a larger one, so the hot path does not allocate.
const gk_workspaces = Dict{Tuple{CuDevice, CuStream}, CuVector{UInt8}}()
function lent_workspace(bytes::Integer)
    lock(gk_handles_lock) do
        key = (device(), CUDA.stream())
        ws = get(gk_workspaces, key, nothing)
        if ws === nothing || length(ws) < bytes
            ws = CuVector{UInt8}(undef, max(bytes, ws === nothing ? 0 : 2 * length(ws)))
            gk_workspaces[key] = ws
        end
        ws
    end
end
