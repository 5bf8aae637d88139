# get_config / Config / ConfigError with the reference's keywords, defaults and rules (src/config.jl),
# plus the B200 engine's tile parameters.  Not executed in this repository's environment (no Julia);
# the executable mirror is gemmkernels_b200/config.py.

struct ConfigError <: Exception
    message::String
end
Base.showerror(io::IO, e::ConfigError) = print(io, "ConfigError: ", e.message)

Base.@kwdef struct Config
    matmul_shape; block_shape; warps_per_block
    mem_a_warp; mem_a_thread; mem_b_warp; mem_b_thread; mem_cd_warp; mem_cd_thread
    compute_warp; compute_op_shape
    global_a_layout; global_b_layout; global_c_layout; global_d_layout
    shared_a_layout; shared_b_layout; shared_c_layout; shared_d_layout
    operator
    is_a_col_major; is_b_col_major
    cta_swizzle
    # B200 engine (0 = take the built-in table)
    tile_n::Int = 0
    cta_group::Int = 0
    stages::Int = 0
    raster_group::Int = 0
end

function heuristic_block_shape(shared_a_layout, shared_b_layout, shared_c_layout, shared_d_layout)
    nbytes(l, s) = prod(Layout.physical_size(l, s)) * sizeof(Layout.eltype(l))
    fits_cd(M, N, K) = max(nbytes(shared_c_layout, (M = M, N = N)), nbytes(shared_d_layout, (M = M, N = N))) <= 64 * 1024
    fits_ab(M, N, K) = nbytes(shared_a_layout, (M = M, K = K)) + nbytes(shared_b_layout, (K = K, N = N)) <= 64 * 1024
    next_MN(M, N, K) = M == N ? (2M, N, K) : (M, 2N, K)
    cur = (1, 1, 1); nxt = next_MN(cur...)
    while fits_cd(nxt...); cur = nxt; nxt = next_MN(cur...); end
    nxt = (cur[1], cur[2], 2cur[3])
    while fits_ab(nxt...); cur = nxt; nxt = (cur[1], cur[2], 2cur[3]); end
    (M = cur[1], N = cur[2], K = cur[3])
end

function adjacent_elements(num, parent_size, is_col_major)
    p = Tuple(parent_size)
    t = is_col_major ? (min(num, p[1]), num ÷ min(num, p[1])) : (num ÷ min(num, p[2]), min(num, p[2]))
    typeof(parent_size)(t)
end

check_operator_config(::Type) = nothing
function check_operator_config(op::Type{<:Operator.GeneralFPUOp})
    s = Operator.base_shape(op)
    s.M * s.N < 32 && throw(ConfigError("The operator shape is too small. The dimensions of the operator shape must adhere to the following constraint: OPERATOR_M * OPERATOR_N ≥ 32."))
    s.mb * s.nb != 32 && throw(ConfigError("The base FPU operator shape should adhere to the following constraint: OPERATOR_M_BASE * OPERATOR_N_BASE = 32."))
    s.kb != 1 && throw(ConfigError("The base FPU operator shape should adhere to the following constraint: OPERATOR_K_BASE = 1."))
    any((s.M, s.N, s.K) .% (s.mb, s.nb, s.kb) .!= 0) && throw(ConfigError("The operator shape should adhere to the following constraint: OPERATOR_M, OPERATOR_N, OPERATOR_K are multiples of OPERATOR_M_BASE, OPERATOR_N_BASE, OPERATOR_K_BASE, respectively."))
end
function check_operator_config(op::Type{<:Union{Operator.WMMAOp, Operator.WMMAComplexOp, Operator.WMMADualOp}})
    s = Operator.shape(op)
    s in [(M = 16, N = 16, K = 16), (M = 8, N = 32, K = 16), (M = 32, N = 8, K = 16)] ||
        throw(ConfigError("Unsupported WMMA Operator shape $(s)!"))
end

require_tile_sized_global(l) = !(Layout.base(l) <: Union{Layout.Zero, Layout.ColMajor, Layout.RowMajor})

function get_config(; gemm_shape, operator, global_a_layout, global_c_layout, kwargs...)
    params = Dict(kwargs)
    global_b_layout = get(params, :global_b_layout, global_a_layout)
    global_d_layout = get(params, :global_d_layout, global_c_layout)
    shared_a_layout = get(params, :shared_a_layout, Layout.Padded{global_a_layout, 16 ÷ sizeof(Layout.eltype(global_a_layout))})
    shared_b_layout = get(params, :shared_b_layout, Layout.Padded{global_b_layout, 16 ÷ sizeof(Layout.eltype(global_b_layout))})
    shared_c_layout = get(params, :shared_c_layout, global_c_layout)
    shared_d_layout = get(params, :shared_d_layout, global_d_layout)
    block_shape = get(params, :block_shape, heuristic_block_shape(shared_a_layout, shared_b_layout, shared_c_layout, shared_d_layout))
    (block_shape.M * block_shape.K < 128 || block_shape.K * block_shape.N < 128 || block_shape.K < 8) &&
        throw(ConfigError("The block shape is too small. The dimensions of the block shape must adhere to the following constraints: BLOCK_M * BLOCK_K ≥ 128, BLOCK_K * BLOCK_N ≥ 128, BLOCK_K ≥ 8."))
    op_shape = Operator.shape(operator)
    (block_shape.M < 2 * op_shape.M || block_shape.N < 2 * op_shape.N || block_shape.K < op_shape.K) &&
        throw(ConfigError("There is a mismatch between the block shape and the operator shape. Their dimensions must adhere to the following constraints: BLOCK_M ≥ 2 * OPERATOR_M, BLOCK_N ≥ 2 * OPERATOR_N, BLOCK_K ≥ OPERATOR_K."))
    check_operator_config(operator)

    warps_default = 8
    compute_warp_default = (M = block_shape.M ÷ 4, N = block_shape.N ÷ 2, K = op_shape.K)
    if (block_shape.M ÷ op_shape.M) < 4 || (block_shape.N ÷ op_shape.N) < 2
        compute_warp_default = (M = max(op_shape.M, block_shape.M ÷ 4), N = max(op_shape.N, block_shape.N ÷ 2), K = op_shape.K)
        warps_default = min(block_shape.M ÷ op_shape.M, 4) * min(block_shape.N ÷ op_shape.N, 2)
    end
    warps_per_block = get(params, :warps_per_block, warps_default)
    compute_warp = get(params, :compute_warp, compute_warp_default)
    is_a_col_major = get(params, :is_a_col_major, true)
    is_b_col_major = get(params, :is_b_col_major, true)
    is_cd_col_major = get(params, :is_cd_col_major, true)

    na = min(16 ÷ sizeof(Layout.eltype(global_a_layout)), (block_shape.M * block_shape.K) ÷ (32 * warps_per_block))
    nb = min(16 ÷ sizeof(Layout.eltype(global_b_layout)), (block_shape.K * block_shape.N) ÷ (32 * warps_per_block))
    nc = min(16 ÷ sizeof(Layout.eltype(global_c_layout)), (block_shape.M * block_shape.N) ÷ (32 * warps_per_block))
    mem_a_warp = get(params, :mem_a_warp, adjacent_elements(32 * na, (M = block_shape.M, K = block_shape.K), is_a_col_major))
    mem_b_warp = get(params, :mem_b_warp, adjacent_elements(32 * nb, (K = block_shape.K, N = block_shape.N), is_b_col_major))
    mem_cd_warp = get(params, :mem_cd_warp, adjacent_elements(32 * nc, (M = block_shape.M, N = block_shape.N), is_cd_col_major))
    mem_a_thread = get(params, :mem_a_thread, adjacent_elements(na, (M = block_shape.M, K = block_shape.K), is_a_col_major))
    mem_b_thread = get(params, :mem_b_thread, adjacent_elements(nb, (K = block_shape.K, N = block_shape.N), is_b_col_major))
    mem_cd_thread = get(params, :mem_cd_thread, adjacent_elements(nc, (M = block_shape.M, N = block_shape.N), is_cd_col_major))

    prod(mem_a_warp) * warps_per_block ≤ block_shape.M * block_shape.K || throw(ConfigError("mem_a_warp is too big for the selected block shape: need at least one iteration in the memory copy loop!"))
    prod(mem_b_warp) * warps_per_block ≤ block_shape.K * block_shape.N || throw(ConfigError("mem_b_warp is too big for the selected block shape: need at least one iteration in the memory copy loop!"))
    prod(mem_cd_warp) * warps_per_block ≤ block_shape.M * block_shape.N || throw(ConfigError("mem_cd_warp is too big for the selected block shape: need at least one iteration in the memory copy loop!"))

    check(num, den, dims, msg) = all(num[d] % den[d] == 0 for d in dims) || throw(ConfigError(msg))
    check(block_shape, compute_warp, [:M, :N, :K], "block_shape must be a multiple of compute_warp!")
    check(compute_warp, op_shape, [:M, :N, :K], "compute_warp must be a multiple of op_shape!")
    require_tile_sized_global(global_a_layout) && check(gemm_shape, block_shape, [:M, :K], "gemm_shape.MK must be a multiple of block_shape.MK!")
    require_tile_sized_global(global_b_layout) && check(gemm_shape, block_shape, [:K, :N], "gemm_shape.KN must be a multiple of block_shape.KN!")
    require_tile_sized_global(global_c_layout) && check(gemm_shape, block_shape, [:M, :N], "gemm_shape.MN must be a multiple of block_shape.MN!")
    require_tile_sized_global(global_d_layout) && check(gemm_shape, block_shape, [:M, :N], "gemm_shape.MN must be a multiple of block_shape.MN!")

    Config(; matmul_shape = gemm_shape, block_shape, warps_per_block,
           mem_a_warp, mem_a_thread, mem_b_warp, mem_b_thread, mem_cd_warp, mem_cd_thread,
           compute_warp, compute_op_shape = op_shape,
           global_a_layout, global_b_layout, global_c_layout, global_d_layout,
           shared_a_layout, shared_b_layout, shared_c_layout, shared_d_layout,
           operator, is_a_col_major, is_b_col_major,
           cta_swizzle = get(params, :cta_swizzle, CTASwizzle.Identity),
           tile_n = get(params, :tile_n, 0), cta_group = get(params, :cta_group, 0),
           stages = get(params, :stages, 0), raster_group = get(params, :raster_group, 0))
end
