"""CPU tests of the host-side mirror of the GemmKernels.jl API: get_config defaults and validity
rules (src/config.jl), create_config's layout/operator choice (src/matmul.jl:66-183), and the
lowering of transforms / epilogues / layouts to the C-ABI descriptor.  No kernel runs here."""
import numpy as np
import pytest
import torch

import gemmkernels_b200 as GK
from gemmkernels_b200 import _lib as L
from gemmkernels_b200 import Epilogue, Kernel, Layout, Operator, Transform, CTASwizzle


def wmma_config(**kw):
    base = dict(gemm_shape=(256, 256, 256), operator=Operator.WMMAOp[16, 16, 16, GK.Float16, GK.Float32],
                global_a_layout=Layout.UnsafeAlignedColMajor[GK.Float16],
                global_c_layout=Layout.UnsafeAlignedColMajor[GK.Float32])
    base.update(kw)
    return GK.get_config(**base)


def test_default_config_matches_reference_heuristics():
    # src/config.jl:84-120, 216-260: (128,128,64) for F16 in / F32 out, 8 warps as 4 x 2,
    # compute_warp = (BM/4, BN/2, OP_K), 16-byte thread tiles, Identity swizzle.
    c = wmma_config()
    assert c.block_shape == {"M": 128, "N": 128, "K": 64}
    assert c.warps_per_block == 8
    assert c.compute_warp == {"M": 32, "N": 64, "K": 16}
    assert c.compute_op_shape == {"M": 16, "N": 16, "K": 16}
    assert c.mem_a_thread == {"M": 8, "K": 1} and c.mem_cd_thread == {"M": 4, "N": 1}
    assert c.mem_a_warp == {"M": 128, "K": 2}
    assert repr(c.shared_a_layout) == "Layout.Padded{Layout.UnsafeAlignedColMajor{Float16}, 8}"
    assert c.global_b_layout == c.global_a_layout and c.global_d_layout == c.global_c_layout
    assert isinstance(c.cta_swizzle, CTASwizzle.Identity)
    assert "matmul_shape" in str(c)


def test_tcgen05_operator_gets_the_same_defaults():
    c = wmma_config(operator=Operator.TCGen05Operator[GK.Float16, GK.Float32])
    assert c.block_shape == {"M": 128, "N": 128, "K": 64} and c.warps_per_block == 8


@pytest.mark.parametrize("kw,fragment", [
    (dict(block_shape=(8, 8, 8)), "block shape is too small"),
    (dict(block_shape=(128, 128, 4)), "block shape is too small"),
    (dict(block_shape=(16, 128, 64)), "mismatch between the block shape and the operator shape"),
    (dict(operator=Operator.WMMAOp[16, 16, 8, GK.Float16, GK.Float32]), "Unsupported WMMA Operator shape"),
    (dict(gemm_shape=(200, 256, 256)), "gemm_shape.MK must be a multiple"),
    (dict(compute_warp=(48, 64, 16)), "block_shape must be a multiple of compute_warp"),
    (dict(warps_per_block=64, block_shape=(32, 32, 16)), "need at least one iteration"),
    (dict(cta_group=3), "cta_group"),
    (dict(tile_n=100), "tile_n"),
])
def test_config_errors(kw, fragment):
    with pytest.raises(GK.ConfigError) as e:
        wmma_config(**kw)
    assert fragment in str(e.value)


@pytest.mark.parametrize("shape,fragment", [
    ((4, 4, 1, 4, 8, 1), "OPERATOR_M * OPERATOR_N"),
    ((8, 8, 1, 4, 4, 1), "OPERATOR_M_BASE * OPERATOR_N_BASE = 32"),
    ((8, 8, 2, 4, 8, 2), "OPERATOR_K_BASE = 1"),
    ((6, 8, 1, 4, 8, 1), "multiples of"),
])
def test_fpu_operator_rules(shape, fragment):
    with pytest.raises(GK.ConfigError) as e:
        GK.get_config(gemm_shape=(128, 128, 128), operator=Operator.FPUOp[(*shape, GK.Float32, GK.Float32)],
                      global_a_layout=Layout.ColMajor[GK.Float32], global_c_layout=Layout.ColMajor[GK.Float32],
                      block_shape=(64, 64, 32))
    assert fragment in str(e.value)


def test_unaligned_layouts_skip_tile_multiple_rule():
    c = GK.get_config(gemm_shape=(10, 1000, 10), operator=Operator.FPUOp[8, 8, 1, 4, 8, 1, GK.Float32, GK.Float32],
                      global_a_layout=Layout.ColMajor[GK.Float32], global_c_layout=Layout.ColMajor[GK.Float32],
                      block_shape=(128, 128, 32))
    assert c.matmul_shape == {"M": 10, "N": 1000, "K": 10}


def test_create_config_picks_operator_layouts_and_kernel():
    F16, F32 = GK.Float16, GK.Float32
    conf, ct, kern = GK.create_config(F16, (2048, 2048), (1, 2048), False, F16, (2048, 2048), (1, 2048), False,
                                      F32, (2048, 2048), (1, 2048), False, True, None)
    assert isinstance(conf.operator, Operator.TCGen05Operator) and ct == F16
    assert conf.global_a_layout == Layout.UnsafeAlignedColMajor[F16]
    assert conf.global_c_layout == Layout.Zero[F32] and conf.shared_c_layout == Layout.Zero[F32]
    assert kern is Kernel.matmul_pipelined
    # unaligned / non-multiple sizes fall back to bounds-checked layouts and the single-stage tag
    conf, _, kern = GK.create_config(F16, (10, 1000), (1, 10), False, F16, (1000, 10), (1, 1000), False,
                                     F32, (10, 10), (1, 10), False, False, True)
    assert conf.global_a_layout == Layout.ColMajor[F16] and conf.global_c_layout == Layout.ColMajor[F32]
    assert kern is Kernel.matmul_singlestage
    # Float32 goes to the FPU operator unless wmma is forced
    conf, _, _ = GK.create_config(F32, (256, 128), (1, 256), True, F32, (256, 512), (1, 256), False,
                                  F32, (128, 512), (1, 128), False, False, None)
    assert isinstance(conf.operator, Operator.FPUOp) and conf.block_shape == {"M": 128, "N": 128, "K": 32}
    assert conf.global_a_layout == Layout.UnsafeAlignedRowMajor[F32] and not conf.is_a_col_major
    # alpha == 0: A and B are not read
    conf, _, _ = GK.create_config(F16, (128, 64), (1, 128), False, F16, (64, 128), (1, 64), False,
                                  F32, (128, 128), (1, 128), True, False, None)
    assert conf.global_a_layout == Layout.Zero[F16] and conf.global_b_layout == Layout.Zero[F16]


def test_dimension_mismatch():
    F16, F32 = GK.Float16, GK.Float32
    with pytest.raises(GK.DimensionMismatch):
        GK.create_config(F16, (128, 64), (1, 128), False, F16, (32, 128), (1, 32), False,
                         F32, (128, 128), (1, 128), False, False, None)


def colmajor(rows, cols, dtype):
    return torch.zeros(cols, rows, dtype=dtype).T


def test_lowering_of_transforms_and_bias():
    conf = wmma_config(gemm_shape=(128, 256, 64), global_a_layout=Layout.UnsafeAlignedRowMajor[GK.Float16],
                       global_b_layout=Layout.UnsafeAlignedColMajor[GK.Float16], is_a_col_major=False)
    a = colmajor(64, 128, torch.float16); b = colmajor(64, 256, torch.float16)
    c = colmajor(128, 256, torch.float32); d = colmajor(128, 256, torch.float32)
    bias = torch.zeros(128)
    hooks = {"shared_to_regs_a": Transform.Elementwise(Transform.Scale(2.0)),
             "shared_to_regs_c": Transform.Elementwise(Transform.Scale(3.0)),
             "shared_to_global_d": Transform.Elementwise(Transform.ReLU())}
    desc, epi, ptrs = GK.lower(conf, a, b, c, d, hooks, Epilogue.Bias(bias, axis="row"), Kernel.matmul_pipelined)
    assert (desc.m, desc.n, desc.k) == (128, 256, 64)
    assert (desc.trans_a, desc.trans_b) == (1, 0) and (desc.lda, desc.ldb, desc.ldd) == (64, 64, 128)
    assert desc.alpha == 2.0 and desc.beta == 3.0 and epi.activation == L.GK_ACT_RELU
    assert epi.bias_axis == L.GK_BIAS_ROW and epi.bias == bias.data_ptr()
    assert desc.op == L.GK_OP_TCGEN05 and desc.compute == L.GK_F16 and desc.dtype_d == L.GK_F32
    assert ptrs[0] == a.data_ptr() and ptrs[3] == d.data_ptr()


def test_arbitrary_functors_are_rejected():
    with pytest.raises(Transform.UnsupportedFunctor):
        Transform.Elementwise(lambda x: x + 1)
    conf = wmma_config(gemm_shape=(128, 128, 64))
    a = colmajor(128, 64, torch.float16); b = colmajor(64, 128, torch.float16)
    d = colmajor(128, 128, torch.float32)
    with pytest.raises(Transform.UnsupportedFunctor):   # an activation on A cannot be fused
        GK.lower(conf, a, b, d, d, {"shared_to_regs_a": Transform.Elementwise(Transform.ReLU())},
                 Epilogue.Default(), Kernel.matmul_singlestage)
    with pytest.raises(Transform.UnsupportedFunctor):   # ReLU before the bias: different math
        GK.lower(conf, a, b, d, d, {"regs_to_shared_d": Transform.Elementwise(Transform.ReLU())},
                 Epilogue.Bias(torch.zeros(128)), Kernel.matmul_singlestage)


def test_pipelined_tag_needs_two_k_steps():
    conf = wmma_config(gemm_shape=(128, 128, 64), block_shape=(128, 128, 16))
    a = colmajor(128, 64, torch.float16); b = colmajor(64, 128, torch.float16); d = colmajor(128, 128, torch.float32)
    with pytest.raises(GK.ConfigError) as e:
        GK.lower(conf, a, b, d, d, {}, Epilogue.Default(), Kernel.matmul_pipelined)
    assert "at least two stages" in str(e.value)


def test_zero_layout_and_wrong_eltype():
    conf = wmma_config(gemm_shape=(128, 128, 64), global_c_layout=Layout.Zero[GK.Float32],
                       global_d_layout=Layout.UnsafeAlignedColMajor[GK.Float32])
    a = colmajor(128, 64, torch.float16); b = colmajor(64, 128, torch.float16); d = colmajor(128, 128, torch.float32)
    desc, _, ptrs = GK.lower(conf, a, b, None, d, {}, Epilogue.Default(), Kernel.matmul_singlestage)
    assert desc.layout_c == L.GK_LAYOUT_ZERO and desc.beta == 0.0 and ptrs[2] is None
    with pytest.raises(GK.ConfigError):
        GK.lower(conf, a.float(), b, None, d, {}, Epilogue.Default(), Kernel.matmul_singlestage)
    with pytest.raises(GK.DimensionMismatch):
        GK.lower(conf, colmajor(64, 64, torch.float16), b, None, d, {}, Epilogue.Default(), Kernel.matmul_singlestage)


def test_planar_complex_lowering():
    conf = GK.get_config(gemm_shape=(128, 128, 64), operator=Operator.WMMAComplexOp[16, 16, 16, GK.Float16, GK.Float32],
                         global_a_layout=Layout.SplitColMajor[GK.Float16], global_c_layout=Layout.SplitColMajor[GK.Float32],
                         block_shape=(64, 64, 32))
    a = torch.zeros(2, 64, 128, dtype=torch.float16).permute(2, 1, 0)   # (128, 64, 2) column-major planes
    b = torch.zeros(2, 128, 64, dtype=torch.float16).permute(2, 1, 0)
    d = torch.zeros(2, 128, 128, dtype=torch.float32).permute(2, 1, 0)
    desc, _, _ = GK.lower(conf, a, b, d, d, {}, Epilogue.Default(), Kernel.matmul_singlestage)
    assert desc.number == L.GK_COMPLEX and desc.plane_a == 128 * 64 and desc.plane_d == 128 * 128


def test_swizzle_visualisation_covers_every_tile_once():
    order = CTASwizzle.visualise_cta_swizzle(CTASwizzle.VerticallyTiled[4], 10, 7)
    flat = sorted(v for row in order for v in row)
    assert flat == list(range(70))
    assert order[0][0] == 0 and order[1][0] == 1 and order[0][1] == 4   # 4 tiles down M, then step along N
    assert CTASwizzle.number_of_blocks(CTASwizzle.Identity(), {"M": 128, "N": 128}, {"M": 1000, "N": 10}) == (8, 1)


def test_every_swizzle_is_a_permutation_and_lebesgue_follows_the_z_curve():
    for sw in (CTASwizzle.Identity(), CTASwizzle.HorizontallyTiled[4], CTASwizzle.VerticallyTiled[3], CTASwizzle.LebesgueCurve()):
        for tm, tn in ((10, 7), (8, 8), (16, 4), (4, 32), (1, 5)):
            order = CTASwizzle.visualise_cta_swizzle(sw, tm, tn)
            assert sorted(v for row in order for v in row) == list(range(tm * tn)), (sw, tm, tn)
    # HorizontallyTiled{4}: four tiles along N, then the next row (src/cta-swizzle.jl:47-90)
    h = CTASwizzle.visualise_cta_swizzle(CTASwizzle.HorizontallyTiled[4], 3, 8)
    assert h[0][:5] == [0, 1, 2, 3, 12] and h[1][0] == 4
    # LebesgueCurve on 8 x 8: the table of src/cta-swizzle.jl:134-143 (1-based there)
    z = CTASwizzle.visualise_cta_swizzle(CTASwizzle.LebesgueCurve(), 8, 8)
    assert [v + 1 for v in z[0]] == [1, 3, 9, 11, 33, 35, 41, 43]
    assert [row[0] + 1 for row in z] == [1, 2, 5, 6, 17, 18, 21, 22]
    # rectangular power-of-two grids: the square curve repeats along the longer side
    r = CTASwizzle.visualise_cta_swizzle(CTASwizzle.LebesgueCurve(), 2, 8)
    assert r[0] == [0, 2, 4, 6, 8, 10, 12, 14] and r[1][0] == 1
    conf = GK.get_config(gemm_shape=(1024, 1024, 64), operator=Operator.TCGen05Operator[GK.Float16, GK.Float32],
                         global_a_layout=Layout.ColMajor[GK.Float16], global_c_layout=Layout.Zero[GK.Float32],
                         global_d_layout=Layout.ColMajor[GK.Float32], cta_swizzle=CTASwizzle.LebesgueCurve())
    a = torch.zeros(64, 1024, dtype=torch.float16).T; b = torch.zeros(1024, 64, dtype=torch.float16).T
    d = torch.zeros(1024, 1024, dtype=torch.float32).T
    desc, _, _ = GK.lower(conf, a, b, None, d, {}, Epilogue.Default(), Kernel.matmul_singlestage)
    assert desc.raster == L.GK_RASTER_LEBESGUE


def test_column_major_helpers_roundtrip():
    x = np.arange(12, dtype=np.float32).reshape(3, 4)
    t = GK.to_cuarray(x, device="cpu")
    assert tuple(t.shape) == (3, 4) and t.stride(0) == 1 and GK.arrays.is_col_major(t)
    assert np.array_equal(GK.to_numpy(t), x)
    z = GK.to_cuarray((x + 1j * x).astype(np.complex64), device="cpu")
    assert tuple(z.shape) == (2, 3, 4) and z.stride(0) == 1 and z.stride(1) == 2
