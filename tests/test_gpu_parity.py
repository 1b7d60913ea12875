"""Parity of the CUDA path (through the C ABI) with the CPU oracle.

Tolerances.  Data whose sums are exactly representable (+-1 and small
integers, the reference tool's own exact mode, tools/single_conv_layer.cpp:
979-1005) must match the oracle BIT FOR BIT.  Uniform / normal data use
poplibs_test::checkIsClose with relative tolerance 1e-3 for half inputs with
float partials and 5e-2 for quarter inputs; the absolute tolerance is
max(1e-5, 2.5e-4 * rms(expected)): an output that is near zero because large
terms cancel cannot be reproduced to 1e-3 of ITSELF by any fp32 accumulation,
so such elements are held to a quarter of the relative tolerance measured
against the typical output magnitude instead.
"""
import os
import zlib

import numpy as np
import pytest

import common as T
import oracle
from poplibs_b200 import capi

pytestmark = pytest.mark.gpu

REL_HALF, REL_QUARTER = T.REL_TOL_HALF, T.REL_TOL_QUARTER


def assert_close(got, exp, rel, what):
    got = np.asarray(got, dtype=np.float64)
    exp = np.asarray(exp, dtype=np.float64).reshape(got.shape)
    rms = float(np.sqrt(np.mean(exp * exp))) if exp.size else 0.0
    abs_tol = max(T.ABS_TOL, 2.5e-4 * rms)
    bad, first, worst = oracle.check_is_close(got, exp, rel, abs_tol)
    assert bad == 0, (f"{what}: {bad}/{got.size} elements outside rel={rel} abs={abs_tol:.2e}; first at "
                      f"{np.unravel_index(first, got.shape)} got {got.ravel()[first]} expected {exp.ravel()[first]}")


def assert_exact(got, exp, what):
    got = np.asarray(got, dtype=np.float64)
    exp = np.asarray(exp, dtype=np.float64).reshape(got.shape)
    diff = got != exp
    assert not diff.any(), f"{what}: {int(diff.sum())}/{got.size} elements differ; first at {np.argwhere(diff)[0]}"


# --------------------------------------------------------------------------- matMul

GEMM_SHAPES = [(128, 64, 64), (1, 8, 1), (1, 1000, 1), (5, 8, 4), (300, 200, 72), (129, 72, 257),
               (256, 128, 128), (128, 64, 256), (640, 320, 520)]


@pytest.mark.parametrize("m,k,n", GEMM_SHAPES)
@pytest.mark.parametrize("tb", [False, True])
def test_matmul_exact(gpu_ctx, m, k, n, tb):
    r = T.rng(m * 7 + k * 3 + n)
    a = T.small_int_half(r, (m, k))
    b = T.small_int_half(r, (n, k) if tb else (k, n), -3, 3)
    got = T.gpu_matmul(a, b, transpose_b=tb, out_dtype=np.float32)
    assert_exact(got, oracle.gemm(a, b, transpose_b=tb), f"matMul {m}x{k}x{n} tb={tb}")


def test_matmul_config1_uniform(gpu_ctx):
    # poplin::matMul fp16 A[512x1024].B[1024x1024], fp32 partials, fp16 out
    r = T.rng(1234 + 1)
    a, b = T.uniform_half(r, (512, 1024)), T.uniform_half(r, (1024, 1024))
    got = T.gpu_matmul(a, b)
    assert_close(got, oracle.gemm(a, b), REL_HALF, "config 1")
    # the gemm tool's own data ranges and D = beta*C + alpha*A*B
    a, b = T.uniform_half(r, (512, 1024), -4, 4), T.uniform_half(r, (1024, 1024), -3, 3)
    c = T.uniform_half(r, (512, 1024), -2, 2)
    got = T.gpu_matmul(a, b, c, alpha=1.0, beta=1.0)
    assert_close(got, oracle.gemm(a, b, c, 1.0, 1.0), REL_HALF, "config 1, alpha=beta=1")


def test_matmul_transposes_groups_alpha_beta(gpu_ctx):
    r = T.rng(11)
    g, m, k, n = 3, 72, 136, 88
    for ta in (False, True):
        for tb in (False, True):
            a = T.small_int_half(r, (g, k, m) if ta else (g, m, k))
            b = T.small_int_half(r, (g, n, k) if tb else (g, k, n), -3, 3)
            c = T.small_int_half(r, (g, m, n), -2, 2)
            got = T.gpu_matmul(a, b, c, transpose_a=ta, transpose_b=tb, alpha=2.0, beta=-1.0,
                               out_dtype=np.float32)
            assert_exact(got, oracle.gemm(a, b, c, 2.0, -1.0, ta, tb), f"grouped ta={ta} tb={tb}")


def test_matmul_empty_dimensions(gpu_ctx):
    r = T.rng(12)
    # gemm_5x0x4: an empty reduction leaves beta*C
    a = np.zeros((5, 0), np.float16)
    b = np.zeros((4, 0), np.float16)
    c = T.small_int_half(r, (5, 4))
    got = T.gpu_matmul(a, b, c, transpose_b=True, beta=1.0, out_dtype=np.float32)
    assert_exact(got, c, "5x0x4")
    got = T.gpu_matmul(np.zeros((0, 8), np.float16), np.zeros((4, 8), np.float16), transpose_b=True)
    assert got.shape == (0, 4)


def test_matmul_quarter_exact_and_scaled(gpu_ctx):
    r = T.rng(13)
    for (m, k, n) in [(128, 128, 64), (300, 256, 72), (256, 512, 256)]:
        av = r.integers(-4, 5, size=(m, k)).astype(np.float64)
        bv = r.integers(-3, 4, size=(k, n)).astype(np.float64)
        a8, b8 = oracle.e4m3_encode(av), oracle.e4m3_encode(bv)
        got = T.gpu_matmul(a8, np.ascontiguousarray(b8.T), transpose_b=True, scale_a=-3, scale_b=-2)
        assert_exact(got, oracle.gemm(av, bv) * 2.0 ** -5, f"quarter {m}x{k}x{n} scaled")
        got = T.gpu_matmul(a8, b8)   # [k][n] right operand goes through the transpose kernel
        assert_exact(got, oracle.gemm(av, bv), f"quarter {m}x{k}x{n} row-major B")


def quantised_normal(r, shape, exponent):
    """N(0,1) data stored as E4M3 with value = stored * 2^exponent: returns the
    bytes and the dequantised doubles the oracle is given."""
    x = r.normal(size=shape)
    bits = oracle.e4m3_encode(x * 2.0 ** (-exponent))
    return bits, oracle.e4m3_decode(bits) * 2.0 ** exponent


def test_matmul_config5_quarter_sampled_rows(gpu_ctx):
    # 8192^3 E4M3, scales 2^-3 and 2^-2, fp16 out: full-size run, oracle on sampled rows
    import torch
    r = T.rng(1234 + 5)
    n = 8192
    a8, av = quantised_normal(r, (n, n), -3)
    b8, bv = quantised_normal(r, (n, n), -2)
    got = T.gpu_matmul(a8, np.ascontiguousarray(b8.T), transpose_b=True, scale_a=-3, scale_b=-2)
    rows = np.sort(r.choice(n, 48, replace=False))
    assert_close(got[rows], oracle.gemm(av[rows], bv), REL_QUARTER, "config 5 fp8 rows")
    torch.cuda.empty_cache()


def test_matmul_config5_half_sampled_rows(gpu_ctx):
    import torch
    r = T.rng(1234 + 6)
    n = 8192
    a = r.normal(size=(n, n)).astype(np.float16)
    b = r.normal(size=(n, n)).astype(np.float16)
    got = T.gpu_matmul(a, b)
    rows = np.sort(r.choice(n, 48, replace=False))
    assert_close(got[rows], oracle.gemm(a[rows], b), REL_HALF, "config 5 fp16 rows")
    # size-independent property: (2A)B == 2(AB) exactly in binary floating point
    got2 = T.gpu_matmul((2 * a).astype(np.float16), b)
    assert (got2[rows].astype(np.float64) == 2 * got[rows].astype(np.float64)).all()
    torch.cuda.empty_cache()


# --------------------------------------------------------------------------- convolution

def conv_case(batch, field, kernel, ci, co, **kw):
    return dict(batch=batch, field=field, kernel=kernel, in_chans=ci, out_chans=co, **kw)


SMALL_CONVS = {
    "3x3_pad1": conv_case(2, [8, 8], [3, 3], 64, 64, padding=1),
    "1x1": conv_case(2, [8, 8], [1, 1], 128, 64),
    "ragged_chans": conv_case(3, [7, 9], [3, 3], 72, 40, padding=1),
    "wide_chans": conv_case(2, [6, 6], [3, 3], 320, 192, padding=1),
    "kernel_dilation": conv_case(2, [12, 12], [3, 3], 64, 64, padding=2, k_dilation=2),
    "asym_padding": conv_case(2, [9, 6], [3, 2], 64, 72, in_pad_lo=[2, 0], in_pad_hi=[0, 1]),
    "flipped_kernel": conv_case(2, [7, 7], [3, 3], 64, 64, padding=1, k_flip=[1, 0]),
    "one_dim": conv_case(4, [33], [5], 64, 96, padding=2),
    "groups2": conv_case(2, [6, 6], [3, 3], 64, 64, padding=1, groups=2),
    "batch1_big_field": conv_case(1, [40, 23], [3, 3], 64, 64, padding=1),
    "5x5_pad2": conv_case(3, [10, 10], [5, 5], 64, 72, padding=2),
}
STRIDED_CONVS = {
    "1x1_s2": conv_case(2, [8, 8], [1, 1], 64, 128, stride=2),
    "3x3_s2": conv_case(2, [9, 9], [3, 3], 64, 64, padding=1, stride=2),
    "3x3_s2x3": conv_case(2, [11, 13], [3, 3], 64, 64, padding=1, stride=[2, 3]),
    "3x3_s1x2": conv_case(5, [10, 13], [3, 3], 64, 64, padding=1, stride=[1, 2]),
    "1x1_s2_even_field": conv_case(3, [12, 10], [1, 1], 64, 128, stride=2),   # last row / column unused
    "3x3_s2_nopad_leftover": conv_case(2, [12, 13], [3, 3], 64, 64, stride=2),
    "5x5_s3_dil1": conv_case(2, [17, 16], [5, 5], 64, 72, padding=2, stride=3),
    "3x3_s2_dil3": conv_case(2, [15, 15], [3, 3], 64, 64, padding=3, stride=2, k_dilation=3),
    "one_dim_s2": conv_case(4, [33], [5], 64, 96, padding=2, stride=2),
}
# Transforms that the reference's canonical form of ordinary layers produces
# (input truncation for unused trailing rows) and its gradient parameters use
# (output truncation / padding); all of them are views and offsets here.
TRANSFORMED_CONVS = {
    "in_trunc": conv_case(2, [11, 12], [3, 3], 64, 64, padding=1, in_trunc_lo=[1, 2], in_trunc_hi=[2, 0]),
    "in_trunc_s2": conv_case(3, [12, 12], [1, 1], 64, 64, stride=2, in_trunc_hi=[1, 1]),
    "out_trunc": conv_case(2, [10, 9], [3, 3], 64, 64, padding=2, out_trunc_lo=[1, 0], out_trunc_hi=[1, 2]),
    "out_pad": conv_case(2, [8, 8], [3, 3], 64, 72, padding=1, out_pad_lo=[1, 0], out_pad_hi=[0, 2]),
    "all_views_s2": conv_case(2, [14, 13], [3, 3], 64, 64, padding=1, stride=2, in_trunc_lo=[1, 0],
                              out_trunc_lo=[2, 0], out_pad_lo=[0, 1], out_pad_hi=[1, 0]),
}


def conv_data(p, kw, r, exact):
    gen = T.binary_half if exact else T.uniform_half
    g = p.groups
    x = gen(r, (p.batch, g * p.in_chans_per_group, *kw["field"]))
    fan_in = p.in_chans_per_group * int(np.prod(kw["kernel"]))
    if exact:
        w = gen(r, (g, p.out_chans_per_group, p.in_chans_per_group, *kw["kernel"]))
    else:
        bound = 1.0 / np.sqrt(fan_in)
        w = T.uniform_half(r, (g, p.out_chans_per_group, p.in_chans_per_group, *kw["kernel"]), -bound, bound)
    dy = gen(r, (p.batch, g * p.out_chans_per_group, *p.output_field()))
    return x, w, dy


@pytest.mark.parametrize("name", sorted({**SMALL_CONVS, **STRIDED_CONVS}))
def test_conv_fwd_small(gpu_ctx, name):
    kw = {**SMALL_CONVS, **STRIDED_CONVS}[name]
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(zlib.crc32(name.encode()) % 1000)
    x, w, _ = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), f"fwd {name} exact")
    x, w, _ = conv_data(p, kw, r, exact=False)
    bias = r.uniform(-2, 6, p.groups * p.out_chans_per_group).astype(np.float32)
    assert_close(T.gpu_conv_fwd(p, x, w, bias=bias), oracle.conv_fwd(spec, x, w, bias), REL_HALF,
                 f"fwd {name} uniform + bias")


@pytest.mark.parametrize("ci,co,groups", [(20, 12, 1), (12, 64, 1), (64, 20, 1), (10, 6, 3), (5, 8, 1)])
def test_conv_channel_counts_that_need_padding(gpu_ctx, ci, co, groups):
    """Channel counts that are not a multiple of 8 run on zero-padded copies."""
    kw = conv_case(3, [9, 10], [3, 3], ci, co, padding=1, groups=groups)   # channels per group
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(ci * 100 + co)
    x, w, dy = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), f"fwd ci={ci} co={co}")
    assert_exact(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), f"bwd ci={ci} co={co}")
    dw16, dw32 = T.gpu_conv_wu(p, x, dy)
    exp = oracle.conv_wu(spec, x, dy)[0]
    assert_exact(dw32, exp, f"wu ci={ci} co={co}")
    assert (dw32.astype(np.float16) == dw16).all()
    bias = r.integers(-3, 4, p.groups * p.out_chans_per_group).astype(np.float32)
    assert_exact(T.gpu_conv_fwd(p, x, w, bias=bias), oracle.conv_fwd(spec, x, w, bias), f"fwd+bias ci={ci} co={co}")


@pytest.mark.parametrize("name", sorted(TRANSFORMED_CONVS))
def test_conv_transform_views(gpu_ctx, name):
    """Input truncation, output truncation and output padding in all three passes."""
    kw = TRANSFORMED_CONVS[name]
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(zlib.crc32(name.encode()) % 1000 + 7)
    x, w, dy = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), f"fwd {name}")
    assert_exact(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), f"bwd {name}")
    _, dw32 = T.gpu_conv_wu(p, x, dy)
    assert_exact(dw32, oracle.conv_wu(spec, x, dy)[0], f"wu {name}")


# 3-D fields: the depth dimension is folded into the channels of a 2-D problem,
# so every transform of that dimension is fair game.
CONVS_3D = {
    "3x3x3_pad1": conv_case(2, [5, 6, 7], [3, 3, 3], 16, 24, padding=1),
    "depth_stride2": conv_case(2, [7, 6, 6], [3, 3, 3], 16, 16, padding=1, stride=[2, 1, 1]),
    "all_s2": conv_case(1, [8, 9, 9], [3, 3, 3], 16, 32, padding=1, stride=2),
    "1x1x1": conv_case(2, [3, 4, 4], [1, 1, 1], 32, 16),
    "depth_only_kernel": conv_case(2, [6, 5, 5], [3, 1, 1], 64, 64, padding=[1, 0, 0]),
    "groups_unaligned": conv_case(2, [4, 5, 5], [2, 3, 3], 6, 10, padding=[0, 1, 1], groups=2),
    "depth_transforms": conv_case(2, [7, 5, 6], [3, 1, 3], 8, 16, in_pad_lo=[2, 0, 1], in_pad_hi=[0, 0, 1],
                                  k_dilation=[2, 1, 1], in_dilation=[2, 1, 1], in_trunc_lo=[1, 0, 0],
                                  k_flip=[1, 0, 0], in_flip=[1, 0, 0], out_pad_lo=[1, 0, 0],
                                  out_trunc_hi=[1, 0, 0], stride=[2, 1, 1]),
    "depth_kernel_trunc_pad": conv_case(1, [6, 4, 4], [4, 3, 3], 8, 8, padding=[2, 1, 1], k_trunc_lo=[1, 0, 0],
                                        k_pad_hi=[1, 0, 0], out_pad_hi=[2, 0, 0]),
}


@pytest.mark.parametrize("name", sorted(CONVS_3D))
def test_conv_3d_all_passes(gpu_ctx, name):
    kw = CONVS_3D[name]
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(zlib.crc32(name.encode()) % 1000 + 11)
    x, w, dy = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), f"3-D fwd {name}")
    assert_exact(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), f"3-D bwd {name}")
    dw16, dw32 = T.gpu_conv_wu(p, x, dy)
    assert_exact(dw32, oracle.conv_wu(spec, x, dy)[0], f"3-D wu {name}")
    assert (dw32.astype(np.float16) == dw16).all()
    x, w, dy = conv_data(p, kw, r, exact=False)
    bias = r.uniform(-2, 6, p.groups * p.out_chans_per_group).astype(np.float32)
    assert_close(T.gpu_conv_fwd(p, x, w, bias=bias), oracle.conv_fwd(spec, x, w, bias), REL_HALF,
                 f"3-D fwd {name} uniform + bias")
    assert_close(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), REL_HALF, f"3-D bwd {name} uniform")
    assert_close(T.gpu_conv_wu(p, x, dy)[0], oracle.conv_wu(spec, x, dy)[0], REL_HALF, f"3-D wu {name} uniform")
    for pass_id in (capi.PASS_TRAINING_FWD, capi.PASS_TRAINING_BWD, capi.PASS_TRAINING_WU):
        assert capi.conv_plan(p, pass_id).flops == 2 * p.macs()


@pytest.mark.parametrize("name", sorted({**SMALL_CONVS, **STRIDED_CONVS}))
def test_conv_bwd_small(gpu_ctx, name):
    kw = {**SMALL_CONVS, **STRIDED_CONVS}[name]
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(zlib.crc32(name.encode()) % 1000 + 1)
    _, w, dy = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), f"bwd {name} exact")
    _, w, dy = conv_data(p, kw, r, exact=False)
    assert_close(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), REL_HALF, f"bwd {name} uniform")


@pytest.mark.parametrize("name", sorted(n for n in {**SMALL_CONVS, **STRIDED_CONVS} if n != "flipped_kernel"))
def test_conv_wu_small(gpu_ctx, name):
    kw = {**SMALL_CONVS, **STRIDED_CONVS}[name]
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(zlib.crc32(name.encode()) % 1000 + 2)
    x, _, dy = conv_data(p, kw, r, exact=True)
    dw16, dw32 = T.gpu_conv_wu(p, x, dy)
    exp, _ = oracle.conv_wu(spec, x, dy)
    assert_exact(dw32, exp, f"wu {name} exact (fp32 sums)")
    x, _, dy = conv_data(p, kw, r, exact=False)
    dw16, dw32 = T.gpu_conv_wu(p, x, dy)
    exp, _ = oracle.conv_wu(spec, x, dy)
    assert_close(dw16, exp, REL_HALF, f"wu {name} uniform")
    # the two outputs of one call agree: half result is the rounded fp32 sum
    assert (dw32.astype(np.float16) == dw16).all()


@pytest.mark.parametrize("name", ["3x3_pad1", "kernel_dilation", "5x5_pad2", "3x3_s1x2", "groups2"])
def test_conv_wu_plan_variants(gpu_ctx, name):
    """One activation strip per filter column (the default where the vertical
    stride is 1) and one box per tap give the same sums; so does any K split."""
    kw = {**SMALL_CONVS, **STRIDED_CONVS}[name]
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(zlib.crc32(name.encode()) % 1000 + 3)
    x, _, dy = conv_data(p, kw, r, exact=True)
    exp, _ = oracle.conv_wu(spec, x, dy)
    assert capi.conv_wu_plan(p).halo_rows == (kw["kernel"][0] - 1) * kw.get("k_dilation", 1)
    for flags, split in ((0, 0), (capi.PLAN_NO_HALO, 0), (0, 1), (0, 3), (capi.PLAN_NO_HALO, 2)):
        opt = capi.ConvOptions.make(plan_flags=flags, split_k=split)
        plan = capi.conv_wu_plan(p, opt)
        assert (plan.halo_rows == 0) == bool(flags & capi.PLAN_NO_HALO)
        _, dw32 = T.gpu_conv_wu(p, x, dy, opt=opt)
        assert_exact(dw32, exp, f"wu {name} flags={flags} split={split}")


PLAN_VARIANTS = {
    "streamed": capi.PLAN_NO_RESIDENT_WEIGHTS,
    "streamed_no_halo": capi.PLAN_NO_RESIDENT_WEIGHTS | capi.PLAN_NO_HALO,
    "resident": capi.PLAN_FORCE_RESIDENT_WEIGHTS | capi.PLAN_NO_HALO,
    "resident_halo": capi.PLAN_FORCE_RESIDENT_WEIGHTS,
    "streamed_pair": capi.PLAN_NO_RESIDENT_WEIGHTS | capi.PLAN_FORCE_CTA_PAIR,
    "resident_pair": capi.PLAN_FORCE_RESIDENT_WEIGHTS | capi.PLAN_NO_HALO | capi.PLAN_FORCE_CTA_PAIR,
    "resident_halo_pair": capi.PLAN_FORCE_RESIDENT_WEIGHTS | capi.PLAN_FORCE_CTA_PAIR,
    "no_pair": capi.PLAN_NO_CTA_PAIR,
}


@pytest.mark.parametrize("variant", sorted(PLAN_VARIANTS))
@pytest.mark.parametrize("name", ["3x3_pad1", "ragged_chans", "kernel_dilation", "asym_padding",
                                  "flipped_kernel", "batch1_big_field", "3x3_s2x3", "one_dim"])
def test_conv_plan_variants_agree_with_oracle(gpu_ctx, name, variant):
    """Every way the planner may run a layer (weights streamed, weights
    resident, resident with halo strips) must give the oracle's result."""
    kw = {**SMALL_CONVS, **STRIDED_CONVS}[name]
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    opt = capi.ConvOptions.make(plan_flags=PLAN_VARIANTS[variant])
    if variant in ("streamed_pair", "resident_pair", "resident_halo_pair"):
        # two CTAs share 256-row MMAs (every case here has at least two pixel tiles)
        plan = capi.conv_plan(p, capi.PASS_TRAINING_FWD, opt)
        pixel_tiles = plan.tiles // -(-p.out_chans_per_group // plan.tile_n)
        assert plan.cta_pair == (1 if pixel_tiles >= 2 else 0)
    r = T.rng(zlib.crc32((name + variant).encode()) % 1000)
    x, w, dy = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w, opt=opt), oracle.conv_fwd(spec, x, w), f"fwd {name} {variant}")
    assert_exact(T.gpu_conv_bwd(p, dy, w, opt=opt), oracle.conv_bwd(spec, dy, w), f"bwd {name} {variant}")


@pytest.mark.parametrize("split", [2, 3, 5])
@pytest.mark.parametrize("variant", ["streamed", "resident_halo", "streamed_pair", "resident_halo_pair", "no_pair"])
@pytest.mark.parametrize("name", ["3x3_pad1", "ragged_chans", "3x3_s2x3", "batch1_big_field"])
def test_conv_split_k_agrees_with_oracle(gpu_ctx, name, variant, split):
    """Forward and backward with several CTAs per output tile (the reduction
    dimension split, fp32 partial sums added by a second kernel in split order)
    under every way the planner may run the layer: the oracle's result, bit for
    bit, with a bias and with fp32 output as well."""
    kw = {**SMALL_CONVS, **STRIDED_CONVS}[name]
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    opt = capi.ConvOptions.make(plan_flags=PLAN_VARIANTS[variant], split_k=split)
    plan = capi.conv_plan(p, capi.PASS_TRAINING_FWD, opt)
    assert 1 <= plan.split_k <= split and (plan.split_k > 1) == (plan.workspace_bytes > 0)
    r = T.rng(zlib.crc32((name + variant).encode()) % 1000 + split)
    x, w, dy = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w, opt=opt), oracle.conv_fwd(spec, x, w), f"fwd {name} {variant} /{split}")
    assert_exact(T.gpu_conv_bwd(p, dy, w, opt=opt), oracle.conv_bwd(spec, dy, w), f"bwd {name} {variant} /{split}")
    bias = r.integers(-3, 4, size=p.groups * p.out_chans_per_group).astype(np.float32)
    pf = capi.ConvParams.make(output_type=capi.FLOAT, **kw)
    assert_exact(T.gpu_conv_fwd(pf, x, w, bias=bias, opt=opt), oracle.conv_fwd(spec, x, w, bias=bias),
                 f"fwd fp32 + bias {name} {variant} /{split}")


def test_matmul_long_k_is_split_by_the_planner(gpu_ctx):
    """Few output tiles and a long reduction: the planner gives each tile to
    several CTAs by itself; results stay exact, also with alpha, beta and C."""
    m, k, n = 256, 8192, 256
    plan = capi.matmul_plan(capi.MatmulDesc.make(m, k, n))
    assert plan.split_k > 1 and plan.grid > plan.tiles
    assert capi.matmul_plan(capi.MatmulDesc.make(512, 1024, 1024)).split_k == 1   # too short to pay
    r = T.rng(5)
    a, b = T.binary_half(r, (m, k)), T.binary_half(r, (k, n))
    assert_exact(T.gpu_matmul(a, b, out_dtype=np.float32), oracle.gemm(a, b), "split matmul")
    bt = np.ascontiguousarray(b.T)
    assert_exact(T.gpu_matmul(a, bt, transpose_b=True, out_dtype=np.float32), oracle.gemm(a, b),
                 "split matmul, transposed B")
    c = T.small_int_half(r, (m, n)).astype(np.float32)
    got = T.gpu_matmul(a, b, c, alpha=0.5, beta=2.0, out_dtype=np.float32)
    assert_exact(got, oracle.gemm(a, b, c, alpha=0.5, beta=2.0), "split matmul with alpha, beta, C")
    # quarter input (half output): sparse right operand keeps the sums exactly representable
    av = r.integers(-1, 2, size=(m, k)).astype(np.float64)
    bv = (r.integers(-2, 3, size=(n, k)) * (r.integers(0, 16, size=(n, k)) == 0)).astype(np.float64)
    got = T.gpu_matmul(oracle.e4m3_encode(av), oracle.e4m3_encode(bv), transpose_b=True)
    assert_exact(got, oracle.gemm(av, bv, transpose_b=True), "split quarter matmul")


@pytest.fixture
def force_cta_pair():
    T.context().set_plan_flags(capi.PLAN_FORCE_CTA_PAIR)
    yield
    T.context().set_plan_flags(0)


@pytest.mark.parametrize("m,k,n,tb", [(384, 192, 200, False), (384, 192, 200, True), (1000, 72, 136, False),
                                      (256, 1024, 512, True), (130, 64, 64, True)])
def test_matmul_cta_pair_exact(gpu_ctx, force_cta_pair, m, k, n, tb):
    """Matrix products on CTA pairs: odd tile counts, ragged N, both B layouts."""
    r = T.rng(m + k + n)
    a = T.binary_half(r, (m, k))
    b = T.binary_half(r, (n, k) if tb else (k, n))
    got = T.gpu_matmul(a, b, transpose_b=tb)
    assert_exact(got, oracle.gemm(a, b, transpose_b=tb), f"pair matmul {m}x{k}x{n} tb={tb}")


def test_matmul_short_k_pairs_under_wide_tiles(gpu_ctx):
    """4 K steps, 256-column tiles, many tiles: the planner pairs CTAs by itself."""
    m, k, n = 4096, 256, 4096
    assert capi.matmul_plan(capi.MatmulDesc.make(m, k, n)).cta_pair == 1
    r = T.rng(77)
    a, b = T.binary_half(r, (m, k)), T.binary_half(r, (k, n))
    got = T.gpu_matmul(a, b)
    rows = np.array([0, 1, 127, 128, 255, 256, 2047, 2048, m - 257, m - 256, m - 1])
    assert_exact(got[rows], oracle.gemm(a[rows], b), "short-K pair matmul, sampled rows")
    assert_exact(got[:, :8].astype(np.float64), a.astype(np.float64) @ b[:, :8].astype(np.float64), "first columns")


def test_matmul_cta_pair_quarter(gpu_ctx, force_cta_pair):
    r = T.rng(5)
    av = r.integers(-3, 4, (384, 256)).astype(np.float64)
    bv = r.integers(-3, 4, (256, 320)).astype(np.float64)
    got = T.gpu_matmul(oracle.e4m3_encode(av), oracle.e4m3_encode(bv))
    assert_exact(got, oracle.gemm(av, bv), "pair quarter matmul")


@pytest.mark.parametrize("fa,fb", [(capi.F152, capi.F152), (capi.F143, capi.F152), (capi.F152, capi.F143)])
def test_matmul_quarter_f152(gpu_ctx, fa, fb):
    """The 1-5-2 quarter format, alone and mixed with 1-4-3, with scales."""
    r = T.rng(40 + fa * 2 + fb)
    m, k, n = 384, 64, 320
    # integers exactly representable in either format; sums stay exact in half
    av = r.integers(-4, 5, (m, k)).astype(np.float64)
    bv = r.integers(-4, 5, (k, n)).astype(np.float64)
    enc = {capi.F143: oracle.e4m3_encode, capi.F152: oracle.e5m2_encode}
    dec = {capi.F143: oracle.e4m3_decode, capi.F152: oracle.e5m2_decode}
    a8, b8 = enc[fa](av), enc[fb](bv)
    assert (dec[fa](a8) == av).all() and (dec[fb](b8) == bv).all()
    got = T.gpu_matmul(a8, b8, format_a=fa, format_b=fb)
    assert_exact(got, oracle.gemm(av, bv), f"quarter matmul formats {fa},{fb}")
    got = T.gpu_matmul(a8, b8, format_a=fa, format_b=fb, scale_a=-2, scale_b=1)
    assert_exact(got, oracle.gemm(av, bv) * 0.5, f"quarter matmul formats {fa},{fb} scaled")
    # fractions the two formats share, and magnitudes only E5M2 reaches (E4M3 stops at 448)
    if fa == capi.F152 and fb == capi.F152:
        vals = r.choice(np.array([1024.0, -2048.0, 4096.0, 0.0, 57344.0, 0.3125, -1.75, 2.0 ** -14]), (128, 64))
        eye = np.eye(64)
        v8 = oracle.e5m2_encode(vals)
        assert (oracle.e5m2_decode(v8) == vals).all()
        got = T.gpu_matmul(v8, oracle.e5m2_encode(eye), format_a=fa, format_b=fb)
        assert_exact(got, vals, "E5M2 range")


def test_conv_quarter_f152_fwd_bwd(gpu_ctx):
    kw = conv_case(2, [9, 8], [3, 3], 16, 32, padding=1, stride=[2, 1])
    p = capi.ConvParams.make(input_type=capi.QUARTER, **kw)
    spec = T.spec_from_params(p)
    r = T.rng(52)
    xv = r.integers(-3, 4, (2, 16, 9, 8)).astype(np.float64)
    wv = r.integers(-2, 3, (1, 32, 16, 3, 3)).astype(np.float64)
    dyv = r.integers(-3, 4, (2, 32, *p.output_field())).astype(np.float64)
    opt = capi.ConvOptions.make(format_in=capi.F152, format_weights=capi.F143, scale_in=1)
    got = T.gpu_conv_fwd(p, oracle.e5m2_encode(xv), oracle.e4m3_encode(wv), opt=opt)
    assert_exact(got, 2 * oracle.conv_fwd(spec, xv, wv), "quarter fwd, F152 activations")
    opt = capi.ConvOptions.make(format_in=capi.F152, format_weights=capi.F152)
    got = T.gpu_conv_bwd(p, oracle.e5m2_encode(dyv), oracle.e5m2_encode(wv), opt=opt)
    assert_exact(got, oracle.conv_bwd(spec, dyv, wv), "quarter bwd (strided), F152 gradients and weights")


def test_conv_bias_update(gpu_ctx):
    """biases += scale * sum over pixels of the output gradients (fp32 sums)."""
    import torch
    ctx = T.context()
    for (n, c, field, dt) in ((4, 64, (9, 7), np.float16), (3, 40, (5, 5), np.float16),
                              (2, 132, (6, 6), np.float32), (5, 3, (4, 4), np.float16)):
        r = T.rng(c)
        dy = T.binary_half(r, (n, c, *field)).astype(dt)
        b0 = r.integers(-4, 5, c).astype(dt)
        ddy = T.to_dev(T.acts_to_device_layout(dy))
        db = T.to_dev(b0.copy())
        torch.cuda.synchronize()
        ctx.conv_bias_update(capi.FLOAT if dt == np.float32 else capi.HALF, ddy, n * field[0] * field[1], c,
                             capi.FLOAT if dt == np.float32 else capi.HALF, db, -0.5)
        ctx.synchronize()
        want = b0.astype(np.float64) - 0.5 * dy.astype(np.float64).sum(axis=(0, 2, 3))
        assert_exact(db.cpu().numpy(), want, f"bias update c={c}")
    # against the model's bias gradient on a convolution
    kw = conv_case(3, [8, 8], [3, 3], 64, 72, padding=1)
    p = capi.ConvParams.make(**kw)
    r = T.rng(9)
    x, _, dy = conv_data(p, kw, r, exact=True)
    _, dbias = oracle.conv_wu(T.spec_from_params(p), x, dy)
    ddy = T.to_dev(T.acts_to_device_layout(dy))
    db = T.to_dev(np.zeros(72, np.float32))
    torch.cuda.synchronize()
    ctx.conv_bias_update(capi.HALF, ddy, 3 * 64, 72, capi.FLOAT, db, 1.0)
    ctx.synchronize()
    assert_exact(db.cpu().numpy(), dbias, "bias gradient vs model")


def test_host_buffer_calls_pipelined_over_two_contexts(gpu_ctx):
    """The asynchronous host-buffer entry points on two alternating contexts
    (upload of one step overlapping the download of the previous one) give the
    same results as the synchronous ones."""
    import torch
    kw = conv_case(4, [20, 20], [3, 3], 64, 64, padding=1)
    p = capi.ConvParams.make(**kw)
    r = T.rng(11)
    ctxs = [capi.Context(0), capi.Context(0)]
    xs, outs, want = [], [], []
    _, w, _ = conv_data(p, kw, r, exact=True)
    wh = torch.from_numpy(T.weights_to_device_layout(w)).pin_memory()
    for i in range(6):
        x, _, _ = conv_data(p, kw, r, exact=True)
        xs.append(torch.from_numpy(T.acts_to_device_layout(x)).pin_memory())
        outs.append(torch.empty((4, 20, 20, 64), dtype=torch.float16).pin_memory())
        want.append(oracle.conv_fwd(T.spec_from_params(p), x, w))
    for i in range(6):
        c = ctxs[i & 1]
        c.synchronize()                      # step i - 2 on this context is complete
        c.conv_fwd_host(p, xs[i], wh, outs[i], sync=False)
    for c in ctxs:
        c.synchronize()
    for i in range(6):
        got = T.acts_from_device_layout(outs[i].numpy())
        assert_exact(got, want[i], f"pipelined host step {i}")
    a = T.binary_half(r, (256, 192))
    b = T.binary_half(r, (192, 128))
    ah, bh = torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory()
    dh = torch.empty((256, 128), dtype=torch.float16).pin_memory()
    ctxs[0].matmul_host(capi.MatmulDesc.make(256, 192, 128), ah, bh, None, dh, sync=False)
    ctxs[0].synchronize()
    assert_exact(dh.numpy(), oracle.gemm(a, b), "async host matmul")


def test_allreduce_over_peer_memory_on_one_gpu(gpu_ctx):
    """plb_allreduce_f32_p2p with all "ranks'" buffers on this GPU and the
    peers' flags already set: checks the flags this rank writes, the rank-order
    sum and the cast.  Then a step whose peers never signal: the kernel's
    bounded wait must run out and report it, leaving the context usable."""
    import torch
    ctx = T.context()
    world, rank, count = 3, 1, 4 * 100003
    words = capi.lib().plb_allreduce_p2p_signal_bytes(world) // 4
    g = torch.Generator().manual_seed(3)
    bufs = [torch.randn(count, generator=g).cuda() for _ in range(world)]
    pads = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(world)]
    for peer in range(world):
        if peer != rank:
            pads[rank][peer] = 1   # "the peers' flags of epoch 1 arrived"
    out32 = torch.empty(count, device="cuda")
    out16 = torch.empty(count, device="cuda", dtype=torch.float16)
    torch.cuda.synchronize()
    ctx.allreduce_f32_p2p(rank, world, [b.data_ptr() for b in bufs], [p.data_ptr() for p in pads], 1,
                          count, out32, out16)
    ctx.synchronize()
    want = (bufs[0] + bufs[1]) + bufs[2]          # rank order, fp32
    assert torch.equal(out32, want)
    assert torch.equal(out16, want.half())
    for peer in range(world):
        if peer != rank:
            assert int(pads[peer][rank]) == 1, "flag not sent"
    # only one output requested
    out32.zero_()
    ctx.allreduce_f32_p2p(rank, world, [b.data_ptr() for b in bufs], [p.data_ptr() for p in pads], 1,
                          count, out32, None)
    ctx.synchronize()
    assert torch.equal(out32, want)
    # epoch 2: nobody signals -> the wait runs out (about two seconds) and is reported
    ctx.allreduce_f32_p2p(rank, world, [b.data_ptr() for b in bufs], [p.data_ptr() for p in pads], 2,
                          count, out32, None)
    with pytest.raises(capi.PlbError):
        ctx.synchronize()
    # the context still works
    ctx.allreduce_f32_p2p(0, 1, [bufs[0].data_ptr()], [pads[0].data_ptr()], 1, count, out32, None)
    ctx.synchronize()
    assert torch.equal(out32, bufs[0])
    with pytest.raises(capi.PlbError):
        ctx.allreduce_f32_p2p(0, 1, [bufs[0].data_ptr()], [pads[0].data_ptr()], 0, count, out32, None)


def test_allreduce_reduce_scatter_form_on_one_gpu(gpu_ctx):
    """plb_allreduce_f32_p2p_rs with all "ranks'" buffers on this GPU and the
    peers' flags of both rounds already set.  Each emulated rank is run in turn:
    it must add its own slice in rank order and store it into every rank's
    result buffer; after all have run once, a second round must give every rank
    the complete sum (fp32 and cast).  Then a step whose peers never signal: the
    bounded wait runs out and is reported, the context stays usable."""
    import torch
    ctx = T.context()
    world, count = 3, 4 * 10007            # slices of unequal length
    words = capi.lib().plb_allreduce_p2p_signal_bytes(world) // 4
    g = torch.Generator().manual_seed(5)
    ins = [torch.randn(count, generator=g).cuda() for _ in range(world)]
    res = [torch.zeros(count, device="cuda") for _ in range(world)]
    pads = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(world)]
    want = (ins[0] + ins[1]) + ins[2]
    out32 = [torch.empty(count, device="cuda") for _ in range(world)]
    out16 = [torch.empty(count, device="cuda", dtype=torch.float16) for _ in range(world)]
    flag1, flag2 = 32, 48

    def run(rank, epoch, o32, o16):
        for peer in range(world):
            if peer != rank:
                pads[rank][flag1 + peer] = epoch
                pads[rank][flag2 + peer] = epoch
        torch.cuda.synchronize()
        ctx.allreduce_f32_p2p_rs(rank, world, [t.data_ptr() for t in ins], [t.data_ptr() for t in res],
                                 [p.data_ptr() for p in pads], epoch, count, o32, o16)
        ctx.synchronize()
    for rank in range(world):
        run(rank, 1, out32[rank], out16[rank])
    # every result buffer now holds every owner's slice
    for r in range(world):
        assert torch.equal(res[r], want), f"result buffer of rank {r}"
    assert torch.equal(out32[world - 1], want)      # the last one already saw all slices
    for rank in range(world):
        run(rank, 2, out32[rank], None if rank == 0 else out16[rank])
        assert torch.equal(out32[rank], want)
        if rank:
            assert torch.equal(out16[rank], want.half())
        for peer in range(world):
            if peer != rank:
                assert int(pads[peer][flag1 + rank]) == 2 and int(pads[peer][flag2 + rank]) == 2, "flag not sent"
    # epoch 3 on rank 1: nobody signals -> reported, not hung
    ctx.allreduce_f32_p2p_rs(1, world, [t.data_ptr() for t in ins], [t.data_ptr() for t in res],
                             [p.data_ptr() for p in pads], 3, count, out32[1], None)
    with pytest.raises(capi.PlbError):
        ctx.synchronize()
    # the context still works (a single rank is its own sum)
    solo_pad = torch.zeros(words, dtype=torch.int32, device="cuda")
    ctx.allreduce_f32_p2p_rs(0, 1, [ins[0].data_ptr()], [res[0].data_ptr()], [solo_pad.data_ptr()], 1, count,
                             out32[0], None)
    ctx.synchronize()
    assert torch.equal(out32[0], ins[0])


def test_weight_update_fused_with_sum_over_ranks_on_one_gpu(gpu_ctx):
    """plb_conv_wu_allreduce with the "peers'" gradient buffers on this GPU,
    already filled, and their chunk flags already set: the call must leave this
    rank's own gradient in its buffer, flag every chunk to every peer and
    return own + peers in rank order (fp32 and cast), for one and for several
    groups.  Then a step whose peers never signal: reported, not hung."""
    import torch
    ctx = T.context()
    world, rank = 3, 1
    r = T.rng(11)
    for kw in (conv_case(6, [12, 12], [3, 3], 64, 72, padding=1),
               conv_case(4, [10, 10], [3, 3], 16, 24, padding=1, groups=3)):
        p = capi.ConvParams.make(**kw)
        g = p.groups
        x = torch.from_numpy(T.binary_half(r, (p.batch, *kw["field"], g * p.in_chans_per_group))).cuda()
        dy = torch.from_numpy(T.binary_half(r, (p.batch, *kw["field"], g * p.out_chans_per_group))).cuda()
        shape = (g, 3, 3, p.out_chans_per_group, p.in_chans_per_group)
        count = int(np.prod(shape))
        local = torch.empty(shape, device="cuda")
        ctx.conv_wu(p, x, dy, None, local)
        ctx.synchronize()
        gen = torch.Generator().manual_seed(4)
        bufs = [torch.randint(-64, 64, (count,), generator=gen).float().cuda() for _ in range(world)]
        words = int(capi.lib().plb_conv_wu_allreduce_flag_bytes(p)) // 4
        assert words > 0
        flags = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(world)]
        flags[rank].fill_(1)                      # "all peers' chunks of step 1 have arrived"
        out32 = torch.empty(shape, device="cuda")
        out16 = torch.empty(shape, device="cuda", dtype=torch.float16)
        torch.cuda.synchronize()
        ctx.conv_wu_allreduce(p, x, dy, rank, world, [b.data_ptr() for b in bufs],
                              [f.data_ptr() for f in flags], 1, out16, out32)
        ctx.synchronize()
        assert torch.equal(bufs[rank].view(shape), local), "own gradient not left in the peer buffer"
        want = ((bufs[0] + bufs[1]) + bufs[2]).view(shape)
        assert torch.equal(out32, want)
        assert torch.equal(out16, want.half())
        chunks = words // 17          # a word per sender and chunk, then a word per chunk
        for peer in range(world):
            if peer != rank:
                sent = flags[peer][:chunks * 16].view(chunks, 16)[:, rank]
                assert bool((sent == 1).all()), "a chunk flag was not sent"
    # step 2: nobody signals -> the bounded wait runs out and is reported
    ctx.conv_wu_allreduce(p, x, dy, rank, world, [b.data_ptr() for b in bufs], [f.data_ptr() for f in flags],
                          2, None, out32)
    with pytest.raises(capi.PlbError):
        ctx.synchronize()
    # the context still works, and a single rank is its own sum
    ctx.conv_wu_allreduce(p, x, dy, 0, 1, [bufs[0].data_ptr()], [flags[0].data_ptr()], 1, None, out32)
    ctx.synchronize()
    assert torch.equal(out32, local)
    # layers that need a preparatory pass are refused with a pointer to the two-call form
    q = capi.ConvParams.make(**conv_case(2, [8, 8], [3, 3], 12, 20, padding=1))
    with pytest.raises(capi.PlbError):
        ctx.conv_wu_allreduce(q, x, dy, 0, 1, [bufs[0].data_ptr()], [flags[0].data_ptr()], 1, None, out32)


def test_small_channel_stem_layers(gpu_ctx):
    # 3-channel inputs go through the space-to-depth path
    for kw in (conv_case(2, [18, 22], [7, 7], 3, 64, padding=3, stride=2),
               conv_case(3, [9, 11], [3, 3], 3, 32, padding=1),
               conv_case(2, [12, 12], [5, 5], 4, 64, padding=2, stride=2),
               conv_case(1, [224, 224], [7, 7], 3, 64, padding=3, stride=2)):
        p = capi.ConvParams.make(**kw)
        spec = T.spec_from_params(p)
        r = T.rng(77)
        x, w, _ = conv_data(p, kw, r, exact=True)
        assert_exact(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), f"stem {kw} exact")
        x, w, _ = conv_data(p, kw, r, exact=False)
        assert_close(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), REL_HALF, f"stem {kw} uniform")


def test_config3a_stem_sampled_images(gpu_ctx):
    # 7x7 stride 2 pad 3, N=256 224x224x3 -> 64: full-size run, oracle on sampled images
    import torch
    kw = conv_case(256, [224, 224], [7, 7], 3, 64, padding=3, stride=2)
    p = capi.ConvParams.make(**kw)
    r = T.rng(1234 + 3)
    x, w, _ = conv_data(p, kw, r, exact=True)
    got = T.gpu_conv_fwd(p, x, w)
    pick = [0, 100, 255]
    p1 = capi.ConvParams.make(**{**kw, "batch": len(pick)})
    assert_exact(got[pick], oracle.conv_fwd(T.spec_from_params(p1), x[pick], w), "config 3a sampled images")
    # every image is an independent problem: a second image set equal to the
    # first must give identical outputs (no cross-image leakage through tiles)
    x[128:] = x[:128]
    got = T.gpu_conv_fwd(p, x, w)
    assert (got[128:] == got[:128]).all()
    del got
    # the same full-size layer on uniform data, the oracle on eight sampled images
    x, w, _ = conv_data(p, kw, r, exact=False)
    got = T.gpu_conv_fwd(p, x, w)
    pick = [0, 1, 37, 100, 127, 128, 200, 255]
    p8 = capi.ConvParams.make(**{**kw, "batch": len(pick)})
    assert_close(got[pick], oracle.conv_fwd(T.spec_from_params(p8), x[pick], w), REL_HALF,
                 "config 3a uniform, sampled images")
    del got
    torch.cuda.empty_cache()


def test_conv_float_output(gpu_ctx):
    kw = conv_case(2, [8, 8], [3, 3], 64, 64, padding=1)
    p = capi.ConvParams.make(output_type=capi.FLOAT, **kw)
    spec = T.spec_from_params(p)
    r = T.rng(21)
    x, w, _ = conv_data(p, kw, r, exact=False)
    got = T.gpu_conv_fwd(p, x, w)
    assert got.dtype == np.float32
    assert_close(got, oracle.conv_fwd(spec, x, w), 1e-4, "fwd fp32 out")


def test_conv_quarter_fwd_bwd(gpu_ctx):
    kw = conv_case(2, [8, 8], [3, 3], 128, 64, padding=1)
    p = capi.ConvParams.make(input_type=capi.QUARTER, **kw)
    spec = T.spec_from_params(p)
    r = T.rng(22)
    xv = r.integers(-2, 3, (2, 128, 8, 8)).astype(np.float64)
    wv = r.integers(-2, 3, (1, 64, 128, 3, 3)).astype(np.float64)
    got = T.gpu_conv_fwd(p, oracle.e4m3_encode(xv), oracle.e4m3_encode(wv))
    assert_exact(got, oracle.conv_fwd(spec, xv, wv), "quarter fwd")
    dyv = r.integers(-2, 3, (2, 64, 8, 8)).astype(np.float64)
    got = T.gpu_conv_bwd(p, oracle.e4m3_encode(dyv), oracle.e4m3_encode(wv))
    assert_exact(got, oracle.conv_bwd(spec, dyv, wv), "quarter bwd")


@pytest.mark.parametrize("name,kw", [
    ("3x3_s2", conv_case(2, [9, 10], [3, 3], 64, 32, padding=1, stride=2)),
    ("1x1_s2", conv_case(2, [8, 8], [1, 1], 32, 64, stride=2)),
    ("5x5_s2x3_groups", conv_case(2, [13, 11], [5, 5], 16, 32, padding=2, stride=[2, 3], groups=2)),
    ("3d_depth_s2", conv_case(2, [5, 6, 6], [3, 3, 3], 16, 16, padding=1, stride=[2, 1, 1])),
])
def test_conv_quarter_strided_and_3d(gpu_ctx, name, kw):
    """8-bit operands in the strided backward pass (sub-filters transposed per
    tap, there is no MN-major operand form for them) and in 3-D layers."""
    p = capi.ConvParams.make(input_type=capi.QUARTER, **kw)
    spec = T.spec_from_params(p)
    r = T.rng(zlib.crc32(name.encode()) % 1000 + 23)
    g = p.groups
    xv = r.integers(-2, 3, (p.batch, g * p.in_chans_per_group, *kw["field"])).astype(np.float64)
    wv = r.integers(-2, 3, (g, p.out_chans_per_group, p.in_chans_per_group, *kw["kernel"])).astype(np.float64)
    dyv = r.integers(-2, 3, (p.batch, g * p.out_chans_per_group, *p.output_field())).astype(np.float64)
    got = T.gpu_conv_fwd(p, oracle.e4m3_encode(xv), oracle.e4m3_encode(wv))
    assert_exact(got, oracle.conv_fwd(spec, xv, wv), f"quarter fwd {name}")
    got = T.gpu_conv_bwd(p, oracle.e4m3_encode(dyv), oracle.e4m3_encode(wv))
    assert_exact(got, oracle.conv_bwd(spec, dyv, wv), f"quarter bwd {name}")
    opt = capi.ConvOptions.make(scale_in=-2, scale_weights=1)
    got = T.gpu_conv_bwd(p, oracle.e4m3_encode(dyv), oracle.e4m3_encode(wv), opt=opt)
    assert_exact(got, oracle.conv_bwd(spec, dyv, wv) * 0.5, f"quarter bwd {name} scaled")


def test_conv_bwd_kernel_dilation_sharing_a_factor_with_the_stride(gpu_ctx):
    """dilation 2 / stride 2, 4 / 2, 2 / 4, 6 / 4: the taps that reach one
    phase are stride / gcd apart and some phases see no tap at all."""
    for i, (dil, stride, k) in enumerate(((2, 2, 3), (4, 2, 3), (2, 4, 4), (6, 4, 3), ([2, 3], [4, 3], 3))):
        dmax = max(dil) if isinstance(dil, list) else dil
        kw = conv_case(2, [19, 17], [k, k], 16, 24, padding=dmax, stride=stride, k_dilation=dil)
        p = capi.ConvParams.make(**kw)
        spec = T.spec_from_params(p)
        r = T.rng(700 + i)
        _, w, dy = conv_data(p, kw, r, exact=True)
        assert_exact(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), f"bwd dil {dil} stride {stride}")


def test_matmul_operands_beyond_4_gib(gpu_ctx):
    """Byte offsets past 2^32 in the left operand (69632 x 32768 half times
    32768 x 64) and element offsets past 2^31 in the output (69632 x 64 times
    64 x 32768, half out), checked on sampled rows including the last ones."""
    import torch
    free, _ = torch.cuda.mem_get_info()
    if free < 12 << 30:
        pytest.skip("needs 12 GiB of free device memory")
    g = torch.Generator(device="cuda").manual_seed(5)
    pm1 = lambda *shape: (torch.randint(0, 2, shape, generator=g, device="cuda", dtype=torch.int8) * 2 - 1).half()  # noqa: E731
    m = 69632
    rows = torch.as_tensor([0, 1, 127, 128, 32767, 65535, 65536, 65537, m - 129, m - 128, m - 2, m - 1], device="cuda")
    for k, n, out_type, dtype in ((32768, 64, capi.FLOAT, torch.float32), (64, 32768, capi.HALF, torch.float16)):
        a, b = pm1(m, k), pm1(k, n)
        out = torch.empty((m, n), device="cuda", dtype=dtype)
        desc = capi.MatmulDesc.make(m, k, n, output_type=out_type)
        torch.cuda.synchronize()
        gpu_ctx.matmul(desc, a, b, None, out)
        gpu_ctx.synchronize()
        torch.cuda.synchronize()
        expect = a[rows].cpu().numpy().astype(np.float64) @ b.cpu().numpy().astype(np.float64)
        assert_exact(out[rows].cpu().numpy(), expect, f"matmul {m}x{k}x{n} sampled rows")
        del a, b, out
        torch.cuda.empty_cache()


# BASELINE configurations at full size -------------------------------------------------

def test_config2_conv3x3_fwd(gpu_ctx):
    kw = conv_case(32, [56, 56], [3, 3], 64, 64, padding=1)
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(1234 + 2)
    x, w, _ = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), "config 2 exact")
    x, w, _ = conv_data(p, kw, r, exact=False)     # x ~ U[-1,1], w ~ U[-1/24, 1/24]
    assert_close(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), REL_HALF, "config 2 uniform")


def test_config3b_pointwise_stride2_fwd(gpu_ctx):
    kw = conv_case(256, [56, 56], [1, 1], 256, 512, stride=2)
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(1234 + 3)
    x, w, _ = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), "config 3b exact")
    # the distributions the configuration names: activations U[-1, 1], weights U[-1/16, 1/16]
    x, w, _ = conv_data(p, kw, r, exact=False)
    assert_close(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), REL_HALF, "config 3b uniform")


def test_config4_fwd_bwd_wu(gpu_ctx):
    kw = conv_case(256, [28, 28], [3, 3], 128, 128, padding=1)
    p = capi.ConvParams.make(**kw)
    spec = T.spec_from_params(p)
    r = T.rng(1234 + 4)
    x, w, dy = conv_data(p, kw, r, exact=True)
    assert_exact(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), "config 4 fwd exact")
    assert_exact(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), "config 4 bwd exact")
    _, dw32 = T.gpu_conv_wu(p, x, dy)
    assert_exact(dw32, oracle.conv_wu(spec, x, dy)[0], "config 4 wu exact (fp32 sums < 2^24)")
    x, w, dy = conv_data(p, kw, r, exact=False)
    assert_close(T.gpu_conv_fwd(p, x, w), oracle.conv_fwd(spec, x, w), REL_HALF, "config 4 fwd uniform")
    assert_close(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), REL_HALF, "config 4 bwd uniform")
    dw16, _ = T.gpu_conv_wu(p, x, dy)
    assert_close(dw16, oracle.conv_wu(spec, x, dy)[0], REL_HALF, "config 4 wu uniform")


# --------------------------------------------------------------------------- plumbing

def test_layout_kernels(gpu_ctx):
    import torch
    r = T.rng(31)
    x = r.integers(0, 60000, (3, 10, 7, 5)).astype(np.uint16)             # [N][C][H][W]
    dx, out = T.to_dev(x.view(np.float16)), T.empty_dev((3, 7, 5, 10), np.float16)
    torch.cuda.synchronize()
    gpu_ctx.acts_to_device(2, 3, 10, 35, dx, out)
    gpu_ctx.synchronize()
    assert (out.cpu().numpy().view(np.uint16) == T.acts_to_device_layout(x)).all()
    back = T.empty_dev((3, 10, 7, 5), np.float16)
    torch.cuda.synchronize()
    gpu_ctx.acts_from_device(2, 3, 10, 35, out, back)
    gpu_ctx.synchronize()
    assert (back.cpu().numpy().view(np.uint16) == x).all()
    w = r.integers(0, 250, (2, 6, 5, 3, 3)).astype(np.uint8)              # [G][Co][Ci][kh][kw]
    dw, wd = T.to_dev(w), T.empty_dev((2, 3, 3, 6, 5), np.uint8)
    torch.cuda.synchronize()
    gpu_ctx.weights_to_device(1, 2, 6, 5, 9, dw, wd)
    gpu_ctx.synchronize()
    assert (wd.cpu().numpy() == T.weights_to_device_layout(w)).all()
    # weightsTransposeChansFlipXY: [G][k][Co][Ci] -> [G][flipped k][Ci][Co]
    wt = T.empty_dev((2, 3, 3, 5, 6), np.uint8)
    torch.cuda.synchronize()
    gpu_ctx.weights_transpose_chans_flip_xy(1, 2, 6, 5, 9, wd, wt)
    gpu_ctx.synchronize()
    expect = np.transpose(T.weights_to_device_layout(w)[:, ::-1, ::-1], (0, 1, 2, 4, 3))
    assert (wt.cpu().numpy() == expect).all()


def test_host_buffer_entry_points(gpu_ctx):
    r = T.rng(32)
    a, b = T.small_int_half(r, (192, 128)), T.small_int_half(r, (128, 136), -3, 3)
    d = np.empty((192, 136), np.float16)
    gpu_ctx.matmul_host(capi.MatmulDesc.make(192, 128, 136), a, b, None, d)
    assert_exact(d, oracle.gemm(a, b), "matmul_host")
    kw = conv_case(2, [8, 8], [3, 3], 64, 64, padding=1)
    p = capi.ConvParams.make(**kw)
    x, w, _ = conv_data(p, kw, r, exact=True)
    y = np.empty((2, 8, 8, 64), np.float16)
    gpu_ctx.conv_fwd_host(p, T.acts_to_device_layout(x), T.weights_to_device_layout(w), y)
    assert_exact(T.acts_from_device_layout(y), oracle.conv_fwd(T.spec_from_params(p), x, w), "conv_fwd_host")


def test_scaled_add_and_cast(gpu_ctx):
    import torch
    r = T.rng(33)
    w = T.uniform_half(r, (1000,))
    d = r.uniform(-1, 1, 1000).astype(np.float32)
    dw, dd = T.to_dev(w), T.to_dev(d)
    torch.cuda.synchronize()
    gpu_ctx.scaled_add_to(capi.HALF, dw, dd, -0.05, 1000)
    gpu_ctx.synchronize()
    expect = (w.astype(np.float32) + np.float32(-0.05) * d).astype(np.float16)
    assert (dw.cpu().numpy() == expect).all()


def test_unsupported_requests_fail_loudly(gpu_ctx):
    # an element type the path does not implement: refused before anything is launched
    p = capi.ConvParams.make(1, [8, 8], [3, 3], 64, 64, input_type=7, output_type=capi.FLOAT)
    with pytest.raises(capi.PlbError) as e:
        gpu_ctx.conv_fwd(p, 0, 0, 0)
    assert e.value.code == 3
    # the weight update in quarter (the reference never runs it either)
    p = capi.ConvParams.make(1, [8, 8], [3, 3], 64, 64, input_type=capi.QUARTER, output_type=capi.HALF)
    with pytest.raises(capi.PlbError) as e:
        gpu_ctx.conv_wu(p, 0, 0, 0, 0)
    assert e.value.code == 3
    # null pointers for tensors that have elements: refused, whatever pre-pass the parameters need
    for kw in (dict(), dict(in_dilation=2), dict(in_flip=1)):
        p = capi.ConvParams.make(1, [8, 8], [3, 3], 64, 64, **kw)
        with pytest.raises(capi.PlbError) as e:
            gpu_ctx.conv_fwd(p, 0, 0, 0)
        assert e.value.code == 1 and "null device pointer" in e.value.message
        with pytest.raises(capi.PlbError):
            gpu_ctx.conv_bwd(p, 0, 0, 0)
        with pytest.raises(capi.PlbError):
            gpu_ctx.conv_wu(p, 0, 0, 0, 0)
    p3 = capi.ConvParams.make(1, [4, 8, 8], [3, 3, 3], 64, 64)
    with pytest.raises(capi.PlbError):
        gpu_ctx.conv_fwd(p3, 0, 0, 0)
    with pytest.raises(capi.PlbError):
        gpu_ctx.matmul(capi.MatmulDesc.make(64, 64, 64), 0, 0, None, 0)
    p = capi.ConvParams.make(1, [8, 8], [3, 3], 64, 64, stride=0)
    with pytest.raises(capi.PlbError) as e:
        gpu_ctx.conv_fwd(p, 0, 0, 0)
    assert e.value.code == 1 and e.value.message == "Stride must be non zero"
    assert gpu_ctx.launch_count() > 0


def test_weight_update_fused_with_owner_ranks_on_one_gpu(gpu_ctx):
    """plb_conv_wu_allreduce_owners with every "rank's" buffers on this GPU and
    all flags already set.  For the chunks it owns (chunk index mod world) the
    emulated rank must add the peers' gradients to its own in rank order, leave
    the sum in its result buffer and flag it to every peer; the other chunks it
    must fetch from their owner's result buffer after flagging its own chunk to
    that owner only.  Then a step whose peers never signal: reported, not hung."""
    import torch
    ctx = T.context()
    world = 3
    r = T.rng(12)
    for kw in (conv_case(6, [12, 12], [3, 3], 64, 72, padding=1),
               conv_case(4, [10, 10], [3, 3], 16, 24, padding=1, groups=3)):
        p = capi.ConvParams.make(**kw)
        g = p.groups
        x = torch.from_numpy(T.binary_half(r, (p.batch, *kw["field"], g * p.in_chans_per_group))).cuda()
        dy = torch.from_numpy(T.binary_half(r, (p.batch, *kw["field"], g * p.out_chans_per_group))).cuda()
        shape = (g, 3, 3, p.out_chans_per_group, p.in_chans_per_group)
        count = int(np.prod(shape))
        per_group = count // g
        local = torch.empty(shape, device="cuda")
        ctx.conv_wu(p, x, dy, None, local)
        ctx.synchronize()
        words = int(capi.lib().plb_conv_wu_allreduce_flag_bytes(p)) // 4
        chunks = words // 17
        per_group_chunks = chunks // g
        # owner of every element: chunk = group * chunks per group + (offset in the group) // 512 floats
        idx = torch.arange(count, device="cuda")
        chunk_of = (idx // per_group) * per_group_chunks + (idx % per_group) // 512
        owner_of = chunk_of % world
        gen = torch.Generator().manual_seed(6)
        for rank in range(world):
            bufs = [torch.randint(-64, 64, (count,), generator=gen).float().cuda() for _ in range(world)]
            res = [torch.randint(-999, 999, (count,), generator=gen).float().cuda() for _ in range(world)]
            fetched = [t.clone() for t in res]
            flags = [torch.zeros(words, dtype=torch.int32, device="cuda") for _ in range(world)]
            flags[rank].fill_(1)                      # every flag this rank waits for has "arrived"
            out32 = torch.empty(shape, device="cuda")
            out16 = torch.empty(shape, device="cuda", dtype=torch.float16)
            torch.cuda.synchronize()
            ctx.conv_wu_allreduce(p, x, dy, rank, world, [b.data_ptr() for b in bufs],
                                  [f.data_ptr() for f in flags], 1, out16, out32,
                                  result_ptrs=[t.data_ptr() for t in res])
            ctx.synchronize()
            assert torch.equal(bufs[rank].view(shape), local), "own gradient not left in the peer buffer"
            summed = ((bufs[0] + bufs[1]) + bufs[2])
            mine = owner_of == rank
            want = summed.clone()
            for o in range(world):
                if o != rank:
                    want[owner_of == o] = fetched[o][owner_of == o]
            assert torch.equal(out32.view(-1), want), f"rank {rank}: fp32 result"
            assert torch.equal(out16.view(-1), want.half()), f"rank {rank}: cast result"
            assert torch.equal(res[rank][mine], summed[mine]), "owned sums not left in the result buffer"
            for o in range(world):
                if o != rank:
                    assert torch.equal(res[o], fetched[o]), "a peer's result buffer was written"
            owners = torch.arange(chunks, device="cuda") % world
            for peer in range(world):
                if peer == rank:
                    continue
                sent = flags[peer][:chunks * 16].view(chunks, 16)[:, rank]
                assert torch.equal(sent == 1, owners == peer), "chunk flags go to the chunk's owner only"
                ready = flags[peer][chunks * 16:chunks * 17]
                assert torch.equal(ready == 1, owners == rank), "result flags of the owned chunks only"
    # step 2 on the last rank: nobody signals -> the bounded wait runs out and is reported
    ctx.conv_wu_allreduce(p, x, dy, rank, world, [b.data_ptr() for b in bufs], [f.data_ptr() for f in flags],
                          2, None, out32, result_ptrs=[t.data_ptr() for t in res])
    with pytest.raises(capi.PlbError):
        ctx.synchronize()
    ctx.conv_wu(p, x, dy, None, local)      # the context still works
    ctx.synchronize()
