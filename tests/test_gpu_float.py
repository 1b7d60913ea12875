"""Float operands (poplar::FLOAT data: lib/poplin/ConvValidation.cpp:11-70 accepts
them, and the reference's tools run "--data-type float").  On this target a
float contraction runs as three bfloat16 terms per product with fp32
accumulation, so a product carries a relative error of about 2^-16.

Tolerances.  Small-integer data (exact in bfloat16, sums exact in fp32) must
match the oracle BIT FOR BIT.  Uniform data are held to
poplibs_test::checkIsClose with the reference's float tolerance for the tools
(relative 1e-3... here tightened to 1e-4, absolute max(1e-5, 2.5e-5 * rms)):
ten times tighter than the half path in both terms.
"""
import zlib

import numpy as np
import pytest

import common as T
import oracle
from poplibs_b200 import capi

pytestmark = pytest.mark.gpu

REL_FLOAT = 1e-4


def assert_close(got, exp, what):
    got = np.asarray(got, dtype=np.float64)
    exp = np.asarray(exp, dtype=np.float64).reshape(got.shape)
    rms = float(np.sqrt(np.mean(exp * exp))) if exp.size else 0.0
    abs_tol = max(T.ABS_TOL, 2.5e-5 * rms)
    bad, first, worst = oracle.check_is_close(got, exp, REL_FLOAT, abs_tol)
    assert bad == 0, (f"{what}: {bad}/{got.size} elements outside rel={REL_FLOAT} abs={abs_tol:.2e}; "
                      f"first at {np.unravel_index(first, got.shape)} got {got.ravel()[first]} "
                      f"expected {exp.ravel()[first]}")


def assert_exact(got, exp, what):
    got = np.asarray(got, dtype=np.float64)
    exp = np.asarray(exp, dtype=np.float64).reshape(got.shape)
    diff = got != exp
    assert not diff.any(), f"{what}: {int(diff.sum())}/{got.size} elements differ; first at {np.argwhere(diff)[0]}"


def ints(r, shape, lo=-4, hi=4):
    return r.integers(lo, hi + 1, size=shape).astype(np.float32)


def uniform(r, shape, lo=-1.0, hi=1.0):
    return r.uniform(lo, hi, size=shape).astype(np.float32)


@pytest.mark.parametrize("m,k,n", [(128, 64, 64), (1, 8, 1), (1, 1000, 1), (5, 8, 4), (300, 200, 72),
                                   (129, 72, 257), (640, 320, 520)])
@pytest.mark.parametrize("tb", [False, True])
def test_float_matmul_exact(gpu_ctx, m, k, n, tb):
    r = T.rng(m * 7 + k * 3 + n)
    a = ints(r, (m, k))
    b = ints(r, (n, k) if tb else (k, n), -3, 3)
    got = T.gpu_matmul(a, b, transpose_b=tb, out_dtype=np.float32)
    assert_exact(got, oracle.gemm(a, b, transpose_b=tb), f"float matMul {m}x{k}x{n} tb={tb}")


def test_float_matmul_transposes_groups_alpha_beta(gpu_ctx):
    r = T.rng(11)
    g, m, k, n = 3, 72, 136, 88
    for ta in (False, True):
        for tb in (False, True):
            a = ints(r, (g, k, m) if ta else (g, m, k))
            b = ints(r, (g, n, k) if tb else (g, k, n), -3, 3)
            c = ints(r, (g, m, n), -2, 2)
            got = T.gpu_matmul(a, b, c, transpose_a=ta, transpose_b=tb, alpha=2.0, beta=-1.0,
                               out_dtype=np.float32)
            assert_exact(got, oracle.gemm(a, b, c, 2.0, -1.0, ta, tb), f"float grouped ta={ta} tb={tb}")


def test_float_matmul_uniform(gpu_ctx):
    # the gemm tool's data ranges; values with full 24-bit significands
    r = T.rng(77)
    a, b = uniform(r, (512, 1024), -4, 4), uniform(r, (1024, 768), -3, 3)
    got = T.gpu_matmul(a, b, out_dtype=np.float32)
    exp = oracle.gemm(a, b)
    assert_close(got, exp, "float matMul 512x1024x768")
    # worst element against the typical magnitude: far inside the half path's tolerance
    rms = float(np.sqrt(np.mean(exp * exp)))
    assert float(np.abs(got - exp).max()) < 1e-4 * rms
    # values spread over many binades keep their relative accuracy (bfloat16 has float's range)
    a = (uniform(r, (64, 256)) * np.exp2(r.integers(-40, 40, size=(64, 1)))).astype(np.float32)
    b = uniform(r, (256, 64))
    got = T.gpu_matmul(a, b, out_dtype=np.float32)
    exp = oracle.gemm(a, b)
    row_rms = np.sqrt(np.mean(exp * exp, axis=1, keepdims=True))
    assert float((np.abs(got - exp) / row_rms).max()) < 1e-4


def test_float_matmul_empty_and_special(gpu_ctx):
    r = T.rng(12)
    c = ints(r, (5, 4))
    got = T.gpu_matmul(np.zeros((5, 0), np.float32), np.zeros((4, 0), np.float32), c, transpose_b=True,
                       beta=1.0, out_dtype=np.float32)
    assert_exact(got, c, "float 5x0x4")
    # an infinity stays an infinity and does not turn the rest of its row into NaN
    a = ints(r, (8, 16))
    b = ints(r, (16, 8), 1, 3)
    a[2, 5] = np.inf
    got = T.gpu_matmul(a, b, out_dtype=np.float32)
    assert np.isinf(got[2]).all() and np.isfinite(np.delete(got, 2, axis=0)).all()


def conv_case(batch, field, kernel, ci, co, **kw):
    return dict(batch=batch, field=field, kernel=kernel, in_chans=ci, out_chans=co, **kw)


FLOAT_CONVS = {
    "3x3_pad1": conv_case(2, [8, 8], [3, 3], 64, 64, padding=1),
    "ragged_chans": conv_case(3, [7, 9], [3, 3], 20, 12, padding=1),
    "stem_like": conv_case(2, [20, 20], [7, 7], 3, 16, padding=3, stride=2),
    "groups2": conv_case(2, [6, 6], [3, 3], 16, 24, padding=1, groups=2),
    "3x3_s2": conv_case(2, [9, 9], [3, 3], 32, 40, padding=1, stride=2),
    "kernel_dilation": conv_case(2, [12, 12], [3, 3], 16, 16, padding=2, k_dilation=2),
    "one_dim": conv_case(4, [33], [5], 24, 32, padding=2),
    "three_dim": conv_case(2, [5, 6, 7], [3, 3, 3], 8, 16, padding=1),
    "in_dilation": conv_case(2, [6, 6], [3, 3], 16, 16, padding=2, in_dilation=2),
    "out_pad_trunc": conv_case(2, [10, 9], [3, 3], 16, 24, padding=2, out_trunc_lo=[1, 0],
                               out_pad_hi=[0, 2]),
}


def conv_data(p, kw, r, exact):
    g = p.groups
    gen = (lambda shape: ints(r, shape, -2, 2)) if exact else (lambda shape: uniform(r, shape))
    x = gen((p.batch, g * p.in_chans_per_group, *kw["field"]))
    w = gen((g, p.out_chans_per_group, p.in_chans_per_group, *kw["kernel"]))
    if not exact:
        w = (w / np.sqrt(p.in_chans_per_group * int(np.prod(kw["kernel"])))).astype(np.float32)
    dy = gen((p.batch, g * p.out_chans_per_group, *p.output_field()))
    return x, w, dy


@pytest.mark.parametrize("name", sorted(FLOAT_CONVS))
def test_float_conv_all_passes(gpu_ctx, name):
    kw = FLOAT_CONVS[name]
    p = capi.ConvParams.make(**kw, input_type=capi.FLOAT, output_type=capi.FLOAT)
    spec = T.spec_from_params(p)
    r = T.rng(zlib.crc32(name.encode()) % 1000)
    for exact in (True, False):
        check = assert_exact if exact else assert_close
        x, w, dy = conv_data(p, kw, r, exact)
        bias = None if exact else r.uniform(-2, 6, p.groups * p.out_chans_per_group).astype(np.float32)
        got = T.gpu_conv_fwd(p, x, w, bias=bias)
        assert got.dtype == np.float32
        check(got, oracle.conv_fwd(spec, x, w, bias), f"float fwd {name} exact={exact}")
        check(T.gpu_conv_bwd(p, dy, w), oracle.conv_bwd(spec, dy, w), f"float bwd {name} exact={exact}")
        dw, dw32 = T.gpu_conv_wu(p, x, dy)
        exp, _ = oracle.conv_wu(spec, x, dy)
        check(dw32, exp, f"float wu {name} exact={exact} (fp32 result)")
        check(dw, exp, f"float wu {name} exact={exact} (result in the input type)")


def test_float_conv_half_output_and_plan(gpu_ctx):
    kw = FLOAT_CONVS["3x3_pad1"]
    p = capi.ConvParams.make(**kw, input_type=capi.FLOAT, output_type=capi.HALF)
    spec = T.spec_from_params(p)
    r = T.rng(5)
    x, w, _ = conv_data(p, kw, r, exact=True)
    got = T.gpu_conv_fwd(p, x, w)
    assert got.dtype == np.float16
    assert_exact(got, oracle.conv_fwd(spec, x, w), "float in, half out")
    # the plan describes what runs: the same FLOPs, a reduction three times as long
    plan = capi.conv_plan(p, pass_=capi.PASS_TRAINING_FWD)
    half = capi.conv_plan(capi.ConvParams.make(**kw), pass_=capi.PASS_TRAINING_FWD)
    assert plan.flops == half.flops and plan.workspace_bytes > half.workspace_bytes


def test_bfloat16_operands(gpu_ctx):
    """The operand type the float route runs in is accepted in its own right."""
    import torch
    r = T.rng(9)
    m, k, n = 96, 128, 72
    a, b = ints(r, (m, k)), ints(r, (k, n), -3, 3)
    desc = capi.MatmulDesc.make(m, k, n, input_type=capi.BFLOAT16, output_type=capi.FLOAT)
    da = torch.from_numpy(a).cuda().to(torch.bfloat16)
    db = torch.from_numpy(b).cuda().to(torch.bfloat16)
    dd = torch.empty((m, n), dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    ctx = T.context()
    ctx.matmul(desc, da, db, None, dd)
    ctx.synchronize()
    assert_exact(dd.cpu().numpy(), oracle.gemm(a, b), "bfloat16 matMul")
