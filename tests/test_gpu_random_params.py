"""Seeded random ConvParams against the oracle, all three passes.

The role of the reference's random-parameter runs
(tools/single_conv_layer_random.py:22-50, tests/poplin/CMakeLists.txt:1040-1065):
every transform of ConvParams is drawn at random -- input truncation, padding
and flip, kernel truncation, dilation, padding and flip, stride, output
truncation and padding, groups, 1-D, 2-D and 3-D fields, and (in runs of its
own: it costs a zero-stuffed copy of the input, or is part of the depth gather
of a 3-D field) input dilation -- and the result must match the oracle bit for
bit on +-1 data (all sums stay below 2048, exact in half).  A drawn combination
that is not a valid convolution (empty output) is redrawn.
"""
import numpy as np
import pytest

import common as T
import oracle
from poplibs_b200 import capi

pytestmark = pytest.mark.gpu


def draw(seed, dims=None, dilate_input=False):
    r = np.random.default_rng(1000 + seed + (50000 if dims else 0) + (90000 if dilate_input else 0))
    for _ in range(200):
        nd = dims or int(r.integers(1, 3))
        vec = lambda lo, hi: [int(v) for v in r.integers(lo, hi + 1, nd)]  # noqa: E731
        kw = dict(
            batch=int(r.integers(1, 5)), field=vec(3, 8) if nd == 3 else vec(5, 14),
            kernel=vec(1, 3) if nd == 3 else vec(1, 5),
            in_chans=int(r.choice([8, 16, 24, 40, 64])), out_chans=int(r.choice([8, 16, 24, 40, 72])),
            groups=int(r.choice([1, 1, 2])),
            in_trunc_lo=vec(0, 2), in_trunc_hi=vec(0, 2), in_pad_lo=vec(0, 3), in_pad_hi=vec(0, 3),
            k_trunc_lo=vec(0, 1), k_trunc_hi=vec(0, 1), k_dilation=vec(1, 3), k_pad_lo=vec(0, 2),
            k_pad_hi=vec(0, 2), k_flip=vec(0, 1), in_flip=vec(0, 1), stride=vec(1, 3), out_trunc_lo=vec(0, 2),
            out_trunc_hi=vec(0, 2), out_pad_lo=vec(0, 2), out_pad_hi=vec(0, 2))
        if nd == 3:
            kw["in_dilation"] = [int(r.integers(1, 3)), 1, 1]
        elif dilate_input:
            kw["in_dilation"] = vec(1, 3)
        # keep the draw simple half of the time: most layers use few transforms
        if r.random() < 0.5:
            for name in ("in_flip", "in_trunc_lo", "in_trunc_hi", "k_trunc_lo", "k_trunc_hi", "k_pad_lo", "k_pad_hi",
                         "out_trunc_lo", "out_trunc_hi", "out_pad_lo", "out_pad_hi"):
                if r.random() < 0.7:
                    kw[name] = [0] * nd
        if any(kw["kernel"][d] - kw["k_trunc_lo"][d] - kw["k_trunc_hi"][d] < 1 for d in range(nd)):
            continue
        if any(kw["field"][d] - kw["in_trunc_lo"][d] - kw["in_trunc_hi"][d] < 1 for d in range(nd)):
            continue
        p = capi.ConvParams.make(**kw)
        try:
            of = p.output_field()
        except capi.PlbError:
            continue
        # a computed (not padded) output must exist
        if any(of[d] - kw["out_pad_lo"][d] - kw["out_pad_hi"][d] < 1 for d in range(nd)):
            continue
        taps = int(np.prod([kw["kernel"][d] for d in range(nd)]))
        if taps * kw["in_chans"] > 2000 or taps * kw["out_chans"] > 2000:
            continue  # sums must stay exactly representable in half
        return kw, p
    raise RuntimeError("no valid parameters drawn")


def data(kw, p, r, dtype=np.float16):
    g = p.groups
    x = T.binary_half(r, (p.batch, g * p.in_chans_per_group, *kw["field"])).astype(dtype)
    w = T.binary_half(r, (g, p.out_chans_per_group, p.in_chans_per_group, *kw["kernel"])).astype(dtype)
    dy = T.binary_half(r, (p.batch, g * p.out_chans_per_group, *p.output_field())).astype(dtype)
    return x, w, dy


def check_all_passes(seed, kw, p):
    spec = T.spec_from_params(p)
    r = T.rng(seed)
    x, w, dy = data(kw, p, r, np.float32 if p.input_type == capi.FLOAT else np.float16)
    what = f"seed {seed}: {kw}"
    got = T.gpu_conv_fwd(p, x, w)
    assert np.array_equal(got.astype(np.float64), oracle.conv_fwd(spec, x, w).reshape(got.shape)), "fwd " + what
    got = T.gpu_conv_bwd(p, dy, w)
    assert np.array_equal(got.astype(np.float64), oracle.conv_bwd(spec, dy, w).reshape(got.shape)), "bwd " + what
    if all(s <= 8 for s in kw["stride"]):
        _, dw32 = T.gpu_conv_wu(p, x, dy)
        assert np.array_equal(dw32.astype(np.float64), oracle.conv_wu(spec, x, dy)[0].reshape(dw32.shape)), "wu " + what


@pytest.mark.parametrize("seed", range(120))
def test_random_conv_params(gpu_ctx, seed):
    kw, p = draw(seed)
    check_all_passes(seed, kw, p)


@pytest.mark.parametrize("seed", range(40))
def test_random_conv_params_3d(gpu_ctx, seed):
    kw, p = draw(seed, dims=3)
    check_all_passes(seed, kw, p)


@pytest.mark.parametrize("seed", range(40))
def test_random_conv_params_dilated_input(gpu_ctx, seed):
    kw, p = draw(seed, dilate_input=True)
    check_all_passes(seed, kw, p)


@pytest.mark.parametrize("seed", range(40))
def test_random_conv_params_float(gpu_ctx, seed):
    """The same draws with float data (three bfloat16 terms per product): +-1 data
    are exact in bfloat16, so the oracle's bits are expected here too."""
    kw, _ = draw(seed, dims=3 if seed % 4 == 3 else None, dilate_input=seed % 4 == 2)
    p = capi.ConvParams.make(**kw, input_type=capi.FLOAT, output_type=capi.FLOAT)
    check_all_passes(seed, kw, p)
