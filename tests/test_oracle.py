"""The CPU oracle (oracle/poplin_oracle.c) against (1) golden vectors produced
by the reference's own models, (2) those models themselves when the build of
them is present, (3) the known-answer tables of the reference's unit tests."""
import json
import os

import numpy as np
import pytest

import oracle
from oracle import ConvSpec

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = np.load(os.path.join(HERE, "golden", "poplibs_test_models.npz"))
META = json.load(open(os.path.join(HERE, "golden", "poplibs_test_models.json")))

CONV_NAMES = sorted(k.split("/", 1)[1] for k in META if k.startswith("conv/"))
GEMM_NAMES = sorted(k.split("/", 1)[1] for k in META if k.startswith("gemm/"))


def spec_of(meta):
    m = dict(meta)
    out_field = m.pop("out_field")
    spec = ConvSpec(m.pop("batch"), m.pop("field"), m.pop("kernel"), m.pop("in_chans"),
                    m.pop("out_chans"), m.pop("groups"), **m)
    assert spec.out_field() == out_field
    return spec


@pytest.mark.parametrize("name", CONV_NAMES)
def test_conv_against_golden(name):
    spec = spec_of(META[f"conv/{name}"])
    g = lambda k: GOLD[f"conv/{name}/{k}"]  # noqa: E731
    np.testing.assert_allclose(oracle.conv_fwd(spec, g("x"), g("w"), g("bias")), g("y"),
                               rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(oracle.conv_bwd(spec, g("dy"), g("w")), g("dx"),
                               rtol=1e-12, atol=1e-12)
    if f"conv/{name}/dw" in GOLD:
        dw, db = oracle.conv_wu(spec, g("x"), g("dy"))
        np.testing.assert_allclose(dw, g("dw"), rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(db, g("db"), rtol=1e-12, atol=1e-12)


@pytest.mark.parametrize("name", GEMM_NAMES)
def test_gemm_against_golden(name):
    m = META[f"gemm/{name}"]
    g = lambda k: GOLD[f"gemm/{name}/{k}"]  # noqa: E731
    d = oracle.gemm(g("a"), g("b"), g("c"), m["alpha"], m["beta"], m["transpose_a"], m["transpose_b"])
    np.testing.assert_allclose(d, g("d"), rtol=1e-12, atol=1e-12)


def random_spec(r):
    """A random valid ConvParams in the spirit of the reference's generator
    (tools/single_conv_layer_random.py:22-50), small enough for its model."""
    nd = int(r.integers(1, 4))
    while True:
        kw = dict(
            field=r.integers(1, 7, nd).tolist(), kernel=r.integers(1, 4, nd).tolist(),
            in_trunc_lo=r.integers(0, 2, nd).tolist(), in_trunc_hi=r.integers(0, 2, nd).tolist(),
            in_dilation=r.integers(1, 3, nd).tolist(), in_pad_lo=r.integers(0, 3, nd).tolist(),
            in_pad_hi=r.integers(0, 3, nd).tolist(), in_flip=r.integers(0, 2, nd).tolist(),
            k_trunc_lo=r.integers(0, 2, nd).tolist(), k_trunc_hi=r.integers(0, 2, nd).tolist(),
            k_dilation=r.integers(1, 3, nd).tolist(), k_pad_lo=r.integers(0, 2, nd).tolist(),
            k_pad_hi=r.integers(0, 2, nd).tolist(), k_flip=r.integers(0, 2, nd).tolist(),
            out_trunc_lo=r.integers(0, 2, nd).tolist(), out_trunc_hi=r.integers(0, 2, nd).tolist(),
            stride=r.integers(1, 4, nd).tolist(), out_pad_lo=r.integers(0, 2, nd).tolist(),
            out_pad_hi=r.integers(0, 2, nd).tolist())
        spec = ConvSpec(int(r.integers(1, 3)), in_chans=int(r.integers(1, 4)),
                        out_chans=int(r.integers(1, 4)), groups=int(r.integers(1, 3)), **kw)
        try:
            if min(spec.out_field()) >= 1:
                return spec
        except ValueError:
            pass


@pytest.mark.skipif(not oracle.have_ref(), reason="build of the reference's models not present")
def test_restatement_against_reference_models_randomised():
    r = np.random.default_rng(42)
    for _ in range(60):
        spec = random_spec(r)
        xs, ws, ys = oracle._shapes(spec)
        x, w, b, dy = r.uniform(-2, 2, xs), r.uniform(-1, 1, ws), r.uniform(-2, 6, ys[1]), r.uniform(-3, 3, ys)
        np.testing.assert_allclose(oracle.conv_fwd(spec, x, w, b), oracle.conv_fwd(spec, x, w, b, use_ref=True),
                                   rtol=1e-12, atol=1e-12, err_msg=str(spec))
        np.testing.assert_allclose(oracle.conv_bwd(spec, dy, w), oracle.conv_bwd(spec, dy, w, use_ref=True),
                                   rtol=1e-12, atol=1e-12, err_msg=str(spec))
        n = spec.normalised()
        if all(s == 1 or (lo == 0 and hi == 0)
               for s, lo, hi in zip(n["stride"], n["out_trunc_lo"], n["out_trunc_hi"])):
            a, c = oracle.conv_wu(spec, x, dy), oracle.conv_wu(spec, x, dy, use_ref=True)
            np.testing.assert_allclose(a[0], c[0], rtol=1e-12, atol=1e-12, err_msg=str(spec))
            np.testing.assert_allclose(a[1], c[1], rtol=1e-12, atol=1e-12)


@pytest.mark.skipif(not oracle.have_ref(), reason="build of the reference's models not present")
def test_gemm_against_reference_model():
    r = np.random.default_rng(7)
    for ta in (False, True):
        for tb in (False, True):
            g, m, k, n = 2, 7, 9, 5
            a = r.uniform(-4, 4, (g, k, m) if ta else (g, m, k))
            b = r.uniform(-3, 3, (g, n, k) if tb else (g, k, n))
            c = r.uniform(-2, 2, (g, m, n))
            np.testing.assert_allclose(oracle.gemm(a, b, c, 1.5, -0.5, ta, tb),
                                       oracle.gemm(a, b, c, 1.5, -0.5, ta, tb, use_ref=True),
                                       rtol=1e-13, atol=1e-13)


# tests/poplin/RangeTest.cpp:33-122 -- getInputIndex(dim, out, kernel, params)
# for a 10-wide input and a 3-wide kernel: (stride, padLo, padHi) -> [(out, k, expected)]
NONE = -1
RANGE_TABLE = {
    (1, 0, 0): [(0, 0, 0), (1, 0, 1), (0, 1, 1), (7, 2, 9)],
    (2, 0, 0): [(1, 0, 2), (3, 2, 8)],
    (1, 1, 0): [(0, 0, NONE), (0, 1, 0), (0, 2, 1), (8, 1, 8), (8, 2, 9)],
    (1, 2, 0): [(0, 0, NONE), (0, 1, NONE), (0, 2, 0), (9, 1, 8), (9, 2, 9)],
    (2, 1, 0): [(0, 0, NONE), (0, 1, 0), (0, 2, 1), (4, 1, 8), (4, 2, 9)],
    (2, 2, 0): [(0, 0, NONE), (0, 1, NONE), (0, 2, 0), (4, 1, 7), (4, 2, 8)],
    (2, 4, 0): [(0, 0, NONE), (0, 1, NONE), (0, 2, NONE), (1, 0, NONE), (1, 1, NONE), (1, 2, 0),
                (5, 1, 7), (5, 2, 8)],
    (1, 1, 1): [(0, 0, NONE), (0, 1, 0), (0, 2, 1), (9, 1, 9), (9, 2, NONE)],
    (2, 1, 2): [(0, 0, NONE), (0, 1, 0), (0, 2, 1), (4, 1, 8), (4, 2, 9), (5, 0, 9), (5, 1, NONE),
                (5, 2, NONE)],
    (3, 2, 2): [(0, 0, NONE), (0, 1, NONE), (0, 2, 0), (3, 1, 8), (3, 2, 9)],
}


def test_input_index_known_answers():
    import ctypes as C
    lib = oracle._lib()
    for (stride, lo, hi), rows in RANGE_TABLE.items():
        spec = ConvSpec(1, [10, 10], [3, 3], 1, 1, in_pad_lo=[lo, lo], in_pad_hi=[hi, hi],
                        stride=[stride, stride])
        p = spec.to_c()
        for out, k, expected in rows:
            assert lib.oracle_conv_input_index(C.byref(p), 0, out, k) == expected, (stride, lo, hi, out, k)


# tests/poplin/RangeTest.cpp:146-168 -- getOutputSize
OUTPUT_DIM_TABLE = [
    ((10, 10), (3, 3), (1, 1), (0, 0), (0, 0), (8, 8)),
    ((10, 10), (2, 2), (1, 1), (0, 0), (0, 0), (9, 9)),
    ((10, 10), (3, 3), (1, 1), (1, 1), (0, 0), (9, 9)),
    ((10, 10), (3, 3), (1, 1), (0, 0), (2, 2), (10, 10)),
    ((10, 10), (3, 3), (1, 1), (3, 3), (2, 2), (13, 13)),
    ((10, 10), (3, 3), (2, 2), (3, 3), (2, 2), (7, 7)),
    ((10, 10), (3, 3), (1, 2), (3, 3), (2, 2), (13, 7)),
    ((10, 12), (3, 5), (1, 1), (0, 1), (0, 2), (8, 11)),
    ((4, 4), (3, 3), (2, 1), (0, 0), (1, 0), (2, 2)),
    ((4, 4), (3, 3), (3, 3), (0, 1), (1, 0), (1, 1)),
]


def test_output_size_known_answers():
    for field, kernel, stride, lo, hi, expected in OUTPUT_DIM_TABLE:
        spec = ConvSpec(1, list(field), list(kernel), 1, 1, in_pad_lo=list(lo), in_pad_hi=list(hi),
                        stride=list(stride))
        assert tuple(spec.out_field()) == expected


def test_macs_exclude_padding():
    # per-dimension counts 166 / 778 / 82 / 28 of the benchmark layers
    assert ConvSpec.simple(1, [56], [3], 1, 1, padding=1).macs() == 166
    assert ConvSpec.simple(1, [224], [7], 1, 1, padding=3, stride=2).macs() == 778
    assert ConvSpec.simple(1, [28], [3], 1, 1, padding=1).macs() == 82
    assert ConvSpec.simple(1, [56], [1], 1, 1, stride=2).macs() == 28
    assert 2 * ConvSpec.simple(32, [56, 56], [3, 3], 64, 64, padding=1).macs() == 7223640064


def test_check_is_close_rule():
    # lib/poplibs_test/Util.cpp:198-217, 316-348
    assert oracle.is_close(1.0, 1.0, 0.0, 0.0)
    assert oracle.is_close(float("nan"), float("nan"), 1e-3)
    assert not oracle.is_close(float("nan"), 1.0, 1e-3)
    assert oracle.is_close(5e-4, -5e-4, 1e-3, 0.0)          # both "small"
    assert oracle.is_close(1.0, 1.0009, 1e-3, 0.0)
    assert not oracle.is_close(1.0, 1.0011, 1e-3, 0.0)
    assert not oracle.is_close(0.0, 2e-3, 1e-3, 0.0)        # strong check: relative to both
    assert oracle.is_close(0.0, 2e-3, 1e-3, 3e-3)           # absolute tolerance rescues
    bad, first, mx = oracle.check_is_close([1.0, 2.0, 3.0], [1.0, 2.5, 3.0], 1e-3, 1e-5)
    assert (bad, first) == (1, 1) and abs(mx - 0.2) < 1e-12


def test_number_formats():
    x = np.array([0.1, -1000.123, 65504.0, 1e-8, 3.0e-5])
    np.testing.assert_array_equal(oracle.round_to_half(x),
                                  [oracle._lib().oracle_round_to_half(float(v)) for v in x])
    codes = np.arange(256, dtype=np.uint8)
    vals = oracle.e4m3_decode(codes)
    assert vals[0x7E] == 448.0 and np.isnan(vals[0x7F]) and vals[0x38] == 1.0 and vals[0x01] == 2.0 ** -9
    finite = ~np.isnan(vals)
    np.testing.assert_array_equal(oracle.e4m3_encode(vals[finite]) & 0x7F, codes[finite] & 0x7F)
    assert oracle.e4m3_encode(np.array([1e6]))[0] == 0x7E      # saturates
    assert oracle.e4m3_encode(np.array([17.0]))[0] == oracle.e4m3_encode(np.array([16.0]))[0]  # tie to even
    r = np.random.default_rng(0)
    v = r.normal(size=20000) * 8
    assert (oracle._e4m3_encode_np(v) ==
            np.array([oracle._lib().oracle_e4m3_from_double(float(t)) for t in v], dtype=np.uint8)).all()


@pytest.mark.parametrize("name", sorted(k[len("norm/"):] for k in META if k.startswith("norm/")))
def test_norm_against_golden(name):
    """The C restatement of the batch-norm models against vectors produced by
    the reference's own lib/poplibs_test/Norms.cpp."""
    m = META[f"norm/{name}"]
    g = lambda k: GOLD[f"norm/{name}/{k}"]   # noqa: E731
    mean, inv = oracle.norm_statistics(g("x"), m["eps"], m["unbiased"], m["stable"])
    assert np.array_equal(mean, g("mean")) and np.array_equal(inv, g("inv_std"))
    y, white = oracle.norm_normalise(g("x"), g("gamma"), g("beta"), mean, inv)
    assert np.array_equal(y, g("y")) and np.array_equal(white, g("whitened"))
    assert np.array_equal(oracle.norm_gradients(white, g("g"), inv, g("gamma")), g("dx"))
    ga, be = oracle.norm_param_update(white, g("g"), m["learning_rate"], g("gamma"), g("beta"))
    assert np.array_equal(ga, g("gamma_updated")) and np.array_equal(be, g("beta_updated"))


@pytest.mark.skipif(not oracle.have_ref(), reason="reference models not built here")
def test_norm_oracle_equals_reference_on_random_shapes():
    r = np.random.default_rng(17)
    for _ in range(20):
        b, c, f = (int(v) for v in r.integers(1, 7, 3))
        x, gr = r.normal(0.3, 1.5, (b, c, f)), r.normal(size=(b, c, f))
        gamma, beta = r.uniform(0.5, 2, c), r.normal(size=c)
        unb, st = bool(r.integers(0, 2)), bool(r.integers(0, 2))
        a = oracle.norm_statistics(x, 1e-4, unb, st)
        b_ = oracle.norm_statistics(x, 1e-4, unb, st, use_ref=True)
        assert np.array_equal(a[0], b_[0]) and np.array_equal(a[1], b_[1])
        y1, w1 = oracle.norm_normalise(x, gamma, beta, *a)
        y2, w2 = oracle.norm_normalise(x, gamma, beta, *a, use_ref=True)
        assert np.array_equal(y1, y2) and np.array_equal(w1, w2)
        assert np.array_equal(oracle.norm_gradients(w1, gr, a[1], gamma),
                              oracle.norm_gradients(w1, gr, a[1], gamma, use_ref=True))
