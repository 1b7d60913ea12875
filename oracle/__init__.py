"""CPU oracle for the poplin dense-contraction path -- TEST INFRASTRUCTURE ONLY.

Python (ctypes + numpy) access to

* ``liboracle.so``: the plain-C restatement in ``poplin_oracle.c`` of the
  reference's CPU models (``lib/poplibs_test/Convolution.cpp:455-895``,
  ``lib/poplibs_test/GeneralMatrixMultiply.cpp:190-283``) and of
  ``checkIsClose`` (``lib/poplibs_test/Util.cpp:198-217, 316-348``);
* ``_ref/libpoplibs_test_ref.so`` (optional): those reference sources
  themselves, compiled unmodified (see ``Makefile``).

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import
this package.  The product package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
MAX_DIMS = 3
_U3 = C.c_uint32 * MAX_DIMS


class _CParams(C.Structure):
    _fields_ = [
        ("num_field_dims", C.c_uint32),
        ("batch", C.c_uint32),
        ("groups", C.c_uint32),
        ("in_chans_per_group", C.c_uint32),
        ("out_chans_per_group", C.c_uint32),
        ("field", _U3), ("kernel", _U3),
        ("in_trunc_lo", _U3), ("in_trunc_hi", _U3), ("in_dilation", _U3),
        ("in_pad_lo", _U3), ("in_pad_hi", _U3), ("in_flip", _U3),
        ("k_trunc_lo", _U3), ("k_trunc_hi", _U3), ("k_dilation", _U3),
        ("k_pad_lo", _U3), ("k_pad_hi", _U3), ("k_flip", _U3),
        ("out_trunc_lo", _U3), ("out_trunc_hi", _U3), ("stride", _U3),
        ("out_pad_lo", _U3), ("out_pad_hi", _U3),
    ]


def _vec(v, n, default):
    if v is None:
        return [default] * n
    if isinstance(v, (int, bool, np.integer)):
        return [int(v)] * n
    v = [int(x) for x in v]
    if len(v) != n:
        raise ValueError(f"expected {n} values, got {v}")
    return v


@dataclass
class ConvSpec:
    """Flat description of a poplin::ConvParams
    (include/poplin/ConvParams.hpp:16-224), channel counts per group."""

    batch: int
    field: Sequence[int]
    kernel: Sequence[int]
    in_chans: int
    out_chans: int
    groups: int = 1
    in_trunc_lo: Optional[Sequence[int]] = None
    in_trunc_hi: Optional[Sequence[int]] = None
    in_dilation: Optional[Sequence[int]] = None
    in_pad_lo: Optional[Sequence[int]] = None
    in_pad_hi: Optional[Sequence[int]] = None
    in_flip: Optional[Sequence[int]] = None
    k_trunc_lo: Optional[Sequence[int]] = None
    k_trunc_hi: Optional[Sequence[int]] = None
    k_dilation: Optional[Sequence[int]] = None
    k_pad_lo: Optional[Sequence[int]] = None
    k_pad_hi: Optional[Sequence[int]] = None
    k_flip: Optional[Sequence[int]] = None
    out_trunc_lo: Optional[Sequence[int]] = None
    out_trunc_hi: Optional[Sequence[int]] = None
    stride: Optional[Sequence[int]] = None
    out_pad_lo: Optional[Sequence[int]] = None
    out_pad_hi: Optional[Sequence[int]] = None

    @staticmethod
    def simple(batch, field, kernel, in_chans, out_chans, padding=0, stride=1,
               groups=1):
        nd = len(field)
        return ConvSpec(batch, list(field), list(kernel), in_chans, out_chans,
                        groups, in_pad_lo=_vec(padding, nd, 0),
                        in_pad_hi=_vec(padding, nd, 0),
                        stride=_vec(stride, nd, 1))

    def normalised(self) -> dict:
        nd = len(self.field)
        d = {"field": list(map(int, self.field)),
             "kernel": list(map(int, self.kernel))}
        ones = ("in_dilation", "k_dilation", "stride")
        for name in ("in_trunc_lo", "in_trunc_hi", "in_dilation", "in_pad_lo",
                     "in_pad_hi", "in_flip", "k_trunc_lo", "k_trunc_hi",
                     "k_dilation", "k_pad_lo", "k_pad_hi", "k_flip",
                     "out_trunc_lo", "out_trunc_hi", "stride", "out_pad_lo",
                     "out_pad_hi"):
            d[name] = _vec(getattr(self, name), nd, 1 if name in ones else 0)
        return d

    def to_c(self) -> _CParams:
        nd = len(self.field)
        if not 1 <= nd <= MAX_DIMS or len(self.kernel) != nd:
            raise ValueError("1..3 field dimensions supported")
        p = _CParams()
        p.num_field_dims = nd
        p.batch, p.groups = self.batch, self.groups
        p.in_chans_per_group, p.out_chans_per_group = self.in_chans, self.out_chans
        for name, vals in self.normalised().items():
            arr = getattr(p, name)
            for i, x in enumerate(vals):
                arr[i] = x
        return p

    def out_field(self):
        lib = _lib()
        p = self.to_c()
        out = [lib.oracle_conv_out_size(C.byref(p), d) for d in range(len(self.field))]
        if any(o < 0 for o in out):
            raise ValueError("invalid convolution parameters")
        return out

    def macs(self) -> int:
        """Multiply-accumulates that touch a real input element (padding is
        not counted), as lib/poplin/PerformanceEstimation.hpp:1641-1666."""
        lib = _lib()
        p = self.to_c()
        per_dim = 1
        for d, (o, k) in enumerate(zip(self.out_field(), self.kernel)):
            n = sum(1 for oi in range(o) for ki in range(k)
                    if lib.oracle_conv_input_index(C.byref(p), d, oi, ki) >= 0)
            per_dim *= n
        return per_dim * self.batch * self.groups * self.in_chans * self.out_chans


_LIB = None
_REF = None
_DP = C.POINTER(C.c_double)


def build(ref: bool = False, reference_dir: str | None = None) -> None:
    """Compile liboracle.so (and, when ``ref`` is set, _ref/libpoplibs_test_ref.so
    from the reference tree at ``reference_dir``) with the Makefile here."""
    targets = ["all"] + (["ref"] if ref else [])
    extra = [f"REFERENCE={reference_dir}"] if reference_dir else []
    subprocess.run(["make", "-s", "-C", _HERE] + extra + targets, check=True)


def _lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        lib = C.CDLL(path)
        PP = C.POINTER(_CParams)
        lib.oracle_conv_out_size.argtypes = [PP, C.c_uint32]
        lib.oracle_conv_input_index.argtypes = [PP, C.c_uint32, C.c_uint32, C.c_uint32]
        lib.oracle_conv_fwd.argtypes = [PP, _DP, _DP, _DP, _DP, C.c_int]
        lib.oracle_conv_bwd.argtypes = [PP, _DP, _DP, _DP, C.c_int]
        lib.oracle_conv_wu.argtypes = [PP, _DP, _DP, _DP, _DP, C.c_int]
        lib.oracle_gemm.argtypes = [C.c_uint32] * 4 + [_DP] * 4 + [C.c_float, C.c_float, C.c_int, C.c_int, C.c_int]
        lib.oracle_is_close.argtypes = [C.c_double] * 4
        lib.oracle_check_is_close.argtypes = [_DP, _DP, C.c_size_t, C.c_double, C.c_double,
                                              C.POINTER(C.c_size_t), C.POINTER(C.c_double)]
        lib.oracle_check_is_close.restype = C.c_size_t
        U = C.c_uint32
        lib.oracle_norm_statistics.argtypes = [_DP, U, U, U, C.c_double, C.c_int, C.c_int, _DP, _DP]
        lib.oracle_norm_statistics.restype = None
        lib.oracle_norm_normalise.argtypes = [_DP] * 5 + [U, U, U, _DP, _DP]
        lib.oracle_norm_normalise.restype = None
        lib.oracle_norm_gradients.argtypes = [_DP] * 4 + [U, U, U, _DP]
        lib.oracle_norm_gradients.restype = None
        lib.oracle_norm_param_update.argtypes = [_DP, _DP, C.c_double, U, U, U, _DP, _DP]
        lib.oracle_norm_param_update.restype = None
        lib.oracle_round_to_half.argtypes = [C.c_double]
        lib.oracle_round_to_half.restype = C.c_double
        lib.oracle_e4m3_from_double.argtypes = [C.c_double]
        lib.oracle_e4m3_from_double.restype = C.c_uint8
        lib.oracle_e4m3_to_double.argtypes = [C.c_uint8]
        lib.oracle_e4m3_to_double.restype = C.c_double
        _LIB = lib
    return _LIB


def have_ref() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libpoplibs_test_ref.so"))


def _ref():
    global _REF
    if _REF is None:
        lib = C.CDLL(os.path.join(_HERE, "_ref", "libpoplibs_test_ref.so"))
        PP = C.POINTER(_CParams)
        lib.ref_conv_fwd.argtypes = [PP, _DP, _DP, _DP, _DP]
        lib.ref_conv_bwd.argtypes = [PP, _DP, _DP, _DP]
        lib.ref_conv_wu.argtypes = [PP, _DP, _DP, _DP, _DP]
        lib.ref_gemm.argtypes = [C.c_uint32] * 4 + [_DP] * 4 + [C.c_float, C.c_float, C.c_int, C.c_int]
        lib.ref_last_error.restype = C.c_char_p
        U = C.c_uint32
        lib.ref_norm_statistics.argtypes = [_DP, U, U, U, C.c_double, C.c_int, C.c_int, _DP, _DP]
        lib.ref_norm_normalise.argtypes = [_DP] * 5 + [U, U, U, _DP, _DP]
        lib.ref_norm_gradients.argtypes = [_DP] * 4 + [U, U, U, _DP]
        lib.ref_norm_param_update.argtypes = [_DP, _DP, C.c_double, U, U, U, _DP, _DP]
        _REF = lib
    return _REF


def _d(a):
    a = np.ascontiguousarray(a, dtype=np.float64)
    return a, a.ctypes.data_as(_DP)


def _shapes(spec: ConvSpec):
    of = spec.out_field()
    ie, ke, oe = int(np.prod(spec.field)), int(np.prod(spec.kernel)), int(np.prod(of))
    return ((spec.batch, spec.groups * spec.in_chans, ie),
            (spec.groups, spec.out_chans, spec.in_chans, ke),
            (spec.batch, spec.groups * spec.out_chans, oe))


def conv_fwd(spec: ConvSpec, x, w, bias=None, threads=0, use_ref=False):
    """out[b][G*Co][prod(outField)] in double; x [b][G*Ci][prod(field)],
    w [G][Co][Ci][prod(kernel)]."""
    xs, ws, ys = _shapes(spec)
    x, xp = _d(np.reshape(x, xs))
    w, wp = _d(np.reshape(w, ws))
    bp = None
    if bias is not None:
        bias, bp = _d(bias)
    y = np.zeros(ys)
    p = spec.to_c()
    if y.size == 0:
        return y
    if use_ref:
        rc = _ref().ref_conv_fwd(C.byref(p), xp, wp, bp, y.ctypes.data_as(_DP))
    else:
        rc = _lib().oracle_conv_fwd(C.byref(p), xp, wp, bp, y.ctypes.data_as(_DP), threads)
    if rc:
        raise RuntimeError(f"oracle conv_fwd failed rc={rc}")
    return y


def conv_bwd(spec: ConvSpec, dy, w, threads=0, use_ref=False):
    xs, ws, ys = _shapes(spec)
    dy, dyp = _d(np.reshape(dy, ys))
    w, wp = _d(np.reshape(w, ws))
    dx = np.zeros(xs)
    p = spec.to_c()
    if dx.size == 0 or dy.size == 0:
        return dx
    if use_ref:
        rc = _ref().ref_conv_bwd(C.byref(p), dyp, wp, dx.ctypes.data_as(_DP))
    else:
        rc = _lib().oracle_conv_bwd(C.byref(p), dyp, wp, dx.ctypes.data_as(_DP), threads)
    if rc:
        raise RuntimeError(f"oracle conv_bwd failed rc={rc}")
    return dx


def conv_wu(spec: ConvSpec, x, dy, threads=0, use_ref=False):
    """(dW [G][Co][Ci][prod(kernel)], dBias [G*Co]) -- the raw gradients."""
    xs, ws, ys = _shapes(spec)
    x, xp = _d(np.reshape(x, xs))
    dy, dyp = _d(np.reshape(dy, ys))
    dw = np.zeros(ws)
    db = np.zeros(ys[1])
    p = spec.to_c()
    if dw.size == 0:
        return dw, db
    if use_ref:
        rc = _ref().ref_conv_wu(C.byref(p), xp, dyp, dw.ctypes.data_as(_DP), db.ctypes.data_as(_DP))
    else:
        rc = _lib().oracle_conv_wu(C.byref(p), xp, dyp, dw.ctypes.data_as(_DP), db.ctypes.data_as(_DP), threads)
    if rc:
        raise RuntimeError(f"oracle conv_wu failed rc={rc}")
    return dw, db


def gemm(a, b, c=None, alpha=1.0, beta=0.0, transpose_a=False, transpose_b=False,
         threads=0, use_ref=False):
    """D = beta*C + alpha*op(A)*op(B) in double; 2-D or grouped 3-D inputs."""
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    squeeze = a.ndim == 2
    if squeeze:
        a, b = a[None], b[None]
        c = None if c is None else np.asarray(c, dtype=np.float64)[None]
    g = a.shape[0]
    m, k = (a.shape[2], a.shape[1]) if transpose_a else (a.shape[1], a.shape[2])
    k2, n = (b.shape[2], b.shape[1]) if transpose_b else (b.shape[1], b.shape[2])
    if k != k2 or b.shape[0] != g:
        raise ValueError("gemm shape mismatch")
    a, ap = _d(a)
    b, bp = _d(b)
    cp = None
    if c is not None:
        c, cp = _d(np.reshape(c, (g, m, n)))
    d = np.zeros((g, m, n))
    if d.size:
        if use_ref:
            rc = _ref().ref_gemm(g, m, k, n, ap, bp, cp, d.ctypes.data_as(_DP), alpha, beta,
                                 int(transpose_a), int(transpose_b))
        else:
            rc = _lib().oracle_gemm(g, m, k, n, ap, bp, cp, d.ctypes.data_as(_DP), alpha, beta,
                                    int(transpose_a), int(transpose_b), threads)
        if rc:
            raise RuntimeError(f"oracle gemm failed rc={rc}")
    return d[0] if squeeze else d


# ---- batch normalisation (poplibs_test::norm, NormType::BatchNorm) -----------------
# Activations are [batch][chans][field...]; statistics are per channel.

def _bcf(a):
    a = np.asarray(a, dtype=np.float64)
    a3 = np.ascontiguousarray(a.reshape(a.shape[0], a.shape[1], -1))
    return a3, a3.ctypes.data_as(_DP), a3.shape


def _check_ref(rc):
    if rc:
        raise RuntimeError(_ref().ref_last_error().decode())


def norm_statistics(acts, eps, unbiased=False, stable=False, use_ref=False):
    """(mean[chans], inv_std_dev[chans])."""
    a, ap, (b, c, f) = _bcf(acts)
    mean, inv = np.zeros(c), np.zeros(c)
    args = (ap, b, c, f, float(eps), int(unbiased), int(stable), mean.ctypes.data_as(_DP), inv.ctypes.data_as(_DP))
    if use_ref:
        _check_ref(_ref().ref_norm_statistics(*args))
    else:
        _lib().oracle_norm_statistics(*args)
    return mean, inv


def norm_normalise(acts, gamma, beta, mean, inv_std, use_ref=False):
    """(normalised, whitened), both shaped like acts."""
    a, ap, (b, c, f) = _bcf(acts)
    out, white = np.zeros_like(a), np.zeros_like(a)
    vecs = [_d(v) for v in (gamma, beta, mean, inv_std)]
    args = (ap, *[v[1] for v in vecs], b, c, f, out.ctypes.data_as(_DP), white.ctypes.data_as(_DP))
    if use_ref:
        _check_ref(_ref().ref_norm_normalise(*args))
    else:
        _lib().oracle_norm_normalise(*args)
    shape = np.asarray(acts).shape
    return out.reshape(shape), white.reshape(shape)


def norm_gradients(whitened, grads_in, inv_std, gamma, use_ref=False):
    """Gradient with respect to the normalisation's input."""
    w, wp, (b, c, f) = _bcf(whitened)
    g, gp, _ = _bcf(grads_in)
    i, ip = _d(inv_std)
    ga, gap = _d(gamma)
    out = np.zeros_like(w)
    args = (wp, gp, ip, gap, b, c, f, out.ctypes.data_as(_DP))
    if use_ref:
        _check_ref(_ref().ref_norm_gradients(*args))
    else:
        _lib().oracle_norm_gradients(*args)
    return out.reshape(np.asarray(whitened).shape)


def norm_param_update(whitened, grads_in, learning_rate, gamma, beta, use_ref=False):
    """(gamma - lr * sum(whitened * grads), beta - lr * sum(grads)) per channel."""
    w, wp, (b, c, f) = _bcf(whitened)
    g, gp, _ = _bcf(grads_in)
    ga = np.array(gamma, dtype=np.float64)
    be = np.array(beta, dtype=np.float64)
    args = (wp, gp, float(learning_rate), b, c, f, ga.ctypes.data_as(_DP), be.ctypes.data_as(_DP))
    if use_ref:
        _check_ref(_ref().ref_norm_param_update(*args))
    else:
        _lib().oracle_norm_param_update(*args)
    return ga, be


def check_is_close(actual, expected, rel_tol, abs_tol=1e-5):
    """poplibs_test::checkIsClose over arrays.  Returns (n_bad, first_bad_index,
    max_relative_error)."""
    a, ap = _d(np.ravel(actual))
    e, ep = _d(np.ravel(expected))
    if a.size != e.size:
        raise ValueError("size mismatch")
    first = C.c_size_t(0)
    mx = C.c_double(0.0)
    bad = _lib().oracle_check_is_close(ap, ep, a.size, rel_tol, abs_tol, C.byref(first), C.byref(mx))
    return int(bad), int(first.value), float(mx.value)


def is_close(actual, expected, rel_tol, abs_tol=1e-5) -> bool:
    return bool(_lib().oracle_is_close(float(actual), float(expected), rel_tol, abs_tol))


def round_to_half(x):
    """Round doubles to the nearest IEEE half value (returned as float64)."""
    return np.asarray(x, dtype=np.float64).astype(np.float16).astype(np.float64)


def e4m3_encode(x) -> np.ndarray:
    """RNE, saturating quantisation of doubles to E4M3 (bias 7, max 448) bytes."""
    x = np.asarray(x, dtype=np.float64)
    lib = _lib()
    flat = np.fromiter((lib.oracle_e4m3_from_double(float(v)) for v in x.ravel()),
                       dtype=np.uint8, count=x.size) if x.size < 4096 else _e4m3_encode_np(x.ravel())
    return flat.reshape(x.shape)


def _e4m3_encode_np(x: np.ndarray) -> np.ndarray:
    ax = np.abs(x)
    sign = (np.signbit(x)).astype(np.uint8) << 7
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(ax > 0, ax, 1.0)))
    e = np.maximum(e, -6.0)
    ulp = np.exp2(e - 3)
    q = np.rint(ax / ulp) * ulp          # rint: ties to even
    q = np.minimum(q, 448.0)
    e2 = np.floor(np.log2(np.where(q > 0, q, 1.0)))
    sub = (q < 2.0 ** -6)
    e2 = np.maximum(e2, -6.0)
    mant_norm = np.rint((q / np.exp2(e2) - 1.0) * 8.0).astype(np.int64)
    code_norm = ((e2.astype(np.int64) + 7) << 3) | mant_norm
    code_sub = np.rint(q / 2.0 ** -9).astype(np.int64)
    code = np.where(sub, code_sub, code_norm)
    code = np.where(q == 0, 0, code)
    code = np.where(np.isnan(x), 0x7F, code)
    return (sign | code.astype(np.uint8)).astype(np.uint8)


def e5m2_encode(x) -> np.ndarray:
    """RNE quantisation of doubles to E5M2 bytes (bias 15; the upper byte of the
    binary16 encoding): round to binary16 first, then drop eight mantissa bits
    with ties to even; values beyond the largest finite code (57344) saturate."""
    x = np.asarray(x, dtype=np.float64)
    h = np.clip(x, -57344.0, 57344.0).astype(np.float16).view(np.uint16).astype(np.uint32)
    lower, upper = h & 0xFF, h >> 8
    round_up = (lower > 0x80) | ((lower == 0x80) & ((upper & 1) == 1))
    code = upper + round_up.astype(np.uint32)
    # rounding must not carry into the infinity code
    code = np.where((code & 0x7F) >= 0x7C, (code & 0x80) | 0x7B, code)
    code = np.where(np.isnan(x), 0x7E, code)
    return code.astype(np.uint8)


def e5m2_decode(bits) -> np.ndarray:
    b = np.asarray(bits, dtype=np.uint8).astype(np.uint16) << 8
    return b.view(np.float16).astype(np.float64)


_E4M3_TABLE = None


def e4m3_decode(bits) -> np.ndarray:
    global _E4M3_TABLE
    if _E4M3_TABLE is None:
        lib = _lib()
        _E4M3_TABLE = np.array([lib.oracle_e4m3_to_double(i) for i in range(256)])
    return _E4M3_TABLE[np.asarray(bits, dtype=np.uint8)]


def num_threads() -> int:
    return int(_lib().oracle_num_threads())
