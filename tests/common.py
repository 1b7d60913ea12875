"""Shared helpers for the parity tests: seeded data in the reference tools'
style, layout changes between poplin's external shapes and the device layouts,
and thin wrappers that run one contraction through the C ABI on cuda:0."""
from __future__ import annotations

import numpy as np

from poplibs_b200 import capi

# BASELINE tolerances: checkIsClose relative tolerance for half data with float
# partials, and for quarter (fp8) data; absolute tolerance as in the reference
# tools (tools/single_conv_layer.cpp:47-50).
REL_TOL_HALF = 1e-3
REL_TOL_QUARTER = 5e-2
ABS_TOL = 1e-5


def rng(seed):
    return np.random.default_rng(seed)


def uniform_half(r, shape, lo=-1.0, hi=1.0):
    """Uniform doubles rounded to half, as the reference rounds its test data
    to the device type before use (lib/poplibs_test/Util.cpp:20-33, 125-130)."""
    return r.uniform(lo, hi, size=shape).astype(np.float16)


def binary_half(r, shape):
    """+-1 data: every product and partial sum is an exactly representable
    integer, so results must match the oracle bit for bit
    (tools/single_conv_layer.cpp:979-1005)."""
    return (r.integers(0, 2, size=shape) * 2 - 1).astype(np.float16)


def small_int_half(r, shape, lo=-4, hi=4):
    return r.integers(lo, hi + 1, size=shape).astype(np.float16)


# ---- layouts ---------------------------------------------------------------
def acts_to_device_layout(x_ncf: np.ndarray) -> np.ndarray:
    """[N][C][field...] -> [N][field...][C]."""
    nd = x_ncf.ndim - 2
    return np.ascontiguousarray(np.moveaxis(x_ncf, 1, -1)) if nd >= 1 else x_ncf


def acts_from_device_layout(x_nfc: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(np.moveaxis(x_nfc, -1, 1))


def weights_to_device_layout(w: np.ndarray) -> np.ndarray:
    """[G][Co][Ci][k...] -> [G][k...][Co][Ci]."""
    nd = w.ndim - 3
    perm = [0] + list(range(3, 3 + nd)) + [1, 2]
    return np.ascontiguousarray(np.transpose(w, perm))


def weights_from_device_layout(w: np.ndarray) -> np.ndarray:
    nd = w.ndim - 3
    perm = [0, 1 + nd, 2 + nd] + list(range(1, 1 + nd))
    return np.ascontiguousarray(np.transpose(w, perm))


# ---- device helpers (torch is only the allocator here) ----------------------
def to_dev(a: np.ndarray):
    import torch
    if a.dtype == np.uint8:
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def empty_dev(shape, dtype):
    import torch
    td = {np.float16: torch.float16, np.float32: torch.float32, np.uint8: torch.uint8}[dtype]
    # poison the buffer so that unwritten elements are caught
    t = torch.empty(shape, dtype=td, device="cuda")
    if t.numel():
        t.view(torch.uint8).fill_(0x7D)
    return t


_CTX = None


def context() -> capi.Context:
    global _CTX
    if _CTX is None:
        _CTX = capi.Context(0)
    return _CTX


def gpu_matmul(a, b, c=None, *, transpose_a=False, transpose_b=False, alpha=1.0, beta=0.0,
               out_dtype=np.float16, scale_a=0, scale_b=0, format_a=0, format_b=0, ctx=None):
    """a: [g][m][k] (or [g][k][m] if transpose_a); b: [g][k][n] (or [g][n][k])."""
    import torch
    ctx = ctx or context()
    squeeze = a.ndim == 2
    if squeeze:
        a, b = a[None], b[None]
        c = None if c is None else c[None]
    g = a.shape[0]
    m, k = (a.shape[2], a.shape[1]) if transpose_a else (a.shape[1], a.shape[2])
    n = b.shape[1] if transpose_b else b.shape[2]
    quarter = a.dtype == np.uint8
    desc = capi.MatmulDesc.make(m, k, n, groups=g,
                                input_type=capi.QUARTER if quarter else
                                capi.FLOAT if a.dtype == np.float32 else capi.HALF,
                                output_type=capi.FLOAT if out_dtype == np.float32 else capi.HALF,
                                transpose_a=transpose_a, transpose_b=transpose_b,
                                alpha=alpha, beta=beta, scale_a=scale_a, scale_b=scale_b,
                                format_a=format_a, format_b=format_b)
    da, db = to_dev(a), to_dev(b)
    dc = to_dev(c.astype(out_dtype)) if c is not None else None
    dd = empty_dev((g, m, n), out_dtype)
    torch.cuda.synchronize()  # inputs were staged on torch's stream
    ctx.matmul(desc, da, db, dc, dd)
    ctx.synchronize()
    torch.cuda.synchronize()
    out = dd.cpu().numpy()
    return out[0] if squeeze else out


def gpu_conv_fwd(p: capi.ConvParams, x_ncf, w_gocik, bias=None, ctx=None, opt=None):
    """x: [N][G*Ci][field...], w: [G][Co][Ci][k...] (poplin external shapes);
    returns [N][G*Co][outField...]."""
    import torch
    ctx = ctx or context()
    out_dtype = np.float32 if p.output_type == capi.FLOAT else np.float16
    of = p.output_field()
    dx = to_dev(acts_to_device_layout(x_ncf))
    dw = to_dev(weights_to_device_layout(w_gocik))
    db = to_dev(np.asarray(bias, dtype=np.float32)) if bias is not None else None
    dy = empty_dev([p.batch] + of + [p.groups * p.out_chans_per_group], out_dtype)
    torch.cuda.synchronize()  # inputs were staged on torch's stream
    ctx.conv_fwd(p, dx, dw, dy, bias=db, opt=opt)
    ctx.synchronize()
    torch.cuda.synchronize()
    return acts_from_device_layout(dy.cpu().numpy())


def gpu_conv_bwd(p: capi.ConvParams, dy_ncf, w_gocik, ctx=None, opt=None):
    import torch
    ctx = ctx or context()
    out_dtype = np.float32 if p.output_type == capi.FLOAT else np.float16
    field = [int(p.field[i]) for i in range(p.num_field_dims)]
    ddy = to_dev(acts_to_device_layout(dy_ncf))
    dw = to_dev(weights_to_device_layout(w_gocik))
    ddx = empty_dev([p.batch] + field + [p.groups * p.in_chans_per_group], out_dtype)
    torch.cuda.synchronize()  # inputs were staged on torch's stream
    ctx.conv_bwd(p, ddy, dw, ddx, opt=opt)
    ctx.synchronize()
    torch.cuda.synchronize()
    return acts_from_device_layout(ddx.cpu().numpy())


def gpu_conv_wu(p: capi.ConvParams, x_ncf, dy_ncf, ctx=None, opt=None, want_f32=True):
    """Returns (dW in the input type, dW fp32), both [G][Co][Ci][k...]."""
    import torch
    ctx = ctx or context()
    in_dtype = (np.uint8 if p.input_type == capi.QUARTER else
                np.float32 if p.input_type == capi.FLOAT else np.float16)
    kernel = [int(p.kernel[i]) for i in range(p.num_field_dims)]
    shape = [p.groups] + kernel + [p.out_chans_per_group, p.in_chans_per_group]
    dx = to_dev(acts_to_device_layout(x_ncf))
    ddy = to_dev(acts_to_device_layout(dy_ncf))
    dw = empty_dev(shape, in_dtype)
    dw32 = empty_dev(shape, np.float32) if want_f32 else None
    torch.cuda.synchronize()  # inputs were staged on torch's stream
    ctx.conv_wu(p, dx, ddy, dw, dw32, opt=opt)
    ctx.synchronize()
    torch.cuda.synchronize()
    a = weights_from_device_layout(dw.cpu().numpy())
    b = weights_from_device_layout(dw32.cpu().numpy()) if want_f32 else None
    return a, b


def spec_from_params(p: capi.ConvParams):
    """The oracle's description of the same convolution."""
    from oracle import ConvSpec
    nd = p.num_field_dims
    kw = {name: [int(getattr(p, name)[i]) for i in range(nd)] for name in capi.ConvParams._VECS}
    return ConvSpec(int(p.batch), [int(p.field[i]) for i in range(nd)],
                    [int(p.kernel[i]) for i in range(nd)], int(p.in_chans_per_group),
                    int(p.out_chans_per_group), int(p.groups), **kw)
