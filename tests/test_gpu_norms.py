"""Batch normalisation kernels (plb_norm_*) through the C ABI against the CPU
oracle (the restatement of lib/poplibs_test/Norms.cpp, pinned to the
reference's own model and its golden vectors by tests/test_oracle.py).

Each stage is checked on its own: the oracle is given what the device was
given (including the device's rounded statistics), so the tolerance is that of
one rounding to the activations' type plus fp32 accumulation: relative 2e-3
for half and 2e-5 for float, absolute floor the same fraction of the
expected values' rms.  The statistics themselves are compared with a looser
5e-3 (half): E[x^2] - mean^2 is formed from the mean rounded to half, as in
the reference's own flow (lib/poplin/codelets/InverseStdDeviation.cpp:43-50).
"""
import numpy as np
import pytest

import common as T
import oracle
from poplibs_b200 import capi

pytestmark = pytest.mark.gpu

SHAPES = [(4, 8, 25), (3, 5, 7), (2, 130, 9), (1, 64, 1), (32, 64, 56 * 56), (6, 3, 50)]


def close(got, want, rel, what):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64).reshape(got.shape)
    rms = float(np.sqrt(np.mean(want * want))) if want.size else 0.0
    bad, first, worst = oracle.check_is_close(got, want, rel, max(1e-7, rel * rms))
    assert bad == 0, f"{what}: {bad}/{got.size} outside rel {rel}; first {got.ravel()[first]} vs {want.ravel()[first]}"


def dev_layout(a):   # [B][C][F] -> [B*F][C]
    return np.ascontiguousarray(np.transpose(a, (0, 2, 1)).reshape(-1, a.shape[1]))


def from_dev(a, b, c, f):
    return np.transpose(a.reshape(b, f, c), (0, 2, 1))


@pytest.mark.parametrize("dtype", ["half", "float"])
@pytest.mark.parametrize("shape", SHAPES)
def test_norm_stages_against_oracle(gpu_ctx, shape, dtype):
    import torch
    ctx = T.context()
    b, c, f = shape
    np_t, plb_t, rel = (np.float16, capi.HALF, 2e-3) if dtype == "half" else (np.float32, capi.FLOAT, 2e-5)
    r = T.rng(b * 1000 + c * 10 + f)
    x = r.normal(0.4, 1.5, shape).astype(np_t)
    g = r.uniform(-1, 1, shape).astype(np_t)
    gamma, beta = r.uniform(0.5, 2.0, c).astype(np_t), r.uniform(-1, 1, c).astype(np_t)
    pixels = b * f
    dx, dg = T.to_dev(dev_layout(x)), T.to_dev(dev_layout(g))
    dgamma, dbeta = T.to_dev(gamma), T.to_dev(beta)
    mean, inv = T.empty_dev([c], np_t), T.empty_dev([c], np_t)
    power = T.empty_dev([c], np.float32)
    xd = x.astype(np.float64)
    for unbiased in (False, True):
        for stable in (False, True):
            n = pixels
            scale = 1.0 / n if n > 1 else 1.0
            scale_var = n / (n - 1) if (unbiased and n > 1) else 1.0
            ctx.norm_moments(plb_t, dx, pixels, c, scale, None, mean, power)
            if stable:
                ctx.norm_moments(plb_t, dx, pixels, c, scale, mean, None, power)
            ctx.norm_inv_std_dev(plb_t, mean, power, c, 1e-3, scale_var, stable, inv)
            ctx.synchronize()
            want_mean, want_inv = oracle.norm_statistics(xd, 1e-3, unbiased, stable)
            if n == 1:
                continue   # a single element: the model defines the variance as 1
            close(mean.cpu().numpy(), want_mean, rel, f"mean {shape} {dtype}")
            # the device applies eps before the unbiased scale, as the reference's vertex does
            close(inv.cpu().numpy(), want_inv, 5e-3 if dtype == "half" else 2e-4,
                  f"inv std dev {shape} {dtype} unbiased={unbiased} stable={stable}")
    m_dev, i_dev = mean.cpu().numpy().astype(np.float64), inv.cpu().numpy().astype(np.float64)
    # whiten + scale and shift, the oracle fed with the device's statistics
    white, out = T.empty_dev([pixels, c], np_t), T.empty_dev([pixels, c], np_t)
    ctx.norm_whiten(plb_t, dx, mean, inv, pixels, c, white)
    ctx.norm_scale_shift(plb_t, white, dgamma, dbeta, pixels, c, out)
    ctx.synchronize()
    _, want_white = oracle.norm_normalise(xd, gamma, beta, m_dev, i_dev)
    w_dev = from_dev(white.cpu().numpy(), b, c, f).astype(np.float64)
    close(w_dev, want_white, rel, f"whitened {shape} {dtype}")
    want_out = gamma.astype(np.float64)[None, :, None] * w_dev + beta.astype(np.float64)[None, :, None]
    close(from_dev(out.cpu().numpy(), b, c, f), want_out, rel, f"normalised {shape} {dtype}")
    # gradients of gamma and beta = what the model's parameter update subtracts at rate 1 from zero
    gd, bd = T.empty_dev([c], np_t), T.empty_dev([c], np_t)
    gd32, bd32 = T.empty_dev([c], np.float32), T.empty_dev([c], np.float32)
    ctx.norm_param_gradients(plb_t, white, dg, pixels, c, 1.0, gd, bd, gd32, bd32)
    ctx.synchronize()
    zero = np.zeros(c)
    ga, be = oracle.norm_param_update(w_dev, g.astype(np.float64), 1.0, zero, zero)
    prel = 4e-3 if dtype == "half" else 1e-4
    if dtype == "float" or np.abs(ga).max() < 6e4:
        close(gd.cpu().numpy(), -ga, prel, f"gamma gradient {shape} {dtype}")
        close(bd.cpu().numpy(), -be, prel, f"beta gradient {shape} {dtype}")
    close(gd32.cpu().numpy(), -ga, 1e-4, f"gamma gradient fp32 {shape} {dtype}")
    close(bd32.cpu().numpy(), -be, 1e-4, f"beta gradient fp32 {shape} {dtype}")
    # gradient through scale, then through the statistics: the model does both at once
    ng, sg = T.empty_dev([pixels, c], np_t), T.empty_dev([pixels, c], np_t)
    ctx.norm_scale_shift(plb_t, dg, dgamma, None, pixels, c, ng)
    ctx.norm_statistics_gradients(plb_t, white, ng, inv, pixels, c, sg)
    ctx.synchronize()
    ng_dev = from_dev(ng.cpu().numpy(), b, c, f).astype(np.float64)
    close(ng_dev, g.astype(np.float64) * gamma.astype(np.float64)[None, :, None], rel, f"norm gradients {shape}")
    ones = np.ones(c)
    want_sg = oracle.norm_gradients(w_dev, ng_dev, i_dev, ones)
    close(from_dev(sg.cpu().numpy(), b, c, f), want_sg, 4e-3 if dtype == "half" else 1e-4,
          f"statistics gradients {shape} {dtype}")
    # the same with the two per-channel means handed in (the distributed form)
    vd = (-(w_dev * ng_dev).sum(axis=(0, 2)) / pixels).astype(np_t)
    md = (-ng_dev.sum(axis=(0, 2)) / pixels).astype(np_t)
    sg2 = T.empty_dev([pixels, c], np_t)
    ctx.norm_statistics_gradients(plb_t, white, ng, inv, pixels, c, sg2, T.to_dev(vd), T.to_dev(md))
    ctx.synchronize()
    want2 = (ng_dev + w_dev * vd.astype(np.float64)[None, :, None] + md.astype(np.float64)[None, :, None]) * \
        i_dev[None, :, None]
    close(from_dev(sg2.cpu().numpy(), b, c, f), want2, rel, f"statistics gradients, given means {shape} {dtype}")
    del torch


def test_norm_rejects_other_types(gpu_ctx):
    ctx = T.context()
    x = T.empty_dev([4, 8], np.uint8)
    with pytest.raises(capi.PlbError):
        ctx.norm_whiten(capi.QUARTER, x, x, x, 4, 8, x)


@pytest.mark.parametrize("dtype", ["half", "float"])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_statistics_and_normalise_give_the_separate_calls_bits(gpu_ctx, shape, dtype):
    """plb_norm_statistics = plb_norm_moments + plb_norm_inv_std_dev, and
    plb_norm_normalise = plb_norm_whiten + plb_norm_scale_shift, bit for bit
    (the separate calls are the ones checked against the oracle above)."""
    import torch
    ctx = T.context()
    b, c, f = shape
    np_t, plb_t = (np.float16, capi.HALF) if dtype == "half" else (np.float32, capi.FLOAT)
    r = T.rng(b * 77 + c * 5 + f)
    x = r.normal(0.4, 1.5, shape).astype(np_t)
    gamma, beta = r.uniform(0.5, 2.0, c).astype(np_t), r.uniform(-1, 1, c).astype(np_t)
    pixels = b * f
    dx, dgamma, dbeta = T.to_dev(dev_layout(x)), T.to_dev(gamma), T.to_dev(beta)
    mean, inv, power = T.empty_dev([c], np_t), T.empty_dev([c], np_t), T.empty_dev([c], np.float32)
    mean2, inv2, power2 = T.empty_dev([c], np_t), T.empty_dev([c], np_t), T.empty_dev([c], np.float32)
    white, out = T.empty_dev([pixels, c], np_t), T.empty_dev([pixels, c], np_t)
    white2, out2, out3 = (T.empty_dev([pixels, c], np_t) for _ in range(3))
    for scale_var in (1.0, pixels / max(pixels - 1, 1)):
        ctx.norm_moments(plb_t, dx, pixels, c, 1.0 / pixels, None, mean, power)
        ctx.norm_inv_std_dev(plb_t, mean, power, c, 1e-3, scale_var, False, inv)
        ctx.norm_statistics(plb_t, dx, pixels, c, 1e-3, scale_var, mean2, inv2, power2)
        ctx.synchronize()
        assert torch.equal(mean, mean2) and torch.equal(power, power2), "mean / power"
        assert torch.equal(inv, inv2), f"inverse standard deviation, scale_var {scale_var}"
    ctx.norm_inv_std_dev(plb_t, mean, power, c, 1e-3, 1.0, False, inv)
    ctx.norm_statistics(plb_t, dx, pixels, c, 1e-3, 1.0, mean2, inv2, None)   # the power is optional
    ctx.norm_whiten(plb_t, dx, mean, inv, pixels, c, white)
    ctx.norm_scale_shift(plb_t, white, dgamma, dbeta, pixels, c, out)
    ctx.norm_normalise(plb_t, dx, mean, inv, dgamma, dbeta, pixels, c, white2, out2)
    ctx.norm_normalise(plb_t, dx, mean, inv, dgamma, dbeta, pixels, c, None, out3)
    ctx.synchronize()
    assert torch.equal(inv, inv2)
    assert torch.equal(white, white2), "whitened activations"
    assert torch.equal(out, out2) and torch.equal(out, out3), "normalised activations"
