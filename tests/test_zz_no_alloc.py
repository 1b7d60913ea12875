"""The weight-update entry point that allocates nothing on the device.

It exists for callers that cannot call cudaMalloc at the moment they need a
weight gradient (everything on the device belongs to their own allocator, or
they run where taking the allocator's lock is not allowed).  The test calls it
through the C ABI twice in a row and checks each result against the ordinary
entry point, plb_conv_wu, on the same inputs.  It is collected last so that a
failure here cannot hide the other tests.
"""
import numpy as np
import pytest

import common as T
from poplibs_b200 import capi

pytestmark = pytest.mark.gpu


def _run_both(ctx, kw, x, dy):
    import torch
    p = capi.ConvParams.make(**kw)
    kernel = [int(p.kernel[i]) for i in range(p.num_field_dims)]
    shape = [p.groups] + kernel + [p.out_chans_per_group, p.in_chans_per_group]
    dx, ddy = T.to_dev(T.acts_to_device_layout(x)), T.to_dev(T.acts_to_device_layout(dy))
    ref16, ref32 = T.empty_dev(shape, np.float16), T.empty_dev(shape, np.float32)
    new16, new32 = T.empty_dev(shape, np.float16), T.empty_dev(shape, np.float32)
    torch.cuda.synchronize()
    ctx.conv_wu(p, dx, ddy, ref16, ref32)
    ctx.synchronize()
    stream = torch.cuda.current_stream()
    capi.conv_wu_static_scratch(0, stream.cuda_stream, p, dx, ddy, new16, new32)
    torch.cuda.synchronize()
    return (ref16.cpu().numpy(), ref32.cpu().numpy(), new16.cpu().numpy(), new32.cpu().numpy())


def test_static_scratch_weight_update_matches_plb_conv_wu_twice(gpu_ctx):
    r = T.rng(91)
    cases = [
        dict(batch=4, field=[14, 14], kernel=[3, 3], in_chans=64, out_chans=64, padding=1),
        dict(batch=64, field=[28, 28], kernel=[3, 3], in_chans=128, out_chans=128, padding=1),
    ]
    # two calls in a row per case: the second finds the first one's partial sums
    # and status word in the shared array
    for kw in cases:
        p = capi.ConvParams.make(**kw)
        of = p.output_field()
        for exact in (True, False):
            gen = T.binary_half if exact else T.uniform_half
            x = gen(r, (kw["batch"], kw["in_chans"], *kw["field"]))
            dy = gen(r, (kw["batch"], kw["out_chans"], *of))
            ref16, ref32, new16, new32 = _run_both(gpu_ctx, kw, x, dy)
            if exact:
                # integer sums below 2^24 are exact whatever the split
                assert (new32 == ref32).all() and (new16 == ref16).all()
            else:
                # the number of K splits may differ, so fp32 sums may differ in
                # their last bits: the tolerance of the other parity tests
                rms = float(np.sqrt(np.mean(ref32.astype(np.float64) ** 2)))
                assert np.abs(new32.astype(np.float64) - ref32).max() <= max(1e-5, 2.5e-4 * rms)
                assert np.abs(new16.astype(np.float64) - ref16.astype(np.float64)).max() <= \
                    max(1e-5, 1e-3 * float(np.abs(ref16.astype(np.float64)).max()))


def test_static_scratch_rejects_gradients_beyond_its_limit(gpu_ctx):
    # 3x3 x 1024 x 1024 fp32 = 36 MiB per group > 32 MiB
    p = capi.ConvParams.make(1, [4, 4], [3, 3], 1024, 1024, padding=1)
    with pytest.raises(capi.PlbError) as e:
        capi.conv_wu_static_scratch(0, 0, p, 0, 0, 0, 0)
    assert e.value.code == 3 and "exceeds the 33554432-byte static scratch" in e.value.message
