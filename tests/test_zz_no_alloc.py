"""The weight-update entry point that allocates nothing on the device.

It exists for callers that cannot call cudaMalloc at the moment they need a
weight gradient (everything on the device belongs to their own allocator, or
they run where taking the allocator's lock is not allowed).  The test calls it
through the C ABI twice in a row and checks each result against the ordinary
entry point, plb_conv_wu, on the same inputs, and against the CPU oracle.  It
also checks the property the entry point exists for: the device's free memory
does not change across a call.  It is collected last so that a failure here
cannot hide the other tests.
"""
import numpy as np
import pytest

import common as T
import oracle
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
        # several groups: the shared array of partial sums is reused group after group
        dict(batch=6, field=[10, 10], kernel=[3, 3], in_chans=16, out_chans=24, padding=1, groups=3),
        # a gradient of 2.25 MiB per K split: the 32 MiB array holds fewer splits than planned
        dict(batch=32, field=[14, 14], kernel=[3, 3], in_chans=256, out_chans=256, padding=1),
    ]
    # two calls in a row per case: the second finds the first one's partial sums
    # and status word in the shared array
    for kw in cases:
        p = capi.ConvParams.make(**kw)
        of = p.output_field()
        for exact in (True, False):
            gen = T.binary_half if exact else T.uniform_half
            g = kw.get("groups", 1)
            x = gen(r, (kw["batch"], g * kw["in_chans"], *kw["field"]))
            dy = gen(r, (kw["batch"], g * kw["out_chans"], *of))
            ref16, ref32, new16, new32 = _run_both(gpu_ctx, kw, x, dy)
            if exact:
                # integer sums below 2^24 are exact whatever the split
                assert (new32 == ref32).all() and (new16 == ref16).all()
                want = oracle.conv_wu(T.spec_from_params(p), x, dy)[0]
                got = T.weights_from_device_layout(new32) if hasattr(T, "weights_from_device_layout") else None
                if got is None:
                    # device layout [G][kh][kw][Co][Ci] -> the oracle's [G][Co][Ci][kh*kw]
                    got = np.transpose(new32, (0, 3, 4, 1, 2)).reshape(want.shape)
                assert (got.astype(np.float64) == want.reshape(got.shape)).all(), "static scratch vs oracle"
            else:
                # the number of K splits may differ, so fp32 sums may differ in
                # their last bits: the tolerance of the other parity tests
                rms = float(np.sqrt(np.mean(ref32.astype(np.float64) ** 2)))
                assert np.abs(new32.astype(np.float64) - ref32).max() <= max(1e-5, 2.5e-4 * rms)
                assert np.abs(new16.astype(np.float64) - ref16.astype(np.float64)).max() <= \
                    max(1e-5, 1e-3 * float(np.abs(ref16.astype(np.float64)).max()))


def test_static_scratch_call_leaves_free_device_memory_unchanged(gpu_ctx):
    import torch
    kw = dict(batch=8, field=[14, 14], kernel=[3, 3], in_chans=64, out_chans=64, padding=1)
    p = capi.ConvParams.make(**kw)
    r = T.rng(5)
    x = T.to_dev(T.acts_to_device_layout(T.binary_half(r, (8, 64, 14, 14))))
    dy = T.to_dev(T.acts_to_device_layout(T.binary_half(r, (8, 64, 14, 14))))
    out32 = T.empty_dev([1, 3, 3, 64, 64], np.float32)
    stream = torch.cuda.current_stream().cuda_stream
    capi.conv_wu_static_scratch(0, stream, p, x, dy, None, out32)    # first call on this device: set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    capi.conv_wu_static_scratch(0, stream, p, x, dy, None, out32)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "the entry point must not allocate or free device memory"


def test_static_scratch_names_the_layers_it_cannot_run(gpu_ctx):
    # channel counts that plb_conv_wu pads in scratch memory are refused up front
    p = capi.ConvParams.make(2, [8, 8], [3, 3], 12, 20, padding=1)
    x, dy = T.empty_dev([2, 8, 8, 12], np.float16), T.empty_dev([2, 8, 8, 20], np.float16)
    out32 = T.empty_dev([1, 3, 3, 20, 12], np.float32)
    with pytest.raises(capi.PlbError) as e:
        capi.conv_wu_static_scratch(0, 0, p, x, dy, None, out32)
    assert e.value.code == 3 and "multiples of 8" in e.value.message and "plb_conv_wu" in e.value.message


def test_static_scratch_rejects_gradients_beyond_its_limit(gpu_ctx):
    # 3x3 x 1024 x 1024 fp32 = 36 MiB per group > 32 MiB
    p = capi.ConvParams.make(1, [4, 4], [3, 3], 1024, 1024, padding=1)
    with pytest.raises(capi.PlbError) as e:
        capi.conv_wu_static_scratch(0, 0, p, 0, 0, 0, 0)
    assert e.value.code == 3 and "exceeds the 33554432-byte static scratch" in e.value.message
