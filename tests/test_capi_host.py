"""Host-side checks that need no GPU: the C ABI library loads and exports every
symbol the header declares, and its host logic (ConvParams algebra, planner,
error reporting) agrees with the oracle and with the reference's messages."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import oracle
from oracle import ConvSpec
from poplibs_b200 import capi
from test_oracle import OUTPUT_DIM_TABLE, RANGE_TABLE, random_spec

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "poplibs_b200.h")).read()
    return sorted(set(re.findall(r"PLB_API[^;(]*?\b(plb_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = capi.lib()
    names = declared_symbols()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/poplibs_b200.h but not exported"
    assert sorted(capi.SYMBOLS) == names
    assert b"sm_100a" in lib.plb_version()


def params_from_spec(spec: ConvSpec) -> capi.ConvParams:
    return capi.ConvParams.make(spec.batch, spec.field, spec.kernel, spec.in_chans, spec.out_chans,
                                spec.groups, **spec.normalised_transforms()) \
        if hasattr(spec, "normalised_transforms") else _params_from_spec(spec)


def _params_from_spec(spec):
    n = spec.normalised()
    n.pop("field"), n.pop("kernel")
    return capi.ConvParams.make(spec.batch, spec.field, spec.kernel, spec.in_chans, spec.out_chans,
                                spec.groups, **n)


def test_input_index_and_output_size_known_answers():
    # the tables of tests/poplin/RangeTest.cpp:33-168
    lib = capi.lib()
    for (stride, lo, hi), rows in RANGE_TABLE.items():
        p = capi.ConvParams.make(1, [10, 10], [3, 3], 1, 1, in_pad_lo=lo, in_pad_hi=hi, stride=stride)
        for out, k, expected in rows:
            assert lib.plb_conv_input_index(C.byref(p), 0, out, k) == expected
    for field, kernel, stride, lo, hi, expected in OUTPUT_DIM_TABLE:
        p = capi.ConvParams.make(1, list(field), list(kernel), 1, 1, in_pad_lo=list(lo),
                                 in_pad_hi=list(hi), stride=list(stride))
        assert tuple(p.output_field()) == expected


def test_geometry_matches_oracle_on_random_params():
    r = np.random.default_rng(3)
    lib, olib = capi.lib(), oracle._lib()
    for _ in range(200):
        spec = random_spec(r)
        p = _params_from_spec(spec)
        assert p.output_field() == spec.out_field()
        assert p.macs() == spec.macs()
        op = spec.to_c()
        for d, (o, k) in enumerate(zip(spec.out_field(), spec.kernel)):
            for oi in range(o):
                for ki in range(k):
                    assert lib.plb_conv_input_index(C.byref(p), d, oi, ki) == \
                        olib.oracle_conv_input_index(C.byref(op), d, oi, ki)


def test_flop_counts_of_the_benchmark_layers():
    mk = capi.ConvParams.make
    assert 2 * mk(32, [56, 56], [3, 3], 64, 64, padding=1).macs() == 7223640064
    assert 2 * mk(256, [28, 28], [3, 3], 128, 128, padding=1).macs() == 56405000192
    assert 2 * mk(256, [56, 56], [1, 1], 256, 512, stride=2).macs() == 52613349376
    assert 2 * mk(256, [224, 224], [7, 7], 3, 64, padding=3, stride=2).macs() == 59501838336  # 2*256*3*64*778^2


def test_validate_messages():
    # lib/poplin/ConvParams.cpp:172-266
    lib = capi.lib()

    def err(**kw):
        p = capi.ConvParams.make(1, [4, 4], [3, 3], 1, 1, **kw)
        rc = lib.plb_conv_validate(C.byref(p))
        return rc, lib.plb_last_error().decode()

    assert err()[0] == 0
    rc, msg = err(stride=[0, 1])
    assert rc == 1 and msg == "Stride must be non zero"
    rc, msg = err(in_dilation=[1, 0])
    assert rc == 1 and msg.startswith("Input dilation must be non zero")
    rc, msg = err(k_dilation=[0, 1])
    assert rc == 1 and msg.startswith("Kernel dilation must be non zero")
    rc, msg = err(in_trunc_lo=[3, 0], in_trunc_hi=[2, 0])
    assert rc == 1 and "truncates by more than the size of the field (4)" in msg
    rc, msg = err(k_trunc_lo=[2, 0], k_trunc_hi=[2, 0])
    assert rc == 1 and "truncates by more than the size of the kernel (3)" in msg
    rc, msg = err(k_trunc_lo=[3, 0])
    assert rc == 1 and msg == "Transformed kernel for dimension 0 has zero size"
    rc, msg = err(k_dilation=[2, 1])
    assert rc == 1 and msg == ("Transformed input size for dimension 0 (4) is less than the "
                               "transformed kernel size (5)")
    rc, msg = err(out_trunc_lo=[2, 0], out_trunc_hi=[1, 0])
    assert rc == 1 and "truncates by more than the size of the convolution output (2)" in msg


def test_planner_choices():
    plan = capi.conv_plan(capi.ConvParams.make(32, [56, 56], [3, 3], 64, 64, padding=1))
    assert (plan.tile_m, plan.tile_n) == (128, 64)
    assert plan.box_w * plan.box_h * plan.box_n == 128
    assert plan.tiles == 784 and plan.grid == 148          # no padded pixels
    assert plan.flops == 7223640064 and plan.bytes == 25763840
    plan = capi.conv_plan(capi.ConvParams.make(256, [28, 28], [3, 3], 128, 128, padding=1))
    assert plan.tile_n == 128 and plan.tiles == 1568
    plan = capi.conv_plan(capi.ConvParams.make(256, [56, 56], [1, 1], 256, 512, stride=2))
    assert plan.tile_n == 256 and plan.bytes == 308543488
    plan = capi.matmul_plan(capi.MatmulDesc.make(8192, 8192, 8192))
    assert plan.tile_n == 256 and plan.tiles == 2048 and plan.b_mn_major == 1
    assert plan.flops == 2 * 8192 ** 3 and plan.bytes == 3 * 8192 * 8192 * 2
    plan = capi.matmul_plan(capi.MatmulDesc.make(8192, 8192, 8192, input_type=capi.QUARTER))
    assert plan.bytes == 2 * 8192 * 8192 + 8192 * 8192 * 2
    plan = capi.matmul_plan(capi.MatmulDesc.make(5, 0, 4))
    assert plan.tiles == 0 and plan.flops == 0


def test_planner_rules_for_pairs_halo_tiles_and_padding():
    """What the closed-form planner picks, per layer shape (no GPU involved)."""
    c2 = capi.conv_plan(capi.ConvParams.make(32, [56, 56], [3, 3], 64, 64, padding=1))
    # small filter, one N tile: weights resident, one strip per filter column, CTA pairs
    assert (c2.resident_weights, c2.halo_rows, c2.cta_pair) == (1, 2, 1)
    c4 = capi.conv_plan(capi.ConvParams.make(256, [28, 28], [3, 3], 128, 128, padding=1))
    # weights too large to keep resident: streamed, but still one activation strip per column
    assert (c4.resident_weights, c4.halo_rows, c4.cta_pair) == (0, 2, 1)
    assert c4.box_w * c4.box_n % 8 == 0 and c4.stages >= 3
    bwd = capi.conv_plan(capi.ConvParams.make(256, [28, 28], [3, 3], 128, 128, padding=1), capi.PASS_TRAINING_BWD)
    assert bwd.b_mn_major == 1 and bwd.cta_pair == 1
    # a short K loop (4 steps) pairs only under 256-column tiles, where the weight tile is
    # most of a stage; with narrower tiles the lockstep costs more than it saves
    c3b = capi.conv_plan(capi.ConvParams.make(256, [56, 56], [1, 1], 256, 512, stride=2))
    assert (c3b.tile_n, c3b.cta_pair, c3b.halo_rows) == (256, 1, 0)
    short128 = capi.conv_plan(capi.ConvParams.make(256, [28, 28], [1, 1], 256, 128))
    assert (short128.tile_n, short128.cta_pair) == (128, 0)
    # a grid of a few tiles takes narrow tiles and no pairs
    c1 = capi.matmul_plan(capi.MatmulDesc.make(512, 1024, 1024))
    assert (c1.tile_n, c1.tiles, c1.grid, c1.cta_pair) == (64, 64, 64, 0)
    big = capi.matmul_plan(capi.MatmulDesc.make(8192, 8192, 8192))
    assert (big.tile_n, big.cta_pair, big.grid) == (256, 1, 148)
    # plan flags
    p = capi.ConvParams.make(256, [28, 28], [3, 3], 128, 128, padding=1)
    off = capi.conv_plan(p, capi.PASS_TRAINING_FWD, capi.ConvOptions.make(plan_flags=capi.PLAN_NO_CTA_PAIR | capi.PLAN_NO_HALO))
    assert (off.cta_pair, off.halo_rows) == (0, 0)
    small = capi.ConvParams.make(2, [12, 12], [3, 3], 64, 64, padding=1)
    assert capi.conv_plan(small).cta_pair == 0
    forced = capi.conv_plan(small, capi.PASS_TRAINING_FWD, capi.ConvOptions.make(plan_flags=capi.PLAN_FORCE_CTA_PAIR))
    assert forced.cta_pair == 1 and forced.grid % 2 == 0
    # channel counts that TMA cannot address are planned on their padded sizes
    odd = capi.conv_plan(capi.ConvParams.make(4, [9, 9], [3, 3], 20, 12, padding=1, groups=2))
    assert odd.tile_n == 64 and odd.tiles > 0
    assert capi.conv_plan(capi.ConvParams.make(4, [9, 9], [3, 3], 20, 12, padding=1), capi.PASS_TRAINING_BWD).tiles > 0
    # the stem goes to the small-channel path
    assert capi.conv_plan(capi.ConvParams.make(8, [224, 224], [7, 7], 3, 64, padding=3, stride=2)).kernel == 2
    # weight update: one strip per filter column with a unit vertical stride, K split to fill the device
    wu = capi.conv_wu_plan(capi.ConvParams.make(256, [28, 28], [3, 3], 128, 128, padding=1))
    assert (wu.kernel, wu.halo_rows, wu.tile_n, wu.split_k, wu.grid) == (1, 2, 384, 49, 147)
    # ... and tap groups sized so that two pipeline stages fit in shared memory
    wide = capi.conv_wu_plan(capi.ConvParams.make(4, [9, 13], [4, 4], 8, 24, stride=3))
    assert wide.halo_rows == 0 and wide.tile_n <= 10 * 32 and wide.stages >= 2


def test_3d_layers_plan_as_2d_layers_with_depth_folded_into_channels():
    """A 3-D field runs as the 2-D problem over the inner dimensions with the
    kernel depth folded into the channels: batch * out-depth images and KD * Ci
    input channels (forward, weight update), batch * depth images and KD * Co
    output channels (backward).  Planning also cross-checks the device-side depth
    index arithmetic against getInputIndex for every (output, kernel) pair."""
    p3 = capi.ConvParams.make(4, [6, 14, 14], [3, 3, 3], 64, 128, padding=1, stride=[2, 1, 1])
    od = p3.output_field()[0]
    assert od == 3
    fwd2 = capi.ConvParams.make(4 * od, [14, 14], [3, 3], 3 * 64, 128, padding=1)
    bwd2 = capi.ConvParams.make(4 * 6, [14, 14], [3, 3], 64, 3 * 128, padding=1)
    same = ("kernel", "tile_m", "tile_n", "stages", "grid", "tiles", "halo_rows", "cta_pair", "split_k")
    for pass_id, p2 in ((capi.PASS_TRAINING_FWD, fwd2), (capi.PASS_TRAINING_BWD, bwd2), (capi.PASS_TRAINING_WU, fwd2)):
        a, b = capi.conv_plan(p3, pass_id).as_dict(), capi.conv_plan(p2, pass_id).as_dict()
        assert {k: a[k] for k in same} == {k: b[k] for k in same}, pass_id
        assert a["flops"] == 2 * p3.macs()
    # every depth transform is accepted (it only changes the gather)
    odd = capi.ConvParams.make(2, [7, 5, 6], [3, 1, 3], 8, 16, in_pad_lo=[2, 0, 1], in_pad_hi=[0, 0, 1],
                               k_dilation=[2, 1, 1], in_dilation=[2, 1, 1], in_trunc_lo=[1, 0, 0],
                               k_flip=[1, 0, 0], in_flip=[1, 0, 0], out_pad_lo=[1, 0, 0], out_trunc_hi=[1, 0, 0],
                               stride=[2, 1, 1])
    for pass_id in (capi.PASS_TRAINING_FWD, capi.PASS_TRAINING_BWD, capi.PASS_TRAINING_WU):
        assert capi.conv_plan(odd, pass_id).flops == 2 * odd.macs()
    # input dilation in an inner dimension runs on the zero-stuffed input (2-D path's fallback)
    inner = capi.ConvParams.make(1, [4, 6, 6], [1, 3, 3], 16, 16, in_dilation=[1, 2, 1])
    stuffed = capi.ConvParams.make(4, [11, 6], [3, 3], 16, 16)
    assert capi.conv_plan(inner).tiles == capi.conv_plan(stuffed).tiles


def test_option_and_type_errors():
    with pytest.raises(capi.PlbError) as e:
        capi.matmul_plan(capi.MatmulDesc.make(4, 4, 4, input_type=capi.QUARTER, output_type=capi.FLOAT))
    assert e.value.code == 1 and "Output type must be half when input type is quarter" in e.value.message
    with pytest.raises(capi.PlbError) as e:
        capi.matmul_plan(capi.MatmulDesc.make(4, 4, 4, partials_type=capi.QUARTER))
    assert e.value.code == 2
    with pytest.raises(capi.PlbError) as e:
        capi.conv_plan(capi.ConvParams.make(1, [4, 4], [3, 3], 8, 8), opt=capi.ConvOptions.make(tile_n=96))
    assert e.value.code == 2


def test_no_silent_fallback_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(capi.PlbError) as e:
        capi.Context(0)
    assert e.value.code == 4  # PLB_ERR_CUDA: fails loudly, nothing is computed on the host


def test_cpulist_parsing():
    """The kernel's cpulist format, as read from a PCI device's local_cpulist."""
    from poplibs_b200 import capi
    assert capi.parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert capi.parse_cpulist("") == set()
    assert capi.parse_cpulist("5") == {5}
