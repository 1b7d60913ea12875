"""Generates tests/golden/*.npz from the REFERENCE's own CPU models.

Run in a container that has the reference tree (it needs
oracle/_ref/libpoplibs_test_ref.so, built by `make -C oracle ref`):

    python tests/golden/make_golden.py

Every case stores its parameters, seeded inputs and the outputs of
poplibs_test::conv::{convolution, convolutionBackward, weightUpdate} /
poplibs_test::gemm::generalGroupedMatrixMultiply, so that the C restatement in
oracle/poplin_oracle.c can be checked where the reference tree is absent.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402
from oracle import ConvSpec  # noqa: E402

# Shapes follow the kinds of layer the reference's own tool tests exercise
# (tests/poplin/CMakeLists.txt: asymmetric strides and padding, dilation of
# input and kernel, truncation, flips, groups, 1-D and 3-D fields, output
# padding), kept small enough for the reference model's speed.
CONV_CASES = {
    "plain_3x3_pad1": ConvSpec.simple(2, [6, 5], [3, 3], 3, 4, padding=1),
    "stem_7x7_s2_p3": ConvSpec.simple(2, [9, 9], [7, 7], 3, 4, padding=3, stride=2),
    "pointwise_s2": ConvSpec.simple(2, [6, 6], [1, 1], 5, 3, stride=2),
    "groups2": ConvSpec.simple(2, [5, 4], [3, 2], 2, 3, padding=1, groups=2),
    "one_dim": ConvSpec(3, [11], [4], 2, 3, in_pad_lo=[2], in_pad_hi=[1], stride=[2]),
    "three_dim": ConvSpec(1, [4, 3, 5], [2, 2, 3], 2, 2, in_pad_lo=[1, 0, 1], in_pad_hi=[0, 1, 1],
                          stride=[1, 2, 1]),
    "asym_stride_pad": ConvSpec(2, [7, 8], [3, 2], 3, 2, in_pad_lo=[2, 0], in_pad_hi=[0, 3],
                                stride=[3, 2]),
    "kernel_dilation": ConvSpec(1, [9, 9], [3, 3], 2, 2, k_dilation=[2, 3], in_pad_lo=[2, 3],
                                in_pad_hi=[2, 3]),
    "input_dilation": ConvSpec(2, [4, 5], [3, 3], 2, 3, in_dilation=[2, 3], in_pad_lo=[2, 2],
                               in_pad_hi=[2, 2]),
    "truncation": ConvSpec(1, [8, 8], [4, 4], 2, 2, in_trunc_lo=[1, 0], in_trunc_hi=[0, 2],
                           k_trunc_lo=[0, 1], k_trunc_hi=[1, 0], out_trunc_lo=[1, 0],
                           out_trunc_hi=[0, 1]),
    "flips": ConvSpec(2, [5, 6], [3, 2], 2, 2, in_flip=[1, 0], k_flip=[0, 1], in_pad_lo=[1, 1],
                      in_pad_hi=[0, 1]),
    "output_padding": ConvSpec(1, [6, 6], [3, 3], 2, 2, stride=[2, 2], out_pad_lo=[1, 0],
                               out_pad_hi=[0, 2]),
    "kernel_padding": ConvSpec(1, [7, 7], [2, 2], 2, 2, k_pad_lo=[1, 0], k_pad_hi=[0, 1]),
    "everything": ConvSpec(2, [7, 6], [3, 3], 2, 2, 2, in_trunc_lo=[1, 0], in_trunc_hi=[0, 1],
                           in_dilation=[2, 1], in_pad_lo=[1, 2], in_pad_hi=[2, 1], in_flip=[0, 1],
                           k_trunc_lo=[0, 1], k_trunc_hi=[0, 0], k_dilation=[1, 2],
                           k_pad_lo=[0, 0], k_pad_hi=[1, 0], k_flip=[1, 0], out_trunc_lo=[0, 1],
                           out_trunc_hi=[1, 0], stride=[2, 1], out_pad_lo=[0, 1],
                           out_pad_hi=[1, 0]),
}

GEMM_CASES = {
    # (groups, m, k, n, alpha, beta, transposeA, transposeB); shapes echo the
    # reference's gemm tool tests (tests/poplin/CMakeLists.txt:515-987)
    "plain": (1, 6, 5, 4, 1.0, 0.0, False, False),
    "alpha_beta": (1, 5, 7, 3, 0.5, 2.0, False, False),
    "left_transposed": (1, 4, 6, 5, 1.0, 1.0, True, False),
    "right_transposed": (1, 4, 6, 5, 1.0, 1.0, False, True),
    "both_transposed_grouped": (3, 3, 4, 5, 2.0, -1.0, True, True),
    "vector_1x1000x1": (1, 1, 1000, 1, 1.0, 1.0, False, False),
    "empty_k_5x0x4": (1, 5, 0, 4, 1.0, 1.0, False, False),
}


NORM_CASES = {
    # (batch, chans, field elements, unbiased variance, stable algorithm)
    "bn_4x8x25": (4, 8, 25, False, False),
    "bn_unbiased": (3, 5, 7, True, False),
    "bn_stable": (2, 16, 9, False, True),
    "bn_stable_unbiased": (5, 3, 4, True, True),
    "bn_single_element": (1, 4, 1, True, False),
}


def main():
    if not oracle.have_ref():
        raise SystemExit("oracle/_ref/libpoplibs_test_ref.so is missing: run `make -C oracle ref`")
    out = {}
    meta = {}
    for idx, (name, spec) in enumerate(sorted(CONV_CASES.items())):
        r = np.random.default_rng(1000 + idx)
        xs, ws, ys = oracle._shapes(spec)
        x = r.uniform(-2, 2, xs)
        w = r.uniform(-1, 1, ws)
        bias = r.uniform(-2, 6, ys[1])
        dy = r.uniform(-3, 3, ys)
        out[f"conv/{name}/x"] = x
        out[f"conv/{name}/w"] = w
        out[f"conv/{name}/bias"] = bias
        out[f"conv/{name}/dy"] = dy
        out[f"conv/{name}/y"] = oracle.conv_fwd(spec, x, w, bias, use_ref=True)
        out[f"conv/{name}/dx"] = oracle.conv_bwd(spec, dy, w, use_ref=True)
        n = spec.normalised()
        # The reference's weightUpdate model mis-sizes the padded gradients when
        # a dimension has both output truncation and a stride above one (it adds
        # the truncation at lib/poplibs_test/Convolution.cpp:792-794 where the
        # forward model subtracts it), so no golden dW is taken for such cases.
        wu_ok = all(s == 1 or (lo == 0 and hi == 0) for s, lo, hi in
                    zip(n["stride"], n["out_trunc_lo"], n["out_trunc_hi"]))
        if wu_ok:
            dw, db = oracle.conv_wu(spec, x, dy, use_ref=True)
            out[f"conv/{name}/dw"] = dw
            out[f"conv/{name}/db"] = db
        d = spec.normalised()
        d.update(batch=spec.batch, in_chans=spec.in_chans, out_chans=spec.out_chans,
                 groups=spec.groups, out_field=spec.out_field())
        meta[f"conv/{name}"] = d
    for idx, (name, (g, m, k, n, alpha, beta, ta, tb)) in enumerate(sorted(GEMM_CASES.items())):
        r = np.random.default_rng(2000 + idx)
        a = r.uniform(-4, 4, (g, k, m) if ta else (g, m, k))
        b = r.uniform(-3, 3, (g, n, k) if tb else (g, k, n))
        c = r.uniform(-2, 2, (g, m, n))
        out[f"gemm/{name}/a"] = a
        out[f"gemm/{name}/b"] = b
        out[f"gemm/{name}/c"] = c
        out[f"gemm/{name}/d"] = oracle.gemm(a, b, c, alpha, beta, ta, tb, use_ref=True)
        meta[f"gemm/{name}"] = dict(groups=g, m=m, k=k, n=n, alpha=alpha, beta=beta,
                                    transpose_a=ta, transpose_b=tb)
    # batch normalisation (lib/poplibs_test/Norms.cpp, BatchNorm): shapes echo the
    # reference's norm layer tests (tests/popnn/BatchNormTest / NormLayerTests:
    # small batches of a few channels, fields of one and two dimensions)
    for idx, (name, (b, c, f, unbiased, stable)) in enumerate(sorted(NORM_CASES.items())):
        r = np.random.default_rng(3000 + idx)
        x = r.normal(0.5, 2.0, (b, c, f))
        g = r.uniform(-1, 1, (b, c, f))
        gamma, beta = r.uniform(0.5, 2.0, c), r.uniform(-1, 1, c)
        mean, inv = oracle.norm_statistics(x, 1e-3, unbiased, stable, use_ref=True)
        y, white = oracle.norm_normalise(x, gamma, beta, mean, inv, use_ref=True)
        dx = oracle.norm_gradients(white, g, inv, gamma, use_ref=True)
        gamma2, beta2 = oracle.norm_param_update(white, g, 0.25, gamma, beta, use_ref=True)
        for key, val in dict(x=x, g=g, gamma=gamma, beta=beta, mean=mean, inv_std=inv, y=y, whitened=white,
                             dx=dx, gamma_updated=gamma2, beta_updated=beta2).items():
            out[f"norm/{name}/{key}"] = val
        meta[f"norm/{name}"] = dict(batch=b, chans=c, field=f, eps=1e-3, unbiased=unbiased, stable=stable,
                                    learning_rate=0.25)
    np.savez_compressed(os.path.join(HERE, "poplibs_test_models.npz"), **out)
    with open(os.path.join(HERE, "poplibs_test_models.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print(f"wrote {len(meta)} cases")


if __name__ == "__main__":
    main()
