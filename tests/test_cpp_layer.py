"""The C++ poplar / poplin layer: host-only checks (graph construction, options,
ConvParams algebra) run here without a GPU; the tool ports run on the GPU and
their dumped tensors are compared with the oracle."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "poplibs_b200")


def compile_cpp(source, output):
    from poplibs_b200 import build
    build.build_poplin()
    cmd = ["g++", "-std=c++17", "-O1", "-I" + os.path.join(ROOT, "include"),
           "-I" + os.path.join(ROOT, "poplibs_b200", "tools"), source, "-o", output,
           "-L" + LIBDIR, "-lpoplin_b200", "-lpoplibs_b200", "-Wl,-rpath," + LIBDIR]
    subprocess.run(cmd, check=True)


def test_poplin_host_layer(tmp_path):
    exe = str(tmp_path / "test_poplin_host")
    compile_cpp(os.path.join(ROOT, "tests", "cpp", "test_poplin_host.cpp"), exe)
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all host checks passed" in out.stdout


def tool(name):
    from poplibs_b200 import build
    build.build_tools()
    return os.path.join(LIBDIR, "tools", "bin", name)


def test_tools_build_graphs_without_a_device():
    out = subprocess.run([tool("single_conv_layer"), "--input-channels=64", "--output-channels=64",
                          "--field={56,56}", "--kernel-size=3", "--padding=1", "--batch-size=32", "--bias=0",
                          "--single-phase=all", "--report-plan", "--compile-only"],
                         capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    assert "CTA tile (pixels x chans)  128 x 64" in out.stdout
    assert "weight update (split-K)" in out.stdout
    out = subprocess.run([tool("general_matrix_multiply"), "--m", "8192", "--k", "8192", "--n", "8192",
                          "--report-plan", "--compile-only"], capture_output=True, text=True, timeout=60)
    assert out.returncode == 0, out.stderr
    assert "128 x 256" in out.stdout
    # the reference tools' error conventions: unknown options and bad option values fail
    bad = subprocess.run([tool("general_matrix_multiply"), "--m", "8", "--k", "8", "--n", "8",
                          "--partials-type", "double", "--compile-only"], capture_output=True, text=True)
    assert bad.returncode == 1 and "Invalid value 'double' for option 'partialsType'" in bad.stderr
    bad = subprocess.run([tool("single_conv_layer"), "--input-channels=8", "--output-channels=8",
                          "--field={4,4}", "--kernel-size=3", "--stride=0", "--compile-only"],
                         capture_output=True, text=True)
    assert bad.returncode == 1 and "Stride must be non zero" in bad.stderr


def load_dump(directory):
    import numpy as np
    tensors = {}
    with open(os.path.join(directory, "manifest.txt")) as f:
        for line in f:
            name, *shape = line.split()
            tensors[name] = np.fromfile(os.path.join(directory, name + ".f64")).reshape([int(s) for s in shape])
    return tensors


@pytest.mark.gpu
def test_general_matrix_multiply_tool_against_oracle(tmp_path):
    import numpy as np
    import oracle
    cases = [
        (["--m", "512", "--k", "1024", "--n", "1024", "--beta", "0"], 1e-3),
        (["--m", "300", "--k", "200", "--n", "72", "--g", "2", "--alpha", "0.5", "--beta", "1"], 1e-3),
        (["--m", "64", "--k", "136", "--n", "40", "--left-matrix-op", "transpose", "--beta", "1", "--integer-data",
          "--output-type", "float"], 0.0),
        (["--m", "64", "--k", "136", "--n", "40", "--right-matrix-op", "transpose", "--beta", "0", "--integer-data",
          "--output-type", "float"], 0.0),
        (["--m", "1", "--k", "1000", "--n", "1", "--beta", "1", "--integer-data", "--output-type", "float"], 0.0),
        (["--m", "5", "--k", "0", "--n", "4", "--beta", "1", "--integer-data"], 0.0),
        # float data (the tool's "--data-type float"): three bfloat16 terms per product
        (["--m", "96", "--k", "200", "--n", "72", "--g", "2", "--data-type", "float", "--alpha", "0.5", "--beta", "1",
          "--integer-data"], 0.0),
        (["--m", "300", "--k", "520", "--n", "136", "--data-type", "float", "--beta", "0"], 1e-4),
        (["--m", "256", "--k", "512", "--n", "256", "--input-type", "quarter", "--fp8-scale-A=-3", "--fp8-scale-B=-2",
          "--beta", "0"], 0.0),
        # the 1-5-2 format (the reference tool's default), alone and mixed with 1-4-3
        (["--m", "256", "--k", "512", "--n", "256", "--input-type", "quarter", "--fp8-format-A=F152",
          "--fp8-format-B=F152", "--fp8-scale-A=-3", "--fp8-scale-B=-2", "--beta", "0"], 0.0),
        (["--m", "200", "--k", "256", "--n", "136", "--input-type", "quarter", "--fp8-format-A=F143",
          "--fp8-format-B=F152", "--fp8-scale-A=1", "--fp8-scale-B=0", "--beta", "0"], 0.0),
    ]
    for i, (flags, tol) in enumerate(cases):
        d = tmp_path / f"gemm{i}"
        d.mkdir()
        out = subprocess.run([tool("general_matrix_multiply"), "--dump-dir", str(d)] + flags,
                             capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, f"{flags}: {out.stderr}"
        t = load_dump(str(d))
        alpha = float(flags[flags.index("--alpha") + 1]) if "--alpha" in flags else 1.0
        beta = float(flags[flags.index("--beta") + 1]) if "--beta" in flags else 1.0
        ta = "--left-matrix-op" in flags
        tb = "--right-matrix-op" in flags
        expect = oracle.gemm(t["A"], t["B"], t["C"], alpha, beta, ta, tb)
        if tol == 0.0:
            assert (t["D"] == expect).all(), flags
        else:
            rms = float(np.sqrt(np.mean(expect * expect)))
            bad, first, worst = oracle.check_is_close(t["D"], expect, tol, max(1e-5, 0.25 * tol * rms))
            assert bad == 0, (flags, bad, worst)


@pytest.mark.gpu
def test_fully_connected_layer_tool_against_oracle(tmp_path):
    """Forward, backward and weight-update passes of a (grouped) fully connected
    layer through matMulGrouped / transposeGroupedMatrix / matMul[Grouped]Acc,
    on small-integer data: every sum is exact, so the dumps must equal the
    model's products bit for bit (after the cast to the output type)."""
    import numpy as np
    import oracle
    cases = [
        ["--input-size", "256", "--output-size", "128", "--batch-size", "64", "--integer-data", "--learning-rate", "0.25"],
        ["--input-size", "72", "--output-size", "40", "--batch-size", "24", "--num-groups", "3", "--integer-data",
         "--learning-rate", "0.5", "--output-type", "float"],
        ["--input-size", "128", "--output-size", "64", "--batch-size", "16", "--bias", "0", "--integer-data",
         "--single-phase", "bwd"],
        ["--input-size", "256", "--output-size", "128", "--batch-size", "32", "--input-type", "quarter",
         "--fp8-scale-fwd=-1", "--fp8-scale-weights=0", "--fp8-scale-bwd=1"],
        ["--input-size", "64", "--output-size", "64", "--batch-size", "8", "--inference-only", "--integer-data"],
    ]
    for i, flags in enumerate(cases):
        d = tmp_path / f"fc{i}"
        d.mkdir()
        out = subprocess.run([tool("fully_connected_layer"), "--dump-dir", str(d)] + flags,
                             capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, f"{flags}: {out.stderr}"
        t = load_dump(str(d))
        lr = float(flags[flags.index("--learning-rate") + 1]) if "--learning-rate" in flags else 0.5
        out_f32 = "float" in flags
        cast = (lambda a: a.astype(np.float32).astype(np.float64)) if out_f32 else \
               (lambda a: a.astype(np.float16).astype(np.float64))
        x, w = t["prevAct"], t["weights"]
        if "nextAct" in t:
            y = oracle.gemm(x, w)
            if "biases" in t:
                # the product is cast to the output type first, then the bias is added in that type
                y = cast(cast(y) + t["biases"][:, None, :])
            assert (t["nextAct"] == cast(y)).all(), flags
        if "prevDeltas" in t:
            dx = oracle.gemm(t["zDeltas"], w, transpose_b=True)
            assert (t["prevDeltas"] == cast(dx)).all(), flags
        if "weightsUpdated" in t:
            dw = oracle.gemm(x, t["zDeltas"], transpose_a=True)
            in_cast = lambda a: a.astype(np.float16).astype(np.float64)  # noqa: E731 weights have the input type
            assert (t["weightsUpdated"] == in_cast(w - lr * dw)).all(), flags
            if "biasesUpdated" in t:
                db = t["zDeltas"].sum(axis=1)
                assert (t["biasesUpdated"] == cast(t["biases"] - lr * db)).all(), flags
        if "--inference-only" in flags:
            assert "prevDeltas" not in t and "weightsUpdated" not in t


@pytest.mark.gpu
def test_single_conv_layer_tool_against_oracle(tmp_path):
    import numpy as np
    import oracle
    from oracle import ConvSpec
    cases = [
        dict(flags=["--input-channels=64", "--output-channels=64", "--field={14,14}", "--kernel-size=3",
                    "--padding=1", "--batch-size=4", "--integer-data", "--learning-rate=0.5"],
             spec=ConvSpec.simple(4, [14, 14], [3, 3], 64, 64, padding=1), bias=True),
        dict(flags=["--input-channels=72", "--output-channels=40", "--field={7,9}", "--kernel-size={3,2}",
                    "--padding-lower={2,0}", "--padding-upper={0,1}", "--batch-size=3", "--bias=0",
                    "--integer-data", "--learning-rate=0.25"],
             spec=ConvSpec(3, [7, 9], [3, 2], 72, 40, in_pad_lo=[2, 0], in_pad_hi=[0, 1]), bias=False),
        dict(flags=["--input-channels=64", "--output-channels=64", "--field={9,9}", "--kernel-size=3",
                    "--padding=1", "--stride=2", "--batch-size=2", "--bias=0", "--integer-data",
                    "--single-phase=fwd"],
             spec=ConvSpec.simple(2, [9, 9], [3, 3], 64, 64, padding=1, stride=2), bias=False),
        # strided layers in all passes; on an even field a 1x1 stride-2 layer leaves the
        # last row and column unused (input truncation in the canonical parameters)
        dict(flags=["--input-channels=64", "--output-channels=128", "--field={12,12}", "--kernel-size=1",
                    "--stride=2", "--batch-size=3", "--bias=0", "--integer-data", "--learning-rate=0.5"],
             spec=ConvSpec.simple(3, [12, 12], [1, 1], 64, 128, stride=2), bias=False),
        dict(flags=["--input-channels=64", "--output-channels=64", "--field={12,11}", "--kernel-size=3",
                    "--padding=1", "--stride=2", "--batch-size=2", "--integer-data", "--learning-rate=0.25"],
             spec=ConvSpec.simple(2, [12, 11], [3, 3], 64, 64, padding=1, stride=2), bias=True),
        # a dilated input without the transpose flag (a transposed convolution written as a
        # forward one) and a flipped input, forward pass
        dict(flags=["--input-channels=64", "--output-channels=72", "--field={6,7}", "--kernel-size=3",
                    "--padding=2", "--in-dilation=2", "--batch-size=2", "--bias=0", "--integer-data",
                    "--single-phase=fwd"],
             spec=ConvSpec(2, [6, 7], [3, 3], 64, 72, in_pad_lo=[2, 2], in_pad_hi=[2, 2], in_dilation=[2, 2]),
             bias=False),
        dict(flags=["--input-channels=64", "--output-channels=64", "--field={7,8}", "--kernel-size=3",
                    "--padding-lower={2,0}", "--padding-upper={0,1}", "--flip-input={1,1}", "--batch-size=2",
                    "--bias=0", "--integer-data", "--learning-rate=0.5"],
             spec=ConvSpec(2, [7, 8], [3, 3], 64, 64, in_pad_lo=[2, 0], in_pad_hi=[0, 1], in_flip=[1, 1]),
             bias=False),
        dict(flags=["--input-channels=32", "--output-channels=32", "--field={6,6}", "--kernel-size=3",
                    "--padding=1", "--conv-groups=2", "--batch-size=2", "--bias=0", "--integer-data",
                    "--learning-rate=0.5"],
             spec=ConvSpec.simple(2, [6, 6], [3, 3], 32, 32, padding=1, groups=2), bias=False),
        # a 3-D field in all three passes
        dict(flags=["--input-channels=16", "--output-channels=24", "--field={5,6,6}", "--kernel-size=3",
                    "--padding=1", "--batch-size=2", "--bias=0", "--integer-data", "--learning-rate=0.5"],
             spec=ConvSpec.simple(2, [5, 6, 6], [3, 3, 3], 16, 24, padding=1), bias=False),
        dict(flags=["--input-channels=16", "--output-channels=16", "--field={6,7,7}", "--kernel-size=3",
                    "--padding=1", "--stride={2,1,2}", "--batch-size=2", "--integer-data", "--learning-rate=0.5"],
             spec=ConvSpec.simple(2, [6, 7, 7], [3, 3, 3], 16, 16, padding=1, stride=[2, 1, 2]), bias=True),
        dict(flags=["--input-channels=128", "--output-channels=64", "--field={8,8}", "--kernel-size=3",
                    "--padding=1", "--batch-size=2", "--bias=0", "--input-type=quarter",
                    "--fp8-scale-fwd=1", "--fp8-scale-weights=0", "--fp8-scale-bwd=1"],
             spec=ConvSpec.simple(2, [8, 8], [3, 3], 128, 64, padding=1), bias=False),
    ]
    cases.append(dict(flags=["--input-channels=24", "--output-channels=40", "--field={9,8}", "--kernel-size=3",
                             "--padding=1", "--stride={2,1}", "--batch-size=3", "--data-type=float",
                             "--integer-data", "--learning-rate=0.5"],
                      spec=ConvSpec.simple(3, [9, 8], [3, 3], 24, 40, padding=1, stride=[2, 1]), bias=True,
                      store=np.float32))
    for i, case in enumerate(cases):
        d = tmp_path / f"conv{i}"
        d.mkdir()
        out = subprocess.run([tool("single_conv_layer"), "--dump-dir", str(d)] + case["flags"],
                             capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, f"{case['flags']}: {out.stderr}"
        t = load_dump(str(d))
        spec = case["spec"]
        flat = lambda a, lead: a.reshape(a.shape[0], a.shape[1], -1) if lead == 2 else a.reshape(*a.shape[:3], -1)  # noqa: E731
        x, w0 = flat(t["prevAct"], 2), flat(t["weights"], 3)
        if "nextAct" in t:
            y = oracle.conv_fwd(spec, x, w0, t.get("biases") if case["bias"] else None)
            assert (flat(t["nextAct"], 2) == y).all(), case["flags"]
        if "prevDeltas" in t:
            dx = oracle.conv_bwd(spec, flat(t["zDeltas"], 2), w0)
            assert (flat(t["prevDeltas"], 2) == dx).all(), case["flags"]
        if "weightDeltas" in t:
            dw, _ = oracle.conv_wu(spec, x, flat(t["zDeltas"], 2))
            assert (flat(t["weightDeltas"], 3) == dw).all(), case["flags"]
            lr = float([f for f in case["flags"] if f.startswith("--learning-rate")][0].split("=")[1])  # exact in half
            store = case.get("store", np.float16)
            expect = (w0 - lr * dw).astype(store).astype(np.float64)
            assert (flat(t["weightsUpdated"], 3) == expect).all(), case["flags"]
            if case["bias"]:
                # biases += -lr * sum of the output gradients (fp32 sums, cast to the bias type)
                _, db = oracle.conv_wu(spec, x, flat(t["zDeltas"], 2))
                expect_b = (t["biases"].ravel() - lr * db).astype(store).astype(np.float64)
                assert (t["biasesUpdated"].ravel() == expect_b).all(), case["flags"]


@pytest.mark.gpu
def test_multiconv_on_gpu_against_oracle(tmp_path):
    """poplin::multiconv (two different layers at once: a padded 3x3 and a
    grouped strided 1x1 with fp32 output) through the Engine: forward outputs,
    weight gradients and updated weights of both must equal the CPU model bit
    for bit on small-integer data."""
    import numpy as np
    import oracle
    from oracle import ConvSpec
    exe = str(tmp_path / "multiconv_gpu")
    compile_cpp(os.path.join(ROOT, "tests", "cpp", "multiconv_gpu.cpp"), exe)
    d = tmp_path / "dump"
    d.mkdir()
    out = subprocess.run([exe, str(d)], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    t = load_dump(str(d))
    specs = [ConvSpec.simple(3, [12, 12], [3, 3], 64, 72, padding=1),
             ConvSpec.simple(2, [9, 10], [1, 1], 32, 48, stride=2, groups=2)]
    for i, spec in enumerate(specs):
        x, w, dy = t[f"in{i}"], t[f"w{i}"], t[f"dy{i}"]
        y = oracle.conv_fwd(spec, x, w).reshape(t[f"out{i}"].shape)
        assert (t[f"out{i}"] == y).all(), f"multiconv forward {i}"
        dw = oracle.conv_wu(spec, x, dy)[0].reshape(w.shape)
        got = t[f"dw{i}"]
        assert (got == dw.astype(np.float16).astype(np.float64)).all(), f"multiconv weight gradient {i}"
        upd = (w + -0.5 * dw).astype(np.float16).astype(np.float64)
        assert (t[f"wUpdated{i}"] == upd).all(), f"multiconv weight update {i}"


@pytest.mark.gpu
def test_convolution_then_batch_norm_on_gpu_against_oracle(tmp_path):
    """poplin::convolution followed by the Norms chain (statistics, whiten,
    normalise; then the three gradients) through the Engine, each stage against
    the CPU models fed with the device's own inputs to that stage."""
    import numpy as np
    import oracle
    from oracle import ConvSpec
    exe = str(tmp_path / "conv_norm_gpu")
    compile_cpp(os.path.join(ROOT, "tests", "cpp", "conv_norm_gpu.cpp"), exe)
    d = tmp_path / "dump"
    d.mkdir()
    run = subprocess.run([exe, str(d)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    t = load_dump(str(d))

    def close(got, want, rel, what):
        want = np.asarray(want, dtype=np.float64).reshape(got.shape)
        rms = float(np.sqrt(np.mean(want * want)))
        bad, first, worst = oracle.check_is_close(got, want, rel, max(1e-6, rel * rms))
        assert bad == 0, (what, bad, got.ravel()[first], want.ravel()[first])
    spec = ConvSpec.simple(4, [10, 10], [3, 3], 16, 32, padding=1)
    close(t["y"], oracle.conv_fwd(spec, t["in"], t["w"]), 1e-3, "convolution")
    mean, inv = oracle.norm_statistics(t["y"], 1e-3, unbiased=True)
    close(t["mean"], mean, 2e-3, "mean")
    close(t["iStdDev"], inv, 5e-3, "inverse standard deviation")
    out, white = oracle.norm_normalise(t["y"], t["gamma"], t["beta"], t["mean"], t["iStdDev"])
    close(t["white"], white, 2e-3, "whitened")
    close(t["out"], t["gamma"][None, :, None, None] * t["white"] + t["beta"][None, :, None, None], 2e-3, "normalised")
    close(t["gradWhite"], t["gradOut"] * t["gamma"][None, :, None, None], 2e-3, "normGradients")
    zero = np.zeros(32)
    ga, be = oracle.norm_param_update(t["white"], t["gradOut"], 1.0, zero, zero)
    close(t["gammaGrad"], -ga, 4e-3, "gamma gradient")
    close(t["betaGrad"], -be, 4e-3, "beta gradient")
    close(t["gradY"], oracle.norm_gradients(t["white"], t["gradWhite"], t["iStdDev"], np.ones(32)), 4e-3,
          "normStatisticsGradients")
