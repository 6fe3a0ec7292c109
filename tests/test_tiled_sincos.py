"""The branch-free sine / cosine of the Tiled broadcast kernel: its CPU restatement (tests/sincos_ref.c, built here
with the constants read from the kernel source) stays within 1.54 ulp of the exact value on strided sweeps of every
f32 argument up to the kernel's limit (the full sweep of all 1.2e9 arguments gives 1.532), and the GPU produces the
restatement's results bit for bit; arguments over the limit, infinities and NaN take the library functions."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def sincos(tmp_path_factory):
    src = open(os.path.join(ROOT, "cutile.jl_b200", "csrc", "tiled.cu")).read()
    body = src[src.index("sincos_reduced(float x) {"):]
    body = body[: body.index("const float ax")]
    defs = dict(re.findall(r"\b(kTwoOverPi|kMagic|P1|P2|P3|S0|S1|S2|C0|C1|C2) = ([-+0-9a-fA-Fxp.e]+f)", body))
    assert len(defs) == 11, defs
    defs["TWO_OVER_PI"], defs["MAGIC"] = defs.pop("kTwoOverPi"), defs.pop("kMagic")
    limit = float(re.search(r"kSinCosLimit = ([0-9.]+)f", src).group(1))
    out = str(tmp_path_factory.mktemp("sincos") / "libsincos_ref.so")
    cmd = ["gcc", "-O2", "-mfma", "-ffp-contract=off", "-shared", "-fPIC", os.path.join(ROOT, "tests", "sincos_ref.c"), "-o", out,
           "-lm"] + [f"-D{k}={v}" for k, v in defs.items()]
    subprocess.run(cmd, check=True)
    lib = C.CDLL(out)
    lib.sincos_max_ulp.restype = C.c_double
    lib.sincos_max_ulp.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32, C.c_int]
    lib.sincos_ref.argtypes = [C.c_void_p, C.c_void_p, C.c_long, C.c_int]
    return lib, limit


def test_restatement_is_within_the_stated_error(sincos):
    lib, limit = sincos
    top = int(np.float32(limit).view(np.uint32))
    for want_cos in (0, 1):
        worst = max(lib.sincos_max_ulp(first, top, 1009, want_cos) for first in (0, 313))     # 2.4e6 arguments
        worst = max(worst, lib.sincos_max_ulp(int(np.float32(1e-3).view(np.uint32)), int(np.float32(8.0).view(np.uint32)), 97, want_cos))
        assert 0.5 < worst <= 1.54, worst


def test_restatement_special_values(sincos):
    lib, _ = sincos
    x = np.array([0.0, -0.0, 1e-45, -1e-45, np.pi, -np.pi / 2], dtype=np.float32)
    for want_cos in (0, 1):
        y = np.empty_like(x)
        lib.sincos_ref(x.ctypes.data, y.ctypes.data, x.size, want_cos)
        if want_cos:
            assert y[0] == 1.0 and y[1] == 1.0 and y[2] == 1.0
        else:
            assert y[0] == 0.0 and not np.signbit(y[0]) and y[1] == 0.0 and np.signbit(y[1])      # sin(-0) = -0
            assert y[2] == x[2] and y[3] == x[3]                                                  # subnormals: sin(x) = x


@pytest.mark.gpu
def test_gpu_matches_the_restatement_bit_for_bit(cuda, sincos):
    import torch
    lib, limit = sincos
    T = cuda.tiled
    g = np.random.default_rng(70)
    n = 1 << 18
    x = np.concatenate([g.uniform(-1, 1, n), g.uniform(-100, 100, n), g.uniform(-limit, limit, n),
                        np.ldexp(g.uniform(-1, 1, n), g.integers(-140, 0, n))]).astype(np.float32)
    x[:4] = [0.0, -0.0, limit, -limit]
    X = torch.from_numpy(x).cuda()
    for want_cos, f in ((0, T.sin), (1, T.cos)):
        want = np.empty_like(x)
        lib.sincos_ref(x.ctypes.data, want.ctypes.data, x.size, want_cos)
        got = T.materialize(f(T.Tiled(X))).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.gpu
def test_gpu_huge_and_non_finite_arguments(cuda):
    import torch
    T = cuda.tiled
    g = np.random.default_rng(71)
    x = g.uniform(-1, 1, 4096).astype(np.float32)
    x[5], x[77], x[1000], x[2049], x[4000] = 3.0e5, -1.0e30, np.inf, np.nan, 1.0e6    # in different threads' groups
    X = torch.from_numpy(x).cuda()
    for f, ref in ((T.sin, np.sin), (T.cos, np.cos)):
        got = T.materialize(f(T.Tiled(X))).cpu().numpy().astype(np.float64)
        with np.errstate(invalid="ignore"):
            want = ref(x.astype(np.float64))
        assert np.isnan(got[1000]) and np.isnan(got[2049])
        ok = np.isfinite(want)
        assert np.abs(got[ok] - want[ok]).max() <= 2.5e-7
