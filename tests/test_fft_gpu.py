"""GPU parity of the batched three-stage FFT against the float64 oracle (the reference example's stages restated with
its own tables) and against the plain DFT the example checks with; tolerance: relative Frobenius norm <= 1e-5 (the
example accepts 1e-4, examples/fft.jl:243-247), the f32 tables bound the error from below at about 5e-8."""
import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _run(cuda, d, D=None, BS=1):
    import torch
    f = d["factors"]
    tabs = ref.fft_make_twiddles(f)
    dev = [torch.from_numpy(t).cuda() for t in tabs]
    x = torch.from_numpy(d["input"]).cuda()
    N = d["n"]
    D = D or min(64, 2 * N)
    xp = torch.view_as_real(x).view(d["batch"], 2 * N // D, D)
    yp = torch.full_like(xp, float("nan"))
    cuda.fft.fft_kernel(xp, yp, *dev, N, f[0], f[1], f[2], BS, D)
    y = torch.view_as_complex(yp.view(d["batch"], N, 2)).cpu().numpy()
    return y, tabs


def _planes(z):
    return np.stack([z.real, z.imag])


# (batch, factors): the example's own cases (main(): 64 and 32 x (8, 8, 8); prepare() defaults 2 x (2, 2, 2) and the
# benchmark 256 x (16, 16, 16)), mixed and degenerate factors, the largest size.
@pytest.mark.parametrize("batch,factors", [(2, (2, 2, 2)), (64, (8, 8, 8)), (32, (8, 8, 8)), (256, (16, 16, 16)),
                                           (5, (4, 8, 16)), (3, (32, 2, 8)), (2, (1, 4, 2)), (1, (1, 1, 1)),
                                           (7, (32, 16, 16)), (3, (16, 32, 8))])
def test_fft_matches_oracle(cuda, batch, factors):
    d = inputs.fft(batch, factors, seed=11 + batch)
    y, tabs = _run(cuda, d)
    want = ref.fft_three_stage(d["input"], *tabs, factors)
    assert ref.rel_fro(_planes(y), _planes(want)) <= TOL
    assert ref.rel_fro(_planes(y), _planes(ref.fft(d["input"]))) <= TOL
    cuda.check_device_status(0)


def test_fft_known_answers(cuda):
    """A unit impulse at position p transforms to exp(-2 pi i p k / N); a constant to N at k = 0."""
    f, N = (8, 8, 8), 512
    x = np.zeros((3, N), dtype=np.complex64)
    x[0, 0] = 1
    x[1, 5] = 1j
    x[2, :] = 1
    y, _ = _run(cuda, dict(input=x, factors=f, batch=3, n=N))
    k = np.arange(N)
    assert np.abs(y[0] - 1).max() <= 1e-5
    assert np.abs(y[1] - 1j * np.exp(-2j * np.pi * 5 * k / N)).max() <= 1e-5
    assert abs(y[2, 0] - N) <= 1e-3 and np.abs(y[2, 1:]).max() <= 1e-3


def test_fft_linearity_and_packing_at_benchmark_size(cuda):
    """fft(a x + b z) = a fft(x) + b fft(z) at batch 256 x 4096 points; the packing dimension D changes nothing."""
    d1, d2 = inputs.fft(256, (16, 16, 16), seed=1), inputs.fft(256, (16, 16, 16), seed=2)
    y1, _ = _run(cuda, d1)
    y2, _ = _run(cuda, d2, D=2)
    mix = dict(d1, input=(np.float32(0.5) * d1["input"] - np.float32(2.0) * d2["input"]).astype(np.complex64))
    y3, _ = _run(cuda, mix, D=8192, BS=4)
    assert ref.rel_fro(_planes(y3), _planes(0.5 * y1 - 2.0 * y2)) <= TOL
    y1b, _ = _run(cuda, d1, D=16)
    assert np.array_equal(y1, y1b)


def test_fft_plan_surface(cuda):
    import torch
    d = inputs.fft(8, (8, 8, 8), seed=3)
    plan = cuda.fft.FftPlan((8, 8, 8), "cuda")
    out = plan(torch.from_numpy(d["input"]).cuda()).cpu().numpy()
    assert ref.rel_fro(_planes(out), _planes(ref.fft(d["input"]))) <= TOL
    for a, b in zip(cuda.fft.make_twiddles((8, 8, 8)), ref.fft_make_twiddles((8, 8, 8))):
        assert np.array_equal(a, b)


def test_fft_rejections(cuda):
    import torch
    lib = cuda._lib
    d = inputs.fft(2, (2, 2, 2))
    tabs = [torch.from_numpy(t).cuda() for t in ref.fft_make_twiddles((2, 2, 2))]
    x = torch.view_as_real(torch.from_numpy(d["input"]).cuda()).view(2, 1, 16)
    y = torch.empty_like(x)
    with pytest.raises(cuda.CtbError) as e:
        cuda.fft.fft_kernel(x, y, *tabs, 8, 2, 2, 4, 1, 16)           # table sizes do not fit the factors
    assert e.value.status == lib.BAD_ARG
    with pytest.raises(cuda.CtbError) as e:
        cuda.fft.fft_kernel(x, y, *tabs, 8, 2, 2, 2, 1, 32)           # 2N not divisible by the packing dimension
    assert e.value.status == lib.BAD_ARG
    with pytest.raises(cuda.CtbError) as e:
        cuda.fft.fft_kernel(x, y, *tabs, 8, 2, 2, 2, 4, 16)           # batch 2 is not a multiple of BS = 4
    assert e.value.status == lib.BAD_ARG
    t3 = [torch.zeros(3, 3, 2, device="cuda")] * 3 + [torch.zeros(3, 9, 2, device="cuda"), torch.zeros(3, 3, 2, device="cuda")]
    x3 = torch.zeros(2, 1, 54, device="cuda")
    with pytest.raises(cuda.CtbError) as e:
        cuda.fft.fft_kernel(x3, torch.empty_like(x3), *t3, 27, 3, 3, 3, 1, 2)  # tile dimensions are powers of two
    assert e.value.status == lib.UNSUPPORTED_TILE
