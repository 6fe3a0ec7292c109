"""GPU parity of the row-softmax kernels against the float64 oracle.

Tolerance (f32): max|out-ref| / max|ref| <= 1e-5; the reference's own check is
per row atol=1e-5, rtol=1e-4 (examples/softmax.jl:185)."""
import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu
TOL = 1e-5


def run(cuda, x, variant, tile=None, out=None):
    import torch
    sm = cuda.softmax
    xin = x if isinstance(x, torch.Tensor) else torch.from_numpy(x).cuda()
    out = torch.empty_like(xin) if out is None else out
    N = xin.shape[1]
    if variant == 0:
        sm.softmax_tma_kernel(out, xin, tile or sm.next_power_of_2(N))
    else:
        sm.softmax_chunked_kernel(out, xin, N, tile or 1024)
    torch.cuda.synchronize()
    return out


# the reference's main() cases (examples/softmax.jl:248-256) + ragged and long rows
@pytest.mark.parametrize("M,N", [(256, 256), (1024, 1024), (4096, 4096), (37, 1000), (3, 8192), (1, 4)])
@pytest.mark.parametrize("variant", [0, 1])
def test_softmax_parity(cuda, M, N, variant):
    x = inputs.softmax(M=M, N=N, seed=1)["input"]
    out = run(cuda, x, variant).cpu().numpy()
    want = ref.softmax(x)
    assert ref.max_abs_over_max(out, want) <= TOL
    assert ref.max_rel(out, want) <= 1e-3  # element-wise relative error with the floor 1e-3 * max|ref|
    assert np.abs(out.astype(np.float64).sum(axis=1) - 1).max() < 1e-5
    # the reference's own per-row criterion
    err = np.linalg.norm(out - want, axis=1)
    assert (err <= np.maximum(1e-5, 1e-4 * np.linalg.norm(want, axis=1))).all()


# rows kept in registers, rows kept whole in shared memory (up to 200 KB), rows that are re-read; odd lengths
@pytest.mark.parametrize("M,N", [(5, 333), (2, 20000), (9, 1), (300, 32768), (3, 51200), (2, 60000), (4, 12004)])
def test_softmax_chunked_any_length(cuda, M, N):
    x = inputs.softmax(M=M, N=N, seed=7)["input"]
    out = run(cuda, x, 1).cpu().numpy()
    want = ref.softmax(x)
    assert ref.max_abs_over_max(out, want) <= TOL
    assert ref.max_rel(out, want) <= 1e-3  # element-wise, floored at 1e-3 of the largest probability
    assert np.abs(out.astype(np.float64).sum(axis=1) - 1).max() < 1e-5


def test_softmax_long_f16_rows(cuda):
    x = inputs.softmax(M=5, N=65536, seed=4)["input"].astype(np.float16)  # 128 KB rows: the shared-memory path
    out = run(cuda, x, 1).cpu().numpy()
    assert ref.max_abs_over_max(out, ref.softmax(x)) <= 1e-3


def test_softmax_f16(cuda):
    x = inputs.softmax(M=64, N=2048, seed=3)["input"].astype(np.float16)
    for variant in (0, 1):
        out = run(cuda, x, variant).cpu().numpy()
        assert out.dtype == np.float16
        assert ref.max_abs_over_max(out, ref.softmax(x)) <= 1e-3  # one f16 rounding of the result


def test_softmax_strided_rows_and_extremes(cuda):
    import torch
    x = inputs.softmax(M=16, N=512, seed=2)["input"]
    x[0, :] = -1e30
    x[1, 5] = 1e30
    x[2, :] = 88.0
    big = torch.zeros(16, 640, device="cuda")
    big[:, :512] = torch.from_numpy(x).cuda()
    outbig = torch.full((16, 768), 7.0, device="cuda")
    want = ref.softmax(x)
    for variant in (0, 1):
        run(cuda, big[:, :512], variant, out=outbig[:, :512])
        assert ref.max_abs_over_max(outbig[:, :512].cpu().numpy(), want) <= TOL
        assert (outbig[:, 512:] == 7.0).all()  # nothing written beyond the row


def test_softmax_rejections(cuda):
    import torch
    lib = cuda._lib
    x = torch.zeros(4, 333, device="cuda")
    with pytest.raises(cuda.CtbError) as e:  # rows not 16-byte multiples: single-tile variant refuses
        cuda.softmax.softmax_tma_kernel(torch.empty_like(x), x, 512)
    assert e.value.status == lib.BAD_ALIGN
    x = torch.zeros(4, 1024, device="cuda")
    with pytest.raises(cuda.CtbError) as e:  # tile must be a power of two (src/compiler/intrinsics/core.jl:10-19)
        cuda.softmax.softmax_tma_kernel(torch.empty_like(x), x, 1000)
    assert e.value.status == lib.UNSUPPORTED_TILE
    with pytest.raises(cuda.CtbError) as e:  # tile smaller than the row
        cuda.softmax.softmax_tma_kernel(torch.empty_like(x), x, 512)
    assert e.value.status == lib.UNSUPPORTED_TILE
    x = torch.zeros(2, 16384, device="cuda")
    with pytest.raises(cuda.CtbError) as e:
        cuda.softmax.softmax_tma_kernel(torch.empty_like(x), x, 16384)
    assert e.value.status == lib.UNSUPPORTED
    cuda.softmax.softmax_chunked_kernel(torch.empty(0, 8, device="cuda"), torch.empty(0, 8, device="cuda"), 8, 8)
