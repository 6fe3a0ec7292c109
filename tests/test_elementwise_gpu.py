"""GPU parity of the element-wise addition and the transpose against the oracle: bit-exact (one rounding per
element for the addition, pure data movement for the transpose), including ragged sizes and strided rows."""
import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,dtype", [(1_024_000, np.float32), (1000003, np.float32), (7, np.float32), (4096 * 33, np.float16)])
def test_vec_add_1d_and_gather(cuda, n, dtype):
    import torch
    d = inputs.vadd((n,), dtype=dtype)
    a, b = torch.from_numpy(d["a"]).cuda(), torch.from_numpy(d["b"]).cuda()
    for fn in (cuda.vadd.vec_add_kernel_1d, cuda.vadd.vec_add_kernel_1d_gather):
        c = torch.full_like(a, float("nan"))
        fn(a, b, c, 1024)
        assert np.array_equal(c.cpu().numpy(), ref.vadd(d["a"], d["b"]))


def test_vec_add_2d_dense_strided_and_unaligned(cuda):
    import torch
    d = inputs.vadd((300, 1000), seed=9)
    a, b = torch.from_numpy(d["a"]).cuda(), torch.from_numpy(d["b"]).cuda()
    c = torch.empty_like(a)
    cuda.vadd.vec_add_kernel_2d(a, b, c, 32, 32)
    assert np.array_equal(c.cpu().numpy(), ref.vadd(d["a"], d["b"]))
    # row views of a wider array (leading dimension > row length), odd row length
    wide_a, wide_b = torch.zeros(300, 1031, device="cuda"), torch.zeros(300, 1031, device="cuda")
    wide_a[:, :999] = a[:, :999]
    wide_b[:, :999] = b[:, :999]
    out = torch.zeros(300, 1031, device="cuda")
    cuda.vadd.vec_add_kernel_2d(wide_a[:, :999], wide_b[:, :999], out[:, :999], 64, 64)
    assert np.array_equal(out[:, :999].cpu().numpy(), ref.vadd(d["a"][:, :999], d["b"][:, :999]))
    assert float(out[:, 999:].abs().max()) == 0.0  # nothing written beyond the rows


@pytest.mark.parametrize("m,n,dtype", [(1024, 512, np.float32), (8192, 8192, np.float32), (100, 37, np.float32),
                                       (257, 1000, np.float16)])
def test_transpose(cuda, m, n, dtype):
    import torch
    d = inputs.transpose(m, n, dtype=dtype)
    x = torch.from_numpy(d["x"]).cuda()
    y = torch.full((m, n), float("nan"), device="cuda", dtype=x.dtype)
    cuda.transpose.transpose_kernel(x, y, 64, 64)
    assert np.array_equal(y.cpu().numpy(), ref.transpose(d["x"]))


def test_elementwise_rejections(cuda):
    import torch
    lib = cuda._lib
    a = torch.zeros(1024, device="cuda")
    with pytest.raises(cuda.CtbError) as e:
        cuda.vadd.vec_add_kernel_1d(a, a, a.clone(), 1000)  # tile sizes are powers of two in the reference
    assert e.value.status == lib.UNSUPPORTED_TILE
    with pytest.raises(cuda.CtbError) as e:
        cuda.vadd.vec_add_kernel_1d(a, a, a.clone(), 1024, num_ctas=3)
    assert e.value.status == lib.BAD_ARG and "power of 2" in str(e.value)
    with pytest.raises(cuda.CtbError) as e:
        cuda.transpose.transpose_kernel(torch.zeros(4, 8, device="cuda"), torch.zeros(4, 8, device="cuda"), 64, 64)
    assert e.value.status == lib.BAD_ARG
