"""GPU parity of the dense / batched GEMM kernels against the float64 oracle.

Tolerances (relative Frobenius error): TF32 operands <= 5e-3, f16 operands
(f32 accumulate, f16 result) <= 2e-3.  The reference's own check is norm-wise
rtol=1e-2 (examples/matmul.jl:100, examples/batchmatmul.jl:105)."""
import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu
TOL_TF32, TOL_F16 = 5e-3, 2e-3


def dense(cuda, d, tiles=(64, 64, 64)):
    import torch
    A, B = torch.from_numpy(d["A"]).cuda(), torch.from_numpy(d["B"]).cuda()
    C = torch.full((d["N"], d["M"]), float("nan"), device="cuda", dtype=A.dtype)
    cuda.matmul.matmul_kernel(A, B, C, *tiles)
    torch.cuda.synchronize()
    return C.cpu().numpy()


# the reference's main() cases (examples/matmul.jl:156-165), ragged edges, K tails, the benchmark shape
@pytest.mark.parametrize("M,N,K,tiles", [(256, 256, 256, (32, 32, 32)), (512, 512, 512, (64, 64, 64)),
                                         (256, 512, 128, (32, 32, 32)), (1024, 1024, 1024, (64, 64, 64)),
                                         (200, 300, 100, (64, 64, 64)), (4, 4, 4, (64, 64, 64)),
                                         (132, 260, 36, (64, 64, 64)), (4096, 4096, 4096, (64, 64, 64)),
                                         (2048, 2048, 256, (64, 64, 64)), (2304, 2600, 100, (64, 64, 64)),
                                         (3000, 1800, 72, (64, 64, 64)), (260, 9000, 40, (64, 64, 64))])
def test_gemm_tf32(cuda, M, N, K, tiles):
    d = inputs.gemm(M, N, K, seed=2)
    C = dense(cuda, d, tiles)
    want = ref.gemm(d["A"], d["B"])
    assert ref.rel_fro(C, want) <= TOL_TF32
    # the kernel sees the operands with the low 13 mantissa bits dropped: against an
    # oracle fed the same truncated operands only f32 accumulation error remains
    assert ref.rel_fro(C, ref.gemm(ref.tf32_trunc(d["A"]), ref.tf32_trunc(d["B"]))) <= 2e-5


def batched(cuda, d, tiles=(128, 128, 64)):
    import torch
    A, B = torch.from_numpy(d["A"]).cuda(), torch.from_numpy(d["B"]).cuda()
    C = torch.full((d["batch"], d["N"], d["M"]), float("nan"), device="cuda", dtype=A.dtype)
    cuda.batchmatmul.batch_matmul_kernel(A, B, C, *tiles)
    torch.cuda.synchronize()
    return C.cpu().numpy()


# examples/batchmatmul.jl:161-169 main() cases, the benchmark shape (both orientations), odd sizes
@pytest.mark.parametrize("M,K,N,batch,dtype,tiles", [
    (256, 128, 256, 4, np.float32, (32, 32, 32)), (512, 256, 512, 4, np.float32, (64, 64, 64)),
    (512, 256, 1024, 4, np.float16, (128, 256, 64)), (1024, 2048, 512, 8, np.float32, (128, 128, 64)),
    (1024, 512, 2048, 8, np.float32, (128, 128, 64)), (100, 72, 36, 3, np.float32, (128, 128, 64)),
    (136, 40, 264, 2, np.float16, (128, 128, 64)),
    (1000, 72, 1300, 5, np.float32, (128, 128, 64)), (1032, 136, 1544, 4, np.float16, (128, 128, 64))])
def test_batched_gemm(cuda, M, K, N, batch, dtype, tiles):
    d = inputs.batched_gemm(M, K, N, batch, seed=2, dtype=dtype)
    C = batched(cuda, d, tiles)
    want = ref.batched_gemm(d["A"], d["B"])
    assert ref.rel_fro(C, want) <= (TOL_TF32 if dtype == np.float32 else TOL_F16)
    for b in range(batch):  # every batch individually (a wrong batch stride would hide in the norm)
        assert ref.rel_fro(C[b], want[b]) <= (TOL_TF32 if dtype == np.float32 else TOL_F16)


def test_gemm_linearity_full_size(cuda):
    """Size-independent property at the benchmark size: (A1+A2)*B == A1*B + A2*B up to TF32 error."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(5)
    n = 4096
    A1 = (torch.rand(n, n, device="cuda", generator=g) - 0.5)
    A2 = (torch.rand(n, n, device="cuda", generator=g) - 0.5)
    B = (torch.rand(n, n, device="cuda", generator=g) - 0.5)
    C1, C2, C3 = (torch.empty(n, n, device="cuda") for _ in range(3))
    mk = cuda.matmul.matmul_kernel
    mk(A1, B, C1, 64, 64, 64); mk(A2, B, C2, 64, 64, 64); mk(A1 + A2, B, C3, 64, 64, 64)
    err = (torch.linalg.norm((C1 + C2 - C3).double()) / torch.linalg.norm(C3.double())).item()
    assert err <= TOL_TF32


def test_gemm_strided_and_rejections(cuda):
    import torch
    lib = cuda._lib
    d = inputs.gemm(96, 80, 64, seed=9)
    Abig = torch.zeros(64, 128, device="cuda"); Abig[:, :96] = torch.from_numpy(d["A"]).cuda()
    Bbig = torch.zeros(80, 68, device="cuda"); Bbig[:, :64] = torch.from_numpy(d["B"]).cuda()
    Cbig = torch.full((80, 100), 7.0, device="cuda")
    cuda.matmul.matmul_kernel(Abig[:, :96], Bbig[:, :64], Cbig[:, :96], 64, 64, 64)
    torch.cuda.synchronize()
    assert ref.rel_fro(Cbig[:, :96].cpu().numpy(), ref.gemm(d["A"], d["B"])) <= TOL_TF32
    assert (Cbig[:, 96:] == 7.0).all()
    A = torch.zeros(64, 96, device="cuda"); B = torch.zeros(80, 64, device="cuda"); C = torch.zeros(80, 96, device="cuda")
    with pytest.raises(cuda.CtbError) as e:
        cuda.matmul.matmul_kernel(A, B, C, 48, 64, 64)  # not a power of two
    assert e.value.status == lib.UNSUPPORTED_TILE
    with pytest.raises(cuda.CtbError) as e:  # leading dimension of A not a multiple of 16 bytes
        cuda.matmul.matmul_kernel(torch.zeros(64, 97, device="cuda")[:, :96], B, C, 64, 64, 64)
    assert e.value.status == lib.BAD_ALIGN
    with pytest.raises(cuda.CtbError) as e:
        cuda.matmul.matmul_kernel(A, torch.zeros(80, 32, device="cuda"), C, 64, 64, 64)
    assert e.value.status == lib.BAD_ARG


@pytest.mark.parametrize("M,N,K,batch", [(256, 256, 256, 1), (200, 300, 100, 1), (1024, 512, 2048, 2), (4096, 4096, 4096, 1)])
def test_gemm_tf32_round_to_nearest_even_option(cuda, M, N, K, batch):
    """With ctb_set_tf32_rounding(1) the operands are rounded like the reference's f32 -> tf32 conversion (nearest even,
    pinned by the bit patterns of tests/golden/tf32_bits.json): against an oracle fed operands rounded that way only
    f32 accumulation error remains, and the error against the exact product is below the truncating default's."""
    import torch
    lib = cuda._lib
    if batch == 1:
        d = inputs.gemm(M, N, K, seed=5)
        run = lambda: dense(cuda, d)
        exact, rounded = ref.gemm(d["A"], d["B"]), ref.gemm(ref.tf32_round(d["A"]), ref.tf32_round(d["B"]))
    else:
        d = inputs.batched_gemm(M, K, N, batch, seed=5)
        run = lambda: batched(cuda, d)
        exact = ref.batched_gemm(d["A"], d["B"])
        rounded = ref.batched_gemm(ref.tf32_round(d["A"]), ref.tf32_round(d["B"]))
    trunc_err = ref.rel_fro(run(), exact)
    lib.set_tf32_rounding(0, True)
    try:
        C = run()
    finally:
        lib.set_tf32_rounding(0, False)
    assert ref.rel_fro(C, rounded) <= 2e-5
    assert ref.rel_fro(C, exact) < trunc_err
    assert lib.lib.ctb_set_tf32_rounding(lib.context(0), 2) == lib.BAD_ARG


@pytest.mark.parametrize("M,K,N,batch", [(256, 128, 256, 1), (136, 40, 264, 2), (2048, 512, 2048, 1), (1024, 2048, 512, 8)])
def test_gemm_bf16(cuda, M, K, N, batch):
    """bfloat16 operands and result, f32 accumulation (the element type is a parameter of the reference's batched example,
    examples/batchmatmul.jl:166): against the oracle on the bf16-rounded inputs, tolerance 1e-2 (8 mantissa bits in the
    result); single-CTA, split-K and CTA-pair kernels."""
    import torch
    d = inputs.batched_gemm(M, K, N, batch, seed=7, dtype=np.float32)
    A, B = (torch.from_numpy(d[k]).cuda().to(torch.bfloat16) for k in ("A", "B"))
    C = torch.full((batch, N, M), float("nan"), device="cuda", dtype=torch.bfloat16)
    cuda.batchmatmul.batch_matmul_kernel(A, B, C, 128, 128, 64)
    torch.cuda.synchronize()
    back = lambda t: t.float().cpu().numpy()
    want = ref.batched_gemm(back(A), back(B))
    assert ref.rel_fro(back(C), want) <= 1e-2
    if batch == 1:
        C2 = torch.empty(N, M, device="cuda", dtype=torch.bfloat16)
        cuda.matmul.matmul_kernel(A[0], B[0], C2, 64, 64, 64)
        assert torch.equal(C2, C[0])
