"""The allocation-free LayerNorm backward entry point (ctb_layernorm_bwd_static).

It exists for callers that cannot allocate device memory where the backward pass runs; its partial dW/dB
scratch is a fixed array inside the library.  Checked here through the C ABI against the ordinary pair of
entry points (caller-provided partial buffers) on two calls in a row with different data, because the built-in
scratch keeps the previous call's contents.  This file sorts last on purpose: a run that stops at the first
failure has then already run every other test."""
import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu
TOL = 1e-5  # the tolerance of the LayerNorm parity tests (max|a-b| / max|b|)


def _run_both(cuda, d):
    import torch
    ln = cuda.layernorm
    M, N = d["M"], d["N"]
    X, W, B, DY = (torch.from_numpy(d[k]).cuda() for k in ("X", "W", "B", "DY"))
    Y = torch.empty_like(X)
    Mean, Rstd = torch.empty(M, device="cuda"), torch.empty(M, device="cuda")
    ln.layer_norm_fwd(X, W, B, Y, Mean, Rstd, float(d["eps"]), 1024)
    # existing entry points: caller-owned partial buffers + final reduce
    DX0 = torch.empty_like(X)
    DWp, DBp = torch.empty(64, N, device="cuda"), torch.empty(64, N, device="cuda")
    FDW0, FDB0 = torch.empty(N, device="cuda"), torch.empty(N, device="cuda")
    ln.layer_norm_bwd_dx_partial_dwdb(DX0, DY, DWp, DBp, X, W, Mean, Rstd, None, 64, 1024)
    ln.layer_norm_bwd_dwdb(DWp, DBp, FDW0, FDB0, 32, 1024)
    # the allocation-free entry point: outputs only, scratch inside the library
    DX1 = torch.full_like(X, float("nan"))
    FDW1, FDB1 = torch.full((N,), float("nan"), device="cuda"), torch.full((N,), float("nan"), device="cuda")
    ln.layer_norm_bwd_static(DX1, DY, X, W, Mean, Rstd, FDW1, FDB1)
    torch.cuda.synchronize()
    return [t.cpu().numpy() for t in (DX0, FDW0, FDB0, DX1, FDW1, FDB1)], (Mean, Rstd)


def test_static_backward_matches_on_two_calls_in_a_row(cuda):
    # the second call is narrower and shorter, so stale partials of the first call sit next to the live ones
    # the last case is as wide as the built-in scratch allows
    for M, N, seed in ((1024, 4096, 0), (300, 1024, 7), (130, 8192, 11)):
        d = inputs.layernorm(M=M, N=N, seed=seed)
        (dx0, dw0, db0, dx1, dw1, db1), _ = _run_both(cuda, d)
        cuda.layernorm.layer_norm_bwd_static_status()  # no kernel of the call gave up a wait
        assert ref.max_abs_over_max(dx1, dx0) <= TOL
        assert ref.max_abs_over_max(dw1, dw0) <= TOL
        assert ref.max_abs_over_max(db1, db0) <= TOL
        rY, rMean, rRstd = ref.layernorm_fwd(d["X"], d["W"], d["B"], d["eps"])
        rDX, rDW, rDB = ref.layernorm_bwd(d["X"], d["W"], d["DY"], rMean, rRstd)
        assert ref.max_abs_over_max(dx1, rDX) <= TOL and ref.max_abs_over_max(dw1, rDW) <= TOL
        assert ref.max_abs_over_max(db1, rDB) <= TOL


def test_static_backward_rejects_what_does_not_fit(cuda):
    import torch
    lib = cuda._lib
    M, N = 4, 16384  # wider than the built-in scratch
    X = torch.zeros(M, N, device="cuda")
    v = torch.zeros(N, device="cuda"); m = torch.zeros(M, device="cuda")
    with pytest.raises(cuda.CtbError) as e:
        cuda.layernorm.layer_norm_bwd_static(torch.empty_like(X), X, X, v, m, m, v.clone(), v.clone())
    assert e.value.status == lib.UNSUPPORTED and "8192" in str(e.value)
    X = torch.zeros(4, 1002, device="cuda")  # rows that cannot be moved by 16-byte bulk copies
    v = torch.zeros(1002, device="cuda")
    with pytest.raises(cuda.CtbError) as e:
        cuda.layernorm.layer_norm_bwd_static(torch.empty_like(X), X, X, v, m, m, v.clone(), v.clone())
    assert e.value.status == lib.BAD_ALIGN
