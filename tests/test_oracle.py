"""CPU tests of the oracle: the one known-answer table the reference holds for
this path (TF32 packing) and self-consistency of the restated formulas."""
import json
import os

import numpy as np
import pytest

from oracle import inputs, ref

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def test_tf32_known_answers():
    gold = json.load(open(os.path.join(GOLD, "tf32_bits.json")))
    for c in gold["cases"]:
        v = float(c["value"])
        assert int(ref.f32_to_tf32_bits(np.float32(v))) == c["bits"], c
    for v in gold["fits_19_bits"]:
        assert int(ref.f32_to_tf32_bits(np.float32(v))) <= 0x7FFFF
    nan = int(ref.f32_to_tf32_bits(np.float32("nan")))
    assert (nan >> 10) & 0xFF == 0xFF and (nan & 0x3FF) != 0


def test_tf32_round_to_nearest_even():
    one = np.float32(1.0).view(np.uint32)
    tie_even = np.uint32(one | 0x1000).view(np.float32)          # kept LSB 0, exactly half -> down
    tie_odd = np.uint32(one | 0x2000 | 0x1000).view(np.float32)  # kept LSB 1, exactly half -> up
    above = np.uint32(one | 0x1001).view(np.float32)
    assert ref.tf32_round(tie_even) == np.float32(1.0)
    assert ref.tf32_round(tie_odd).view(np.uint32) == one + 0x4000
    assert ref.tf32_round(above).view(np.uint32) == one + 0x2000
    assert ref.tf32_trunc(above) == np.float32(1.0)


def test_layernorm_matches_direct_formula():
    d = inputs.layernorm(M=33, N=100, seed=11)
    Y, mean, rstd = ref.layernorm_fwd(d["X"], d["W"], d["B"], d["eps"])
    X = d["X"].astype(np.float64)
    assert np.allclose(mean, X.mean(axis=1))
    assert np.allclose(rstd, 1 / np.sqrt(X.var(axis=1) + 1e-5), rtol=1e-9)
    # gradient check of dX against finite differences of sum(Y*dY)
    DX, DW, DB = ref.layernorm_bwd(d["X"], d["W"], d["DY"], mean, rstd)
    f = lambda Z: (ref.layernorm_fwd(Z, d["W"], d["B"], d["eps"])[0] * d["DY"]).sum()
    Z = d["X"].astype(np.float64)
    for (i, j) in [(0, 0), (5, 17), (32, 99)]:
        h = 1e-6
        Zp = Z.copy(); Zp[i, j] += h
        Zm = Z.copy(); Zm[i, j] -= h
        assert abs((f(Zp) - f(Zm)) / (2 * h) - DX[i, j]) < 1e-5
    assert np.allclose(DB, d["DY"].astype(np.float64).sum(axis=0))


def test_softmax_rows_sum_to_one():
    x = inputs.softmax(M=7, N=50)["input"]
    s = ref.softmax(x)
    assert np.allclose(s.sum(axis=1), 1.0) and (s >= 0).all()


def test_gemm_layout():
    d = inputs.gemm(M=8, N=5, K=3)
    C = ref.gemm(d["A"], d["B"])  # [N, M]
    A_jl = d["A"].T  # Julia A(M,K)
    B_jl = d["B"].T  # Julia B(K,N)
    assert np.allclose(C.T, A_jl.astype(np.float64) @ B_jl.astype(np.float64))


def test_swizzle_covers_grid_once():
    M, N, tm, tn = 1000, 700, 64, 64
    nm, nn = -(-M // tm), -(-N // tn)
    seen = {ref.swizzle_2d(M, N, tm, tn, 8, b) for b in range(1, nm * nn + 1)}
    assert seen == {(i, j) for i in range(1, nm + 1) for j in range(1, nn + 1)}


def test_fmha_causal_first_row_and_gqa():
    d = inputs.fmha(batch=1, heads=4, seq_q=16, seq_kv=16, d=8, kv_heads=2, seed=5)
    o = ref.fmha(d["Q"], d["K"], d["V"], causal=True)
    # query 0 sees only key 0 -> output = V[0] of its KV head (heads 0,1 -> kv 0; 2,3 -> kv 1)
    for h in range(4):
        assert np.allclose(o[0, h, 0], d["V"][0, h // 2, 0].astype(np.float64))
    full = ref.fmha(d["Q"], d["K"], d["V"], causal=False)
    assert np.allclose(o[0, :, -1], full[0, :, -1])  # the last query sees every key either way


def test_moe_align_matches_hand_case():
    # 3 tokens, top-2, 4 experts, tile 4.  ids[topk, T]
    ids = np.array([[1, 3, 1], [3, 2, 4]], dtype=np.int32)
    tok, exp = ref.moe_align_tile_size(ids, 4, 4)
    # flat (slot fastest): t0:(1,3) t1:(3,2) t2:(1,4) -> [1,3,3,2,1,4]; flat ids 1..6
    assert exp.tolist() == [1, 2, 3, 4]
    assert tok.tolist() == [1, 5, 7, 7, 4, 7, 7, 7, 2, 3, 7, 7, 6, 7, 7, 7]


def test_moe_router_and_ffn_small():
    d = inputs.moe(tokens=12, hidden=64, experts=8, inter=32, topk=2, seed=9)
    ids, gates, logits = ref.moe_router(d["X"], d["Wr"], 2)
    assert ids.shape == (2, 12) and ids.min() >= 1 and ids.max() <= 8
    assert (ids[0] != ids[1]).all()
    srt = np.sort(logits, axis=1)
    assert np.array_equal(logits[np.arange(12), ids[0] - 1], srt[:, -1])
    assert np.array_equal(logits[np.arange(12), ids[1] - 1], srt[:, -2])
    assert np.allclose(gates.astype(np.float64).sum(axis=0), 1.0, atol=2e-3)
    out = ref.moe_ffn(d["X"], d["w1"], d["w2"], gates, ids)
    # direct per-token evaluation
    I = 32
    for t in (0, 5, 11):
        acc = np.zeros(64)
        for s in range(2):
            e = ids[s, t] - 1
            x = d["X"][t].astype(np.float64)
            g = d["w1"][e, :I].astype(np.float64) @ x
            u = d["w1"][e, I:].astype(np.float64) @ x
            acc += float(gates[s, t]) * (d["w2"][e].astype(np.float64) @ (g / (1 + np.exp(-g)) * u))
        assert np.allclose(out[t], acc)


def test_vadd_and_transpose_restatements():
    d = inputs.vadd((1000,), seed=1)
    assert np.array_equal(ref.vadd(d["a"], d["b"]), d["a"] + d["b"]) and ref.vadd(d["a"], d["b"]).dtype == np.float32
    t = inputs.transpose(5, 3)
    y = ref.transpose(t["x"])
    assert y.shape == (5, 3) and y[4, 2] == t["x"][2, 4] and y.flags.c_contiguous


@pytest.mark.parametrize("batch,factors", [(2, (2, 2, 2)), (4, (8, 8, 8)), (3, (4, 8, 16)), (2, (16, 16, 16)), (2, (1, 4, 2)),
                                           (2, (32, 2, 8))])
def test_fft_three_stage_restatement_is_the_dft(batch, factors):
    """The stage-by-stage restatement of the example's kernel, fed the example's own f32 tables, reproduces the DFT that
    the example verifies against (FFTW there, numpy's pocketfft here) and closed-form answers."""
    d = inputs.fft(batch, factors)
    tabs = ref.fft_make_twiddles(factors)
    y = ref.fft_three_stage(d["input"], *tabs, factors)
    want = ref.fft(d["input"])
    assert ref.rel_fro(np.stack([y.real, y.imag]), np.stack([want.real, want.imag])) <= 2e-7
    n = d["n"]
    imp = np.zeros((1, n), dtype=np.complex64)
    imp[0, n // 2 + (n > 1)] = 1
    p = n // 2 + (n > 1)
    yi = ref.fft_three_stage(imp, *tabs, factors)[0]
    assert np.abs(yi - np.exp(-2j * np.pi * p * np.arange(n) / n)).max() <= 1e-6
    # tables: symmetric DFT matrices with unit-modulus entries, first row/column of every table equal to 1
    for t in tabs:
        assert np.allclose(np.hypot(t[..., 0], t[..., 1]), 1.0, atol=1e-6)
        assert np.array_equal(t[0, :, 0], np.ones(t.shape[1], np.float32)) and not t[0, :, 1].any()


def test_tiled_restatements_follow_julia_dimension_order():
    """numpy arrays hold the Julia arrays with the dimensions reversed: Julia dims=1 is numpy's LAST axis, and Julia's
    broadcast of A(N) with B(N, M) is numpy's broadcast of a[N] with b[M, N]."""
    a = np.arange(24, dtype=np.float64).reshape(2, 3, 4)          # Julia (4, 3, 2)
    r = ref.tiled_mapreduce("identity", "add", a, (1,))
    assert r.shape == (2, 3, 1) and np.array_equal(r[..., 0], a.sum(axis=2))
    r = ref.tiled_mapreduce("abs2", "add", a, (1, 3))
    assert r.shape == (1, 3, 1) and np.array_equal(r[0, :, 0], (a * a).sum(axis=(0, 2)))
    assert np.array_equal(ref.tiled_mapreduce("identity", "max", a, (2, 7)), a.max(axis=1, keepdims=True))  # dims > ndims ignored
    assert np.array_equal(ref.tiled_mapreduce("identity", "mul", a, ()), a)
    v, m = np.arange(4.0), np.ones((3, 4))
    out = ref.tiled_broadcast(("add", v, ("mul", m, ("sin", v))))
    want = np.array([[v[j] + np.sin(v[j]) for j in range(4)] for _ in range(3)])
    assert out.shape == (3, 4) and np.allclose(out, want, rtol=0, atol=1e-15)
