"""Seeded synthetic inputs for the six benchmark workloads.

TEST INFRASTRUCTURE ONLY (see the package docstring).

Every array is returned as a C-contiguous numpy array whose *memory* is the
reference's Julia column-major array; the numpy shape is therefore the Julia
shape reversed (Julia ``X(N, M)`` is numpy ``X[M, N]``).  The reference draws
its inputs with cuRAND inside each example's ``prepare`` (for instance
``examples/layernorm.jl:211-229``); nothing there is reproducible on a CPU, so
the generator here is numpy's PCG64 ``default_rng(seed)`` with the arrays drawn
in the order listed in each function, in float32, then cast.
"""
import numpy as np


def layernorm(M=4096, N=4096, seed=0):
    """X ~ N(0,1), W ~ U(0.5,1.5), B ~ N(0,0.1), dY ~ N(0,1); eps = 1e-5.

    Shapes follow ``examples/layernorm.jl:211-229`` (X, dY are Julia (N, M))."""
    g = np.random.default_rng(seed)
    X = g.standard_normal((M, N), dtype=np.float32)
    W = g.uniform(0.5, 1.5, N).astype(np.float32)
    B = (0.1 * g.standard_normal(N, dtype=np.float32)).astype(np.float32)
    DY = g.standard_normal((M, N), dtype=np.float32)
    return dict(X=X, W=W, B=B, DY=DY, eps=np.float32(1e-5), M=M, N=N)


def softmax(M=4096, N=4096, seed=1):
    """logits ~ N(0, 2^2); Julia (N, M) (``examples/softmax.jl:116-128``)."""
    g = np.random.default_rng(seed)
    return dict(input=(2.0 * g.standard_normal((M, N), dtype=np.float32)).astype(np.float32), M=M, N=N)


def gemm(M=4096, N=4096, K=4096, seed=2):
    """A(M,K), B(K,N) ~ U(-1,1) f32, Julia column-major
    (``examples/matmul.jl:66-77``): numpy A[K, M], B[N, K]."""
    g = np.random.default_rng(seed)
    A = g.uniform(-1.0, 1.0, (K, M)).astype(np.float32)
    B = g.uniform(-1.0, 1.0, (N, K)).astype(np.float32)
    return dict(A=A, B=B, M=M, N=N, K=K)


def batched_gemm(M=1024, K=2048, N=512, batch=8, seed=2, dtype=np.float32):
    """A(M,K,Batch), B(K,N,Batch), batch last (``examples/batchmatmul.jl:62-74``):
    numpy A[batch, K, M], B[batch, N, K]."""
    g = np.random.default_rng(seed)
    A = g.uniform(-1.0, 1.0, (batch, K, M)).astype(np.float32).astype(dtype)
    B = g.uniform(-1.0, 1.0, (batch, N, K)).astype(np.float32).astype(dtype)
    return dict(A=A, B=B, M=M, N=N, K=K, batch=batch)


def fmha(batch=8, heads=16, seq_q=1024, seq_kv=1024, d=64, kv_heads=None, seed=3):
    """Q(D,Sq,H,B), K/V(D,Skv,KVH,B) f16 ~ N(0,1) (``examples/fmha.jl:226-252``):
    numpy Q[B, H, Sq, D]."""
    kv_heads = heads if kv_heads is None else kv_heads
    g = np.random.default_rng(seed)
    Q = g.standard_normal((batch, heads, seq_q, d), dtype=np.float32).astype(np.float16)
    K = g.standard_normal((batch, kv_heads, seq_kv, d), dtype=np.float32).astype(np.float16)
    V = g.standard_normal((batch, kv_heads, seq_kv, d), dtype=np.float32).astype(np.float16)
    return dict(Q=Q, K=K, V=V, batch=batch, heads=heads, kv_heads=kv_heads,
                seq_q=seq_q, seq_kv=seq_kv, d=d)


def moe(tokens=256, hidden=1024, experts=32, inter=2048, topk=2, seed=4):
    """hidden(H,T) ~ N(0,1); W_r(H,E) ~ N(0,0.02); w1(H,2I,E) = [gate | up],
    w2(I,H,E), all ~ N(0,0.02), f16 (``examples/moe.jl:311-345`` for the shapes).
    numpy: X[T,H], Wr[E,H], w1[E,2I,H], w2[E,H,I]."""
    g = np.random.default_rng(seed)
    X = g.standard_normal((tokens, hidden), dtype=np.float32).astype(np.float16)
    Wr = (0.02 * g.standard_normal((experts, hidden), dtype=np.float32)).astype(np.float16)
    w1 = np.empty((experts, 2 * inter, hidden), dtype=np.float16)
    w2 = np.empty((experts, hidden, inter), dtype=np.float16)
    for e in range(experts):  # gate then up of every expert, then all down projections
        w1[e] = (0.02 * g.standard_normal((2 * inter, hidden), dtype=np.float32)).astype(np.float16)
    for e in range(experts):
        w2[e] = (0.02 * g.standard_normal((hidden, inter), dtype=np.float32)).astype(np.float16)
    return dict(X=X, Wr=Wr, w1=w1, w2=w2, tokens=tokens, hidden=hidden,
                experts=experts, inter=inter, topk=topk)


def vadd(shape=(2 ** 27,), seed=5, dtype=np.float32):
    """a, b ~ U(0,1) (``examples/vadd.jl:52-64``: cuRAND.rand); benchmark shape 2^27 elements."""
    g = np.random.default_rng(seed)
    a = g.random(shape, dtype=np.float32).astype(dtype)
    b = g.random(shape, dtype=np.float32).astype(dtype)
    return dict(a=a, b=b, shape=tuple(shape))


def transpose(m=8192, n=8192, seed=6, dtype=np.float32):
    """x(M, N) ~ U(0,1) (``examples/transpose.jl:25-36``), numpy x[N, M]; benchmark shape 8192 x 8192."""
    g = np.random.default_rng(seed)
    return dict(x=g.random((n, m), dtype=np.float32).astype(dtype), m=m, n=n)


def fft(batch=256, factors=(16, 16, 16), seed=7):
    """input ~ complex standard normal (``examples/fft.jl:182-190``: cuRAND.randn(ComplexF32, N, batch)), numpy
    complex64 [batch, N]; benchmark shape batch 256, factors (16, 16, 16)."""
    g = np.random.default_rng(seed)
    n = int(np.prod(factors))
    re = g.standard_normal((batch, n), dtype=np.float32)
    im = g.standard_normal((batch, n), dtype=np.float32)
    return dict(input=(re + 1j * im).astype(np.complex64) * np.float32(np.sqrt(0.5)), factors=tuple(factors), batch=batch, n=n)
