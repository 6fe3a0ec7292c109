"""numpy restatement of the CPU references in the reference's examples.

TEST INFRASTRUCTURE ONLY (see the package docstring).  Arrays are in the memory
order of the Julia column-major originals, i.e. numpy shapes are the Julia
shapes reversed.  ``dtype=np.float64`` is the parity oracle; ``np.float32`` is
the timed CPU baseline (numpy's OpenBLAS does every contraction, as Julia's
``mul!`` would).
"""
import numpy as np


# --------------------------------------------------------------------------- TF32
def f32_to_tf32_bits(x):
    """19-bit TF32 pattern sign(1)|exp(8)|mant(10): the float32 pattern with the
    low 13 mantissa bits dropped, round-to-nearest-even.  Known answers:
    ``test/types.jl:203-245``; conversion rule:
    ``src/compiler/intrinsics/conversions.jl:188-197``."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    isnan = ((u >> 23) & 0xFF == 0xFF) & ((u & 0x7FFFFF) != 0)
    r = (u + 0xFFF + ((u >> 13) & 1)) >> 13
    r = np.where(isnan, (u >> 13) | 1, r)
    return (r & 0x7FFFF).astype(np.uint32)


def tf32_round(x):
    """float32 values rounded (RNE) to TF32 precision, returned as float32."""
    return (f32_to_tf32_bits(x).astype(np.uint32) << 13).view(np.float32).reshape(np.shape(x))


def tf32_trunc(x):
    """float32 values with the low 13 mantissa bits cleared (what a tensor core
    that reads raw float32 from shared memory sees)."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return u.view(np.float32)


# ---------------------------------------------------------------------- LayerNorm
def layernorm_fwd(X, W, B, eps, dtype=np.float64):
    """``examples/layernorm.jl:284-298``: population variance, rstd = 1/sqrt(var+eps).
    X[M, N] (rows normalised over N).  Returns Y[M,N], mean[M], rstd[M]."""
    X = X.astype(dtype)
    N = X.shape[1]
    mean = X.sum(axis=1, keepdims=True) / N
    var = ((X - mean) ** 2).sum(axis=1, keepdims=True) / N
    rstd = 1.0 / np.sqrt(var + dtype(eps))
    Y = (X - mean) * rstd * W.astype(dtype) + B.astype(dtype)
    return Y, mean[:, 0], rstd[:, 0]


def layernorm_bwd(X, W, DY, mean, rstd, dtype=np.float64):
    """``examples/layernorm.jl:302-313``.  Returns DX[M,N], DW[N], DB[N]."""
    X = X.astype(dtype); DY = DY.astype(dtype); W = W.astype(dtype)
    N = X.shape[1]
    xhat = (X - mean.astype(dtype)[:, None]) * rstd.astype(dtype)[:, None]
    wdy = W * DY
    c1 = (xhat * wdy).sum(axis=1, keepdims=True) / N
    c2 = wdy.sum(axis=1, keepdims=True) / N
    DX = (wdy - (xhat * c1 + c2)) * rstd.astype(dtype)[:, None]
    return DX, (DY * xhat).sum(axis=0), DY.sum(axis=0)


# ------------------------------------------------------------------------ softmax
def softmax(x, dtype=np.float64):
    """``examples/softmax.jl:175-188``: per row subtract max, exp, normalise."""
    x = x.astype(dtype)
    e = np.exp(x - x.max(axis=1, keepdims=True))
    return e / e.sum(axis=1, keepdims=True)


# --------------------------------------------------------------------------- GEMM
def gemm(A, B, dtype=np.float64):
    """``examples/matmul.jl:98-101``: C = A*B with Julia A(M,K), B(K,N).
    Memory-order inputs A[K,M], B[N,K]; returns C[N,M]."""
    return B.astype(dtype) @ A.astype(dtype)


def batched_gemm(A, B, dtype=np.float64):
    """``examples/batchmatmul.jl:97-106``; A[b,K,M], B[b,N,K] -> C[b,N,M]."""
    return np.matmul(B.astype(dtype), A.astype(dtype))


def swizzle_2d(M, N, tm, tn, group_size_m, bid):
    """``examples/matmul.jl:13-24``: 1-based block id -> 1-based (bid_m, bid_n)."""
    cld = lambda a, b: -(-a // b)
    num_bid_m, num_bid_n = cld(M, tm), cld(N, tn)
    in_group = group_size_m * num_bid_n
    bid0 = bid - 1
    first = (bid0 // in_group) * group_size_m
    gsz = min(num_bid_m - first, group_size_m)
    return first + bid0 % gsz + 1, (bid0 % in_group) // gsz + 1


# --------------------------------------------------------------------------- FMHA
def fmha(Q, K, V, qk_scale=None, causal=False, input_pos=0, dtype=np.float64):
    """``examples/fmha.jl:175-220``.  Q[B,H,Sq,D], K/V[B,KVH,Skv,D] -> Out[B,H,Sq,Dv].
    KV head of query head h (1-based) is cld(h, H/KVH).  The causal rule with a
    query offset is the kernel's (``examples/fmha.jl:45-47,99-101``): key j is
    visible to query i when i + input_pos >= j; ``ref_fmha`` is the
    input_pos = 0 case."""
    Bn, H, Sq, D = Q.shape
    KVH, Skv = K.shape[1], K.shape[2]
    scale = dtype(1.0 / np.sqrt(D)) if qk_scale is None else dtype(qk_scale)
    out = np.zeros((Bn, H, Sq, V.shape[3]), dtype=dtype)
    group = H // KVH
    if causal:
        hidden = np.arange(Skv)[None, :] > (np.arange(Sq)[:, None] + input_pos)
    for b in range(Bn):
        for h in range(H):
            kh = h // group
            s = (Q[b, h].astype(dtype) @ K[b, kh].astype(dtype).T) * scale
            if causal:
                s = np.where(hidden, -np.inf, s)
            m = s.max(axis=1, keepdims=True)
            m = np.where(np.isinf(m), 0.0, m)
            p = np.exp(s - m)
            out[b, h] = (p / p.sum(axis=1, keepdims=True)) @ V[b, kh].astype(dtype)
    return out


# ---------------------------------------------------------------------------- MoE
def moe_router(X, Wr, topk):
    """Router of the benchmark configuration (the reference draws ids with
    ``randperm``, ``examples/moe.jl:323-332``, so this step is specified here).
    logits[t,e] = sum_k X[t,k]*Wr[e,k] in float32 in a fixed order: 32 partial
    sums, partial l taking the k with (k mod 256) in [8l, 8l+8) in ascending k
    (each f16*f16 product is exact in float32, so a fused multiply-add and
    multiply-then-add agree), combined by the butterfly v += v[l ^ o] for
    o = 16, 8, 4, 2, 1.  Top-k by value, ties to the smallest expert index (the
    reference's arg-reduction rule, ``src/language/operations.jl:1675-1677``);
    gates = softmax over the k chosen logits in float32, stored as f16.
    X[T,H] f16, Wr[E,H] f16 -> ids[topk,T] int32 (1-based), gates[topk,T] f16,
    logits[T,E] float32."""
    T, H = X.shape
    E = Wr.shape[0]
    Hp = -(-H // 256) * 256
    Xf = np.zeros((T, Hp), np.float32); Xf[:, :H] = X.astype(np.float32)
    Wf = np.zeros((E, Hp), np.float32); Wf[:, :H] = Wr.astype(np.float32)
    lanes = np.arange(32)
    part = np.zeros((T, E, 32), dtype=np.float32)
    for c in range(Hp // 256):
        for j in range(8):
            k = c * 256 + lanes * 8 + j
            part = part + Xf[:, None, k] * Wf[None, :, k]
    for o in (16, 8, 4, 2, 1):
        part = part + part[:, :, lanes ^ o]
    acc = np.ascontiguousarray(part[:, :, 0])
    work = acc.copy()
    ids = np.empty((topk, T), dtype=np.int32)
    sel = np.empty((topk, T), dtype=np.float32)
    rows = np.arange(T)
    for s in range(topk):
        j = np.argmax(work, axis=1)  # first maximum -> smallest index on ties
        ids[s] = j + 1
        sel[s] = work[rows, j]
        work[rows, j] = -np.inf
    e = np.exp(sel - sel[0:1])
    gates = (e / e.sum(axis=0, keepdims=True)).astype(np.float32).astype(np.float16)
    return ids, gates, acc


def moe_align_tile_size(topk_ids, tile_m, num_experts):
    """``examples/moe.jl:142-183``.  topk_ids[topk,T] (memory of Julia (T,topk)),
    1-based.  Flat slot id = token*topk + slot (slot fastest), stable sort by
    expert, each expert padded to a multiple of tile_m with the sentinel
    T*topk+1.  Returns sorted_token_ids int32[blocks*tile_m] (1-based),
    sorted_expert_ids int32[blocks] (1-based)."""
    topk, T = topk_ids.shape
    total = T * topk
    flat = np.ascontiguousarray(topk_ids.T).reshape(-1).astype(np.int64)
    perm = np.argsort(flat, kind="stable") + 1
    counts = np.bincount(flat - 1, minlength=num_experts)
    blocks = -(-counts // tile_m)
    nblk = int(blocks.sum())
    tok = np.full(nblk * tile_m, total + 1, dtype=np.int32)
    exp = np.zeros(nblk, dtype=np.int32)
    cb = ct = 0
    for e in range(num_experts):
        exp[cb:cb + blocks[e]] = e + 1
        tok[cb * tile_m: cb * tile_m + counts[e]] = perm[ct:ct + counts[e]]
        ct += counts[e]; cb += blocks[e]
    return tok, exp


def silu_and_mul(gate, up, dtype=np.float64):
    """``examples/moe.jl:110-128``: gate/(1+exp(-gate)) * up."""
    g = gate.astype(dtype)
    return g / (1.0 + np.exp(-g)) * up.astype(dtype)


def moe_ffn(X, w1, w2, topk_weights, topk_ids, dtype=np.float64):
    """``examples/moe.jl:264-304``.  X[T,H], w1[E,2I,H] (gate rows then up rows),
    w2[E,H,I], topk_weights/topk_ids[topk,T] -> out[T,H]."""
    T, H = X.shape
    E, I = w2.shape[0], w2.shape[2]
    out = np.zeros((T, H), dtype=dtype)
    Xd = X.astype(dtype)
    tw = topk_weights.astype(dtype)
    for e in range(E):
        slot, tok = np.nonzero(topk_ids == e + 1)
        if tok.size == 0:
            continue
        w1e = w1[e].astype(dtype)
        x = Xd[tok]
        act = silu_and_mul(x @ w1e[:I].T, x @ w1e[I:].T, dtype)
        y = act @ w2[e].astype(dtype).T
        np.add.at(out, tok, y * tw[slot, tok][:, None])
    return out


# ------------------------------------------------------------------- error norms
def vadd(a, b):
    """c = a + b in the element type (``examples/vadd.jl:127-129``: ``Array(result.c) ≈ Array(a) + Array(b)``)."""
    return a + b


def transpose(x):
    """y = transpose(x) (``examples/transpose.jl:58-60``).  numpy x[N, M] holds Julia x(M, N); the result holds y(N, M)."""
    return np.ascontiguousarray(x.T)


def fft_dft_matrix(size, dtype=np.float32):
    """``dft_matrix`` (``examples/fft.jl:128-138``): W[i, j] = exp(-2 pi i ij / size), rounded to ComplexF32 and split
    into Float32 planes.  Julia (2, size, size) is numpy [size, size, 2]."""
    w = np.zeros((size, size), dtype=np.complex64)
    for i in range(size):
        for j in range(size):
            w[i, j] = np.exp(-2j * np.pi * i * j / size)
    return np.stack([w.real, w.imag], axis=-1).astype(dtype)


def fft_make_twiddles(factors, dtype=np.float32):
    """``make_twiddles`` (``examples/fft.jl:141-176``).  T0 Julia (2, F1F2, F0) is numpy [F0, F1F2, 2] with
    [i, j] = exp(-2 pi i ij / N); T1 Julia (2, F2, F1) is numpy [F1, F2, 2] with [j, k] = exp(-2 pi i jk / F1F2)."""
    F0, F1, F2 = factors
    N, F1F2 = F0 * F1 * F2, F1 * F2
    T0 = np.zeros((F0, F1F2, 2), dtype=dtype)
    for i in range(F0):
        for j in range(F1F2):
            v = np.exp(-2j * np.pi * i * j / N)
            T0[i, j, 0], T0[i, j, 1] = v.real, v.imag
    T1 = np.zeros((F1, F2, 2), dtype=dtype)
    for j in range(F1):
        for k in range(F2):
            v = np.exp(-2j * np.pi * j * k / F1F2)
            T1[j, k, 0], T1[j, k, 1] = v.real, v.imag
    return fft_dft_matrix(F0, dtype), fft_dft_matrix(F1, dtype), fft_dft_matrix(F2, dtype), T0, T1


def _jl(a, shape):
    """Julia ``reshape`` (column-major)."""
    return np.reshape(a, shape, order="F")


def fft_three_stage(x, W0, W1, W2, T0, T1, factors, dtype=np.float64):
    """``fft_kernel`` (``examples/fft.jl:22-126``) stage by stage with Julia's column-major reshapes and permutes:
    F0-point DFT, twiddle T0, permute, F1-point DFT, twiddle T1, permute, F2-point DFT, final permute.
    x: complex numpy [batch, N] (Julia (N, batch)); tables as numpy arrays in the layouts of ``fft_make_twiddles``.
    Returns complex [batch, N]."""
    F0, F1, F2 = factors
    N, F1F2, F0F2, F0F1 = F0 * F1 * F2, F1 * F2, F0 * F2, F0 * F1
    ct = np.complex128 if dtype == np.float64 else np.complex64
    BS = x.shape[0]
    cplx = lambda t: (t[..., 0].astype(dtype) + 1j * t[..., 1].astype(dtype)).astype(ct)
    # numpy [j, i] of a (2, F, F) table is Julia W(i, j)
    w0, w1, w2 = cplx(W0).T, cplx(W1).T, cplx(W2).T            # now indexed [i, j] like Julia
    t0 = _jl(cplx(T0).T, (N,))                                   # Julia T0(j, i) flattened column-major
    t1 = _jl(cplx(T1).T, (F1F2,))                                # Julia T1(k, j) flattened
    X = x.astype(ct).T                                           # Julia (N, BS)
    X = _jl(X, (F1F2, F0, BS))
    X = np.einsum("jnb,nk->jkb", X, w0)                          # X * W0 per batch (:80-83)
    X = _jl(X, (N, BS)) * t0[:, None]                            # (:86-87)
    X = np.transpose(_jl(X, (F2, F1, F0, BS)), (2, 0, 1, 3))     # permutedims (3, 1, 2, 4) (:90-91)
    X = _jl(X, (F0F2, F1, BS))
    X = np.einsum("rnb,nk->rkb", X, w1)                          # (:95-98)
    X = _jl(X, (F0, F1F2, BS)) * t1[None, :, None]               # (:101-102)
    X = np.transpose(_jl(X, (F0, F2, F1, BS)), (2, 0, 1, 3))     # (:105-106)
    X = _jl(X, (F0F1, F2, BS))
    X = np.einsum("qnb,nk->qkb", X, w2)                          # (:110-113)
    X = np.transpose(_jl(X, (F1, F0, F2, BS)), (1, 0, 2, 3))     # permutedims (2, 1, 3, 4) (:116-117)
    return np.ascontiguousarray(_jl(X, (N, BS)).T)


def fft(x):
    """The example's check (``examples/fft.jl:243-247``): ``FFTW.fft(input, 1)``, the DFT along the N dimension."""
    return np.fft.fft(np.asarray(x, dtype=np.complex128), axis=-1)


# ---------------------------------------------------------------------- ct.Tiled host operations
TILED_UNARY = {"identity": lambda x: x, "neg": lambda x: -x, "abs": np.abs, "sqrt": np.sqrt, "exp": np.exp, "exp2": np.exp2,
               "log": np.log, "log2": np.log2, "sin": np.sin, "cos": np.cos, "tanh": np.tanh, "inv": lambda x: 1.0 / x,
               "abs2": lambda x: x * x}
TILED_BINARY = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide, "max": np.maximum,
                "min": np.minimum, "pow": np.power}


def tiled_broadcast(expr, dtype=np.float64):
    """Value of a broadcast expression tree (``src/broadcast.jl:19-23``: ``ct.Tiled(C) .= f.(args...)`` means the plain
    Julia broadcast of the same expression).  expr: a numpy array, a Python scalar, or a tuple (name, arg) /
    (name, lhs, rhs).  numpy arrays hold the Julia arrays with the dimensions reversed, so numpy's alignment of
    TRAILING dimensions is Julia's alignment of LEADING dimensions: plain numpy broadcasting gives Julia's result."""
    if isinstance(expr, tuple):
        if len(expr) == 2:
            return TILED_UNARY[expr[0]](tiled_broadcast(expr[1], dtype))
        return TILED_BINARY[expr[0]](tiled_broadcast(expr[1], dtype), tiled_broadcast(expr[2], dtype))
    return np.asarray(expr, dtype=dtype)


def tiled_mapreduce(f, op, x, julia_dims, dtype=np.float64):
    """``mapreduce(f, op, ct.Tiled(A); dims)`` (``src/mapreduce.jl:66-203``; sum / prod / maximum / minimum are the
    cases f = identity).  x: numpy array whose axes are the Julia dimensions reversed; julia_dims: 1-based Julia
    dimensions to reduce (dimensions beyond ndims are ignored like in Julia).  Keeps the reduced dimensions with
    extent 1."""
    y = TILED_UNARY[f](np.asarray(x, dtype=dtype))
    axes = tuple(x.ndim - d for d in julia_dims if 1 <= d <= x.ndim)
    red = {"add": np.sum, "mul": np.prod, "max": np.max, "min": np.min}[op]
    if not axes:
        return y
    if op in ("max", "min") and any(y.shape[a] == 0 for a in axes):
        shape = [1 if i in axes else n for i, n in enumerate(y.shape)]
        return np.full(shape, -np.inf if op == "max" else np.inf, dtype=dtype)
    return red(y, axis=axes, keepdims=True)


def rel_fro(out, ref):
    """||out-ref||_F / ||ref||_F, the norm-wise measure Julia's ``isapprox`` uses
    on arrays (``examples/matmul.jl:100``)."""
    out = np.asarray(out, dtype=np.float64); ref = np.asarray(ref, dtype=np.float64)
    return float(np.linalg.norm(out - ref) / max(np.linalg.norm(ref), 1e-300))


def max_rel(out, ref, floor=1e-3):
    """max |out-ref| / max(|ref|, floor*max|ref|): element-wise relative error
    with a floor, so that entries that cancel to ~0 do not dominate."""
    out = np.asarray(out, dtype=np.float64); ref = np.asarray(ref, dtype=np.float64)
    den = np.maximum(np.abs(ref), floor * np.abs(ref).max())
    return float((np.abs(out - ref) / den).max())


def max_abs_over_max(out, ref):
    """max |out-ref| / max |ref|."""
    out = np.asarray(out, dtype=np.float64); ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(out - ref).max() / np.abs(ref).max())
