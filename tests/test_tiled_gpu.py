"""GPU parity of the host-level array operations (ct.Tiled broadcast and mapreduce) against numpy in float64, on the
cases of the reference's own tests (test/host/broadcast.jl, test/host/mapreduce.jl).  Tolerance: 1e-6 relative for the
element-wise expressions (f32 arithmetic, accurate math functions), 1e-5 for sums of 10^5..10^7 f32 terms; data
movement and max/min are exact."""
import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu


def rnd(shape, seed, dtype=np.float32, lo=-1.0, hi=1.0):
    g = np.random.default_rng(seed)
    return (g.random(shape, dtype=np.float32) * (hi - lo) + lo).astype(dtype)


def close(got, want, tol):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape
    denom = max(np.abs(want).max(), 1e-30) if want.size else 1.0
    assert (np.abs(got - want).max() if want.size else 0.0) <= tol * denom


def test_broadcast_elementwise_and_fused(cuda):
    import torch
    T = cuda.tiled
    a, b = rnd((1 << 20,), 1), rnd((1 << 20,), 2)
    A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    C = torch.empty_like(A)
    assert T.assign(C, T.Tiled(A) + T.Tiled(B)) is C                                   # 1D element-wise
    assert np.array_equal(C.cpu().numpy(), a + b)
    T.assign(C, T.Tiled(A) + T.Tiled(A) * T.sin(T.Tiled(A)))                           # fused multi-op: one kernel
    close(C.cpu().numpy(), ref.tiled_broadcast(("add", a, ("mul", a, ("sin", a)))), 1e-6)
    T.assign(C, T.Tiled(A) + 1.0)                                                      # scalar broadcast
    assert np.array_equal(C.cpu().numpy(), a + np.float32(1))
    T.assign(C, 2.5)                                                                   # scalar fill
    assert np.array_equal(C.cpu().numpy(), np.full_like(a, 2.5))
    T.assign(C, T.exp(-abs(T.Tiled(A))) / (1.0 + T.Tiled(B) ** 2.0) - T.tmax(T.Tiled(A), T.Tiled(B)))
    want = ref.tiled_broadcast(("sub", ("div", ("exp", ("neg", ("abs", a))), ("add", 1.0, ("pow", b, 2.0))), ("max", a, b)))
    close(C.cpu().numpy(), want, 2e-6)


@pytest.mark.parametrize("shape", [(64, 32), (8, 16, 32), (33, 1001), (3, 5, 7), (1, 257), (1, 1, 100), (4, 64)])
def test_broadcast_shapes_2d_3d_unaligned_and_leading_singletons(cuda, shape):
    import torch
    T = cuda.tiled
    a, b = rnd(shape, 3), rnd(shape, 4)
    A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    out = T.materialize(T.Tiled(A) * T.Tiled(B) + T.Tiled(A))                          # allocating form
    close(out.cpu().numpy(), a * b + a, 1e-6)
    assert out.shape == A.shape


def test_broadcast_size_one_expansion_and_rank_expansion(cuda):
    import torch
    T = cuda.tiled
    # Julia A(1, 64) .+ B(32, 1) -> (32, 64): torch [64, 1] and [1, 32]
    a, b = rnd((64, 1), 5), rnd((1, 32), 6)
    out = T.materialize(T.Tiled(torch.from_numpy(a).cuda()) + T.Tiled(torch.from_numpy(b).cuda()))
    close(out.cpu().numpy(), a + b, 1e-6)
    # row expansion into a given destination, with a nested function of the expanded operand
    m = rnd((48, 100), 7)
    row = rnd((1, 100), 8)      # Julia (100, 1)
    C = torch.empty(48, 100, device="cuda")
    T.assign(C, T.Tiled(torch.from_numpy(m).cuda()) + T.sin(T.Tiled(torch.from_numpy(row).cuda())))
    close(C.cpu().numpy(), m + np.sin(row.astype(np.float64)), 1e-6)
    # size-1 expansion only: C(M, N) .= A(1, N) .+ 1
    col = rnd((100, 1), 9)      # Julia (1, 100)
    C2 = torch.empty(100, 48, device="cuda")
    T.assign(C2, T.Tiled(torch.from_numpy(col).cuda()) + 1.0)
    close(C2.cpu().numpy(), np.broadcast_to(col + 1, (100, 48)), 1e-6)
    # rank expansion: vector (N,) + matrix (N, M)
    v, mat = rnd((64,), 10), rnd((20, 64), 11)
    out = T.materialize(T.Tiled(torch.from_numpy(v).cuda()) + T.Tiled(torch.from_numpy(mat).cuda()))
    close(out.cpu().numpy(), v + mat, 1e-6)
    # f16 arrays compute in f32 and round once
    h1, h2 = rnd((40, 72), 12, np.float16), rnd((40, 72), 13, np.float16)
    out = T.materialize(T.Tiled(torch.from_numpy(h1).cuda()) * T.Tiled(torch.from_numpy(h2).cuda()) + 0.5)
    want = (h1.astype(np.float32) * h2.astype(np.float32) + np.float32(0.5)).astype(np.float16)
    assert np.array_equal(out.cpu().numpy(), want)


def _tree_to_expr(T, tree, leaves):
    """(name, ...) trees with integer leaves (operand index) and float leaves (constants) -> a Tiled expression."""
    if isinstance(tree, int):
        return T.Tiled(leaves[tree])
    if isinstance(tree, float):
        return tree
    args = [_tree_to_expr(T, c, leaves) for c in tree[1:]]
    if len(args) == 1:
        return {"neg": lambda x: -x, "abs": abs}.get(tree[0], getattr(T, tree[0], None))(T.Expr.wrap(args[0]))
    a, b = T.Expr.wrap(args[0]), T.Expr.wrap(args[1])
    return {"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b, "div": lambda: a / b, "pow": lambda: a ** b,
            "max": lambda: T.tmax(a, b), "min": lambda: T.tmin(a, b)}[tree[0]]()


def _tree_to_oracle(tree, arrays):
    if isinstance(tree, int):
        return arrays[tree]
    if isinstance(tree, float):
        return tree
    return (tree[0],) + tuple(_tree_to_oracle(c, arrays) for c in tree[1:])


# one tree per kernel variant: operands held (1, 2, 3-4), accumulator only or with the stack, reversed operators
VARIANT_TREES = [
    ("sub", 2.0, ("exp", 0)),                                             # 1 operand, constant on the left (reversed)
    ("div", 0, ("add", ("abs2", 0), 1.5)),                                # 1 operand, input on the left (reversed)
    ("mul", ("sin", 0), ("cos", 0)),                                      # 1 operand, two computed sides (stack)
    ("min", ("max", 0, 1), ("mul", 1, 0.5)),                              # 2 operands, stack
    ("sub", ("mul", 0, 1), 1),                                            # 2 operands, accumulator only
    ("add", ("mul", 0, 1), ("sub", 2, 3)),                                # 4 operands, stack
    ("sub", 3, ("div", 2, ("add", ("abs", 1), ("exp", 0)))),              # 4 operands, accumulator only, reversed twice
    ("sub", ("sub", ("sin", 0), ("cos", 1)), ("sub", ("tanh", 2), ("mul", ("exp", 0), ("abs", 1)))),   # 3 live values
    ("pow", 1.5, ("abs", 0)),                                             # reversed pow
]


@pytest.mark.parametrize("n", [4 * 256 * 4 * 3 + 4, 1000, 1 << 20, (1 << 20) + 12])
@pytest.mark.parametrize("k", range(len(VARIANT_TREES)))
def test_broadcast_every_kernel_variant(cuda, n, k):
    """Sizes around the group structure (G groups of four elements per thread and trip, a grid apart): ragged last
    trips, fewer groups than threads, unaligned n (scalar path: n = 1000 is a multiple of four, 1 << 20 + 12 too;
    the odd case is in the shapes test)."""
    import torch
    T = cuda.tiled
    tree = VARIANT_TREES[k]
    arrays = [rnd((n,), 40 + j) for j in range(4)]
    leaves = [torch.from_numpy(a).cuda() for a in arrays]
    out = torch.full((n,), float("nan"), device="cuda")
    T.assign(out, _tree_to_expr(T, tree, leaves))
    close(out.cpu().numpy(), ref.tiled_broadcast(_tree_to_oracle(tree, arrays)), 2e-6)


def test_broadcast_in_place(cuda):
    """The destination may be an operand: every thread reads the elements of a trip before it writes them, and reads
    ahead only elements it has not written (several trips per thread at this size)."""
    import torch
    T = cuda.tiled
    a, b = rnd((1 << 24,), 30), rnd((1 << 24,), 31)
    A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    T.assign(A, T.Tiled(A) * 2.0 + T.Tiled(B))
    assert np.array_equal(A.cpu().numpy(), a * np.float32(2) + b)
    T.assign(B, T.sin(T.Tiled(B)) * T.cos(T.Tiled(A)) + T.Tiled(B))                    # stack in use, two operands
    want = np.sin(b.astype(np.float64)) * np.cos((a * np.float32(2) + b).astype(np.float64)) + b
    close(B.cpu().numpy(), want, 2e-6)


def test_broadcast_variants_f16_and_expanded(cuda):
    import torch
    T = cuda.tiled
    # Julia (64, 48) with a column operand (64, 1) and a row operand (1, 48): the non-dense vector path, two operands
    a, col, row = rnd((48, 64), 50), rnd((1, 64), 51), rnd((48, 1), 52)
    A, Cc, R = (torch.from_numpy(v).cuda() for v in (a, col, row))
    out = T.materialize((T.Tiled(A) - T.Tiled(Cc)) * T.Tiled(R) + T.sin(T.Tiled(A)) * T.cos(T.Tiled(Cc)))
    close(out.cpu().numpy(), (a - col) * row + np.sin(a.astype(np.float64)) * np.cos(col.astype(np.float64)), 2e-6)
    for tree in VARIANT_TREES[:6]:
        arrays = [rnd((4099 * 4,), 60 + j, dtype=np.float16) for j in range(4)]
        leaves = [torch.from_numpy(v).cuda() for v in arrays]
        out = torch.empty(4099 * 4, device="cuda", dtype=torch.float16)
        T.assign(out, _tree_to_expr(T, tree, leaves))
        want = ref.tiled_broadcast(_tree_to_oracle(tree, [v.astype(np.float64) for v in arrays]))
        close(out.cpu().numpy(), want, 1.5e-3)                                # one f16 rounding of the f32 result


def test_broadcast_empty_zero_dim_and_rejections(cuda):
    import torch
    T = cuda.tiled
    E = torch.empty(0, device="cuda")
    assert T.assign(E, T.Tiled(E) + 1.0) is E                                          # empty: no launch
    Z = torch.zeros((), device="cuda")
    T.assign(Z, 1.0)                                                                   # 0-dim arrays
    assert Z.item() == 1.0
    A = torch.ones(16, device="cuda")
    C = torch.arange(32, device="cuda", dtype=torch.float32)
    with pytest.raises(ValueError, match="DimensionMismatch"):
        T.assign(C, T.Tiled(A))
    with pytest.raises(ValueError, match="DimensionMismatch"):
        T.assign(C, T.Tiled(C) + T.Tiled(A))
    with pytest.raises(ValueError, match="device memory"):
        T.assign(C, T.Tiled(torch.ones(32)) * 2.0)                                     # host-side leaf
    with pytest.raises(TypeError):
        T.assign(C, T.Tiled(C) + range(16))                                            # no device storage
    with pytest.raises(ValueError, match="device memory"):
        T.assign(torch.ones(32), 0)                                                    # CPU destination
    lib = cuda._lib
    # six pushes deep as a postfix program, one live value after the library re-orders it
    D = torch.empty_like(C)
    T.assign(D, T.Tiled(C) + (T.Tiled(C) + (T.Tiled(C) + (T.Tiled(C) + (T.Tiled(C) + T.Tiled(C))))))
    np.testing.assert_array_equal(D.cpu().numpy(), 6 * C.cpu().numpy())
    long = T.Tiled(C)
    for _ in range(17):                                                                # 35 operations: over the limit
        long = long + T.Tiled(C)
    with pytest.raises(cuda.CtbError) as e:
        T.assign(D, long)
    assert e.value.status == lib.UNSUPPORTED


@pytest.mark.parametrize("shape,dims", [((1000,), None), ((1000,), 1), ((64, 32), 1), ((64, 32), 2), ((8, 16, 32), (1, 2)),
                                        ((8, 16, 32), (1, 3)), ((8, 16, 32), (2, 3)), ((8, 16, 32), (1, 2, 3)),
                                        ((33, 1001), 2), ((33, 1001), 1), ((7, 5, 3), None), ((64, 32), (2, 3)),
                                        ((4096, 4096), None), ((3, 2_000_003), 1), ((2_000_003, 3), 1),
                                        ((1000, 260), 2), ((37, 11, 64), (2, 3)), ((5000, 8), 2), ((2048, 2048), 2)])
def test_mapreduce_sum(cuda, shape, dims):
    import torch
    T = cuda.tiled
    a = rnd(shape, 21, lo=0.0, hi=1.0)
    A = torch.from_numpy(a).cuda()
    got = T.tsum(T.Tiled(A), dims=dims)
    jd = tuple(range(1, a.ndim + 1)) if dims is None else ((dims,) if isinstance(dims, int) else dims)
    want = ref.tiled_mapreduce("identity", "add", a, jd)
    if dims is None:
        assert got.dim() == 0
        close(got.cpu().numpy().reshape(()), want.reshape(()), 1e-5)
    else:
        close(got.cpu().numpy(), want, 1e-5)
    assert torch.equal(got, T.tsum(T.Tiled(A), dims=dims))                             # fixed order: bitwise repeatable


def test_mapreduce_prod_max_min_mapped_and_edge_cases(cuda):
    import torch
    T = cuda.tiled
    a = rnd((7, 5, 3), 22, lo=0.5, hi=1.5)
    A = torch.from_numpy(a).cuda()
    close(T.tprod(T.Tiled(A), dims=2).cpu().numpy(), ref.tiled_mapreduce("identity", "mul", a, (2,)), 1e-6)
    assert np.array_equal(T.tmaximum(T.Tiled(A), dims=(1, 3)).cpu().numpy(), a.max(axis=(0, 2), keepdims=True))
    assert np.array_equal(T.tminimum(T.Tiled(A)).cpu().numpy(), a.min())
    assert np.array_equal(T.tprod(T.Tiled(A), dims=()).cpu().numpy(), a)                # no-op dims: a copy
    assert np.array_equal(T.tmaximum(T.Tiled(A), dims=()).cpu().numpy(), a)
    b = rnd((300, 200), 23)
    B = torch.from_numpy(b).cuda()
    close(T.tmapreduce("abs2", "add", T.Tiled(B), dims=1).cpu().numpy(), ref.tiled_mapreduce("abs2", "add", b, (1,)), 1e-5)
    close(T.tmapreduce("abs", "max", T.Tiled(B)).cpu().numpy(), np.abs(b).max(), 0.0)
    h = rnd((128, 96), 24, np.float16)
    got = T.tsum(T.Tiled(torch.from_numpy(h).cuda()), dims=1)                          # f16 in, f32 accumulate, f16 out
    want = h.astype(np.float32).sum(axis=1, keepdims=True)
    close(got.cpu().numpy(), want, 2e-3)
    assert got.dtype == torch.float16
    # first dimension kept and a multiple of four: four outputs per thread, f32 and f16, every reduction
    c = rnd((333, 40), 25, lo=0.9, hi=1.1)
    Cc = torch.from_numpy(c).cuda()
    close(T.tprod(T.Tiled(Cc), dims=2).cpu().numpy(), ref.tiled_mapreduce("identity", "mul", c, (2,)), 1e-5)
    assert np.array_equal(T.tmaximum(T.Tiled(Cc), dims=2).cpu().numpy(), c.max(axis=0, keepdims=True))
    assert np.array_equal(T.tminimum(T.Tiled(Cc), dims=2).cpu().numpy(), c.min(axis=0, keepdims=True))
    close(T.tmapreduce("abs2", "add", T.Tiled(Cc), dims=2).cpu().numpy(), ref.tiled_mapreduce("abs2", "add", c, (2,)), 1e-5)
    h2 = rnd((301, 64), 26, np.float16)
    got = T.tsum(T.Tiled(torch.from_numpy(h2).cuda()), dims=2)
    close(got.cpu().numpy(), h2.astype(np.float32).sum(axis=0, keepdims=True), 2e-3)
    view = torch.from_numpy(rnd((64, 36), 27)).cuda()[:, 1:33].contiguous()            # aligned copy ...
    close(T.tsum(T.Tiled(view), dims=2).cpu().numpy(), view.cpu().numpy().sum(axis=0, keepdims=True), 1e-5)
    with pytest.raises(ValueError, match="ArgumentError"):
        T.tsum(T.Tiled(A), dims=0)
    with pytest.raises(TypeError):
        T.tsum(T.Tiled(A), dims=(1.0,))
    E = torch.empty(0, 4, device="cuda")                                              # Julia (4, 0)
    assert np.array_equal(T.tsum(T.Tiled(E), dims=2).cpu().numpy(), np.zeros((1, 4), np.float32))
