"""The broadcast expression compiler of the library (postfix program -> accumulator-machine instructions), without a
GPU: ctb_tiled_compile returns the instruction words the kernel would run; a small numpy machine with the documented
meaning of a word (include/cutile_b200.h) runs them and the result must equal the oracle's value of the expression
(src/broadcast.jl:19-23: the fused kernel means the plain Julia broadcast).  Bit-exact in float64: the compiler only
re-orders evaluation and commutes + and *."""
import ctypes as C

import numpy as np
import pytest

from oracle import ref

OPS = {"input": 0, "const": 1, "identity": 16, "neg": 17, "abs": 18, "sqrt": 19, "exp": 20, "exp2": 21, "log": 22,
       "log2": 23, "sin": 24, "cos": 25, "tanh": 26, "inv": 27, "abs2": 28, "add": 64, "sub": 65, "mul": 66, "div": 67,
       "max": 68, "min": 69, "pow": 70}
NAMES = {v: k for k, v in OPS.items()}
SAFE_UNARY = ["identity", "neg", "abs", "sin", "cos", "tanh", "abs2", "exp"]
BINARY = ["add", "sub", "mul", "div", "max", "min"]


def lib():
    from cutile_b200 import _lib
    return _lib


def postfix(tree, out):
    """tree: ("in", i) | ("c", j) | (unary, t) | (binary, l, r)"""
    if tree[0] == "in":
        out += [OPS["input"], tree[1]]
    elif tree[0] == "c":
        out += [OPS["const"], tree[1]]
    else:
        for c in tree[1:]:
            postfix(c, out)
        out += [OPS[tree[0]], 0]
    return out


def compile_words(prog, n_inputs, n_consts):
    L = lib()
    words = (C.c_uint32 * 32)()
    n = C.c_int(0)
    st = L.lib.ctb_tiled_compile((C.c_int32 * len(prog))(*prog), len(prog) // 2, n_inputs, n_consts, words, C.byref(n))
    return st, list(words[: n.value])


def run_words(words, inputs, consts):
    """The machine of the header comment; also checks the stack never holds more than four values."""
    stack = []
    for w in words:
        kind, src, rev, code, arg = w & 3, (w >> 2) & 3, (w >> 4) & 1, (w >> 8) & 0xFF, (w >> 16) & 0xFF
        if kind == 1:
            stack[-1] = ref.TILED_UNARY[NAMES[code]](stack[-1])
            continue
        if src == 1:
            t = inputs[arg]
        elif src == 2:
            t = np.float64(consts[arg])
        else:
            assert kind == 2 and len(stack) >= 2
            t = stack.pop(-2)
        if kind == 0:
            stack.append(t)
            assert len(stack) <= 4
        else:
            a, b = (t, stack[-1]) if rev else (stack[-1], t)
            stack[-1] = ref.TILED_BINARY[NAMES[code]](a, b)
    assert len(stack) == 1
    return stack[0]


def to_oracle(tree, inputs, consts):
    if tree[0] == "in":
        return inputs[tree[1]]
    if tree[0] == "c":
        return float(consts[tree[1]])
    return (tree[0],) + tuple(to_oracle(c, inputs, consts) for c in tree[1:])


def random_tree(g, budget):
    if budget <= 1 or g.random() < 0.15:
        return ("in", int(g.integers(0, 4))) if g.random() < 0.75 else ("c", int(g.integers(0, 3)))
    if g.random() < 0.35:
        return (SAFE_UNARY[int(g.integers(0, len(SAFE_UNARY)))], random_tree(g, budget - 1))
    left = int(g.integers(1, budget - 1)) if budget > 2 else 1
    return (BINARY[int(g.integers(0, len(BINARY)))], random_tree(g, left), random_tree(g, budget - 1 - left))


def size(tree):
    return 1 if tree[0] in ("in", "c") else 1 + sum(size(c) for c in tree[1:])


def test_fused_example_takes_four_instructions():
    # A .+ A .* sin.(A): load, sin, multiply by the input in place, add the input in place
    tree = ("add", ("in", 0), ("mul", ("in", 0), ("sin", ("in", 0))))
    st, words = compile_words(postfix(tree, []), 1, 0)
    assert st == 0 and len(words) == 4
    assert [w & 3 for w in words] == [0, 1, 2, 2] and all(((w >> 4) & 1) == 0 for w in words)


def test_non_commutative_leaf_on_the_left_is_reversed():
    g = np.random.default_rng(0)
    x = [g.random(7) + 0.5 for _ in range(2)]
    for name in ("sub", "div", "max", "min", "pow"):
        tree = (name, ("in", 0), ("exp", ("in", 1)))
        st, words = compile_words(postfix(tree, []), 2, 0)
        assert st == 0 and len(words) == 3 and (words[-1] >> 4) & 1 == 1
        np.testing.assert_array_equal(run_words(words, x, []), ref.tiled_broadcast(to_oracle(tree, x, [])))


def test_random_expressions_match_the_oracle():
    g = np.random.default_rng(1)
    L = lib()
    inputs = [g.random((3, 5)) * 2 - 1 for _ in range(4)]
    consts = [0.5, -1.25, 3.0]
    done = 0
    for _ in range(400):
        tree = random_tree(g, int(g.integers(1, 30)))
        if size(tree) > 32:
            continue
        st, words = compile_words(postfix(tree, []), 4, 3)
        assert st == 0, L.last_error()
        with np.errstate(all="ignore"):
            got = run_words(words, inputs, consts)
            want = ref.tiled_broadcast(to_oracle(tree, inputs, consts))
        np.testing.assert_array_equal(np.broadcast_to(got, want.shape), want)
        done += 1
    assert done > 350


def test_identity_is_dropped_and_a_lone_leaf_loads():
    st, words = compile_words(postfix(("identity", ("c", 0)), []), 0, 1)
    assert st == 0 and len(words) == 1 and words[0] & 3 == 0 and (words[0] >> 2) & 3 == 2


def test_deep_right_nested_chain_needs_no_stack():
    # a - (b - (c - (d - (a - (b - (c - d)))))): seven pushes deep as a postfix program, one live value compiled
    tree = ("in", 3)
    for i in (2, 1, 0, 3, 2, 1, 0):
        tree = ("sub", ("in", i), tree)
    st, words = compile_words(postfix(tree, []), 4, 0)
    assert st == 0 and sum(1 for w in words if w & 3 == 0) == 1
    g = np.random.default_rng(2)
    x = [g.random(9) for _ in range(4)]
    np.testing.assert_array_equal(run_words(words, x, []), ref.tiled_broadcast(to_oracle(tree, x, [])))


def test_the_largest_live_set_of_32_operations_fits():
    # A full binary tree over computed values is the worst case: depth 3 (23 operations) needs four live values, and
    # depth 4 would take 47 operations, more than a program may have: no valid program is refused for its depth.
    def full(depth):
        return ("sin", ("in", 0)) if depth == 0 else ("sub", full(depth - 1), full(depth - 1))
    tree = full(3)
    st, words = compile_words(postfix(tree, []), 1, 0)
    assert st == 0 and len(words) == 23
    x = [np.random.default_rng(3).random(5)]
    np.testing.assert_array_equal(run_words(words, x, []), ref.tiled_broadcast(to_oracle(tree, x, [])))


@pytest.mark.parametrize("prog,frag", [
    ([64, 0], "needs two values"),
    ([0, 0, 24, 0, 64, 0], "needs two values"),
    ([24, 0], "empty stack"),
    ([0, 2], "input that was not given"),
    ([1, 0], "constant that was not given"),
    ([0, 0, 0, 0], "exactly one value"),
    ([0, 0, 99, 0], "not an operation code"),
])
def test_malformed_programs(prog, frag):
    L = lib()
    st, _ = compile_words(prog, 1, 0)
    assert st == L.BAD_ARG and frag in L.last_error()
