"""GPU parity of the MoE kernels against the oracle.

Routing (top-k ids, sorted slot ids, expert ids per block) must be bit-exact;
router logits are compared bit for bit with the float32 CPU loop; gate weights
within one f16 ulp (expf differs between CPU and GPU); FFN outputs within a
relative Frobenius error of 2e-3 (f16 operands, f32 accumulation, f16 output).
The reference's own check is norm-wise rtol=1e-2, atol=1e-2 (examples/moe.jl:370-374)."""
import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu
TOL = 2e-3


def random_routing(T, E, topk, seed):
    """ids and weights drawn the way the reference's prepare() does (examples/moe.jl:323-332)."""
    g = np.random.default_rng(seed)
    ids = np.stack([g.permutation(E)[:topk] + 1 for _ in range(T)], axis=1).astype(np.int64)  # [topk, T]
    raw = np.exp(g.random((topk, T), dtype=np.float32))
    return ids, (raw / raw.sum(axis=0, keepdims=True)).astype(np.float16)


@pytest.mark.parametrize("T,H,E,topk", [(256, 1024, 32, 2), (48, 512, 64, 8), (4096, 1024, 32, 2), (7, 64, 40, 3)])
def test_router_bit_exact(cuda, T, H, E, topk):
    import torch
    d = inputs.moe(tokens=T, hidden=H, experts=E, inter=8, topk=topk, seed=4)
    w, ids, logits = cuda.moe.moe_router(torch.from_numpy(d["X"]).cuda(), torch.from_numpy(d["Wr"]).cuda(), topk,
                                         return_logits=True)
    rids, rgates, rlogits = ref.moe_router(d["X"], d["Wr"], topk)
    assert np.array_equal(logits.cpu().numpy().view(np.uint32), rlogits.view(np.uint32))  # same f32 bits
    assert np.array_equal(ids.cpu().numpy(), rids)
    ulp = np.abs(w.cpu().numpy().view(np.int16).astype(np.int32) - rgates.view(np.int16).astype(np.int32))
    assert ulp.max() <= 1


def test_router_tie_goes_to_smallest_index(cuda):
    import torch
    X = np.zeros((3, 64), np.float16); X[:, 0] = 1
    Wr = np.zeros((16, 64), np.float16); Wr[[3, 5, 9], 0] = 2.0  # three equal maxima, the rest tie at 0
    w, ids = cuda.moe.moe_router(torch.from_numpy(X).cuda(), torch.from_numpy(Wr).cuda(), 4)
    assert ids.cpu().numpy()[:, 0].tolist() == [4, 6, 10, 1]


@pytest.mark.parametrize("T,E,topk,tile_m,dtype", [(48, 64, 8, 128, np.int64), (128, 32, 4, 128, np.int64),
                                                   (64, 64, 8, 128, np.int32), (256, 32, 2, 128, np.int32),
                                                   (4096, 32, 2, 128, np.int32), (1000, 7, 3, 16, np.int64),
                                                   (1, 4, 1, 32, np.int32)])
def test_align_bit_exact(cuda, T, E, topk, tile_m, dtype):
    import torch
    ids, _ = random_routing(T, E, topk, seed=T + E)
    tok, exp = cuda.moe.moe_align_tile_size(torch.from_numpy(ids.astype(dtype)).cuda(), tile_m, E)
    rtok, rexp = ref.moe_align_tile_size(ids, tile_m, E)
    assert np.array_equal(tok.cpu().numpy(), rtok)
    assert np.array_equal(exp.cpu().numpy(), rexp)


def test_align_skewed_and_empty_experts(cuda):
    import torch
    ids = np.ones((2, 300), np.int32); ids[1] = 5  # every token picks experts 1 and 5 only
    tok, exp = cuda.moe.moe_align_tile_size(torch.from_numpy(ids).cuda(), 128, 8)
    rtok, rexp = ref.moe_align_tile_size(ids, 128, 8)
    assert np.array_equal(tok.cpu().numpy(), rtok) and np.array_equal(exp.cpu().numpy(), rexp)
    bad = ids.copy(); bad[0, 7] = 9  # expert id out of range is reported, not silently used
    with pytest.raises(cuda.CtbError):
        cuda.moe.moe_align_tile_size(torch.from_numpy(bad).cuda(), 128, 8)


def dev(d, *names):
    import torch
    return [torch.from_numpy(d[n]).cuda() for n in names]


# examples/moe.jl:402-410 main() cases (random routing as in its prepare())
# the reference's main() cases, then cases with some hundred slots per expert: several full blocks per expert, ragged
# last blocks, an intermediate size that is not a multiple of the tile
@pytest.mark.parametrize("T,H,E,I,topk", [(48, 512, 64, 1024, 8), (128, 512, 32, 1024, 4), (64, 1024, 64, 2048, 8),
                                          (1024, 256, 4, 384, 2), (600, 512, 2, 256, 1), (1500, 320, 5, 136, 1)])
def test_cutile_moe_reference_cases(cuda, T, H, E, I, topk):
    import torch
    d = inputs.moe(tokens=T, hidden=H, experts=E, inter=I, topk=topk, seed=4)
    ids, w = random_routing(T, E, topk, seed=1)
    X, w1, w2 = dev(d, "X", "w1", "w2")
    out = cuda.moe.cutile_moe(X, w1, w2, torch.from_numpy(w).cuda(), torch.from_numpy(ids).cuda(), 128, 128, 64)
    torch.cuda.synchronize()
    want = ref.moe_ffn(d["X"], d["w1"], d["w2"], w, ids)
    assert ref.rel_fro(out.cpu().numpy(), want) <= TOL


def test_moe_benchmark_config_with_router(cuda):
    import torch
    d = inputs.moe()  # 256 tokens, hidden 1024, 32 experts, inter 2048, top-2, seed 4
    X, Wr, w1, w2 = dev(d, "X", "Wr", "w1", "w2")
    w, ids = cuda.moe.moe_router(X, Wr, 2)
    out = cuda.moe.cutile_moe(X, w1, w2, w, ids, 128, 128, 64)
    torch.cuda.synchronize()
    rids, rgates, _ = ref.moe_router(d["X"], d["Wr"], 2)
    assert np.array_equal(ids.cpu().numpy(), rids)
    want = ref.moe_ffn(d["X"], d["w1"], d["w2"], rgates, rids)
    assert ref.rel_fro(out.cpu().numpy(), want) <= TOL
    out2 = cuda.moe.cutile_moe(X, w1, w2, w, ids, 128, 128, 64)
    assert torch.equal(out, out2)  # no atomics anywhere: bitwise repeatable


def test_moe_three_kernel_path_matches_reference_structure(cuda):
    """The reference's own decomposition (examples/moe.jl:228-256): grouped GEMM -> SiLU*mul -> grouped GEMM with
    routing weights -> sum over slots, through the per-kernel entry points."""
    import torch
    T, H, E, I, topk = 96, 256, 16, 512, 4
    d = inputs.moe(tokens=T, hidden=H, experts=E, inter=I, topk=topk, seed=8)
    ids, w = random_routing(T, E, topk, seed=2)
    X, w1, w2 = dev(d, "X", "w1", "w2")
    tok, exp = cuda.moe.moe_align_tile_size(torch.from_numpy(ids).cuda(), 64, E)
    total = T * topk
    cache1 = torch.zeros(total, 2 * I, device="cuda", dtype=torch.float16)
    cache2 = torch.zeros(total, I, device="cuda", dtype=torch.float16)
    cache3 = torch.zeros(total, H, device="cuda", dtype=torch.float16)
    wflat = torch.from_numpy(np.ascontiguousarray(w.T).reshape(-1)).cuda()  # vec(permutedims(topk_weights))
    cuda.moe.fused_moe_kernel(X, w1, cache1, wflat, tok, exp, topk, False, 64, 128, 64)
    cuda.moe.silu_and_mul_kernel(cache1[:, :I], cache1[:, I:], cache2, 512)
    cuda.moe.fused_moe_kernel(cache2, w2, cache3, wflat, tok, exp, 1, True, 64, 128, 64)
    out = cache3.view(T, topk, H).float().sum(dim=1)
    torch.cuda.synchronize()
    want = ref.moe_ffn(d["X"], d["w1"], d["w2"], w, ids)
    assert ref.rel_fro(out.cpu().numpy(), want) <= 3e-3  # three f16 roundings of intermediates, as in the reference
    fused = cuda.moe.cutile_moe(X, w1, w2, torch.from_numpy(w).cuda(), torch.from_numpy(ids).cuda(), 64, 128, 64)
    assert ref.rel_fro(fused.cpu().numpy(), want) <= TOL


def test_moe_full_size_token_permutation(cuda):
    """4096-token configuration: a token's output depends only on its own row and routing, so permuting the tokens
    permutes the output bit for bit; a 256-token sample is also checked against the oracle."""
    import torch
    d = inputs.moe(tokens=4096, seed=4)
    X, Wr, w1, w2 = dev(d, "X", "Wr", "w1", "w2")
    w, ids = cuda.moe.moe_router(X, Wr, 2)
    out = cuda.moe.cutile_moe(X, w1, w2, w, ids, 128, 128, 64)
    perm = torch.randperm(4096, device="cuda", generator=torch.Generator(device="cuda").manual_seed(0))
    outp = cuda.moe.cutile_moe(X[perm].contiguous(), w1, w2, w[:, perm].contiguous(), ids[:, perm].contiguous(),
                               128, 128, 64)
    assert torch.equal(outp, out[perm])
    sample = np.arange(0, 4096, 16)
    idn, wn = ids.cpu().numpy(), w.cpu().numpy()
    want = ref.moe_ffn(d["X"][sample], d["w1"], d["w2"], wn[:, sample], idn[:, sample])
    assert ref.rel_fro(out.cpu().numpy()[sample], want) <= TOL


def test_moe_rejections(cuda):
    import torch
    lib = cuda._lib
    d = inputs.moe(tokens=8, hidden=64, experts=4, inter=64, topk=2, seed=1)
    X, w1, w2 = dev(d, "X", "w1", "w2")
    ids, w = random_routing(8, 4, 2, 0)
    idd, wd = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    with pytest.raises(cuda.CtbError) as e:
        cuda.moe.cutile_moe(X, w1, w2, wd, idd, 100, 128, 64)
    assert e.value.status == lib.UNSUPPORTED_TILE
    with pytest.raises(cuda.CtbError) as e:
        cuda.moe.cutile_moe(X, w1, w2[:, :, :32].contiguous(), wd, idd, 128, 128, 64)
    assert e.value.status == lib.BAD_ARG
