"""GPU parity of the flash-attention forward kernel against the float64 oracle.

Tolerance: relative Frobenius error <= 2e-3 (f16 operands, f32 softmax state and
accumulation, f16 output).  The reference's own check is norm-wise rtol=1e-2,
atol=1e-3 (examples/fmha.jl:277-282)."""
import numpy as np
import pytest

from oracle import inputs, ref

pytestmark = pytest.mark.gpu
TOL = 2e-3


def run(cuda, d, **kw):
    import torch
    Q, K, V = (torch.from_numpy(d[k]).cuda() for k in ("Q", "K", "V"))
    out = cuda.fmha.cutile_fmha(Q, K, V, **kw)
    torch.cuda.synchronize()
    return out.cpu().numpy()


# examples/fmha.jl:314-325 main() cases, then the benchmark shape
@pytest.mark.parametrize("batch,heads,seq,causal", [(2, 8, 128, False), (2, 8, 128, True), (4, 16, 256, True),
                                                    (8, 16, 1024, True), (1, 2, 1024, False)])
def test_fmha_reference_cases(cuda, batch, heads, seq, causal):
    d = inputs.fmha(batch, heads, seq, seq, 64, seed=3)
    out = run(cuda, d, causal=causal)
    want = ref.fmha(d["Q"], d["K"], d["V"], causal=causal)
    assert out.dtype == np.float16
    assert ref.rel_fro(out, want) <= TOL
    err = np.linalg.norm(out.astype(np.float64) - want)
    assert err <= max(1e-3, 1e-2 * np.linalg.norm(want))  # the reference's own criterion


@pytest.mark.parametrize("seq_q,seq_kv,causal,input_pos,heads,kv_heads", [
    (200, 300, False, 0, 4, 4),    # ragged Q and K tiles (EVEN_K false)
    (200, 200, True, 0, 4, 4),     # ragged + causal
    (128, 384, True, 256, 4, 4),   # prefill with a cache: queries sit at positions 256..383
    (100, 333, True, 233, 2, 2),   # ragged everything with an offset
    (256, 256, True, 0, 8, 2),     # grouped-query attention, group of 4
    (256, 512, False, 0, 6, 3),    # GQA, non-causal, rectangular
    (1, 1, True, 0, 1, 1),         # a single query and key
])
def test_fmha_options(cuda, seq_q, seq_kv, causal, input_pos, heads, kv_heads):
    d = inputs.fmha(2, heads, seq_q, seq_kv, 64, kv_heads=kv_heads, seed=13)
    out = run(cuda, d, causal=causal, input_pos=input_pos, query_group_size=heads // kv_heads)
    want = ref.fmha(d["Q"], d["K"], d["V"], causal=causal, input_pos=input_pos)
    assert ref.rel_fro(out, want) <= TOL
    for h in range(heads):  # per head, so that a wrong KV-head mapping cannot hide in the norm
        assert ref.rel_fro(out[:, h], want[:, h]) <= TOL


def test_fmha_scale_and_large_scores(cuda):
    d = inputs.fmha(1, 2, 256, 256, 64, seed=21)
    d["Q"] = (d["Q"].astype(np.float32) * 6).astype(np.float16)  # sharp softmax: exercises the running max
    out = run(cuda, d, causal=True, qk_scale=0.3)
    want = ref.fmha(d["Q"], d["K"], d["V"], qk_scale=0.3, causal=True)
    assert ref.rel_fro(out, want) <= TOL


def test_fmha_causal_prefix_property_full_size(cuda):
    """Size-independent property at the benchmark shape: under the causal mask the output of the first 512
    queries does not depend on the later keys/values, so it equals the result on the truncated problem."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(3)
    Q, K, V = (torch.randn(8, 16, 1024, 64, device="cuda", generator=g).half() for _ in range(3))
    full = cuda.fmha.cutile_fmha(Q, K, V, causal=True)
    half = cuda.fmha.cutile_fmha(Q[:, :, :512].contiguous(), K[:, :, :512].contiguous(), V[:, :, :512].contiguous(),
                                 causal=True)
    assert torch.equal(full[:, :, :512], half)
    assert torch.isfinite(full).all()


def test_fmha_rejections(cuda):
    import torch
    lib = cuda._lib
    q = torch.zeros(1, 2, 128, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(cuda.CtbError) as e:
        cuda.fmha.cutile_fmha(q, q, q, tile_m=96)
    assert e.value.status == lib.UNSUPPORTED_TILE
    with pytest.raises(cuda.CtbError) as e:
        cuda.fmha.cutile_fmha(q, q, q, query_group_size=3)
    assert e.value.status == lib.BAD_ARG
    q32 = torch.zeros(1, 2, 128, 32, device="cuda", dtype=torch.float16)
    with pytest.raises(cuda.CtbError) as e:
        cuda.fmha.cutile_fmha(q32, q32, q32)
    assert e.value.status == lib.UNSUPPORTED


@pytest.mark.parametrize("batch,heads,seq_q,seq_kv,causal,input_pos,kv_heads", [
    (2, 8, 128, 128, True, 0, 8), (8, 16, 1024, 1024, True, 0, 16), (2, 4, 200, 333, True, 133, 2), (1, 2, 256, 512, False, 0, 2)])
def test_fmha_bf16(cuda, batch, heads, seq_q, seq_kv, causal, input_pos, kv_heads):
    """bfloat16 operands (examples/fmha.jl takes the element type as a parameter, :236): the same kernel with bf16 MMAs,
    probabilities and output rounded to bf16.  The oracle is fed the bf16-rounded inputs; tolerance 1e-2 (8 mantissa
    bits in P and in the output)."""
    import torch
    d = inputs.fmha(batch, heads, seq_q, seq_kv, 64, kv_heads=kv_heads, seed=17)
    Q, K, V = (torch.from_numpy(d[k].astype(np.float32)).cuda().to(torch.bfloat16) for k in ("Q", "K", "V"))
    out = cuda.fmha.cutile_fmha(Q, K, V, causal=causal, input_pos=input_pos, query_group_size=heads // kv_heads)
    torch.cuda.synchronize()
    assert out.dtype == torch.bfloat16
    back = lambda t: t.float().cpu().numpy()
    want = ref.fmha(back(Q), back(K), back(V), causal=causal, input_pos=input_pos)
    assert ref.rel_fro(back(out), want) <= 1e-2
    cuda.check_device_status(0)
