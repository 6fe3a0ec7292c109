# Flash attention forward through libcutile_b200; interface of examples/fmha.jl (cutile_fmha allocates and returns Out).
# Not executed in the build environment.
using CUDA
using CuTileB200: cutile_fmha, timed

function prepare(; benchmark::Bool=false, D_k::Int=64, SeqLen_Q::Int=benchmark ? 1024 : 256, Heads::Int=benchmark ? 16 : 4,
                 Batch::Int=benchmark ? 8 : 2, D_v::Int=D_k, SeqLen_KV::Int=SeqLen_Q, KV_Heads::Int=Heads,
                 causal::Bool=true, T::DataType=Float16)
    return (; Q=T.(CUDA.randn(Float32, D_k, SeqLen_Q, Heads, Batch)), K=T.(CUDA.randn(Float32, D_k, SeqLen_KV, KV_Heads, Batch)),
            V=T.(CUDA.randn(Float32, D_v, SeqLen_KV, KV_Heads, Batch)), D_k, D_v, SeqLen_Q, SeqLen_KV, Heads, KV_Heads, Batch,
            causal, query_group_size=Heads ÷ KV_Heads)
end

function run(data; tile_m::Int=128, tile_n::Int=128, nruns::Int=1, warmup::Int=0)
    call() = cutile_fmha(data.Q, data.K, data.V; tile_m, tile_n, data.causal, data.query_group_size)
    out = call()
    times = timed(call; nruns, warmup)
    return (; out, times)
end

function verify(data, result)
    Q, K, V = (Float64.(Array(a)) for a in (data.Q, data.K, data.V))
    got = Float64.(Array(result.out))
    scale = 1 / sqrt(data.D_k)
    num = den = 0.0
    for b in 1:data.Batch, h in 1:data.Heads
        kv = cld(h, data.query_group_size)
        s = (Q[:, :, h, b]' * K[:, :, kv, b]) .* scale                     # (SeqLen_Q, SeqLen_KV)
        data.causal && (s[[i < j for i in 1:data.SeqLen_Q, j in 1:data.SeqLen_KV]] .= -Inf)
        p = exp.(s .- maximum(s; dims=2))
        p ./= sum(p; dims=2)
        want = V[:, :, kv, b] * p'                                         # (D_v, SeqLen_Q)
        num += sum(abs2, got[:, :, h, b] .- want)
        den += sum(abs2, want)
    end
    @assert sqrt(num / den) <= 2e-3
end

# the reference's convention: 4 * B * H * Sq * Skv * D, not halved for the causal mask
metric(data) = (4 * data.Batch * data.Heads * data.SeqLen_Q * data.SeqLen_KV * data.D_k, "TFLOPS")
