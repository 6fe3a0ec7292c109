# Mixture-of-experts FFN through libcutile_b200; interface of examples/moe.jl (cutile_moe, moe_align_tile_size), with the
# benchmark configuration's router in front (top-2 over 32 experts).  Not executed in the build environment.
using CUDA
using CuTileB200: cutile_moe, moe_router, moe_align_tile_size, timed

function prepare(; benchmark::Bool=false, num_tokens::Int=256, hidden_size::Int=benchmark ? 1024 : 256,
                 num_experts::Int=benchmark ? 32 : 8, intermediate_size::Int=benchmark ? 2048 : 512, topk::Int=2)
    h16(s, dims...) = Float16.(s .* CUDA.randn(Float32, dims...))
    hidden_states = h16(1f0, hidden_size, num_tokens)
    W_r = h16(0.02f0, hidden_size, num_experts)
    w1 = h16(0.02f0, hidden_size, 2 * intermediate_size, num_experts)     # gate rows, then up rows
    w2 = h16(0.02f0, intermediate_size, hidden_size, num_experts)
    topk_weights, topk_ids = moe_router(hidden_states, W_r, topk)
    return (; hidden_states, W_r, w1, w2, topk_weights, topk_ids, num_tokens, hidden_size, num_experts, intermediate_size, topk)
end

function run(data; tile_m::Int=128, tile_n::Int=128, tile_k::Int=64, nruns::Int=1, warmup::Int=0)
    call() = cutile_moe(data.hidden_states, data.w1, data.w2, data.topk_weights, data.topk_ids, tile_m, tile_n, tile_k)
    out = call()
    times = timed(call; nruns, warmup)
    return (; out, times)
end

function verify(data, result)
    X, w1, w2 = Float64.(Array(data.hidden_states)), Float64.(Array(data.w1)), Float64.(Array(data.w2))
    gates, ids = Float64.(Array(data.topk_weights)), Array(data.topk_ids)
    I = data.intermediate_size
    want = zeros(data.hidden_size, data.num_tokens)
    for t in 1:data.num_tokens, s in 1:data.topk
        e = ids[t, s]
        g, u = w1[:, 1:I, e]' * X[:, t], w1[:, I+1:2I, e]' * X[:, t]
        want[:, t] .+= gates[t, s] .* (w2[:, :, e]' * ((g ./ (1 .+ exp.(-g))) .* u))
    end
    @assert sqrt(sum(abs2, Float64.(Array(result.out)) .- want) / sum(abs2, want)) <= 2e-3
end

metric(data) = (2 * data.num_tokens * data.topk * data.hidden_size * data.intermediate_size * 3, "TFLOPS")
