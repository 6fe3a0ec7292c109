# Row softmax through libcutile_b200: same harness interface (prepare / run / verify / metric) and the same kernel
# names and argument order as examples/softmax.jl of cuTile.jl, so that the reference's benchmark driver can time it.
# Not executed in the build environment.
using CUDA
using CuTileB200: softmax_tma_kernel, softmax_chunked_kernel, timed

function prepare(; benchmark::Bool=false, M::Int=benchmark ? 4096 : 256, N::Int=benchmark ? 4096 : 256, T::DataType=Float32)
    input = T(2) .* CUDA.randn(T, N, M)          # logits ~ N(0, 2^2); (N, M): a column is one softmax problem
    return (; input, output_tma=similar(input), output_chunked=similar(input), M, N)
end

function run(data; tile_tma::Int=nextpow(2, data.N), tile_chunked::Int=1024, nruns::Int=1, warmup::Int=0)
    (; input, output_tma, output_chunked, N) = data
    times = Dict{String,Vector{Float64}}(
        "B200 single tile" => timed(() -> softmax_tma_kernel(output_tma, input, tile_tma); nruns, warmup),
        "B200 chunked" => timed(() -> softmax_chunked_kernel(output_chunked, input, N, tile_chunked); nruns, warmup))
    return (; output_tma, output_chunked, times)
end

function verify(data, result)
    x = Float64.(Array(data.input))
    want = exp.(x .- maximum(x; dims=1))
    want ./= sum(want; dims=1)
    for out in (result.output_tma, result.output_chunked)
        @assert maximum(abs.(Float64.(Array(out)) .- want)) <= 1e-5 * maximum(want)
    end
end

# one read and one write of the matrix for both variants (the chunked variant's re-reads hit on-chip memory)
metric(data) = (2 * data.M * data.N * sizeof(eltype(data.input)), "GB/s")
