# Matrix transpose through libcutile_b200; interface of examples/transpose.jl.  Not executed in the build environment.
using CUDA
using CuTileB200: transpose_kernel, timed

function prepare(; benchmark::Bool=false, m::Int=benchmark ? 8192 : 1024, n::Int=benchmark ? 8192 : 512, T::DataType=Float32)
    x = CUDA.rand(T, m, n)
    return (; x, y=similar(x, n, m), m, n)
end

function run(data; tm::Int=64, tn::Int=64, nruns::Int=1, warmup::Int=0)
    return (; data.y, times=timed(() -> transpose_kernel(data.x, data.y, tm, tn); nruns, warmup))
end

verify(data, result) = @assert Array(result.y) == permutedims(Array(data.x))

metric(data) = (2 * data.m * data.n * sizeof(eltype(data.x)), "GB/s")
