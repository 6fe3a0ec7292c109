# Vector / matrix addition through libcutile_b200; interface of examples/vadd.jl.  Not executed in the build environment.
using CUDA
using CuTileB200: vec_add_kernel_1d, vec_add_kernel_1d_gather, vec_add_kernel_2d, timed

function prepare(; benchmark::Bool=false, shape::Tuple=benchmark ? (2^27,) : (1_024_000,), use_gather::Bool=false,
                 T::DataType=Float32)
    a = CUDA.rand(T, shape...)
    return (; a, b=CUDA.rand(T, shape...), c=similar(a), shape, use_gather)
end

function run(data; tile::Union{Int,Tuple{Int,Int}}=1024, nruns::Int=1, warmup::Int=0)
    (; a, b, c, shape, use_gather) = data
    call = if length(shape) == 2
        tx, ty = tile isa Tuple ? tile : (tile, tile)
        () -> vec_add_kernel_2d(a, b, c, tx, ty)
    elseif use_gather
        () -> vec_add_kernel_1d_gather(a, b, c, first(tile))
    else
        () -> vec_add_kernel_1d(a, b, c, first(tile))
    end
    return (; c, times=timed(call; nruns, warmup))
end

verify(data, result) = @assert Array(result.c) == Array(data.a) .+ Array(data.b)

metric(data) = (3 * prod(data.shape) * sizeof(eltype(data.a)), "GB/s")
