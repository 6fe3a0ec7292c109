# Batched GEMM (batch last) through libcutile_b200; interface of examples/batchmatmul.jl.  The benchmark shape is the
# benchmark configuration's (batch 8 of A[1024 x 2048] * B[2048 x 512]).  Not executed in the build environment.
using CUDA
using CuTileB200: batch_matmul_kernel, timed

function prepare(; benchmark::Bool=false, Batch::Int=benchmark ? 8 : 4, M::Int=benchmark ? 1024 : 256,
                 K::Int=benchmark ? 2048 : 128, N::Int=benchmark ? 512 : 256, T::DataType=Float32)
    u(dims...) = T(2) .* CUDA.rand(T, dims...) .- T(1)
    return (; A=u(M, K, Batch), B=u(K, N, Batch), C=CuArray{T}(undef, M, N, Batch), M, K, N, Batch)
end

function run(data; tm::Int=128, tn::Int=128, tk::Int=64, nruns::Int=1, warmup::Int=0)
    times = timed(() -> batch_matmul_kernel(data.A, data.B, data.C, tm, tn, tk); nruns, warmup)
    return (; data.C, times)
end

function verify(data, result)
    A, B, C = Float64.(Array(data.A)), Float64.(Array(data.B)), Float64.(Array(result.C))
    tol = eltype(data.A) == Float32 ? 5e-3 : 2e-3
    for b in 1:data.Batch
        want = A[:, :, b] * B[:, :, b]
        @assert sqrt(sum(abs2, C[:, :, b] .- want) / sum(abs2, want)) <= tol
    end
end

metric(data) = (2 * data.M * data.N * data.K * data.Batch, "TFLOPS")
