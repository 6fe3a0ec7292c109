# Dense GEMM C = A * B (f32 storage, TF32 tensor-core operands) through libcutile_b200; interface of examples/matmul.jl.
# Not executed in the build environment.
using CUDA
using CuTileB200: matmul_kernel, timed

function prepare(; benchmark::Bool=false, M::Int=benchmark ? 4096 : 256, N::Int=benchmark ? 4096 : 256,
                 K::Int=benchmark ? 4096 : 256, T::DataType=Float32)
    u(dims...) = T(2) .* CUDA.rand(T, dims...) .- T(1)      # U(-1, 1)
    return (; A=u(M, K), B=u(K, N), C=CuArray{T}(undef, M, N), M, N, K)
end

function run(data; tm::Int=64, tn::Int=64, tk::Int=64, nruns::Int=1, warmup::Int=0)
    times = timed(() -> matmul_kernel(data.A, data.B, data.C, tm, tn, tk); nruns, warmup)
    return (; data.C, times)
end

function verify(data, result)
    want = Float64.(Array(data.A)) * Float64.(Array(data.B))
    err = sqrt(sum(abs2, Float64.(Array(result.C)) .- want) / sum(abs2, want))
    @assert err <= 5e-3      # TF32 operands, f32 accumulation
end

metric(data) = (2 * data.M * data.N * data.K, "TFLOPS")
