# Batched complex FFT through libcutile_b200; interface of examples/fft.jl.  Not executed in the build environment.
using CUDA, FFTW
using CuTileB200: fft_kernel, timed

planes(z) = (out = zeros(Float32, 2, size(z)...); out[1, :, :] = real.(z); out[2, :, :] = imag.(z); out)
root(i, j, n) = ComplexF32(cispi(-2 * i * j / n))
dft_matrix(n) = planes([root(i, j, n) for i in 0:n-1, j in 0:n-1])

function make_twiddles((F0, F1, F2)::NTuple{3,Int})
    N, F1F2 = F0 * F1 * F2, F1 * F2
    T0 = planes([root(i, j, N) for j in 0:F1F2-1, i in 0:F0-1])      # (2, F1F2, F0)
    T1 = planes([root(j, k, F1F2) for k in 0:F2-1, j in 0:F1-1])     # (2, F2, F1)
    return dft_matrix(F0), dft_matrix(F1), dft_matrix(F2), T0, T1
end

function prepare(; benchmark::Bool=false, batch::Int=benchmark ? 256 : 2,
                 factors::NTuple{3,Int}=benchmark ? (16, 16, 16) : (2, 2, 2),
                 atom_packing_dim::Int=min(64, 2 * prod(factors)))
    N, D = prod(factors), atom_packing_dim
    @assert 2N % D == 0 "2 * N must be divisible by atom_packing_dim"
    input = CUDA.randn(ComplexF32, N, batch)
    tables = map(CuArray, make_twiddles(factors))
    x_packed = reshape(reinterpret(reshape, Float32, input), D, 2N ÷ D, batch)
    y_packed = CuArray{Float32}(undef, D, 2N ÷ D, batch)
    return (; input, x_packed, y_packed, tables, factors, batch, N, D)
end

function run(data; nruns::Int=1, warmup::Int=0)
    (; x_packed, y_packed, tables, factors, batch, N, D) = data
    times = timed(() -> fft_kernel(x_packed, y_packed, tables..., N, factors..., 1, D); nruns, warmup)
    output = copy(reinterpret(reshape, ComplexF32, reshape(y_packed, 2, N, batch)))
    return (; output, times)
end

verify(data, result) = @assert isapprox(Array(result.output), FFTW.fft(Array(data.input), 1), rtol=1e-4)

metric(data) = (0, "μs")   # a latency benchmark: the time is the figure
