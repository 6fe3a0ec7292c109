# LayerNorm forward / backward through libcutile_b200; harness interface and kernel signatures of examples/layernorm.jl.
# Not executed in the build environment.
using CUDA
using CuTileB200: layer_norm_fwd, layer_norm_bwd_dx_partial_dwdb, layer_norm_bwd_dwdb, timed

function prepare(; benchmark::Bool=false, M::Int=benchmark ? 4096 : 256, N::Int=benchmark ? 4096 : 256,
                 eps::Float32=1f-5, GROUP_SIZE_M::Int=64)
    f32(dims...) = CuArray{Float32}(undef, dims...)
    return (; X=CUDA.randn(Float32, N, M), W=0.5f0 .+ CUDA.rand(Float32, N), B=0.1f0 .* CUDA.randn(Float32, N),
            DY=CUDA.randn(Float32, N, M), Y=f32(N, M), Mean=f32(M), Rstd=f32(M), DX=f32(N, M),
            DW_partial=f32(N, GROUP_SIZE_M), DB_partial=f32(N, GROUP_SIZE_M), Locks=CuArray{Int}(undef, GROUP_SIZE_M),
            FINAL_DW=f32(N), FINAL_DB=f32(N), M, N, eps, GROUP_SIZE_M)
end

function run(data; TILE_N::Int=1024, TILE_M::Int=32, nruns::Int=1, warmup::Int=0)
    d = data
    fwd() = layer_norm_fwd(d.X, d.W, d.B, d.Y, d.Mean, d.Rstd, d.eps, TILE_N)
    function bwd()   # no zero-fills: every partial column has a single writer, the locks are not used
        layer_norm_bwd_dx_partial_dwdb(d.DX, d.DY, d.DW_partial, d.DB_partial, d.X, d.W, d.Mean, d.Rstd, d.Locks,
                                       d.GROUP_SIZE_M, TILE_N)
        layer_norm_bwd_dwdb(d.DW_partial, d.DB_partial, d.FINAL_DW, d.FINAL_DB, TILE_M, TILE_N)
    end
    fwd()
    times_fwd = timed(fwd; nruns, warmup)
    times_bwd = timed(bwd; nruns, warmup)
    return (; d.Y, d.Mean, d.Rstd, d.DX, d.FINAL_DW, d.FINAL_DB, times_fwd, times_bwd)
end

function verify(data, result)
    X, W, B, DY = (Float64.(Array(a)) for a in (data.X, data.W, data.B, data.DY))
    N = data.N
    mu = sum(X; dims=1) ./ N
    rstd = 1 ./ sqrt.(sum((X .- mu) .^ 2; dims=1) ./ N .+ data.eps)
    xhat = (X .- mu) .* rstd
    close(got, want) = maximum(abs.(Float64.(Array(got)) .- want)) <= 1e-5 * maximum(abs.(want))
    @assert close(result.Y, xhat .* W .+ B)
    wdy = W .* DY
    c1 = sum(xhat .* wdy; dims=1) ./ N
    c2 = sum(wdy; dims=1) ./ N
    @assert close(result.DX, (wdy .- (xhat .* c1 .+ c2)) .* rstd)
    @assert close(result.FINAL_DW, vec(sum(DY .* xhat; dims=2)))
    @assert close(result.FINAL_DB, vec(sum(DY; dims=2)))
end

# forward: read X, write Y; backward: read X and dY, write dX (vectors are negligible)
metric(data) = Dict("cuTile Fwd" => (2 * data.M * data.N * 4, "GB/s"), "cuTile Bwd" => (3 * data.M * data.N * 4, "GB/s"))
