# CuTileB200.jl — Julia call surface of libcutile_b200.so.
#
# Drop-in replacements for the entry points of cuTile.jl's examples
# (examples/{layernorm,softmax,matmul,batchmatmul,fmha,moe}.jl): same function
# names, same positional arguments, CuArray in / CuArray out.  Where the
# reference call is `@cuda backend=cuTile blocks=g kernel(args..., ct.Constant(x))`
# the replacement is `kernel(args..., x)`: constants are plain integers and the
# launch geometry is chosen by the library.
#
# NOT EXECUTED IN THE BUILD ENVIRONMENT (no Julia there).  Every wrapper is a
# size unpack plus one `ccall`; the same C ABI is exercised by the Python ctypes
# mirror (../../../cutile_b200), which is the tested path.
#
# Launch keywords of `@cuda backend=cuTile ...` (src/launch.jl:855-869) are accepted by
# every kernel function as keyword arguments: `num_ctas`, `occupancy`, `opt_level`,
# `num_worker_warps` are checked with the reference's ranges and are advisory,
# `stream` is honoured, `dependent`, `sm_arch` and `name` are accepted.
module CuTileB200

using CUDA

const LIB = get(ENV, "CUTILE_B200_LIB", joinpath(@__DIR__, "..", "..", "..", "cutile_b200", "libcutile_b200.so"))

const CTB_F32 = Cint(0)
const CTB_F16 = Cint(1)

struct CtbError <: Exception
    status::Cint
    msg::String
end
Base.showerror(io::IO, e::CtbError) = print(io, "libcutile_b200 status $(e.status): $(e.msg)")

check(st::Cint) = st == 0 ? nothing :
    throw(CtbError(st, unsafe_string(ccall((:ctb_last_error, LIB), Cstring, ()))))

const CONTEXTS = Dict{Int,Ptr{Cvoid}}()
function context()
    dev = CUDA.deviceid(CUDA.device())
    get!(CONTEXTS, dev) do
        out = Ref{Ptr{Cvoid}}(C_NULL)
        check(ccall((:ctb_create, LIB), Cint, (Ref{Ptr{Cvoid}}, Cint), out, dev))
        out[]
    end
end
stream() = reinterpret(Ptr{Cvoid}, CUDA.stream().handle)

"Checks the launch keywords of a call like the reference's validate_hint (src/language/types.jl:864-882) and returns the
raw stream handle to launch on."
function launch_opts(; num_ctas=nothing, occupancy=nothing, opt_level=nothing, num_worker_warps=nothing,
                     stream=nothing, dependent::Bool=false, sm_arch=nothing, name=nothing)
    for (k, v) in (:num_ctas => num_ctas, :occupancy => occupancy, :opt_level => opt_level, :num_worker_warps => num_worker_warps)
        v === nothing || v isa Integer || throw(ArgumentError("$k must be an integer, got $(typeof(v))"))
    end
    unset(v) = v === nothing ? Cint(-1) : Cint(v)
    st = ccall((:ctb_validate_hints, LIB), Cint, (Cint, Cint, Cint, Cint),
               unset(num_ctas), unset(occupancy), unset(opt_level), unset(num_worker_warps))
    st == 0 || throw(ArgumentError(unsafe_string(ccall((:ctb_last_error, LIB), Cstring, ()))))
    return stream === nothing ? CuTileB200.stream() : reinterpret(Ptr{Cvoid}, stream.handle)
end
dptr(a) = reinterpret(Ptr{Cvoid}, pointer(a))
dtype(::Type{Float32}) = CTB_F32
dtype(::Type{Float16}) = CTB_F16
dtype(::Type{Core.BFloat16}) = Cint(2)  # CTB_BF16 (flash attention)

"""
    timed(f; nruns=1, warmup=0) -> Vector{Float64}

`warmup` untimed calls of `f` (followed by a synchronize), then `nruns` calls each bracketed by CUDA events; the times
in milliseconds.  The measurement protocol of the reference's examples (examples/benchmarks.jl:12-13,104,159-171).
"""
function timed(f; nruns::Int=1, warmup::Int=0)
    for _ in 1:warmup
        f()
    end
    CUDA.synchronize()
    return Float64[1000 * (CUDA.@elapsed f()) for _ in 1:nruns]
end

"Synchronises the current stream and throws if a kernel recorded a bounded-wait expiry or a bad index."
check_device_status() = check(ccall((:ctb_check_device_status, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}), context(), stream()))

"f32 GEMM operands: `false` = truncated to TF32 by the tensor core (default), `true` = rounded to nearest even first."
set_tf32_rounding(nearest_even::Bool) =
    check(ccall((:ctb_set_tf32_rounding, LIB), Cint, (Ptr{Cvoid}, Cint), context(), nearest_even ? 1 : 0))

"How long kernels wait for another rank's flag before they give up (nanoseconds; 2 s by default)."
set_flag_wait_limit(ns::Integer) =
    check(ccall((:ctb_set_flag_wait_limit, LIB), Cint, (Ptr{Cvoid}, UInt64), context(), UInt64(ns)))

function versioninfo()
    buf = Vector{UInt8}(undef, 256)
    check(ccall((:ctb_version_info, LIB), Cint, (Ptr{UInt8}, Csize_t), buf, 256))
    unsafe_string(pointer(buf))
end

# ---- examples/softmax.jl ---------------------------------------------------
function softmax_tma_kernel(output::CuArray{T,2}, input::CuArray{T,2}, TILE_SIZE::Int; opts...) where {T}
    N, M = size(input)
    check(ccall((:ctb_softmax, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(output), dptr(input), N, M, stride(output, 2), stride(input, 2), 0, TILE_SIZE, dtype(T)))
end
function softmax_chunked_kernel(output::CuArray{T,2}, input::CuArray{T,2}, n_elems::Int, TILE_SIZE::Int; opts...) where {T}
    N, M = size(input)
    @assert n_elems == N
    check(ccall((:ctb_softmax, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(output), dptr(input), N, M, stride(output, 2), stride(input, 2), 1, TILE_SIZE, dtype(T)))
end

# ---- examples/layernorm.jl -------------------------------------------------
function layer_norm_fwd(X, W, B, Y, Mean, Rstd, eps::Float32, TILE_N::Int; opts...)
    N, M = size(X)
    check(ccall((:ctb_layernorm_fwd, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int64, Int64, Int64, Int64, Cfloat, Cint),
        context(), launch_opts(; opts...), dptr(X), dptr(W), dptr(B), dptr(Y), dptr(Mean), dptr(Rstd), N, M,
        stride(X, 2), stride(Y, 2), eps, TILE_N))
end
function layer_norm_bwd_dx_partial_dwdb(DX, DY, DW, DB, X, W, Mean, Rstd, Locks, GROUP_SIZE_M::Int, TILE_N::Int; opts...)
    N, M = size(X)
    check(ccall((:ctb_layernorm_bwd_dx_partial_dwdb, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Cint, Cint),
        context(), launch_opts(; opts...), dptr(DX), dptr(DY), dptr(DW), dptr(DB), dptr(X), dptr(W), dptr(Mean), dptr(Rstd),
        dptr(Locks), N, M, stride(X, 2), stride(DY, 2), stride(DX, 2), GROUP_SIZE_M, TILE_N))
end
function layer_norm_bwd_dwdb(DW, DB, FINAL_DW, FINAL_DB, TILE_M::Int, TILE_N::Int; opts...)
    N, G = size(DW)
    check(ccall((:ctb_layernorm_bwd_dwdb, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(DW), dptr(DB), dptr(FINAL_DW), dptr(FINAL_DB), N, G, TILE_M, TILE_N))
end

# ---- examples/matmul.jl, examples/batchmatmul.jl -----------------------------
function matmul_kernel(A::CuArray{T,2}, B::CuArray{T,2}, C::CuArray{T,2}, tm::Int, tn::Int, tk::Int; opts...) where {T}
    M, K = size(A); N = size(B, 2)
    check(ccall((:ctb_gemm, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Int64,
         Cint, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(A), dptr(B), dptr(C), M, N, K, stride(A, 2), stride(B, 2), stride(C, 2),
        dtype(T), tm, tn, tk))
end
function batch_matmul_kernel(A::CuArray{T,3}, B::CuArray{T,3}, C::CuArray{T,3}, tm::Int, tn::Int, tk::Int; opts...) where {T}
    M, K, Batch = size(A); N = size(B, 2)
    check(ccall((:ctb_gemm_batched, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Int64, Int64,
         Int64, Int64, Int64, Cint, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(A), dptr(B), dptr(C), M, N, K, Batch, stride(A, 2), stride(B, 2), stride(C, 2),
        stride(A, 3), stride(B, 3), stride(C, 3), dtype(T), tm, tn, tk))
end

# ---- examples/fmha.jl ------------------------------------------------------
function cutile_fmha(Q::CuArray{T}, K::CuArray{T}, V::CuArray{T};
                     qk_scale::Union{Float32,Nothing}=nothing, input_pos::Int=0,
                     tile_m::Int=128, tile_n::Int=128, query_group_size::Int=1, causal::Bool=false) where {T}
    D_k, SeqLen_Q, Heads, Batch = size(Q)
    D_v, SeqLen_KV, KV_Heads, _ = size(V)
    qk_scale === nothing && (qk_scale = Float32(1.0 / sqrt(D_k)))
    Out = CuArray{T}(undef, D_v, SeqLen_Q, Heads, Batch)
    check(ccall((:ctb_fmha_fwd, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64,
         Int64, Int64, Cfloat, Int32, Cint, Cint, Cint, Cint, Cint),
        context(), stream(), dptr(Q), dptr(K), dptr(V), dptr(Out), D_k, D_v, SeqLen_Q, SeqLen_KV, Heads, KV_Heads,
        Batch, qk_scale, Int32(input_pos), tile_m, tile_n, query_group_size, causal, dtype(T)))
    return Out
end

# ---- examples/moe.jl -------------------------------------------------------
ids_bits(::CuArray{Int32}) = Cint(32)
ids_bits(::CuArray{Int64}) = Cint(64)

"Router of the benchmark configuration: returns (topk_weights::CuArray{Float16}(T, topk), topk_ids::CuArray{Int32}(T, topk))."
function moe_router(hidden_states::CuArray{Float16,2}, W_r::CuArray{Float16,2}, topk::Int)
    H, T = size(hidden_states); E = size(W_r, 2)
    ids = CuArray{Int32}(undef, T, topk); w = CuArray{Float16}(undef, T, topk)
    check(ccall((:ctb_moe_router, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Cint),
        context(), stream(), dptr(hidden_states), dptr(W_r), dptr(ids), dptr(w), C_NULL, T, H, E, topk))
    return w, ids
end

function moe_align_tile_size(topk_ids::CuArray, tile_m::Int, num_experts::Int)
    T, topk = size(topk_ids)
    cap = ccall((:ctb_moe_max_blocks, LIB), Int64, (Int64, Int64, Int64, Cint), T, topk, num_experts, tile_m)
    tok = CuArray{Int32}(undef, cap * tile_m); ex = CuArray{Int32}(undef, cap); nb = CUDA.zeros(Int32, 1)
    check(ccall((:ctb_moe_align, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Cint, Int64, Int64, Int64, Cint, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64),
        context(), stream(), dptr(topk_ids), ids_bits(topk_ids), T, topk, num_experts, tile_m, dptr(tok), dptr(ex),
        dptr(nb), cap))
    n = Int(Array(nb)[1])
    return tok[1:n*tile_m], ex[1:n]
end

function fused_moe_kernel(A, B, C, topk_weights, sorted_token_ids, sorted_expert_ids,
                          num_token_replicas::Int, mul_routed_weight::Bool, TILE_M::Int, TILE_N::Int, TILE_K::Int; opts...)
    K, a_cols = size(A); N = size(B, 2); E = size(B, 3); c_cols = size(C, 2)
    check(ccall((:ctb_moe_fused_gemm, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64,
         Int64, Int64, Int64, Int64, Cint, Cint, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(A), dptr(B), dptr(C), dptr(topk_weights), dptr(sorted_token_ids),
        dptr(sorted_expert_ids), length(sorted_token_ids), K, N, E, a_cols, c_cols, num_token_replicas,
        mul_routed_weight, TILE_M, TILE_N, TILE_K))
end

function silu_and_mul_kernel(A, B, C, TILE_N::Int; opts...)   # A, B may be views of the halves of the gate/up buffer
    n, cols = size(C)
    check(ccall((:ctb_moe_silu_and_mul, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Cint),
        context(), launch_opts(; opts...), dptr(A), dptr(B), dptr(C), n, cols, stride(A, 2), stride(B, 2), stride(C, 2), TILE_N))
end

function cutile_moe(hidden_states::CuArray{T}, w1, w2, topk_weights, topk_ids, tile_m, tile_n, tile_k) where {T}
    hidden_size, num_tokens = size(hidden_states)
    intermediate_size = size(w2, 1); num_experts = size(w1, 3); _, topk = size(topk_ids)
    out = CuArray{T}(undef, hidden_size, num_tokens)
    check(ccall((:ctb_moe_ffn, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Cint, Ptr{Cvoid}, Int64,
         Int64, Int64, Int64, Int64, Cint, Cint, Cint),
        context(), stream(), dptr(hidden_states), dptr(w1), dptr(w2), dptr(topk_weights), dptr(topk_ids),
        ids_bits(topk_ids), dptr(out), num_tokens, hidden_size, intermediate_size, num_experts, topk,
        tile_m, tile_n, tile_k))
    return out
end

# ---- examples/vadd.jl, examples/transpose.jl --------------------------------
function vec_add_kernel_1d(a::CuArray{T,1}, b::CuArray{T,1}, c::CuArray{T,1}, tile::Int; opts...) where {T}
    n = length(a)
    check(ccall((:ctb_vadd, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Cint, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(a), dptr(b), dptr(c), n, 1, n, n, n, tile, 1, 0, dtype(T)))
end
function vec_add_kernel_1d_gather(a::CuArray{T,1}, b::CuArray{T,1}, c::CuArray{T,1}, tile::Int; opts...) where {T}
    n = length(a)
    check(ccall((:ctb_vadd, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Cint, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(a), dptr(b), dptr(c), n, 1, n, n, n, tile, 1, 1, dtype(T)))
end
function vec_add_kernel_2d(a::CuArray{T,2}, b::CuArray{T,2}, c::CuArray{T,2}, tile_x::Int, tile_y::Int; opts...) where {T}
    m, n = size(a)
    check(ccall((:ctb_vadd, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Cint, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(a), dptr(b), dptr(c), m, n, stride(a, 2), stride(b, 2), stride(c, 2),
        tile_x, tile_y, 0, dtype(T)))
end
function transpose_kernel(x::CuArray{T,2}, y::CuArray{T,2}, tm::Int, tn::Int; opts...) where {T}
    m, n = size(x)
    check(ccall((:ctb_transpose, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Cint, Cint, Cint),
        context(), launch_opts(; opts...), dptr(x), dptr(y), m, n, stride(x, 2), stride(y, 2), tm, tn, dtype(T)))
end

# ---- examples/fft.jl ---------------------------------------------------------
"fft_kernel of examples/fft.jl:22-126; the tables are the caller's (make_twiddles there)."
function fft_kernel(x_packed_in::CuArray{Float32,3}, y_packed_out::CuArray{Float32,3}, W0::CuArray{Float32,3},
                    W1::CuArray{Float32,3}, W2::CuArray{Float32,3}, T0::CuArray{Float32,3}, T1::CuArray{Float32,3},
                    N::Int, F0::Int, F1::Int, F2::Int, BS::Int, D::Int; opts...)
    size(x_packed_in) == size(y_packed_out) || throw(ArgumentError("fft_kernel: x and y differ in shape"))
    batch = length(x_packed_in) ÷ 2N
    check(ccall((:ctb_fft, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int64, Cint, Cint, Cint, Int64, Cint, Cint),
        context(), launch_opts(; opts...), dptr(x_packed_in), dptr(y_packed_out), dptr(W0), dptr(W1), dptr(W2), dptr(T0),
        dptr(T1), N, F0, F1, F2, batch, BS, D))
end

# ---- building blocks of the expert-parallel MoE ----
"dst(:, i) = src(:, cld(ids[i], num_token_replicas)); ids out of range give zero rows."
function moe_gather_rows(dst::CuArray{Float16,2}, src::CuArray{Float16,2}, ids::CuArray{Int32,1}, num_token_replicas::Int)
    check(ccall((:ctb_moe_gather_rows, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Cint, Int64),
        context(), stream(), dptr(dst), dptr(src), dptr(ids), length(ids), size(src, 1), num_token_replicas, size(src, 2)))
end

"dst(:, ids[i]) = src(:, i)."
function moe_scatter_rows(dst::CuArray{Float16,2}, src::CuArray{Float16,2}, ids::CuArray{Int32,1})
    check(ccall((:ctb_moe_scatter_rows, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64),
        context(), stream(), dptr(dst), dptr(src), dptr(ids), length(ids), size(src, 1), size(dst, 2)))
end

"out(:, t) = sum of the topk slot rows of token t; slots is (H, topk, T) (examples/moe.jl:256)."
function moe_combine(slots::CuArray{Float16,3}, out::CuArray{Float16,2})
    H, topk, T = size(slots)
    check(ccall((:ctb_moe_combine, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64),
        context(), stream(), dptr(slots), dptr(out), T, H, topk))
end

# ---- LayerNorm backward with built-in scratch (no context, no partial buffers; N <= 8192) ----
function layer_norm_bwd_static(DX, DY, X, W, Mean, Rstd, FINAL_DW, FINAL_DB)
    N, M = size(X)
    check(ccall((:ctb_layernorm_bwd_static, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int64, Int64, Int64, Int64, Int64),
        stream(), dptr(DX), dptr(DY), dptr(X), dptr(W), dptr(Mean), dptr(Rstd), dptr(FINAL_DW), dptr(FINAL_DB),
        N, M, stride(X, 2), stride(DY, 2), stride(DX, 2)))
end

"Reads and clears the status word of layer_norm_bwd_static on the current device (throws on a bounded-wait expiry)."
layer_norm_bwd_static_status() = check(ccall((:ctb_layernorm_bwd_static_status, LIB), Cint, (Ptr{Cvoid},), stream()))

# ---- several GPUs ------------------------------------------------------------
# One process, several devices: `g = Group([0, 1, ...])` creates a context per device, enables peer access and gives
# every device an NCCL communicator owned by the library.  All arrays of a call are vectors with one CuArray per device.
mutable struct Group
    handle::Ptr{Cvoid}
    devices::Vector{Int}
    eps::Dict{NTuple{3,Int},Vector{Ptr{Cvoid}}}
end
function Group(devices::Vector{Int})
    out = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:ctb_create_multi, LIB), Cint, (Ref{Ptr{Cvoid}}, Ptr{Cint}, Cint), out, Cint.(devices), length(devices)))
    Group(out[], devices, Dict())
end
function Base.close(g::Group)
    for v in values(g.eps), e in v
        ccall((:ctb_ep_destroy, LIB), Cvoid, (Ptr{Cvoid},), e)
    end
    empty!(g.eps)
    ccall((:ctb_destroy_multi, LIB), Cvoid, (Ptr{Cvoid},), g.handle)
    g.handle = C_NULL
end
streams(g::Group) = [begin CUDA.device!(d); stream() end for d in g.devices]
ptrs(xs) = Ptr{Cvoid}[dptr(x) for x in xs]

"batch_matmul_kernel over the group: A[i], B[i], C[i] hold device i's batches (batch-last: contiguous slabs)."
function batch_matmul_sharded(g::Group, A::Vector, B::Vector, C::Vector, tm::Int=128, tn::Int=128, tk::Int=64)
    M, K, _ = size(A[1]); N = size(B[1], 2); T = eltype(A[1])
    check(ccall((:ctb_gemm_batched_sharded, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Int64, Int64, Int64, Ptr{Int64},
         Int64, Int64, Int64, Int64, Int64, Int64, Cint, Cint, Cint, Cint),
        g.handle, streams(g), ptrs(A), ptrs(B), ptrs(C), M, N, K, Int64[size(a, 3) for a in A], M, K, M, M * K, K * N, M * N,
        dtype(T), tm, tn, tk))
    return C
end

"cutile_fmha over the group, split by batch: Q[i], K[i], V[i] hold device i's batches; returns the vector of outputs."
function cutile_fmha_sharded(g::Group, Q::Vector, K::Vector, V::Vector; qk_scale=nothing, input_pos::Int=0,
                             tile_m::Int=128, tile_n::Int=128, query_group_size::Int=1, causal::Bool=false)
    D_k, Sq, Heads, _ = size(Q[1]); D_v, Skv, KVH, _ = size(V[1]); T = eltype(Q[1])
    qk_scale === nothing && (qk_scale = Float32(1.0 / sqrt(D_k)))
    Out = [begin CUDA.device!(d); CuArray{T}(undef, D_v, Sq, Heads, size(q, 4)) end for (d, q) in zip(g.devices, Q)]
    check(ccall((:ctb_fmha_fwd_sharded, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Int64, Int64, Int64,
         Int64, Int64, Int64, Ptr{Int64}, Cfloat, Int32, Cint, Cint, Cint, Cint, Cint),
        g.handle, streams(g), ptrs(Q), ptrs(K), ptrs(V), ptrs(Out), D_k, D_v, Sq, Skv, Heads, KVH,
        Int64[size(q, 4) for q in Q], qk_scale, Int32(input_pos), tile_m, tile_n, query_group_size, causal, dtype(T)))
    return Out
end

function ep_states(g::Group, T_local::Int, H::Int, topk::Int)
    get!(g.eps, (T_local, H, topk)) do
        eps = Ptr{Cvoid}[]
        for i in 0:length(g.devices)-1
            out = Ref{Ptr{Cvoid}}(C_NULL)
            ctx = ccall((:ctb_group_ctx, LIB), Ptr{Cvoid}, (Ptr{Cvoid}, Cint), g.handle, i)
            check(ccall((:ctb_ep_create, LIB), Cint, (Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Ref{Ptr{Cvoid}}),
                        ctx, length(g.devices), i, T_local, H, topk, out))
            push!(eps, out[])
        end
        check(ccall((:ctb_ep_connect_local, LIB), Cint, (Ptr{Ptr{Cvoid}}, Cint), eps, length(eps)))
        eps
    end
end

const A2A_NCCL = Cint(0)
const A2A_PEER = Cint(1)

"Expert-parallel cutile_moe over the group (experts [r*E/N, (r+1)*E/N) on device r, tokens sharded by device).
 hidden_states[i] (H, T_local), w1[i] (H, 2I, E/N), w2[i] (I, H, E/N), topk_weights[i] / topk_ids[i] (T_local, topk) with global
 1-based expert ids (Int32).  a2a = A2A_PEER: stores into peer memory; A2A_NCCL: NCCL send/receive pairs."
function cutile_moe_ep(g::Group, hidden_states::Vector, w1::Vector, w2::Vector, topk_weights::Vector, topk_ids::Vector,
                       num_experts::Int, tile_m::Int, tile_n::Int, tile_k::Int; a2a::Cint=A2A_PEER)
    H, T_local = size(hidden_states[1]); I = size(w2[1], 1); topk = size(topk_ids[1], 2)
    out = [begin CUDA.device!(d); CuArray{Float16}(undef, H, T_local) end for d in g.devices]
    check(ccall((:ctb_moe_ffn_ep_group, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}},
         Ptr{Ptr{Cvoid}}, Ptr{Ptr{Cvoid}}, Int64, Int64, Int64, Int64, Int64, Cint, Cint, Cint, Cint),
        g.handle, ep_states(g, T_local, H, topk), streams(g), ptrs(hidden_states), ptrs(w1), ptrs(w2), ptrs(topk_weights),
        ptrs(topk_ids), ptrs(out), T_local, H, I, num_experts, topk, tile_m, tile_n, tile_k, a2a))
    return out
end

# ---- one process per GPU ----------------------------------------------------
# The library owns the NCCL communicator and the exchange buffers; the host program only carries two byte strings
# between its processes by its own means (MPI.jl, Distributed, files): the NCCL unique id drawn by rank 0, and every
# rank's buffer handle.  `exchange(bytes) -> Vector{Vector{UInt8}}` below is that means: it must return the byte
# strings of all ranks, in rank order, on every rank (an all-gather).
const UNIQUE_ID_BYTES = 128
const EP_HANDLE_BYTES = 64

"Rank 0 draws the NCCL unique id (ncclGetUniqueId) that `comm_init_rank` takes on every rank."
function comm_unique_id()
    id = zeros(UInt8, UNIQUE_ID_BYTES)
    check(ccall((:ctb_comm_unique_id, LIB), Cint, (Ptr{UInt8},), id))
    return id
end
"Attaches a communicator of `world` ranks to this process's context (collective: every rank calls it with the same id)."
comm_init_rank(id::Vector{UInt8}, rank::Int, world::Int) =
    check(ccall((:ctb_comm_init_rank, LIB), Cint, (Ptr{Cvoid}, Ptr{UInt8}, Cint, Cint), context(), id, rank, world))
"Tears the communicator down without waiting for outstanding operations (after a host-side failure of another rank)."
comm_abort() = check(ccall((:ctb_comm_abort, LIB), Cint, (Ptr{Cvoid},), context()))
"(rank, world, NCCL version) of this context's communicator; world == 1 when there is none."
function comm_info()
    r, w, v = Ref{Cint}(0), Ref{Cint}(0), Ref{Cint}(0)
    check(ccall((:ctb_comm_info, LIB), Cint, (Ptr{Cvoid}, Ref{Cint}, Ref{Cint}, Ref{Cint}), context(), r, w, v))
    return (Int(r[]), Int(w[]), Int(v[]))
end

"One rank's exchange buffers for a fixed (T_local, H, topk), mapped into every rank through CUDA IPC handles."
mutable struct EpRank
    handle::Ptr{Cvoid}
    rank::Int
    world::Int
    shape::NTuple{3,Int}
end
function EpRank(T_local::Int, H::Int, topk::Int, rank::Int, world::Int, exchange; with_nccl::Bool=true)
    if with_nccl && world > 1 && comm_info()[2] == 1   # no communicator on the context yet
        ids = exchange(rank == 0 ? comm_unique_id() : zeros(UInt8, UNIQUE_ID_BYTES))
        comm_init_rank(ids[1], rank, world)
    end
    out = Ref{Ptr{Cvoid}}(C_NULL)
    check(ccall((:ctb_ep_create, LIB), Cint, (Ptr{Cvoid}, Cint, Cint, Int64, Int64, Int64, Ref{Ptr{Cvoid}}),
                context(), world, rank, T_local, H, topk, out))
    mine = zeros(UInt8, EP_HANDLE_BYTES)
    check(ccall((:ctb_ep_export, LIB), Cint, (Ptr{Cvoid}, Ptr{UInt8}), out[], mine))
    for (q, h) in enumerate(exchange(mine))
        q - 1 == rank || check(ccall((:ctb_ep_import, LIB), Cint, (Ptr{Cvoid}, Cint, Ptr{UInt8}), out[], q - 1, h))
    end
    CUDA.synchronize()
    exchange(UInt8[])   # a barrier: every rank's flags are zero and mapped before anyone's first step
    return EpRank(out[], rank, world, (T_local, H, topk))
end
function Base.close(e::EpRank)
    e.handle == C_NULL || ccall((:ctb_ep_destroy, LIB), Cvoid, (Ptr{Cvoid},), e.handle)
    e.handle = C_NULL
end

"This rank's call of the expert-parallel cutile_moe (every rank must make it): hidden_states (H, T_local), w1 (H, 2I, E/N),
 w2 (I, H, E/N), topk_weights / topk_ids (T_local, topk) with global 1-based expert ids (Int32).  Returns (H, T_local) f16,
 bit-identical to cutile_moe on the gathered problem."
function cutile_moe_ep(e::EpRank, hidden_states::CuArray{Float16,2}, w1::CuArray{Float16,3}, w2::CuArray{Float16,3},
                       topk_weights::CuArray{Float16,2}, topk_ids::CuArray{Int32,2}, num_experts::Int,
                       tile_m::Int, tile_n::Int, tile_k::Int; a2a::Cint=A2A_PEER)
    H, T_local = size(hidden_states); I = size(w2, 1); topk = size(topk_ids, 2)
    (T_local, H, topk) == e.shape || throw(ArgumentError("cutile_moe_ep: shapes do not match the buffers"))
    out = CuArray{Float16}(undef, H, T_local)
    check(ccall((:ctb_moe_ffn_ep, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64,
         Int64, Int64, Cint, Cint, Cint, Cint),
        e.handle, stream(), dptr(hidden_states), dptr(w1), dptr(w2), dptr(topk_weights), dptr(topk_ids), dptr(out),
        T_local, H, I, num_experts, topk, tile_m, tile_n, tile_k, a2a))
    return out
end

"Releases this process's contexts (and their communicators and scratch)."
function destroy_contexts()
    for ctx in values(CONTEXTS)
        ccall((:ctb_destroy, LIB), Cvoid, (Ptr{Cvoid},), ctx)
    end
    empty!(CONTEXTS)
end
status_string(st::Integer) = unsafe_string(ccall((:ctb_status_string, LIB), Cstring, (Cint,), st))

"Bytes of context scratch `cutile_moe` needs for this shape; `reserve_workspace` sizes it up front (before a graph capture)."
moe_workspace_bytes(T, H, I, E, topk, tile_m) =
    ccall((:ctb_workspace_bytes, LIB), Csize_t, (Cint, Ptr{Int64}, Cint), 1, Int64[T, H, I, E, topk, tile_m], 6)
reserve_workspace(bytes) =
    check(ccall((:ctb_reserve_workspace, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}, Csize_t), context(), stream(), bytes))

# ---- ct.Tiled: host-level broadcast and mapreduce (src/broadcast.jl, src/mapreduce.jl) -------------------------
# `Tiled(A) .= f.(Tiled(B), ...)` flattens the Broadcasted tree into a postfix program that the library evaluates in one
# kernel; `sum(Tiled(A); dims)`, `prod`, `maximum`, `minimum` and `mapreduce(f, op, Tiled(A); dims)` go to
# ctb_tiled_mapreduce.  Arrays of up to three dimensions, Float32 or Float16.
import Base.Broadcast: BroadcastStyle, Broadcasted

struct Tiled{A<:CuArray}
    parent::A
end
Base.parent(t::Tiled) = t.parent
Base.size(t::Tiled) = size(t.parent)
Base.axes(t::Tiled) = axes(t.parent)
Base.ndims(::Type{<:Tiled{A}}) where {A} = ndims(A)
Base.eltype(::Type{<:Tiled{A}}) where {A} = eltype(A)
Base.Broadcast.broadcastable(t::Tiled) = t

struct TiledStyle{N} <: BroadcastStyle end
TiledStyle{M}(::Val{N}) where {N,M} = TiledStyle{N}()
BroadcastStyle(::Type{<:Tiled{A}}) where {A} = TiledStyle{ndims(A)}()
BroadcastStyle(::TiledStyle{N}, ::Base.Broadcast.DefaultArrayStyle{M}) where {N,M} = TiledStyle{max(N, M)}()
BroadcastStyle(::TiledStyle{N}, ::TiledStyle{M}) where {N,M} = TiledStyle{max(N, M)}()

const TILED_UNARY = Dict{Any,Cint}(identity => 16, (-) => 17, abs => 18, sqrt => 19, exp => 20, exp2 => 21, log => 22,
                                   log2 => 23, sin => 24, cos => 25, tanh => 26, inv => 27, abs2 => 28)
const TILED_BINARY = Dict{Any,Cint}((+) => 64, (-) => 65, (*) => 66, (/) => 67, max => 68, min => 69, (^) => 70)

function tiled_compile!(prog::Vector{Int32}, inputs::Vector{Any}, consts::Vector{Float32}, x)
    if x isa Tiled
        i = findfirst(a -> a === parent(x), inputs)
        i === nothing && (push!(inputs, parent(x)); i = length(inputs))
        append!(prog, (0, i - 1))
    elseif x isa Number
        v = Float32(x)
        i = findfirst(==(v), consts)
        i === nothing && (push!(consts, v); i = length(consts))
        append!(prog, (1, i - 1))
    elseif x isa Base.RefValue
        tiled_compile!(prog, inputs, consts, x[])
    elseif x isa Broadcasted
        foreach(a -> tiled_compile!(prog, inputs, consts, a), x.args)
        table = length(x.args) == 1 ? TILED_UNARY : TILED_BINARY
        haskey(table, x.f) || throw(ArgumentError("Tiled broadcast: no device code for $(x.f) with $(length(x.args)) argument(s)"))
        append!(prog, (table[x.f], 0))
    elseif x isa AbstractArray
        throw(ArgumentError("Tiled broadcast: host-side array leaf of type $(typeof(x))"))
    else
        throw(TypeError(:Tiled, "broadcast leaf", Union{Tiled,Number}, x))
    end
end

shape3(a) = Int64[size(a, 1), size(a, 2), size(a, 3)]

function tiled_broadcast!(dest::CuArray{T}, bc) where {T}
    ndims(dest) <= 3 || throw(ArgumentError("Tiled: at most three dimensions"))
    axes(dest) == axes(bc) || all(d -> size(dest, d) == get(map(length, axes(bc)), d, 1) || get(map(length, axes(bc)), d, 1) == 1, 1:3) ||
        throw(DimensionMismatch("destination $(size(dest)) and broadcast expression $(map(length, axes(bc)))"))
    isempty(dest) && return dest
    prog, inputs, consts = Int32[], Any[], Float32[]
    tiled_compile!(prog, inputs, consts, bc)
    strides = Int64[]
    for a in inputs
        eltype(a) == T || throw(ArgumentError("Tiled: operands and destination must share one element type"))
        run = 1
        for d in 1:3
            push!(strides, size(a, d) == 1 ? 0 : run)
            run *= size(a, d)
        end
    end
    check(ccall((:ctb_tiled_broadcast, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Int64}, Ptr{Ptr{Cvoid}}, Ptr{Int64}, Cint, Ptr{Int32}, Cint, Ptr{Float32}, Cint, Cint),
        context(), stream(), dptr(dest), shape3(dest), Ptr{Cvoid}[dptr(a) for a in inputs], strides, length(inputs), prog,
        length(prog) ÷ 2, consts, length(consts), dtype(T)))
    return dest
end

Base.Broadcast.materialize!(dest::Tiled, bc::Broadcasted) = tiled_broadcast!(parent(dest), bc)
Base.Broadcast.materialize!(dest::Tiled, x::Number) = tiled_broadcast!(parent(dest), Broadcasted(identity, (x,)))
function Base.copy(bc::Broadcasted{TiledStyle{N}}) where {N}
    find(t::Tiled) = parent(t)
    find(x) = nothing
    find(b::Broadcasted) = (for a in b.args; r = find(a); r === nothing || return r; end; nothing)
    arr = find(bc)
    arr === nothing && error("tiled broadcast requires at least one Tiled() argument")
    return tiled_broadcast!(similar(arr, eltype(arr), axes(bc)), bc)
end

function tiled_mapreduce(f, op, t::Tiled; dims=:)
    A = parent(t)
    T = eltype(A)
    ds = dims === Colon() ? (1:ndims(A)) : dims
    mask = 0
    for d in ds
        d isa Integer || throw(ArgumentError("dims must be integers"))
        d >= 1 || throw(ArgumentError("reduced dimension(s) must be >= 1"))
        d <= ndims(A) && (mask |= 1 << (d - 1))
    end
    R = similar(A, T, ntuple(d -> (mask >> (d - 1)) & 1 == 1 ? 1 : size(A, d), ndims(A)))
    haskey(TILED_UNARY, f) || throw(ArgumentError("Tiled mapreduce: no device code for $f"))
    code = op === (+) || op === Base.add_sum ? 64 : op === (*) || op === Base.mul_prod ? 66 : op === max ? 68 : op === min ? 69 :
           throw(ArgumentError("Tiled mapreduce: the reduction must be +, *, max or min"))
    check(ccall((:ctb_tiled_mapreduce, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Int64}, Cint, Cint, Cint, Cint),
        context(), stream(), dptr(R), dptr(A), shape3(A), mask, TILED_UNARY[f], code, dtype(T)))
    return dims === Colon() ? Array(R)[1] : R
end
Base.mapreduce(f, op, t::Tiled; dims=:) = tiled_mapreduce(f, op, t; dims)
Base.sum(t::Tiled; dims=:) = tiled_mapreduce(identity, +, t; dims)
Base.prod(t::Tiled; dims=:) = tiled_mapreduce(identity, *, t; dims)
Base.maximum(t::Tiled; dims=:) = tiled_mapreduce(identity, max, t; dims)
Base.minimum(t::Tiled; dims=:) = tiled_mapreduce(identity, min, t; dims)

end # module
