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
# mirror (../cutile_b200), which is the tested path.
module CuTileB200

using CUDA

const LIB = get(ENV, "CUTILE_B200_LIB", joinpath(@__DIR__, "..", "cutile_b200", "libcutile_b200.so"))

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
dptr(a) = reinterpret(Ptr{Cvoid}, pointer(a))
dtype(::Type{Float32}) = CTB_F32
dtype(::Type{Float16}) = CTB_F16

function versioninfo()
    buf = Vector{UInt8}(undef, 256)
    check(ccall((:ctb_version_info, LIB), Cint, (Ptr{UInt8}, Csize_t), buf, 256))
    unsafe_string(pointer(buf))
end

# ---- examples/softmax.jl ---------------------------------------------------
function softmax_tma_kernel(output::CuArray{T,2}, input::CuArray{T,2}, TILE_SIZE::Int) where {T}
    N, M = size(input)
    check(ccall((:ctb_softmax, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Cint, Cint, Cint),
        context(), stream(), dptr(output), dptr(input), N, M, stride(output, 2), stride(input, 2), 0, TILE_SIZE, dtype(T)))
end
function softmax_chunked_kernel(output::CuArray{T,2}, input::CuArray{T,2}, n_elems::Int, TILE_SIZE::Int) where {T}
    N, M = size(input)
    @assert n_elems == N
    check(ccall((:ctb_softmax, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Cint, Cint, Cint),
        context(), stream(), dptr(output), dptr(input), N, M, stride(output, 2), stride(input, 2), 1, TILE_SIZE, dtype(T)))
end

# ---- examples/layernorm.jl -------------------------------------------------
function layer_norm_fwd(X, W, B, Y, Mean, Rstd, eps::Float32, TILE_N::Int)
    N, M = size(X)
    check(ccall((:ctb_layernorm_fwd, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Int64, Int64, Int64, Int64, Cfloat, Cint),
        context(), stream(), dptr(X), dptr(W), dptr(B), dptr(Y), dptr(Mean), dptr(Rstd), N, M,
        stride(X, 2), stride(Y, 2), eps, TILE_N))
end
function layer_norm_bwd_dx_partial_dwdb(DX, DY, DW, DB, X, W, Mean, Rstd, Locks, GROUP_SIZE_M::Int, TILE_N::Int)
    N, M = size(X)
    check(ccall((:ctb_layernorm_bwd_dx_partial_dwdb, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid},
         Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Cint, Cint),
        context(), stream(), dptr(DX), dptr(DY), dptr(DW), dptr(DB), dptr(X), dptr(W), dptr(Mean), dptr(Rstd),
        dptr(Locks), N, M, stride(X, 2), stride(DY, 2), stride(DX, 2), GROUP_SIZE_M, TILE_N))
end
function layer_norm_bwd_dwdb(DW, DB, FINAL_DW, FINAL_DB, TILE_M::Int, TILE_N::Int)
    N, G = size(DW)
    check(ccall((:ctb_layernorm_bwd_dwdb, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Cint, Cint, Cint),
        context(), stream(), dptr(DW), dptr(DB), dptr(FINAL_DW), dptr(FINAL_DB), N, G, TILE_M, TILE_N))
end

# ---- examples/matmul.jl, examples/batchmatmul.jl -----------------------------
function matmul_kernel(A::CuArray{T,2}, B::CuArray{T,2}, C::CuArray{T,2}, tm::Int, tn::Int, tk::Int) where {T}
    M, K = size(A); N = size(B, 2)
    check(ccall((:ctb_gemm, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Int64,
         Cint, Cint, Cint, Cint),
        context(), stream(), dptr(A), dptr(B), dptr(C), M, N, K, stride(A, 2), stride(B, 2), stride(C, 2),
        dtype(T), tm, tn, tk))
end
function batch_matmul_kernel(A::CuArray{T,3}, B::CuArray{T,3}, C::CuArray{T,3}, tm::Int, tn::Int, tk::Int) where {T}
    M, K, Batch = size(A); N = size(B, 2)
    check(ccall((:ctb_gemm_batched, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Int64, Int64,
         Int64, Int64, Int64, Cint, Cint, Cint, Cint),
        context(), stream(), dptr(A), dptr(B), dptr(C), M, N, K, Batch, stride(A, 2), stride(B, 2), stride(C, 2),
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
                          num_token_replicas::Int, mul_routed_weight::Bool, TILE_M::Int, TILE_N::Int, TILE_K::Int)
    K, a_cols = size(A); N = size(B, 2); E = size(B, 3); c_cols = size(C, 2)
    check(ccall((:ctb_moe_fused_gemm, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64,
         Int64, Int64, Int64, Int64, Cint, Cint, Cint, Cint, Cint),
        context(), stream(), dptr(A), dptr(B), dptr(C), dptr(topk_weights), dptr(sorted_token_ids),
        dptr(sorted_expert_ids), length(sorted_token_ids), K, N, E, a_cols, c_cols, num_token_replicas,
        mul_routed_weight, TILE_M, TILE_N, TILE_K))
end

function silu_and_mul_kernel(A, B, C, TILE_N::Int)   # A, B may be views of the halves of the gate/up buffer
    n, cols = size(C)
    check(ccall((:ctb_moe_silu_and_mul, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Int64, Cint),
        context(), stream(), dptr(A), dptr(B), dptr(C), n, cols, stride(A, 2), stride(B, 2), stride(C, 2), TILE_N))
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

# ---- building blocks of the expert-parallel MoE (the all-to-all itself is the host's, e.g. NCCL.jl) ----
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

# ---- expert-parallel MoE over peer memory (one process per GPU) ----
# Mirrors `ctb_ep_buffers`: addresses of every rank's buffers, valid on the calling device (the host obtains them from
# a symmetric-memory allocator or from CUDA IPC / VMM mappings).
struct EpBuffers
    world::Cint
    rank::Cint
    recv_rows::NTuple{8,Ptr{Cvoid}}
    recv_ids::NTuple{8,Ptr{Cvoid}}
    recv_gates::NTuple{8,Ptr{Cvoid}}
    slot_out::NTuple{8,Ptr{Cvoid}}
    flags::NTuple{8,Ptr{Cvoid}}
    epoch::Ptr{Cvoid}
end

function moe_ep_dispatch(bufs::EpBuffers, hidden_states::CuArray{Float16,2}, topk_ids::CuArray{Int32,2},
                         topk_weights::CuArray{Float16,2}, num_experts::Int)
    H, T = size(hidden_states); topk = size(topk_ids, 2)
    check(ccall((:ctb_moe_ep_dispatch, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ref{EpBuffers}, Ptr{Cvoid}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64),
        context(), stream(), Ref(bufs), dptr(hidden_states), dptr(topk_ids), dptr(topk_weights), T, H, num_experts, topk))
end

moe_ep_barrier(bufs::EpBuffers) =
    check(ccall((:ctb_moe_ep_barrier, LIB), Cint, (Ptr{Cvoid}, Ptr{Cvoid}, Ref{EpBuffers}), context(), stream(), Ref(bufs)))

function moe_ep_experts(bufs::EpBuffers, w1_local, w2_local, cap::Int, tile_m::Int, tile_n::Int, tile_k::Int)
    I, H, El = size(w2_local)
    check(ccall((:ctb_moe_ep_experts, LIB), Cint,
        (Ptr{Cvoid}, Ptr{Cvoid}, Ref{EpBuffers}, Ptr{Cvoid}, Ptr{Cvoid}, Int64, Int64, Int64, Int64, Cint, Cint, Cint),
        context(), stream(), Ref(bufs), dptr(w1_local), dptr(w2_local), cap, H, I, El, tile_m, tile_n, tile_k))
end

end # module
