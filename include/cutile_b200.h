/* libcutile_b200: C ABI of the sm_100a kernel suite that stands in for the
 * kernels of cuTile.jl's examples (LayerNorm, softmax, GEMM, FMHA, MoE).
 *
 * Each entry point replaces one `@cuda backend=cuTile ... kernel(args...)`
 * launch (reference: src/launch.jl:788-814, the TileKernel call) or one host
 * wrapper of the examples' .jl files; the comment above each declaration names it.
 *
 * Conventions
 *  - Arrays are Julia column-major: the first listed dimension is contiguous.
 *    Leading dimensions (ld*) and strides are in ELEMENTS, like TileArray
 *    strides (src/language/types.jl:326-357).
 *  - All array arguments are DEVICE pointers owned by the caller; a host pointer
 *    is rejected with CTB_BAD_ARG (the reference raises ArgumentError,
 *    src/language/types.jl:371-376).
 *  - `stream` is the raw CUstream/cudaStream_t handle (NULL = default stream).
 *    Calls only enqueue work; they never synchronise unless stated.
 *  - Tile-size constants keep the reference's rule: powers of two
 *    (src/compiler/intrinsics/core.jl:10-19).  They are validated and otherwise
 *    advisory: the hand-written kernels choose their own blocking.
 *  - Index arrays (MoE) are 1-based, as in the reference.
 *  - Every function returns CTB_OK (0) or a positive ctb_status;
 *    ctb_last_error() gives the message of the calling thread's last failure.
 *  - There is no CPU fallback: without a usable sm_100 device ctb_create fails.
 */
#ifndef CUTILE_B200_H
#define CUTILE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum ctb_status {
  CTB_OK = 0,
  CTB_BAD_ARG = 1,          /* null/host pointer, non-positive size, bad enum      */
  CTB_BAD_ALIGN = 2,        /* pointer or leading dimension not aligned as needed  */
  CTB_UNSUPPORTED_TILE = 3, /* tile constant not a power of two / out of range     */
  CTB_UNSUPPORTED = 4,      /* shape or option outside what the kernels implement  */
  CTB_CUDA_ERROR = 5,
  CTB_NCCL_ERROR = 6,
  CTB_TIMEOUT = 7,          /* a bounded device-side wait ran out                  */
  CTB_NO_DEVICE = 8         /* no sm_100 device / driver                           */
} ctb_status;

typedef enum ctb_dtype { CTB_F32 = 0, CTB_F16 = 1, CTB_BF16 = 2 } ctb_dtype;

typedef struct ctb_ctx ctb_ctx;

/* Context = one device + its scratch + its device status word.  Replaces the
 * per-process state of the reference launch layer (compile cache and module
 * loading, src/launch.jl:616-625,663-687): kernels are built ahead of time. */
int ctb_create(ctb_ctx** out, int device);
void ctb_destroy(ctb_ctx* ctx);
const char* ctb_last_error(void);
const char* ctb_status_string(int status);
/* Counterpart of cuTile.versioninfo() (src/launch.jl:891-903). */
int ctb_version_info(char* buf, size_t n);
/* Synchronises `stream`, then reads and clears the device status word.  Returns
 * CTB_OK, or CTB_TIMEOUT / CTB_BAD_ARG if a kernel recorded a bounded-wait
 * expiry or a bad index since the last call. */
int ctb_check_device_status(ctb_ctx* ctx, void* stream);
/* How long the kernels of this context wait for a flag that another rank writes (the barrier of the peer-memory
 * expert-parallel step) before they record a timeout in the status word and return; 1 microsecond to 10 seconds,
 * 2 seconds by default.  A host that learns of a lost rank by other means lowers it so that the surviving ranks'
 * next step ends quickly with CTB_TIMEOUT from ctb_check_device_status instead of waiting out the default. */
int ctb_set_flag_wait_limit(ctb_ctx* ctx, uint64_t nanoseconds);
/* How ctb_gemm / ctb_gemm_batched turn f32 operands into TF32.  0 (default): the tensor core reads the f32 bits and
 * ignores the low 13 mantissa bits (truncation; no extra pass).  1: round to nearest even like the reference's
 * f32 -> tf32 conversion (src/compiler/intrinsics/conversions.jl:188-197, bit patterns of test/types.jl:203-245): a
 * pass of its own writes rounded copies of A and B into the context's scratch first (about one fifth more time at
 * 4096^3), after which the products are those of the reference's operands. */
int ctb_set_tf32_rounding(ctb_ctx* ctx, int nearest_even);

/* Launch hints of the reference's launch layer (`@cuda backend=cuTile num_ctas=... occupancy=... opt_level=...
 * num_worker_warps=...`, src/launch.jl:855-869), validated with the reference's ranges (validate_hint,
 * src/language/types.jl:864-882): num_ctas a power of two in [1, 16], occupancy in [1, 32], opt_level in [0, 3],
 * num_worker_warps 4 or 8; CTB_HINT_UNSET for a keyword that was not given.  The hints are advisory here: the
 * hand-written kernels choose cluster size, occupancy and warp roles themselves, so the host bindings check the
 * values (CTB_BAD_ARG with the reference's message for a bad one) and pass nothing on.  `stream` is honoured: it is
 * the stream argument of every entry point.  `dependent` (programmatic dependent launch) is accepted and ignored. */
#define CTB_HINT_UNSET (-1)
int ctb_validate_hints(int num_ctas, int occupancy, int opt_level, int num_worker_warps);

/* ---- Row softmax -------------------------------------------------------- */
/* softmax_tma_kernel(output, input, TILE_SIZE)      examples/softmax.jl:18-42
 * softmax_chunked_kernel(output, input, n_elems, TILE_SIZE)   :48-100
 * input/output (N, M): M rows of N contiguous elements, row stride ld.
 * variant 0: whole row staged in shared memory by bulk async copies (needs
 *            tile_size >= N, N*elemsize % 16 == 0, 16-byte aligned rows);
 * variant 1: any N; tile_size is advisory: rows that qualify for variant 0's
 *            kernel (N <= 8192, aligned) take it, longer or unaligned rows run
 *            chunks with a running max/sum per thread.
 * dtype: CTB_F32 or CTB_F16 (computes in f32, like the reference). */
int ctb_softmax(ctb_ctx* ctx, void* stream, void* output, const void* input, int64_t N, int64_t M, int64_t ld_out,
                int64_t ld_in, int variant, int tile_size, int dtype);

/* ---- Element-wise addition and transpose ----------------------------------- */
/* vec_add_kernel_1d(a, b, c, tile)                    examples/vadd.jl:10-17
 * vec_add_kernel_2d(a, b, c, tile_x, tile_y)          examples/vadd.jl:20-28
 * vec_add_kernel_1d_gather(a, b, c, tile)             examples/vadd.jl:31-45
 * c = a + b over `rows` rows of n contiguous elements (1-D: rows = 1); row strides lda/ldb/ldc in elements.  The
 * gather/scatter variant addresses the same contiguous elements and runs the same kernel.  dtype CTB_F32 or CTB_F16
 * (the sum is formed in the element type, like the reference's tile addition). */
int ctb_vadd(ctb_ctx* ctx, void* stream, const void* a, const void* b, void* c, int64_t n, int64_t rows, int64_t lda,
             int64_t ldb, int64_t ldc, int tile_x, int tile_y, int use_gather, int dtype);
/* transpose_kernel(x, y, tm, tn)                      examples/transpose.jl:11-19
 * y(n, m) = transpose of x(m, n), column-major with leading dimensions ldx/ldy; CTB_F32 or CTB_F16. */
int ctb_transpose(ctb_ctx* ctx, void* stream, const void* x, void* y, int64_t m, int64_t n, int64_t ldx, int64_t ldy, int tm,
                  int tn, int dtype);

/* ---- FFT -------------------------------------------------------------------- */
/* fft_kernel(x_packed_in, y_packed_out, W0, W1, W2, T0, T1, N, F0, F1, F2, BS, D)   examples/fft.jl:22-126
 * Batched complex FFT of length N = F0 * F1 * F2 along the first dimension as three DFT-matrix stages.  x and y are
 * f32 (D, 2N / D, batch): per batch item N interleaved (re, im) pairs, whatever D.  W0/W1/W2 are the (2, F, F) DFT
 * matrices and T0 (2, F1 * F2, F0), T1 (2, F2, F1) the twiddle factors of make_twiddles (examples/fft.jl:128-176); the
 * kernel uses the values it is given.  Factors are powers of two up to 32, N <= 8192; BS (batch items per block of the
 * reference launch, batch % BS == 0) and D (2N % D == 0) are validated and otherwise advisory.  f32 FMA arithmetic. */
int ctb_fft(ctb_ctx* ctx, void* stream, const void* x, void* y, const void* W0, const void* W1, const void* W2, const void* T0,
            const void* T1, int64_t N, int F0, int F1, int F2, int64_t batch, int BS, int D);

/* ---- Host-level array operations (ct.Tiled) ---------------------------------- */
/* ct.Tiled(C) .= f.(ct.Tiled(A), ...)                 src/broadcast.jl:19-23,92-165 (one fused kernel per expression)
 * sum / prod / maximum / minimum / mapreduce(f, op, ct.Tiled(A); dims)     src/mapreduce.jl:66-203
 * Arrays have up to three dimensions (shape[3], unused trailing extents = 1), column-major and dense; f32 or f16,
 * arithmetic in f32.  The broadcast expression is a postfix program of (code, argument) pairs with the meaning of a
 * stack machine: CTB_TILED_INPUT pushes inputs[argument] (its three strides in elements, 0 along a dimension where
 * the operand has extent 1 and is expanded), CTB_TILED_CONST pushes constants[argument], a unary code replaces the
 * top, a binary code replaces the two top values (second-from-top OP top).  The program must leave exactly one value.
 * The library re-orders the evaluation (an input or constant operand of a binary operator is read in place, the
 * deeper side of an operator between two computed values goes first; a + b and a * b may be evaluated as b + a and
 * b * a); it then holds at most four intermediate values at once, which every program of CTB_TILED_MAX_OPS
 * operations fits.  Empty arrays launch nothing. */
enum {
  CTB_TILED_INPUT = 0, CTB_TILED_CONST = 1,
  CTB_TILED_IDENTITY = 16, CTB_TILED_NEG, CTB_TILED_ABS, CTB_TILED_SQRT, CTB_TILED_EXP, CTB_TILED_EXP2, CTB_TILED_LOG,
  CTB_TILED_LOG2, CTB_TILED_SIN, CTB_TILED_COS, CTB_TILED_TANH, CTB_TILED_INV, CTB_TILED_ABS2,
  CTB_TILED_ADD = 64, CTB_TILED_SUB, CTB_TILED_MUL, CTB_TILED_DIV, CTB_TILED_MAX, CTB_TILED_MIN, CTB_TILED_POW
};
#define CTB_TILED_MAX_OPS 32
#define CTB_TILED_MAX_INPUTS 4
#define CTB_TILED_MAX_CONSTS 8
int ctb_tiled_broadcast(ctb_ctx* ctx, void* stream, void* dest, const int64_t* shape, const void* const* inputs,
                        const int64_t* input_strides, int n_inputs, const int32_t* program, int n_ops, const float* constants,
                        int n_constants, int dtype);
/* Diagnostic: the instruction words ctb_tiled_broadcast would run for this program (no GPU needed).  A word is
 * kind | source << 2 | reversed << 4 | code << 8 | argument << 16 with kind 0 = push the operand, 1 = top = code(top),
 * 2 = top = top code operand (operand code top when reversed); source 0 = the value below the top (popped), 1 =
 * inputs[argument], 2 = constants[argument]; the argument has eight bits, bits 24-31 repeat kind, source, reversed and
 * code as one dense index for the kernel's jump table.  instructions has room for CTB_TILED_MAX_OPS words. */
int ctb_tiled_compile(const int32_t* program, int n_ops, int n_inputs, int n_constants, uint32_t* instructions,
                      int* n_instructions);
/* dest = reduction with `op` (CTB_TILED_ADD, _MUL, _MAX or _MIN) of f(src) (a unary code, CTB_TILED_IDENTITY for none)
 * over the dimensions whose bit is set in reduce_mask (bit 0 = first dimension); dest is dense with extent 1 along
 * the reduced dimensions.  Fixed summation order (bitwise repeatable); an empty reduction gives the neutral element. */
int ctb_tiled_mapreduce(ctb_ctx* ctx, void* stream, void* dest, const void* src, const int64_t* shape, int reduce_mask, int f,
                        int op, int dtype);

/* ---- LayerNorm ---------------------------------------------------------- */
/* layer_norm_fwd(X, W, B, Y, Mean, Rstd, eps, TILE_N)   examples/layernorm.jl:27-68
 * X, Y (N, M) f32; W, B (N); Mean, Rstd (M). */
int ctb_layernorm_fwd(ctb_ctx* ctx, void* stream, const float* X, const float* W, const float* B, float* Y,
                      float* Mean, float* Rstd, int64_t N, int64_t M, int64_t ldx, int64_t ldy, float eps,
                      int tile_n);
/* layer_norm_bwd_dx_partial_dwdb(DX, DY, DW, DB, X, W, Mean, Rstd, Locks,
 *                                GROUP_SIZE_M, TILE_N)   examples/layernorm.jl:118-171
 * DW, DB are the (N, group_size_m) partial buffers (scratch owned by the caller);
 * on return column g holds the sum of dy*xhat (resp. dy) over the rows assigned
 * to group g.  They need no zero-fill and `locks` is unused (may be NULL): each
 * partial column is written once by the thread-block cluster that owns it. */
int ctb_layernorm_bwd_dx_partial_dwdb(ctb_ctx* ctx, void* stream, float* DX, const float* DY, float* DW, float* DB,
                                      const float* X, const float* W, const float* Mean, const float* Rstd,
                                      void* locks, int64_t N, int64_t M, int64_t ldx, int64_t lddy, int64_t lddx,
                                      int group_size_m, int tile_n);
/* layer_norm_bwd_dwdb(DW, DB, FINAL_DW, FINAL_DB, TILE_M, TILE_N)   examples/layernorm.jl:186-205
 * Column sums of the (N, group_size_m) partials, in fixed order (deterministic). */
int ctb_layernorm_bwd_dwdb(ctb_ctx* ctx, void* stream, const float* DW, const float* DB, float* FINAL_DW,
                           float* FINAL_DB, int64_t N, int group_size_m, int tile_m, int tile_n);

/* ---- GEMM ---------------------------------------------------------------- */
/* matmul_kernel(A, B, C, tm, tn, tk)                 examples/matmul.jl:28-60
 * C(M,N) = A(M,K) * B(K,N), column-major with leading dimensions lda/ldb/ldc.
 * dtype CTB_F32: TF32 tensor-core operands (low 13 mantissa bits ignored), f32
 * accumulate, f32 result.  dtype CTB_F16 / CTB_BF16: 16-bit operands, f32 accumulate, result in the operands' type.
 * A and B need 16-byte aligned bases and leading dimensions (TMA). */
int ctb_gemm(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
             int64_t lda, int64_t ldb, int64_t ldc, int dtype, int tm, int tn, int tk);
/* batch_matmul_kernel(A, B, C, tm, tn, tk)           examples/batchmatmul.jl:15-56
 * A(M,K,batch), B(K,N,batch), C(M,N,batch), batch last; stride* = elements
 * between consecutive batches. */
int ctb_gemm_batched(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, int64_t M, int64_t N,
                     int64_t K, int64_t batch, int64_t lda, int64_t ldb, int64_t ldc, int64_t strideA,
                     int64_t strideB, int64_t strideC, int dtype, int tm, int tn, int tk);

/* ---- Flash attention forward ------------------------------------------------ */
/* fmha_kernel(Q, K, V, Out, qk_scale, input_pos, TILE_D, H, TILE_M, TILE_N,
 *             QUERY_GROUP_SIZE, CAUSAL, EVEN_K)      examples/fmha.jl:20-139
 * as launched by cutile_fmha(Q, K, V; ...)           examples/fmha.jl:146-168
 * Q, Out (D, seq_q, heads, batch); K, V (D, seq_kv, kv_heads, batch), dense,
 * f16 or bf16.  heads = kv_heads * query_group_size.  Query i sits at position
 * i + input_pos for the causal rule.  EVEN_K is derived from seq_kv here.
 * Implemented: dtype CTB_F16 and CTB_BF16 (operands, probabilities and output in that type; f32 scores, softmax
 * state and accumulation), d_k = d_v = 64. */
int ctb_fmha_fwd(ctb_ctx* ctx, void* stream, const void* Q, const void* K, const void* V, void* Out, int64_t d_k,
                 int64_t d_v, int64_t seq_q, int64_t seq_kv, int64_t heads, int64_t kv_heads, int64_t batch,
                 float qk_scale, int32_t input_pos, int tile_m, int tile_n, int query_group_size, int causal,
                 int dtype);

/* ---- Mixture of experts -------------------------------------------------------- */
/* Upper bound on the number of tile_m-slot blocks moe_align can emit:
 * ceil(T*topk / tile_m) + E.  Size sorted_token_ids / sorted_expert_ids with it. */
int64_t ctb_moe_max_blocks(int64_t T, int64_t topk, int64_t E, int tile_m);

/* Router of the benchmark configuration (no counterpart kernel in the reference,
 * which draws ids with randperm, examples/moe.jl:323-332).  hidden (H, T) f16,
 * W_r (H, E) f16.  Each logit is summed in f32 in a fixed order that a CPU loop can
 * reproduce bit for bit: 32 partial sums, partial l taking the hidden indices k with
 * (k mod 256) in [8l, 8l+8) in ascending k, then v += v[l xor o] for o = 16, 8, 4, 2, 1 over
 * the partials (every f16*f16 product is exact in f32).  Top-k by value, ties
 * to the smallest index (the reference's arg-reduction rule,
 * src/language/operations.jl:1675-1677); gates = softmax over the chosen logits.
 * Outputs: topk_ids (T, topk) int32, 1-based; topk_weights (T, topk) f16;
 * logits (E, T) f32 or NULL. */
int ctb_moe_router(ctb_ctx* ctx, void* stream, const void* hidden, const void* W_r, int32_t* topk_ids,
                   void* topk_weights, float* logits, int64_t T, int64_t H, int64_t E, int topk);

/* moe_align_tile_size(topk_ids, tile_m, num_experts)      examples/moe.jl:142-183
 * Runs on the device (the reference copies the ids to the host and sorts there).
 * topk_ids (T, topk), 1-based, 32- or 64-bit integers (ids_bits).  Outputs, sized
 * for capacity_blocks >= ctb_moe_max_blocks(...): sorted_token_ids
 * [capacity_blocks*tile_m] (flat slot ids, sentinel T*topk+1), sorted_expert_ids
 * [capacity_blocks] (0 marks unused blocks), num_blocks[1] (device). */
int ctb_moe_align(ctb_ctx* ctx, void* stream, const void* topk_ids, int ids_bits, int64_t T, int64_t topk, int64_t E,
                  int tile_m, int32_t* sorted_token_ids, int32_t* sorted_expert_ids, int32_t* num_blocks,
                  int64_t capacity_blocks);

/* fused_moe_kernel(A, B, C, topk_weights, sorted_token_ids, sorted_expert_ids,
 *                  num_token_replicas, mul_routed_weight, TILE_M, TILE_N, TILE_K)
 *                                                          examples/moe.jl:45-105
 * A (K, a_cols) f16; B (K, N, E) f16; C (N, c_cols) f16; topk_weights flat
 * [c_cols] f16 (used when mul_routed_weight); sorted_token_ids [num_slots_padded],
 * sorted_expert_ids [num_slots_padded / tile_m].  Column id of C receives
 * B_e * A[:, cld(id, num_token_replicas)]; ids > c_cols are padding. */
int ctb_moe_fused_gemm(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, const void* topk_weights,
                       const int32_t* sorted_token_ids, const int32_t* sorted_expert_ids, int64_t num_slots_padded,
                       int64_t K, int64_t N, int64_t E, int64_t a_cols, int64_t c_cols, int num_token_replicas,
                       int mul_routed_weight, int tile_m, int tile_n, int tile_k);

/* silu_and_mul_kernel(A, B, C, TILE_N)                     examples/moe.jl:110-128
 * C(:, j) = silu(A(:, j)) * B(:, j) for n rows and `cols` columns (views with
 * leading dimensions lda/ldb/ldc), f16 in and out, f32 arithmetic. */
int ctb_moe_silu_and_mul(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, int64_t n, int64_t cols,
                         int64_t lda, int64_t ldb, int64_t ldc, int tile_n);

/* cutile_moe(hidden_states, w1, w2, topk_weights, topk_ids, tile_m, tile_n, tile_k)
 *                                                          examples/moe.jl:218-257
 * hidden (H, T); w1 (H, 2I, E) with gate rows then up rows; w2 (I, H, E);
 * topk_weights (T, topk) f16; topk_ids (T, topk) 1-based (ids_bits 32 or 64);
 * out (H, T) f16.  Device-side align, gate/up GEMM with fused SwiGLU, down GEMM
 * scaled by the routing weight, top-k sum; scratch comes from the context. */
int ctb_moe_ffn(ctb_ctx* ctx, void* stream, const void* hidden, const void* w1, const void* w2,
                const void* topk_weights, const void* topk_ids, int ids_bits, void* out, int64_t T, int64_t H,
                int64_t I, int64_t E, int64_t topk, int tile_m, int tile_n, int tile_k);

/* Building blocks of the expert-parallel MoE (one process per GPU; experts
 * [r*E/N, (r+1)*E/N) live on rank r; tokens start sharded by rank).  The reference
 * is single-GPU; the sharding comes from the benchmark configuration.  The
 * exchange itself (all-to-all of token rows and of their outputs) is done by the
 * host binding with NCCL.
 * ctb_moe_gather_rows : dst(:, i) = src(:, cld(ids[i], replicas)), the gather half
 *   of fused_moe_kernel (examples/moe.jl:62-70) as a stand-alone copy: packs the
 *   token rows of the locally routed slots, sorted by destination expert, into the
 *   send buffer.  Out-of-range ids give zero rows.
 * ctb_moe_scatter_rows: dst(:, ids[i]) = src(:, i): puts the returned slot outputs
 *   back in flat slot order (the scatter half, examples/moe.jl:99-102).
 * ctb_moe_combine     : out(:, t) = sum over the topk slots of token t, slots
 *   (H, topk, T) f16 (examples/moe.jl:256). */
int ctb_moe_gather_rows(ctb_ctx* ctx, void* stream, void* dst, const void* src, const int32_t* ids, int64_t n_ids,
                        int64_t row_elems, int num_token_replicas, int64_t src_rows);
int ctb_moe_scatter_rows(ctb_ctx* ctx, void* stream, void* dst, const void* src, const int32_t* ids, int64_t n_ids,
                         int64_t row_elems, int64_t dst_rows);
int ctb_moe_combine(ctb_ctx* ctx, void* stream, const void* slots, void* out, int64_t T, int64_t H, int64_t topk);

/* ---- Expert-parallel MoE over peer memory ---------------------------------------- */
/* The reference's MoE is single-GPU (examples/moe.jl); the sharding (one process per
 * GPU, experts [r*E/N, (r+1)*E/N) on rank r, tokens sharded by rank) comes from the
 * benchmark configuration.  Every pointer below is an address that is valid on the
 * calling device: rank q's buffers are peer memory mapped into this process (NVLink
 * peer access or a CUDA VMM mapping; the host binding obtains them, e.g. from a
 * symmetric-memory allocator).  cap = T * topk is the number of slots per rank.
 *   recv_rows[q] : (H, N*cap) f16 on rank q; column r*cap + s holds the token row of
 *                  slot s of rank r when the slot's expert lives on q
 *   recv_ids[q]  : (N*cap) int32 on rank q; the local expert id (1-based) of that
 *                  column, 0 when the slot belongs to another rank
 *   recv_gates[q]: (N*cap) f16 routing weights of the columns
 *   slot_out[q]  : (H, cap) f16 on rank q: the weighted expert outputs of its own
 *                  slots, summed over topk by ctb_moe_combine
 * ctb_moe_ep_dispatch: for every local slot writes the token row (the gather half of
 *   fused_moe_kernel, examples/moe.jl:62-70), its gate and its id entries straight
 *   into the owners' buffers.  Needs a barrier over the ranks before
 *   ctb_moe_ep_experts, and another one between ctb_moe_ep_experts and
 *   ctb_moe_combine(slot_out[rank]): ctb_moe_ep_barrier, or any collective of the
 *   host binding's library.
 * ctb_moe_ep_barrier : one small kernel per rank: it advances the rank's epoch
 *   counter, stores the epoch into entry `rank` of every rank's flag array
 *   (flags[q], N uint32 each, zero before the first use) and waits until all N
 *   entries of its own array have reached the epoch.  The wait is bounded (2 s);
 *   when it runs out the kernel records CTB_TIMEOUT in the context's status word
 *   and returns.  Stream-ordered and free of host state, so it can be captured in
 *   a CUDA graph and replayed.
 * ctb_moe_ep_experts : align + gate/up GEMM with SwiGLU + down GEMM of the received
 *   columns with the local experts; the down projection's epilogue writes each
 *   weighted output row into slot_out of the rank that sent the slot (the scatter
 *   half, examples/moe.jl:99-102, as bulk stores to peer memory). */
#define CTB_EP_MAX_RANKS 8
typedef struct ctb_ep_buffers {
  int world, rank;
  void* recv_rows[CTB_EP_MAX_RANKS];
  int32_t* recv_ids[CTB_EP_MAX_RANKS];
  void* recv_gates[CTB_EP_MAX_RANKS];
  void* slot_out[CTB_EP_MAX_RANKS];
  uint32_t* flags[CTB_EP_MAX_RANKS]; /* barrier flags of every rank (peer memory), N entries each */
  uint32_t* epoch;                   /* this rank's barrier counter (one uint32 in its own memory) */
} ctb_ep_buffers;
int ctb_moe_ep_dispatch(ctb_ctx* ctx, void* stream, const ctb_ep_buffers* bufs, const void* hidden,
                        const int32_t* topk_ids, const void* topk_weights, int64_t T, int64_t H, int64_t E,
                        int64_t topk);
int ctb_moe_ep_barrier(ctb_ctx* ctx, void* stream, const ctb_ep_buffers* bufs);
int ctb_moe_ep_experts(ctb_ctx* ctx, void* stream, const ctb_ep_buffers* bufs, const void* w1_local,
                       const void* w2_local, int64_t cap, int64_t H, int64_t I, int64_t E_local, int tile_m, int tile_n,
                       int tile_k);

/* ---- Several GPUs ------------------------------------------------------------------ */
/* The reference is single-GPU; the partitioning below is that of the benchmark configuration (batched GEMM and
 * FMHA split by batch with no communication; MoE expert-parallel with experts [r*E/N, (r+1)*E/N) on rank r and
 * the tokens sharded by rank).  The host wrapper that a multi-GPU cutile_moe replaces is examples/moe.jl:218-257.
 *
 * One process, several devices: ctb_create_multi creates one context per listed device, enables peer access
 * between all of them and, for more than one device, an NCCL communicator per device (ncclCommInitAll).  The
 * group owns its contexts: ctb_group_ctx(g, i) is the context to pass to the single-device entry points for
 * device i (make that device current first); ctb_destroy_multi frees everything. */
typedef struct ctb_group ctb_group;
int ctb_create_multi(ctb_group** out, const int* devices, int ndev);
void ctb_destroy_multi(ctb_group* g);
int ctb_group_size(const ctb_group* g);
ctb_ctx* ctb_group_ctx(ctb_group* g, int i);

/* One process per GPU: rank 0 draws an id (ncclGetUniqueId), the host language's own means carry the
 * CTB_UNIQUE_ID_BYTES bytes to the other processes, and every rank attaches a communicator to its context
 * (ncclCommInitRank; collective: all ranks must call).  ctb_destroy destroys the communicator;
 * ctb_comm_abort tears it down without waiting for outstanding operations (after a host-side failure of
 * another rank).  NCCL is loaded at run time (libnccl.so.2); CTB_NCCL_ERROR when it is missing or fails. */
#define CTB_UNIQUE_ID_BYTES 128
int ctb_comm_unique_id(void* id);
int ctb_comm_init_rank(ctb_ctx* ctx, const void* id, int rank, int world);
int ctb_comm_abort(ctb_ctx* ctx);
int ctb_comm_info(ctb_ctx* ctx, int* rank, int* world, int* nccl_version);

/* batch_matmul_kernel (examples/batchmatmul.jl:15-56) over the devices of a group: device i runs the
 * batch_per_dev[i] batches whose arrays are A[i], B[i], C[i] (device pointers on device i; batch-last layout makes a
 * shard a contiguous slab of the whole array) on streams[i].  No communication. */
int ctb_gemm_batched_sharded(ctb_group* g, void* const* streams, const void* const* A, const void* const* B,
                             void* const* C, int64_t M, int64_t N, int64_t K, const int64_t* batch_per_dev, int64_t lda,
                             int64_t ldb, int64_t ldc, int64_t strideA, int64_t strideB, int64_t strideC, int dtype,
                             int tm, int tn, int tk);
/* cutile_fmha's launch (examples/fmha.jl:146-168) over the devices of a group: device i runs batch_per_dev[i]
 * batches (all heads) of Q[i], K[i], V[i] -> Out[i]; (D, S, H, B) arrays split along B are contiguous slabs. */
int ctb_fmha_fwd_sharded(ctb_group* g, void* const* streams, const void* const* Q, const void* const* K,
                         const void* const* V, void* const* Out, int64_t d_k, int64_t d_v, int64_t seq_q,
                         int64_t seq_kv, int64_t heads, int64_t kv_heads, const int64_t* batch_per_dev, float qk_scale,
                         int32_t input_pos, int tile_m, int tile_n, int query_group_size, int causal, int dtype);

/* Expert-parallel cutile_moe.  ctb_ep holds one rank's exchange buffers for a fixed (T_local, H, topk): a single
 * device allocation that the other ranks map -- ctb_ep_connect_local inside one process (after ctb_create_multi),
 * or ctb_ep_export / ctb_ep_import across processes (a CUDA IPC handle of CTB_EP_HANDLE_BYTES bytes per rank,
 * carried by the host; every rank imports every other rank's).  ctb_ep_table gives the ctb_ep_buffers table for
 * the building-block calls above.
 * ctb_moe_ffn_ep runs one rank's step: hidden (H, T_local), w1_local (H, 2I, E/N), w2_local (I, H, E/N),
 * topk_weights / topk_ids (T_local, topk) with GLOBAL 1-based expert ids, out (H, T_local).
 *   a2a_mode CTB_A2A_NCCL: rows are packed by destination rank and cross as grouped ncclSend/ncclRecv pairs, outputs
 *     come back the same way.  The per-pair counts cross first and are read on the host: the call synchronises
 *     `stream` once and cannot be captured in a graph.  Needs a communicator on the context.
 *   a2a_mode CTB_A2A_PEER: the dispatch kernel stores each token row into the owning rank's buffer, the down
 *     projection's epilogue stores each weighted output row into the sender's buffer (plain peer stores over
 *     NVLink), two flag barriers with bounded waits in between.  Kernel launches only.
 * Both give results bit-identical to ctb_moe_ffn on the gathered problem.  Every rank must make the call.
 * ctb_moe_ffn_ep_group makes the calls of all ranks of a single-process group from one thread (NCCL requires its
 * send/receive pairs of several devices driven by one thread to sit in one group call). */
#define CTB_EP_HANDLE_BYTES 64
typedef enum ctb_a2a_mode { CTB_A2A_NCCL = 0, CTB_A2A_PEER = 1 } ctb_a2a_mode;
typedef struct ctb_ep ctb_ep;
int ctb_ep_create(ctb_ctx* ctx, int world, int rank, int64_t T_local, int64_t H, int64_t topk, ctb_ep** out);
void ctb_ep_destroy(ctb_ep* ep);
int ctb_ep_export(ctb_ep* ep, void* handle);
int ctb_ep_import(ctb_ep* ep, int peer_rank, const void* handle);
int ctb_ep_connect_local(ctb_ep* const* eps, int n);
const ctb_ep_buffers* ctb_ep_table(const ctb_ep* ep);
int ctb_moe_ffn_ep(ctb_ep* ep, void* stream, const void* hidden, const void* w1_local, const void* w2_local,
                   const void* topk_weights, const int32_t* topk_ids, void* out, int64_t T_local, int64_t H, int64_t I,
                   int64_t E, int64_t topk, int tile_m, int tile_n, int tile_k, int a2a_mode);
int ctb_moe_ffn_ep_group(ctb_group* g, ctb_ep* const* eps, void* const* streams, const void* const* hidden,
                         const void* const* w1_local, const void* const* w2_local, const void* const* topk_weights,
                         const int32_t* const* topk_ids, void* const* out, int64_t T_local, int64_t H, int64_t I,
                         int64_t E, int64_t topk, int tile_m, int tile_n, int tile_k, int a2a_mode);

/* Scratch of the context.  ctb_moe_ffn and the expert-parallel calls keep their intermediates (sorted slot ids,
 * activations, per-slot outputs) in scratch owned by the context, grown on demand; growing frees and reallocates
 * after a device synchronise, so a CUDA graph captured earlier must be captured again, and it is refused
 * (CTB_UNSUPPORTED) while the stream is being captured.  Size it once up front instead:
 * ctb_workspace_bytes(op, dims, ndims) with dims = {T, H, I, E, topk, tile_m} for CTB_OP_MOE_FFN and
 * {T_local, H, I, E_local, topk, tile_m, world} for CTB_OP_MOE_EP (0 for an unknown op), then
 * ctb_reserve_workspace.  One context serves one stream at a time. */
typedef enum ctb_op { CTB_OP_MOE_FFN = 1, CTB_OP_MOE_EP = 2 } ctb_op;
size_t ctb_workspace_bytes(int op, const int64_t* dims, int ndims);
int ctb_reserve_workspace(ctb_ctx* ctx, void* stream, size_t bytes);

/* ---- LayerNorm backward without any allocation --------------------------------- */
/* No counterpart in the reference.  For callers that cannot obtain device memory
 * at the point where the backward pass runs (a plug-in inside another runtime's
 * memory plan, a latency-critical loop that must not block in the allocator, a
 * section of code that is being recorded into a stream capture) this fuses
 * layer_norm_bwd_dx_partial_dwdb and layer_norm_bwd_dwdb with GROUP_SIZE_M = 64
 * and keeps the (N, 64) partial dW/dB buffers in a fixed 4 MiB array inside the
 * library image, so neither the caller nor the library calls cudaMalloc/cudaFree
 * (nor any allocating library routine) and no context object is needed.
 *  - Limit: N <= 8192 (the size of the built-in scratch); larger N returns
 *    CTB_UNSUPPORTED.  N and the leading dimensions must be multiples of 4 and
 *    X, DY, DX, W 16-byte aligned (CTB_BAD_ALIGN otherwise).
 *  - Works on the current device.  The first call on each device looks up the
 *    device address of the built-in array; make that first call before starting
 *    any stream capture.
 *  - The scratch is shared by every call on the device and keeps the previous
 *    call's contents.  Nothing in it has to start at zero (each partial column is
 *    fully rewritten), but two calls that overlap on the GPU (different streams,
 *    or one still running when the next starts on another stream) race on it:
 *    keep calls on one stream or order them with events. */
int ctb_layernorm_bwd_static(void* stream, float* DX, const float* DY, const float* X, const float* W,
                             const float* Mean, const float* Rstd, float* FINAL_DW, float* FINAL_DB, int64_t N,
                             int64_t M, int64_t ldx, int64_t lddy, int64_t lddx);
/* No counterpart in the reference.  The allocation-free call above has no context, so the bounded waits of its
 * kernels report into a status word that lives next to the scratch inside the library.  This call synchronises
 * `stream`, reads that word on the current device and clears it: CTB_OK, or CTB_TIMEOUT when a kernel of
 * ctb_layernorm_bwd_static gave up a wait since the last check (its outputs are then not valid).  It allocates
 * nothing either. */
int ctb_layernorm_bwd_static_status(void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CUTILE_B200_H */
