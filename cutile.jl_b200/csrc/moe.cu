// Mixture-of-experts FFN for sm_100a (counterparts of examples/moe.jl):
//   moe_router_kernel   logits = X^T * W_r in f32 in a fixed, warp-shaped summation
//                       order that a CPU float32 loop reproduces bit for bit,
//                       top-k by value with ties to the smallest index,
//                       softmax-renormalised gates stored as f16.  (The reference example draws its ids
//                       at random, examples/moe.jl:323-332; the router belongs to
//                       the benchmark configuration.)
//   moe_align_kernel    device version of moe_align_tile_size (:142-183): stable
//                       sort of the flat slot ids by expert, each expert padded to
//                       a multiple of tile_m with the sentinel total+1.
//   moe_gemm_kernel     fused_moe_kernel (:45-105): per (slot block, 128 weight
//                       rows) acc(N,M) += W_e(N,K) * A(K,M); weights stream by TMA,
//                       token rows are gathered by slot id with cp.async into
//                       128B-swizzled shared memory (completion arrives on the
//                       stage's mbarrier), tcgen05.mma accumulates in TMEM.  The
//                       instruction's N extent is the block's valid slot count
//                       rounded up to 16, so sparsely filled blocks (16 of 128
//                       slots at top-2 over 32 experts) cost little tensor time.
//                       Epilogues: plain f16 scatter with optional routing weight
//                       (the reference kernel), SwiGLU over a gate/up row pair
//                       (fuses silu_and_mul_kernel, :110-128), or weighted f32.
//   moe_combine_kernel  sum over the top-k slots of a token (:256).
// At 256 tokens the FFN is bound by streaming 403 MB of expert weights from HBM.
#include <cooperative_groups.h>
#include <math.h>

#include <type_traits>

#include "ctx.h"
#include "ptx.cuh"

using namespace ctb;
using namespace ctb_internal;
namespace cg = cooperative_groups;

namespace {

// ------------------------------------------------------------------ router
// One warp per token.  The accumulation order of a logit is fixed and shaped
// like the warp: lane l owns the hidden indices k with (k mod 256) in
// [8l, 8l+8) and adds their products x[k]*w[e][k] in ascending k into one f32
// partial sum (a fused multiply-add chain; every f16*f16 product is exact in
// f32); the 32 partials are then combined by a butterfly, v += v[lane ^ o] for
// o = 16, 8, 4, 2, 1.  The CPU oracle performs the same operations in the same
// order, so logits and therefore top-k ids agree bit for bit.  Every load is a
// coalesced 16-byte access; W_r (64 KB at 32 experts x 1024) stays in L1/L2.
constexpr int kRouterEPL = 256 / 32;
// Top-k selection and gate weights of one token from its logits (lane l holds experts l, l+32, ...).
template <int EPL>  // experts per lane: E <= 32 * EPL
__device__ __forceinline__ void route_one(float (&mine)[EPL], int t, int* __restrict__ ids,
                                          __half* __restrict__ gates, float* __restrict__ logits_out, int T, int E,
                                          int topk, int lane) {
  if (logits_out) {
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (lane + 32 * i < E) logits_out[(long long)t * E + lane + 32 * i] = mine[i];
  }
  float mysel = 0.f, top = 0.f, sum = 0.f;  // lane s keeps the s-th selected logit
  int myid = 0;
  for (int s = 0; s < topk; ++s) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (mine[i] > bv || (mine[i] == bv && e < bi))) {
        bv = mine[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (s == 0) top = bv;
    const float ex = expf(bv - top);
    sum += ex;
    if (lane == s) {
      mysel = ex;
      myid = bi;
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (lane + 32 * i == bi) mine[i] = -INFINITY;
  }
  if (lane < topk) {
    ids[(long long)lane * T + t] = myid + 1;
    gates[(long long)lane * T + t] = __float2half_rn(mysel / sum);
  }
}

constexpr int kRouterWarps = 16;  // four per scheduler: the logit loop is latency-bound with fewer
constexpr int kRouterThreads = kRouterWarps * 32;
constexpr int kMaxRouterE = 256;
constexpr int kRouterTE = 4;  // experts a warp carries through the hidden dimension at a time

__device__ __forceinline__ void cvt8(const uint4& u, float* f) {
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __half22float2(h[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

// A CTA works on groups of G = TT * tw tokens.  Its 16 warps form tw token-warps x ew expert-warps (tw * ew = 16):
// a warp owns TT tokens and every ew-th block of four experts, computes those logits in the fixed order (lane l
// = partial sum l, its 8 elements of each 256-chunk are one 16-byte shared-memory read, conflict-free without any
// permutation) and leaves them in shared memory; after a barrier the warps take the group's tokens in turn for
// top-k and gates.  Few tokens: small groups split over expert-warps, so that a 256-token batch still fills the
// GPU; many tokens: TT = 4 tokens per warp, so that every weight vector read from shared memory feeds four
// multiply-adds.  Rows are staged as f16 with cp.async (zero-filled up to a multiple of 256 elements); W_r stays
// resident for the CTA's lifetime when it fits, else it passes through in slices of eg experts.
template <int TT>
__global__ void __launch_bounds__(kRouterThreads)
    moe_router_kernel(const __half* __restrict__ X, const __half* __restrict__ Wr, int* __restrict__ ids,
                      __half* __restrict__ gates, float* __restrict__ logits_out, int T, int H, int E, int topk,
                      int eg, int tw) {
  extern __shared__ __align__(16) unsigned char rsm_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nchunk = (H + 255) / 256, Hp = nchunk * 256;
  const int ew = kRouterWarps / tw, G = TT * tw;
  __half* sx = reinterpret_cast<__half*>(rsm_raw);                     // [G][Hp]
  __half* sw = sx + (size_t)G * Hp;                                    // [eg][Hp]
  float* sl = reinterpret_cast<float*>(sw + (size_t)eg * Hp);          // [G][E] logits of the group
  const int vpr = Hp / 8;                                              // 16-byte vectors per padded row
  const int ngroups = (T + G - 1) / G;
  constexpr int EPL = kRouterEPL;
  auto stage_rows = [&](__half* dst, const __half* src, int nrows, int row_limit) {
    for (int i = tid; i < nrows * vpr; i += kRouterThreads) {
      const int r = i / vpr, v = i - r * vpr;
      const bool valid = r < row_limit && v * 8 < H;
      cp_async16(dst + (size_t)r * Hp + v * 8, valid ? (const void*)(src + (long long)r * H + v * 8) : (const void*)src,
                 valid ? 16u : 0u);
    }
  };
  const bool resident = eg >= E;  // all of W_r stays in shared memory for the CTA's lifetime
  if (resident) stage_rows(sw, Wr, E, E);
  const int wt = warp / ew, we = warp - wt * ew;
#pragma unroll 1
  for (int grp = blockIdx.x; grp < ngroups; grp += gridDim.x) {
    const int tbase = grp * G;
    __syncthreads();  // the previous group's token rows and logits have been consumed
    stage_rows(sx, X + (long long)tbase * H, G, T - tbase);
    const uint4* xrow[TT];
#pragma unroll
    for (int u = 0; u < TT; ++u) xrow[u] = reinterpret_cast<const uint4*>(sx + (size_t)(wt * TT + u) * Hp) + lane;
#pragma unroll 1
    for (int g0 = 0; g0 < E; g0 += eg) {
      const int ge = min(eg, E - g0);
      if (!resident) {
        __syncthreads();  // the previous expert rows have been consumed
        stage_rows(sw, Wr + (long long)g0 * H, ge, ge);
      }
      cp_async_wait_all();
      __syncthreads();
      // four experts at a time in rolled loops (the body runs a few times per warp: keep it small for the
      // instruction cache)
      constexpr int TE = kRouterTE;
#pragma unroll 1
      for (int e0 = we * TE; e0 < ge; e0 += ew * TE) {
        float acc[TT][TE];
#pragma unroll
        for (int u = 0; u < TT; ++u)
#pragma unroll
          for (int e = 0; e < TE; ++e) acc[u][e] = 0.f;
        const uint4* wrow[TE];
#pragma unroll
        for (int e = 0; e < TE; ++e) wrow[e] = reinterpret_cast<const uint4*>(sw + (size_t)min(e0 + e, ge - 1) * Hp) + lane;
#pragma unroll 2
        for (int c = 0; c < nchunk; ++c) {
          float xf[TT][8];
#pragma unroll
          for (int u = 0; u < TT; ++u) cvt8(xrow[u][c * 32], xf[u]);
#pragma unroll
          for (int e = 0; e < TE; ++e) {
            float wf[8];
            cvt8(wrow[e][c * 32], wf);
#pragma unroll
            for (int j = 0; j < 8; ++j)  // ascending k inside the lane
#pragma unroll
              for (int u = 0; u < TT; ++u) acc[u][e] = fmaf(xf[u][j], wf[j], acc[u][e]);
          }
        }
        // The 32 partial sums of each of the TT * TE logits meet in the butterfly v += v[lane ^ o], o = 16, 8, 4, 2, 1.
        // Every lane of a pair computes the same sum (a + b = b + a), so at each level a lane keeps half of its
        // logits and hands the other half to its partner: the same additions in the same order for the logit a
        // lane ends up holding, a quarter of the shuffles.
        constexpr int NV = TT * TE;
        float v[NV];
#pragma unroll
        for (int u = 0; u < TT; ++u)
#pragma unroll
          for (int e = 0; e < TE; ++e) v[u * TE + e] = acc[u][e];
        int held = 0;  // index of the logit this lane holds at the end
        int cnt = NV;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          if (cnt > 1) {
            const int half = cnt / 2;
            const bool upper = (lane & o) != 0;
#pragma unroll
            for (int j = 0; j < NV / 2; ++j) {
              if (j < half) {
                const float send = upper ? v[j] : v[j + half];
                const float keep = upper ? v[j + half] : v[j];
                v[j] = keep + __shfl_xor_sync(0xffffffffu, send, o);
              }
            }
            if (upper) held += half;
            cnt = half;
          } else {
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
          }
        }
        static_assert(NV <= 16, "the last butterfly level must be a plain exchange");
        {
          const int u = held / TE, e = held - u * TE;
          if ((lane & ((32 / NV) - 1)) == 0 && e0 + e < ge) sl[(size_t)(wt * TT + u) * E + g0 + e0 + e] = v[0];
        }
      }
    }
    __syncthreads();
#pragma unroll 1
    for (int tl = warp; tl < G; tl += kRouterWarps) {
      const int t = tbase + tl;
      if (t >= T) break;
      auto route = [&](auto epl) {  // as few experts per lane as E needs: the selection loops run over all of them
        constexpr int N = decltype(epl)::value;
        float lg[N];
#pragma unroll
        for (int i = 0; i < N; ++i) lg[i] = lane + 32 * i < E ? sl[(size_t)tl * E + lane + 32 * i] : -INFINITY;
        route_one<N>(lg, t, ids, gates, logits_out, T, E, topk, lane);
      };
      if (E <= 32) route(std::integral_constant<int, 1>{});
      else if (E <= 64) route(std::integral_constant<int, 2>{});
      else if (E <= 128) route(std::integral_constant<int, 4>{});
      else route(std::integral_constant<int, EPL>{});
    }
  }
  cp_async_wait_all();  // a CTA without any group still has its copy of W_r in flight
}

// ------------------------------------------------------------------ align
constexpr int kAlignThreads = 1024;
constexpr int kAlignWarps = kAlignThreads / 32;
constexpr int kMaxExperts = 256;
constexpr int kAlignRegIds = 8;   // ids a lane keeps in registers between the two passes

// Mask of the lanes of the (converged) warp that hold the same value v; v uses `bits` bits (lanes with v < 0 form a
// group of their own).  One ballot per bit: much cheaper than match.any, whose cost grows with the number of
// distinct values in the warp (about 20 of 32 experts at top-2).
__device__ __forceinline__ unsigned same_value_mask(int v, int bits) {
  unsigned m = __ballot_sync(0xffffffffu, v < 0);
  m = v < 0 ? m : ~m;
  for (int b = 0; b < bits; ++b) {
    const unsigned bal = __ballot_sync(0xffffffffu, (v >> b) & 1);
    m &= ((v >> b) & 1) ? bal : ~bal;
  }
  return m;
}

// One thread-block cluster of C CTAs (C = 1 for small batches).  CTA r counts and later scatters the ids
// [r*chunk, (r+1)*chunk); between the two passes every CTA reads the others' per-expert counts through
// distributed shared memory and derives the same block layout and its own offset inside every expert's range.
// A single CTA spent its time issuing instructions for 32 warps on one SM; the cluster spreads that over C SMs.
template <typename IdT>
__global__ void __launch_bounds__(kAlignThreads)
    moe_align_kernel(const IdT* __restrict__ topk_ids, int T, int topk, int E, int tile_m,
                     int* __restrict__ sorted_token_ids, int* __restrict__ sorted_expert_ids,
                     int* __restrict__ num_blocks, int capacity_blocks, int skip_empty, int* status,
                     const unsigned char* __restrict__ warm, long long warm_bytes) {
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  if ((int)blockIdx.x >= C) {
    // The clusters after the first do not sort: they ask the L2 to fetch the head of the expert weights that the next
    // kernel streams (HBM is idle while the ids are sorted), one 128-byte line per request, and leave.
    const long long nlines = warm_bytes >> 7;
    const long long first = (long long)((int)blockIdx.x - C) * kAlignThreads + threadIdx.x;
    const long long step = (long long)((int)gridDim.x - C) * kAlignThreads;
    for (long long c = first; c < nlines; c += step)
      asm volatile("prefetch.global.L2 [%0];" ::"l"(warm + (c << 7)) : "memory");
    return;
  }
  extern __shared__ int sm[];
  int* wcount = sm;                       // [kAlignWarps][E]: per-warp counts, then running offsets
  int* estart = sm + kAlignWarps * E;     // [E]: first padded position of expert e
  int* bstart = estart + E;               // [E+1]: first block of expert e
  int* ctot = bstart + E + 1;             // [E]: ids of expert e in this CTA's range (read by the peers)
  int* coff = ctot + E;                   // [E]: ids of expert e in the ranges of the CTAs before this one
  int* etot = coff + E;                   // [E]: ids of expert e over all CTAs
  __shared__ int bad;                     // read by the peers as well
  __shared__ int bad_any;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total = T * topk;
  const int chunk = ((total + C - 1) / C + kAlignThreads - 1) / kAlignThreads * kAlignThreads;  // ids per CTA
  const int seg = chunk / kAlignWarps;                                                           // ids per warp
  const int lo = min(total, rank * chunk + warp * seg), hi = min(total, lo + seg);
  const int niter = lo < hi ? (hi - lo + 31) / 32 : 0;
  int ebits = 1;
  while ((1 << ebits) < E) ++ebits;
  if (tid == 0) bad = 0;
  for (int i = tid; i < kAlignWarps * E; i += kAlignThreads) wcount[i] = 0;
  // flat id i (0-based) = token*topk + slot; topk_ids is (T, topk) column-major
  auto expert_of = [&](int i) -> int {
    const int tok = i / topk, slot = i - tok * topk;
    return (int)topk_ids[(long long)slot * T + tok] - 1;
  };
  int ecache[kAlignRegIds];  // this lane's experts, loaded up front so that the loads overlap
#pragma unroll
  for (int q = 0; q < kAlignRegIds; ++q) {
    const int i = lo + q * 32 + lane;
    ecache[q] = (q < niter && i < hi) ? expert_of(i) : -1;
  }
  if (C == 1) {
    // a single CTA orders its own writes: everything gets the sentinel now, under the latency of the id loads, and
    // the scatter at the end overwrites the positions that hold ids
    for (int i = tid; i < capacity_blocks * tile_m; i += kAlignThreads) sorted_token_ids[i] = total + 1;
    for (int i = tid; i < capacity_blocks; i += kAlignThreads) sorted_expert_ids[i] = 0;
  }
  __syncthreads();
#pragma unroll 1
  for (int q0 = 0; q0 < niter; q0 += kAlignRegIds) {
#pragma unroll
    for (int qq = 0; qq < kAlignRegIds; ++qq) {
      const int q = q0 + qq;
      if (q < niter) {
        const int i = lo + q * 32 + lane;
        int e = q0 == 0 ? ecache[qq] : (i < hi ? expert_of(i) : -1);
        if (i < hi && (e < 0 || e >= E)) {
          if (!(skip_empty && e == -1)) bad = 1;  // skip_empty: id 0 marks a slot that belongs to nobody here
          e = -1;
        }
        const unsigned grp = same_value_mask(e, ebits);
        if (e >= 0 && (grp & ((1u << lane) - 1)) == 0) wcount[warp * E + e] += __popc(grp);
        __syncwarp();  // the next iteration's group leader may be another lane
      }
    }
  }
  __syncthreads();
  // per expert: exclusive prefix over this CTA's warps
  if (tid < E) {
    int run = 0;
    for (int w = 0; w < kAlignWarps; ++w) {
      const int c = wcount[w * E + tid];
      wcount[w * E + tid] = run;
      run += c;
    }
    ctot[tid] = run;
  }
  cluster.sync();  // every CTA's counts (and its `bad`) are in place
  if (tid < E) {
    int before = 0, all = 0;
    for (int k = 0; k < C; ++k) {
      const int c = cluster.map_shared_rank(ctot, k)[tid];
      if (k < rank) before += c;
      all += c;
    }
    coff[tid] = before;
    etot[tid] = all;
    estart[tid] = (all + tile_m - 1) / tile_m;  // blocks of this expert, replaced by the start below
  }
  if (tid == 0) {
    int any = 0;
    for (int k = 0; k < C; ++k) any |= *cluster.map_shared_rank(&bad, k);
    bad_any = any;
  }
  __syncthreads();
  if (warp == 0) {  // exclusive scan over experts of the block counts (the same in every CTA)
    int carry = 0;
    for (int e0 = 0; e0 < E; e0 += 32) {
      const int e = e0 + lane;
      const int nb = e < E ? estart[e] : 0;
      int inc = nb;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += v;
      }
      if (e < E) bstart[e] = carry + inc - nb;
      carry += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) {
      bstart[E] = carry;
      if (carry > capacity_blocks) bad_any = 1;
      if (rank == 0) *num_blocks = min(carry, capacity_blocks);
    }
  }
  cluster.sync();  // the peers have read this CTA's counts: from here on nobody touches remote shared memory
  const int gtid = rank * kAlignThreads + tid, gthreads = C * kAlignThreads;
  if (bad_any) {
    if (gtid == 0) {
      atomicMax(status, DEV_BAD_INDEX);
      *num_blocks = 0;
    }
    for (int i = gtid; i < capacity_blocks * tile_m; i += gthreads) sorted_token_ids[i] = total + 1;
    for (int i = gtid; i < capacity_blocks; i += gthreads) sorted_expert_ids[i] = 0;
    return;
  }
  if (tid < E) estart[tid] = bstart[tid] * tile_m;
  __syncthreads();
  auto expert_of_block = [&](int b) {  // last e with bstart[e] <= b
    int l = 0, h = E - 1;
    while (l < h) {
      const int mid = (l + h + 1) >> 1;
      if (bstart[mid] <= b) l = mid; else h = mid - 1;
    }
    return l;
  };
  // One warp per block: its expert id, and the sentinel in every position that no id will be written to (each
  // position has one writer, so this needs no ordering against the scatter below).
  const int used_blocks = bstart[E];
  if (C == 1) {
    for (int b = tid; b < used_blocks; b += kAlignThreads) sorted_expert_ids[b] = expert_of_block(b) + 1;
    __syncthreads();  // the early sentinel fill of this CTA is ordered before the scatter
  }
  for (int b = rank * kAlignWarps + warp; C > 1 && b < capacity_blocks; b += C * kAlignWarps) {
    int e = -1, valid = 0;
    if (b < used_blocks) {
      e = expert_of_block(b);
      valid = min(tile_m, max(0, etot[e] - (b - bstart[e]) * tile_m));
    }
    if (lane == 0) sorted_expert_ids[b] = e + 1;
    for (int sl = valid + lane; sl < tile_m; sl += 32) sorted_token_ids[(long long)b * tile_m + sl] = total + 1;
  }
#pragma unroll 1
  for (int q0 = 0; q0 < niter; q0 += kAlignRegIds) {
#pragma unroll
    for (int qq = 0; qq < kAlignRegIds; ++qq) {
      const int q = q0 + qq;
      if (q < niter) {
        const int i = lo + q * 32 + lane;
        const int e = q0 == 0 ? ecache[qq] : (i < hi ? expert_of(i) : -1);
        const unsigned grp = same_value_mask(e, ebits);
        if (e >= 0) {
          const int rk = __popc(grp & ((1u << lane) - 1));
          sorted_token_ids[estart[e] + coff[e] + wcount[warp * E + e] + rk] = i + 1;
        }
        __syncwarp();
        if (e >= 0 && (grp & ((1u << lane) - 1)) == 0) wcount[warp * E + e] += __popc(grp);
        __syncwarp();
      }
    }
  }
}

// ------------------------------------------------------------------ grouped GEMM
constexpr int kRows = 128;  // weight rows per tile = MMA M
constexpr int kBK = 64;     // K elements per stage (128 bytes of f16)
constexpr int kMaxTileM = 128;  // slots per block at most = MMA M
constexpr int kGatherWarps = 8;
constexpr int kGatherThreads = kGatherWarps * 32;
constexpr int kEpiWarps = 8;  // two per TMEM lane quadrant: each takes half of the output rows of the item
constexpr int kGemmThreads = 64 + kGatherThreads + 32 * kEpiWarps;  // producer + MMA warps, gather warps, epilogue warps
constexpr int kWTile = kRows * kBK * 2;  // 16 KiB

enum Epilogue : int { EPI_F16 = 0, EPI_SWIGLU = 1 };

struct GemmParams {
  const __half* A;        // token rows, K contiguous
  long long lda;
  int a_rows;             // rows of A
  const int* sorted_ids;  // 1-based flat slot ids, padded with total+1
  const int* expert_ids;  // 1-based expert per block (0 = unused block)
  const int* num_blocks_dev;
  int num_blocks_host;    // >= 0: use this instead of *num_blocks_dev
  const __half* topk_w;   // routing weights, may be null
  int w_tokens, w_topk;   // w_tokens == 0: topk_w is flat, indexed by id-1; else (T, topk) column-major
  int replicas, mul_weight;
  int K, N;               // N = output rows per expert (SwiGLU: the weight tensor holds 2N rows)
  int E, tile_m, total;
  __half* C;              // element (n, id-1) at C[(id-1)*ldc + n]
  int c_vec;              // 1: columns of C start on 16-byte boundaries (ldc % 8 == 0, aligned base)
  // Expert-parallel down projection: column id-1 lives on rank (id-1) / c_split, at column (id-1) % c_split of that
  // rank's buffer c_peer[rank] (an address of peer memory mapped into this process).  c_split == 0: plain C.
  __half* c_peer[CTB_EP_MAX_RANKS];
  int c_split;
  long long ldc;
  int n_tiles, stages, stage_bytes;
};

// number of leading slots of the block that have to take part (last valid + 1)
__device__ __forceinline__ int block_extent(const int* ids, int tile_m, int total, int lane) {
  int last = 0;
  for (int r = lane; r < tile_m; r += 32)
    if (ids[r] >= 1 && ids[r] <= total) last = r + 1;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) last = max(last, __shfl_xor_sync(0xffffffffu, last, o));
  return last;
}

constexpr int kPassCols = 32;                      // output columns an epilogue thread stages per bulk copy
constexpr int kStagePitch = kPassCols * 2 + 16;    // bytes between staging rows
constexpr int kEpiStageBytes = kEpiWarps * 32 * kStagePitch;
constexpr int kMetaItems = 64;  // work items whose block metadata a CTA caches per round
constexpr int kIssue = 1;      // k-blocks the weight producer requests at a time (2 measured no faster)

// EPI: epilogue.  NW: 128-row weight tiles per work item (2 for SwiGLU = gate tile + up tile; 2 for the plain
// epilogues when the expert has at least 256 output rows, so that a gathered token tile is used by 256 rows).
template <int EPI, int NW>
__global__ void __launch_bounds__(kGemmThreads, 1)
    moe_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const GemmParams p, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kMaxStages = 8;
  // full[s]: one arrival with the TMA byte count from the weight producer + one arrival per gather thread
  __shared__ __align__(8) uint64_t full[kMaxStages], empty[kMaxStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s, tok_rows_s;
  __shared__ int meta_e[kMetaItems], meta_ext[kMetaItems];  // expert (0-based, -1 = skip) and slot extent per item
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_s = 0;
    tok_rows_s = 16;
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&full[s], 1 + kGatherThreads);  // gather threads arrive when their cp.async copies have landed
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], kEpiWarps);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  volatile int* abort = &abort_s;
  const int nblocks = p.num_blocks_host >= 0 ? p.num_blocks_host : *p.num_blocks_dev;
  const int base_items = nblocks * p.n_tiles;
  // Work items [0, split_from) are whole (block, NW weight tiles) pairs; item split_from + q is weight tile q & 1 of
  // pair split_from + q / 2.  The pairs of a last, less than half-filled round over the CTAs are handed out as
  // single tiles, so that the round costs about half an item instead of a whole one (320 pairs on 148 SMs are the
  // down projection at 4096 tokens: 2.6 rounds instead of 3).
  int split_from = base_items;
  if (EPI == EPI_F16 && NW == 2) {
    const int rest = base_items % (int)gridDim.x;
    if (rest > 0 && base_items > (int)gridDim.x && 2 * rest <= (int)gridDim.x) split_from = base_items - rest;
  }
  const int items = base_items + (base_items - split_from);
  const int my_items = (int)blockIdx.x < items ? (items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int nk = (p.K + kBK - 1) / kBK;
  constexpr int wbytes = NW * kWTile;    // offset of the token tile inside a stage
  constexpr int kRowsItem = NW * kRows;  // for SwiGLU: 128 gate rows + the matching 128 up rows
  // item index -> block, weight-tile pair, first weight tile inside the pair and number of weight tiles
  auto decode = [&](int it, int& bm, int& nt, int& w0, int& nw) {
    int pair = it;
    w0 = 0;
    nw = NW;
    if (it >= split_from) {
      const int q = it - split_from;
      pair = split_from + (q >> 1);
      w0 = q & 1;
      nw = 1;
    }
    bm = pair / p.n_tiles;
    nt = pair - bm * p.n_tiles;
  };

  // Ring geometry of this CTA.  A stage holds the weight tile(s) and as many token rows as the fullest block among
  // this CTA's items needs (a multiple of 16): with few tokens per expert the stages shrink and more of them, i.e.
  // more weight bytes in flight, fit the same shared memory.  The MMA still reads 128 token rows; the rows past the
  // stage's token part are whatever follows in shared memory (the next stage or the output staging, always inside
  // the allocation) and only feed accumulator rows that nobody reads.
  for (int n = warp; n < my_items; n += kGemmThreads / 32) {
    int bm, nt_, w0_, nw_;
    decode(blockIdx.x + n * gridDim.x, bm, nt_, w0_, nw_);
    const int e = p.expert_ids[bm] - 1;
    const int ext = (e < 0 || e >= p.E) ? 0 : block_extent(p.sorted_ids + (long long)bm * p.tile_m, p.tile_m, p.total, lane);
    if (lane == 0 && ext > 0) atomicMax(&tok_rows_s, min(kMaxTileM, (ext + 15) & ~15));
  }
  __syncthreads();
  const int ring_bytes = p.stages * p.stage_bytes;  // the host's budget, sized for full 128-row token tiles
  const int stage_bytes = wbytes + tok_rows_s * 128;
  const int stages = min(kMaxStages, ring_bytes / stage_bytes);

  // pipeline state of each role persists across rounds
  int stage = 0, nacc = 0;
  uint32_t phase = 0;

  for (int r0 = 0; r0 < my_items; r0 += kMetaItems) {
    const int rn = min(kMetaItems, my_items - r0);
    // ---- every warp: cache the metadata of this round's items (global-load latency paid once, in parallel)
    for (int n = warp; n < rn; n += kGemmThreads / 32) {
      int bm, nt_, w0_, nw_;
      decode(blockIdx.x + (r0 + n) * gridDim.x, bm, nt_, w0_, nw_);
      int e = p.expert_ids[bm] - 1;
      if (e < 0 || e >= p.E) e = -1;
      const int ext = block_extent(p.sorted_ids + (long long)bm * p.tile_m, p.tile_m, p.total, lane);
      if (lane == 0) {
        meta_e[n] = ext > 0 ? e : -1;
        meta_ext[n] = ext;
      }
    }
    __syncthreads();

    if (warp == 0) {
      // ---- weight producer: the whole warp walks the loop, one elected lane issues
      for (int n = 0; n < rn && !*abort; ++n) {
        const int e = meta_e[n];
        if (e < 0) continue;
        int bm_, nt, w0, nw;
        decode(blockIdx.x + (r0 + n) * gridDim.x, bm_, nt, w0, nw);
        bool ok = true;
        // kIssue k-blocks are requested at a time (with 2, the two 128-byte pieces of a weight row reach the memory
        // controller together)
        for (int kb = 0; kb < nk; kb += kIssue) {
          const int nb = min(kIssue, nk - kb);
          int s2 = stage;
          uint32_t ph2 = phase;
          for (int b = 0; b < nb && ok; ++b) {
            ok = CTB_WARP_WAIT(&empty[s2], ph2 ^ 1, status, DEV_TIMEOUT_SLOT, abort);
            if (++s2 == stages) { s2 = 0; ph2 ^= 1; }
          }
          if (!ok) break;
          if (elect_one()) {
            int s3 = stage;
            for (int b = 0; b < nb; ++b) {
              unsigned char* dst = smem + (size_t)s3 * stage_bytes;
              mbar_expect_tx(&full[s3], nw * kWTile);
              if (EPI == EPI_SWIGLU) {
                tma_load_3d(dst, &tmW, (kb + b) * kBK, nt * kRows, e, &full[s3]);
                tma_load_3d(dst + kWTile, &tmW, (kb + b) * kBK, p.N + nt * kRows, e, &full[s3]);
              } else {
#pragma unroll
                for (int w = 0; w < NW; ++w)
                  if (w < nw)
                    tma_load_3d(dst + w * kWTile, &tmW, (kb + b) * kBK, nt * kRowsItem + (w0 + w) * kRows, e, &full[s3]);
              }
              if (++s3 == stages) s3 = 0;
            }
          }
          __syncwarp();
          stage = s2;
          phase = ph2;
        }
        if (!ok) break;
      }
    } else if (warp == 1) {
      // ---- MMA issuer: the whole warp walks the loop, one elected lane issues.
      // The gathered token tile is the A operand (M = 128 slots = TMEM lanes), the weight tile(s) the B operand
      // (N = NW * 128 weight rows = accumulator columns): one 128 x N x 16 instruction per k-step.
      constexpr uint32_t idesc_pair = make_idesc(FMT_F16, kRows, (uint32_t)(NW * kRows), 0, 0);
      constexpr uint32_t idesc_one = make_idesc(FMT_F16, kRows, (uint32_t)kRows, 0, 0);
      for (int n = 0; n < rn && !*abort; ++n) {
        if (meta_e[n] < 0) continue;
        const uint32_t idesc = (int)(blockIdx.x + (r0 + n) * gridDim.x) >= split_from ? idesc_one : idesc_pair;
        const int acc = nacc & 1;
        const uint32_t acc_phase = (nacc >> 1) & 1;
        ++nacc;
        if (!CTB_WARP_WAIT(&acc_empty[acc], acc_phase ^ 1, status, DEV_TIMEOUT_SLOT, abort)) break;
        tc_fence_after();
        const uint32_t d = tmem + acc * 256;
        bool ok = true;
        for (int kb = 0; kb < nk; ++kb) {
          ok = CTB_WARP_WAIT(&full[stage], phase, status, DEV_TIMEOUT_TMA, abort);
          if (!ok) break;
          fence_proxy_async_smem();  // the gathered rows were written through the generic proxy
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + (size_t)stage * stage_bytes);
          const uint32_t st = sw + wbytes;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              mma_f16_ss(d, make_sdesc_sw128(st + k * 32, 0, 1024), make_sdesc_sw128(sw + k * 32, 0, 1024), idesc,
                         (kb | k) != 0);
            tc_commit(&empty[stage]);
          }
          __syncwarp();
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (elect_one()) tc_commit(&acc_full[acc]);
        __syncwarp();
      }
    } else if (warp < 2 + kGatherWarps) {
      // ---- token-row gather into the swizzled B operand (cp.async; the copy engine arrives on the stage's
      // barrier when a thread's copies have landed, so no thread waits for its data).
      // Thread g copies the 16-byte chunks g, g+256, ... of the (slots x 8 chunks) tile, so one warp instruction
      // moves four whole 128-byte row segments (full cache lines, conflict-free stores).  The loop is the critical
      // path of a k-block when few warps share it: everything that does not depend on the k-block (source rows,
      // byte counts, the chunk's place inside a stage) is computed once per work item.
      const int g = threadIdx.x - 64;  // 0..255
      const int cch = g & 7;           // chunk inside the 128-byte row segment (the same for every copy of the thread)
      constexpr int kQ = kMaxTileM * 8 / kGatherThreads;   // copies per thread and k-block at most
      constexpr int kRowStep = kGatherThreads / 8;   // block rows between two copies of a thread
      // byte offset of the thread's first chunk inside the B part of a stage: row g/8, 128-byte swizzle
      const uint32_t chunk_off = (uint32_t)((g >> 6) * 1024 + ((g >> 3) & 7) * 128 + ((cch ^ ((g >> 3) & 7)) << 4));
      // The slot ids of an item are fetched while the previous item is being gathered (raw[] holds them), so that
      // the first copies of an item do not wait for a dependent global load.
      auto fetch_ids = [&](int n, int (&raw)[kQ]) {
        const int nrows = max(16, (meta_ext[n] + 15) & ~15);
        int bm, nt_, w0_, nw_;
        decode(blockIdx.x + (r0 + n) * gridDim.x, bm, nt_, w0_, nw_);
#pragma unroll
        for (int q = 0; q < kQ; ++q) {
          const int r = q * kRowStep + (g >> 3);
          raw[q] = (r < p.tile_m && r < nrows) ? p.sorted_ids[(long long)bm * p.tile_m + r] : 0;
        }
      };
      auto next_valid = [&](int n) {
        while (n < rn && meta_e[n] < 0) ++n;
        return n;
      };
      int raw[kQ];
      int n = next_valid(0);
      if (n < rn) fetch_ids(n, raw);
      while (n < rn) {
        // rows up to the block's extent carry tokens; the others are not copied: whatever they hold only produces
        // accumulator rows (TMEM lanes) that nobody reads
        const int nrows = max(16, (meta_ext[n] + 15) & ~15);
        const __half* src[kQ];  // row q*kRowStep + g/8 of the block; invalid rows read nothing (zero fill)
        uint32_t nbytes[kQ];
#pragma unroll
        for (int q = 0; q < kQ; ++q) {
          src[q] = p.A;
          nbytes[q] = 0;
          const int id = raw[q];
          if (id >= 1 && id <= p.total) {
            const int tok = (id - 1) / p.replicas;  // cld(id, replicas) - 1
            if (tok < p.a_rows) {
              src[q] = p.A + (long long)tok * p.lda + cch * 8;
              nbytes[q] = 16;
            }
          }
        }
        const int n_next = next_valid(n + 1);
        if (n_next < rn) fetch_ids(n_next, raw);
        bool ok = true;
        for (int kb = 0; kb < nk; ++kb) {
          ok = CTB_WARP_WAIT1(&empty[stage], phase ^ 1, status, DEV_TIMEOUT_SLOT, abort);
          if (!ok) break;
          const uint32_t base = smem_u32(smem + (size_t)stage * stage_bytes + wbytes) + chunk_off;
          const bool in_k = kb * kBK + cch * 8 < p.K;  // K is a multiple of 8: a chunk is inside or outside as a whole
#pragma unroll
          for (int q = 0; q < kQ; ++q) {
            if (q * kRowStep + (g >> 3) < nrows) {  // the same for the whole warp (nrows is a multiple of 16)
              cp_async16_s(base + q * (kRowStep / 8) * 1024, src[q], in_k ? nbytes[q] : 0u);
              src[q] += kBK;
            }
          }
          cp_async_arrive_noinc(&full[stage]);  // fires when this thread's copies have landed
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        n = n_next;
      }
    } else {
      // ---- epilogue: thread = slot (TMEM lane), accumulator columns = output rows of the item.  The two warps of
      // a lane quadrant split the columns; a thread's outputs are contiguous in C, so they leave as 16-byte stores.
      const int sub = warp & 3;
      const int half = (warp - (2 + kGatherWarps)) >> 2;
      const uint32_t lane_addr = (uint32_t)(sub * 32) << 16;
      const int slot = sub * 32 + lane;
      constexpr int kOutCols = EPI == EPI_SWIGLU ? kRows : NW * kRows;  // output rows per item
      constexpr int kMyCols = kOutCols / 2;                            // ... of which this warp writes half
      // this thread's row of its warp's staging tile (rows 16 bytes apart from a multiple of 128: no bank conflicts)
      unsigned char* stg = smem + (size_t)ring_bytes +
                           ((size_t)(warp - (2 + kGatherWarps)) * 32 + lane) * kStagePitch;
      for (int n = 0; n < rn; ++n) {
        if (meta_e[n] < 0) continue;
        int bm, nt, w0, nw;
        decode(blockIdx.x + (r0 + n) * gridDim.x, bm, nt, w0, nw);
        // output columns this warp writes: half of the item's (a single-tile item has half the columns of a pair)
        const int my_cols = EPI == EPI_SWIGLU ? kMyCols : nw * (kRows / 2);
        const int acc = nacc & 1;
        const uint32_t acc_phase = (nacc >> 1) & 1;
        ++nacc;
        // slot id and routing weight of this thread's slot (loaded before the wait)
        int id = slot < p.tile_m ? p.sorted_ids[(long long)bm * p.tile_m + slot] : 0;
        if (id < 1 || id > p.total) id = 0;
        float wt = 1.f;
        if (p.mul_weight && id) {
          const int f = id - 1;
          wt = __half2float(p.topk_w[p.w_tokens ? (long long)(f % p.w_topk) * p.w_tokens + f / p.w_topk : f]);
        }
        const int col = id ? id - 1 : 0;
        __half* crow = p.c_split ? p.c_peer[col / p.c_split] + (long long)(col % p.c_split) * p.ldc
                                 : p.C + (long long)col * p.ldc;
        bool ok = CTB_WARP_WAIT1(&acc_full[acc], acc_phase, status, DEV_TIMEOUT_MMA, abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem + lane_addr + acc * 256;
        const int n_base = nt * kOutCols + w0 * kRows + half * my_cols;
        // kPassCols outputs at a time: registers -> this thread's row of the staging tile -> one bulk copy to the
        // slot's row of C.  (Stored straight from registers, 32 lanes hit 32 different rows of C with every
        // instruction; those scattered stores kept the load/store unit busy for about 2000 clocks per item, during
        // which the gather's copies and the MMA warp's proxy fence queued up behind them.)
#pragma unroll 1
        for (int ps = 0; ps < my_cols / kPassCols; ++ps) {
          uint32_t pk[kPassCols / 2];
#pragma unroll
          for (int c = 0; c < kPassCols / 16; ++c) {
            const int col = half * my_cols + ps * kPassCols + c * 16;
            uint32_t ga[16], up[16];
            tmem_ld16(taddr + col, ga);
            if (EPI == EPI_SWIGLU) tmem_ld16(taddr + kRows + col, up);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              float o0, o1;
              const float v0 = __uint_as_float(ga[j]), v1 = __uint_as_float(ga[j + 1]);
              if (EPI == EPI_SWIGLU) {
                // silu(g) * u with flush-to-zero and an approximate reciprocal (examples/moe.jl:117-124)
                o0 = v0 * rcp_approx_ftz(1.0f + __expf(-v0)) * __uint_as_float(up[j]);
                o1 = v1 * rcp_approx_ftz(1.0f + __expf(-v1)) * __uint_as_float(up[j + 1]);
              } else {
                o0 = v0 * wt;
                o1 = v1 * wt;
              }
              pk[c * 8 + (j >> 1)] = pack_f16x2(o0, o1);
            }
          }
          const int n0 = n_base + ps * kPassCols;
          bulk_wait_read<0>();  // the previous pass's copy has read this thread's staging row
          if (id) {
            if (p.c_vec && n0 + kPassCols <= p.N) {
              uint4* srow = reinterpret_cast<uint4*>(stg);
#pragma unroll
              for (int v = 0; v < kPassCols / 8; ++v) srow[v] = make_uint4(pk[4 * v], pk[4 * v + 1], pk[4 * v + 2], pk[4 * v + 3]);
              fence_proxy_async_smem();
              bulk_s2g(crow + n0, stg, kPassCols * 2);
            } else {
#pragma unroll
              for (int j = 0; j < kPassCols; ++j)
                if (n0 + j < p.N)
                  crow[n0 + j] = __ushort_as_half((unsigned short)((j & 1) ? (pk[j >> 1] >> 16) : (pk[j >> 1] & 0xffffu)));
            }
          }
          bulk_commit();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
      }
    }
    __syncthreads();  // the metadata cache is rewritten in the next round
    if (*abort) break;
  }
  if (warp >= 2 + kGatherWarps) bulk_wait<0>();  // this thread's output copies are complete
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ------------------------------------------------------------------ small kernels
// out(:, t) = sum over the top-k slot outputs of token t.  The slot outputs are f16 like the reference's cache3
// (examples/moe.jl:230,256); they are added in f32 in ascending slot order and rounded once.
__global__ void moe_combine_kernel(const __half* __restrict__ slots, __half* __restrict__ out, int T, int H, int topk) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;  // over T*H/8
  const int h8 = H / 8;
  if (i >= (long long)T * h8) return;
  const int t = (int)(i / h8), h = (int)(i - (long long)t * h8) * 8;
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  for (int s = 0; s < topk; ++s) {  // ascending slot: fixed order
    const uint4 v = *reinterpret_cast<const uint4*>(slots + ((long long)t * topk + s) * H + h);
    const __half2* hv = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(hv[j]);
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  }
  uint4 o;
  o.x = pack_f16x2(acc[0], acc[1]); o.y = pack_f16x2(acc[2], acc[3]);
  o.z = pack_f16x2(acc[4], acc[5]); o.w = pack_f16x2(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(out + (long long)t * H + h) = o;
}

// dst row i = src row (ids[i]-1)/replicas (zero when the id is out of range); rows of `vecs` 16-byte vectors
__global__ void moe_gather_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                       const int* __restrict__ ids, long long n, int vecs, int replicas,
                                       long long src_rows) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * vecs) return;
  const long long r = i / vecs;
  const int v = (int)(i - r * vecs);
  const long long id = ids[r];
  const long long sr = id >= 1 ? (id - 1) / replicas : -1;
  dst[i] = (sr >= 0 && sr < src_rows) ? src[sr * vecs + v] : make_uint4(0, 0, 0, 0);
}
// dst row ids[i]-1 = src row i (ids out of range are skipped)
__global__ void moe_scatter_rows_kernel(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                        const int* __restrict__ ids, long long n, int vecs, long long dst_rows) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * vecs) return;
  const long long r = i / vecs;
  const int v = (int)(i - r * vecs);
  const long long id = ids[r];
  if (id >= 1 && id <= dst_rows) dst[(id - 1) * vecs + v] = src[i];
}

__global__ void moe_silu_and_mul_kernel(const __half* __restrict__ A, const __half* __restrict__ B,
                                        __half* __restrict__ C, int n, long long cols, long long lda, long long ldb,
                                        long long ldc) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= cols * n) return;
  const long long col = i / n;
  const int r = (int)(i - col * n);
  const float a = __half2float(A[col * lda + r]), b = __half2float(B[col * ldb + r]);
  const float sig = rcp_approx_ftz(1.0f + __expf(-a));
  C[col * ldc + r] = __float2half_rn(a * sig * b);
}

// ------------------------------------------------------------------ expert-parallel dispatch over peer memory
struct EpPtrs {
  uint4* rows[CTB_EP_MAX_RANKS];
  int* ids[CTB_EP_MAX_RANKS];
  __half* gates[CTB_EP_MAX_RANKS];
};
// One warp per slot (token t, choice k): the token row goes straight into the receive buffer of the rank that owns
// the chosen expert (stores to peer memory, 512 contiguous bytes per warp instruction), at row rank*cap + slot, the
// position that names its sender; every rank's id array gets the local expert id (owner) or 0 (others) for the
// slot, so receivers need neither counts nor a cleared buffer.
__global__ void __launch_bounds__(256)
    moe_ep_dispatch_kernel(const uint4* __restrict__ X, const int* __restrict__ topk_ids,
                           const __half* __restrict__ topk_w, const EpPtrs pp, int T, int topk, int vecs, int E, int El,
                           int world, int rank, int* status) {
  const int lane = threadIdx.x & 31;
  const int cap = T * topk;
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  for (int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); slot < cap; slot += nwarps) {
    const int t = slot / topk, k = slot - t * topk;
    const int e = topk_ids[(long long)k * T + t];
    const long long row = (long long)rank * cap + slot;
    int owner = -1, le = 0;
    if (e >= 1 && e <= E) {
      owner = (e - 1) / El;
      le = e - owner * El;
    } else if (lane == 0) {
      atomicMax(status, DEV_BAD_INDEX);
    }
    if (lane < world) pp.ids[lane][row] = lane == owner ? le : 0;
    if (owner < 0) continue;
    if (lane == 0) pp.gates[owner][row] = topk_w[(long long)k * T + t];
    const uint4* src = X + (long long)t * vecs;
    uint4* dst = pp.rows[owner] + row * vecs;
    for (int v = lane; v < vecs; v += 32) dst[v] = src[v];
  }
}

// Barrier over the ranks (one launch per rank, on different GPUs).  Lane q publishes this rank's new epoch in
// rank q's flag array and then waits for rank q's epoch in its own array.  The release store follows the kernels
// that ran before this one on the stream, whose stores to peer memory are complete at that point; the acquire load
// precedes the kernels after it.  Epochs only grow, so a replayed CUDA graph needs no host-side state.
struct EpFlags {
  uint32_t* flags[CTB_EP_MAX_RANKS];
};
__global__ void moe_ep_barrier_kernel(const EpFlags f, uint32_t* epoch, int world, int rank, int* status,
                                      unsigned long long limit_ns) {
  const int lane = threadIdx.x;
  uint32_t e = 0;
  if (lane == 0) {
    e = *epoch + 1;
    *epoch = e;
  }
  e = __shfl_sync(0xffffffffu, e, 0);
  if (lane < world) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.flags[lane] + rank), "r"(e) : "memory");
    const uint32_t* mine = f.flags[rank] + lane;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 0;; ++it) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if ((int32_t)(v - e) >= 0) break;
      if ((it & 255u) == 255u && globaltimer_ns() - t0 > limit_ns) {
        atomicMax(status, DEV_TIMEOUT_SLOT);
        break;
      }
    }
  }
}

// ------------------------------------------------------------------ host side
int launch_gemm(ctb_ctx* ctx, cudaStream_t st, int epi, const __half* A, long long lda, int a_rows, const __half* W,
                int K, int wrows, int N, int E, const __half* topk_w, const int* sorted_ids, const int* expert_ids,
                const int* nblocks_dev, int nblocks_host, int max_blocks, int replicas, int mul_weight, int tile_m,
                int total, void* C, long long ldc, int w_tokens = 0, int w_topk = 1, void* const* c_peer = nullptr,
                int c_split = 0, int expect_blocks = -1) {
  if (expect_blocks < 0) expect_blocks = max_blocks;
  CUtensorMap tw;
  uint64_t dims[3] = {(uint64_t)K, (uint64_t)wrows, (uint64_t)E};
  uint64_t str[2] = {(uint64_t)K * 2, (uint64_t)K * wrows * 2};
  uint32_t box[3] = {kBK, kRows, 1};
  int r = make_tmap(&tw, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, W, dims, str, box);
  if (r) return r;
  GemmParams p;
  p.A = A; p.lda = lda; p.a_rows = a_rows;
  p.sorted_ids = sorted_ids; p.expert_ids = expert_ids;
  p.num_blocks_dev = nblocks_dev; p.num_blocks_host = nblocks_host;
  p.topk_w = topk_w; p.replicas = replicas; p.mul_weight = mul_weight;
  p.w_tokens = w_tokens; p.w_topk = w_topk;
  p.K = K; p.N = N; p.E = E; p.tile_m = tile_m; p.total = total;
  p.C = (__half*)C; p.ldc = ldc;
  p.c_vec = (ldc % 8 == 0 && (uintptr_t)C % 16 == 0) ? 1 : 0;
  p.c_split = c_split;
  for (int q = 0; q < CTB_EP_MAX_RANKS; ++q) {
    p.c_peer[q] = c_peer ? (__half*)c_peer[q] : nullptr;
    if (c_split && c_peer && c_peer[q] && (uintptr_t)c_peer[q] % 16) p.c_vec = 0;
  }
  // Two 128-row weight tiles per item share one gathered token tile (MMA N = 256), unless the (block, tile pair) items
  // would leave more than half of the SMs without work: then single tiles, twice as many items.  `expect_blocks` is
  // the caller's estimate of the blocks that will actually hold slots (max_blocks is only the capacity).
  const int pairs = (N + 2 * kRows - 1) / (2 * kRows);
  const int nw = (epi == EPI_SWIGLU) ? 2 : (N >= 2 * kRows && (long long)expect_blocks * pairs * 2 > ctx->sm_count) ? 2 : 1;
  p.n_tiles = epi == EPI_SWIGLU ? (N + kRows - 1) / kRows : (N + nw * kRows - 1) / (nw * kRows);
  // the token tile is the MMA's A operand with M = 128 rows whatever tile_m is: the instruction reads all of them
  p.stage_bytes = nw * kWTile + kRows * 128;
  p.stages = std::min(8, (int)((225 * 1024 - kEpiStageBytes) / p.stage_bytes));
  const size_t smem = (size_t)p.stages * p.stage_bytes + kEpiStageBytes + 1024;
  const long long items = (long long)max_blocks * p.n_tiles;
  const int grid = (int)std::max<long long>(1, std::min<long long>(items, ctx->sm_count));
  cudaError_t e;
#define CTB_LAUNCH_MOE(EPI, NWV)                                                                              \
  e = cudaFuncSetAttribute(moe_gemm_kernel<EPI, NWV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
  if (e != cudaSuccess) return cuda_fail(e, "moe gemm: shared memory opt-in");                                \
  moe_gemm_kernel<EPI, NWV><<<grid, kGemmThreads, smem, st>>>(tw, p, ctx->dev_status);
  if (epi == EPI_SWIGLU) { CTB_LAUNCH_MOE(EPI_SWIGLU, 2) }
  else if (nw == 2) { CTB_LAUNCH_MOE(EPI_F16, 2) }
  else { CTB_LAUNCH_MOE(EPI_F16, 1) }
#undef CTB_LAUNCH_MOE
  CTB_CHECK_LAUNCH("moe gemm launch");
  return CTB_OK;
}

// Bytes of the gate/up weights worth fetching into the L2 ahead of the expert GEMM: with few slots that GEMM streams
// the weights once and is bound by HBM, which sits idle during the sort; the blocks are ordered by expert, so the GEMM
// starts at the head of the tensor.  48 MB is what a sort of that size gives the memory time to deliver and a safe
// share of the L2.  With many slots the GEMM is bound by the tensor cores and nothing is fetched.
long long warm_bytes(long long slots, long long weight_bytes) {
  return slots <= 2048 ? std::min<long long>(weight_bytes, 48ll << 20) : 0;
}

// `warm`, `warm_bytes`: memory (16-byte aligned) that extra CTAs of the launch ask the L2 to fetch while the ids are
// sorted; null for none.
int launch_align(ctb_ctx* ctx, cudaStream_t st, const void* topk_ids, int ids_bits, int T, int topk, int E, int tile_m,
                 int* sorted_token_ids, int* sorted_expert_ids, int* num_blocks, int capacity, int skip_empty = 0,
                 const void* warm = nullptr, long long warm_bytes = 0) {
  const size_t smem = (size_t)(kAlignWarps * E + 5 * E + 1) * sizeof(int);
  const long long total = (long long)T * topk;
  const int C = total >= 4096 ? 8 : total >= 2048 ? 4 : 1;  // CTAs in the cluster: about 1024 ids each at least
  if (!warm || warm_bytes <= 0 || (uintptr_t)warm % 16) {
    warm = nullptr;
    warm_bytes = 0;
  }
  const int extra = warm ? std::max(1, (ctx->sm_count - C) / C) : 0;  // whole clusters that only warm the L2
  const unsigned char* warm_p = static_cast<const unsigned char*>(warm);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(C * (1 + extra));
  cfg.blockDim = dim3(kAlignThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cfg.numAttrs = C > 1 ? 1 : 0;  // a single CTA is launched as an ordinary grid (a cluster of one by default)
  cudaError_t e;
  if (ids_bits == 32)
    e = cudaLaunchKernelEx(&cfg, moe_align_kernel<int>, (const int*)topk_ids, T, topk, E, tile_m, sorted_token_ids,
                           sorted_expert_ids, num_blocks, capacity, skip_empty, ctx->dev_status, warm_p, warm_bytes);
  else
    e = cudaLaunchKernelEx(&cfg, moe_align_kernel<long long>, (const long long*)topk_ids, T, topk, E, tile_m,
                           sorted_token_ids, sorted_expert_ids, num_blocks, capacity, skip_empty, ctx->dev_status, warm_p,
                           warm_bytes);
  if (e != cudaSuccess) return cuda_fail(e, "moe align launch");
  return CTB_OK;
}

int check_tile(const char* who, int tile_m, int tile_n, int tile_k) {
  if (!is_pow2(tile_m) || !is_pow2(tile_n) || !is_pow2(tile_k))
    return fail(CTB_UNSUPPORTED_TILE, "%s: tile sizes must be powers of two (got %d,%d,%d)", who, tile_m, tile_n, tile_k);
  if (tile_m < 16 || tile_m > kMaxTileM)
    return fail(CTB_UNSUPPORTED_TILE, "%s: tile_m must be between 16 and %d (got %d)", who, kMaxTileM, tile_m);
  return CTB_OK;
}

}  // namespace

namespace ctb_internal {

size_t moe_experts_rows_workspace(int64_t R, int64_t I, int64_t E_local, int tile_m) {
  const int64_t blocks_cap = ctb_moe_max_blocks(R, 1, E_local, tile_m);
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  return up((size_t)blocks_cap * tile_m * 4) + up((size_t)blocks_cap * 4) + 256 + up((size_t)R * I * 2);
}

// The expert phase of the expert-parallel paths: `R` token rows (row i at rows + i*ld_rows, H f16 each) that made ONE
// choice each, ids[i] = local expert (1-based; 0 = the row is not for this rank), gates[i] = its routing weight.
// align + gate/up GEMM with SwiGLU + down GEMM; the weighted output row of token i goes to C + i*ldc, or, with
// c_split > 0, to c_peer[i / c_split] + (i % c_split)*ldc (peer memory: the buffer of the rank that sent the row).
int moe_experts_rows(ctb_ctx* ctx, cudaStream_t st, const void* rows, int64_t ld_rows, const int32_t* ids,
                     const void* gates, int64_t R, int64_t H, int64_t I, int64_t E_local, const void* w1_local,
                     const void* w2_local, int tile_m, void* C, int64_t ldc, void* const* c_peer, int64_t c_split) {
  if (R <= 0 || H <= 0 || I <= 0 || E_local <= 0 || R > (1 << 24)) return fail(CTB_BAD_ARG, "expert phase: bad shape");
  if (E_local > kMaxExperts) return fail(CTB_UNSUPPORTED, "expert phase: at most %d local experts", kMaxExperts);
  if (H % 8 || I % 8 || ld_rows % 8) return fail(CTB_BAD_ALIGN, "expert phase: hidden and intermediate sizes must be multiples of 8");
  CTB_CHECK_DEV(w1_local); CTB_CHECK_DEV(w2_local);
  if ((uintptr_t)w1_local % 16 || (uintptr_t)w2_local % 16 || (uintptr_t)rows % 16)
    return fail(CTB_BAD_ALIGN, "expert phase: 16-byte alignment of the weights and token rows");
  const int blocks_cap = (int)ctb_moe_max_blocks(R, 1, E_local, tile_m);
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  const size_t o_tok = 0, o_exp = up((size_t)blocks_cap * tile_m * 4), o_nb = o_exp + up((size_t)blocks_cap * 4),
               o_act = o_nb + 256, bytes = o_act + up((size_t)R * I * 2);
  void* ws;
  int r = workspace(ctx, bytes, &ws, st);
  if (r) return r;
  unsigned char* w = (unsigned char*)ws;
  int* s_tok = (int*)(w + o_tok);
  int* s_exp = (int*)(w + o_exp);
  int* s_nb = (int*)(w + o_nb);
  __half* act = (__half*)(w + o_act);
  // with rows from `world` ranks in the buffer (c_split rows each), about one rank's worth is for this rank's experts
  const int expect_blocks = c_split > 0 ? (int)(c_split / tile_m + E_local) : blocks_cap;
  r = launch_align(ctx, st, ids, 32, (int)R, 1, (int)E_local, tile_m, s_tok, s_exp, s_nb, blocks_cap, /*skip_empty=*/1,
                   w1_local, warm_bytes(R, 2 * I * H * E_local * 2));
  if (r) return r;
  r = launch_gemm(ctx, st, EPI_SWIGLU, (const __half*)rows, ld_rows, (int)R, (const __half*)w1_local, (int)H,
                  (int)(2 * I), (int)I, (int)E_local, nullptr, s_tok, s_exp, s_nb, -1, blocks_cap, 1, 0, tile_m, (int)R,
                  act, I);
  if (r) return r;
  return launch_gemm(ctx, st, EPI_F16, act, I, (int)R, (const __half*)w2_local, (int)I, (int)H, (int)H, (int)E_local,
                     (const __half*)gates, s_tok, s_exp, s_nb, -1, blocks_cap, 1, 1, tile_m, (int)R, C, ldc, 0, 1, c_peer,
                     (int)c_split, expect_blocks);
}

}  // namespace ctb_internal

extern "C" {

int64_t ctb_moe_max_blocks(int64_t T, int64_t topk, int64_t E, int tile_m) {
  if (T < 0 || topk <= 0 || E <= 0 || tile_m <= 0) return 0;
  return (T * topk + tile_m - 1) / tile_m + E;  // sum_e ceil(c_e / tile_m) <= total/tile_m + E
}

int ctb_moe_router(ctb_ctx* ctx, void* stream, const void* hidden, const void* W_r, int32_t* topk_ids,
                   void* topk_weights, float* logits, int64_t T, int64_t H, int64_t E, int topk) {
  CTB_CHECK_CTX(ctx);
  if (T < 0 || H <= 0 || E <= 0 || topk <= 0) return fail(CTB_BAD_ARG, "ctb_moe_router: non-positive dimension");
  if (E > kMaxRouterE) return fail(CTB_UNSUPPORTED, "ctb_moe_router: at most %d experts", kMaxRouterE);
  if (topk > 32 || topk > E) return fail(CTB_UNSUPPORTED, "ctb_moe_router: topk must be <= min(32, E)");
  if (H % 8) return fail(CTB_BAD_ALIGN, "ctb_moe_router: hidden size must be a multiple of 8");
  if (T == 0) return CTB_OK;
  CTB_CHECK_DEV(hidden); CTB_CHECK_DEV(W_r); CTB_CHECK_DEV(topk_ids); CTB_CHECK_DEV(topk_weights);
  if ((uintptr_t)hidden % 16 || (uintptr_t)W_r % 16) return fail(CTB_BAD_ALIGN, "ctb_moe_router: 16-byte alignment");
  // Group shape: (tokens per warp, token-warps).  Cost model: rounds of groups over the SMs x tokens per group x
  // shared-memory reads per token-expert block, (TT + 4) / TT.
  static const int cand[5][2] = {{2, 1}, {2, 2}, {2, 4}, {2, 8}, {4, 8}};
  int best = 0;
  double best_cost = 1e300;
  for (int c = 0; c < 5; ++c) {
    const int G = cand[c][0] * cand[c][1];
    const long long groups = (T + G - 1) / G, rounds = (groups + ctx->sm_count - 1) / ctx->sm_count;
    const double cost = (double)rounds * G * (cand[c][0] + kRouterTE) / cand[c][0];
    if (cost < best_cost * 0.999) { best_cost = cost; best = c; }
  }
  const int TT = cand[best][0], tw = cand[best][1], G = TT * tw;
  // shared memory: G token rows + eg expert rows as f16, rows padded to a multiple of 256 elements, + G x E logits
  const int64_t Hp = (H + 255) / 256 * 256;
  const size_t budget = 220 * 1024, rowbytes = (size_t)Hp * 2, fixed = (size_t)G * rowbytes + (size_t)G * E * 4;
  if (fixed + kRouterTE * rowbytes > budget)
    return fail(CTB_UNSUPPORTED, "ctb_moe_router: hidden size %lld too large", (long long)H);
  const int eg = (int)std::min<size_t>((size_t)E, (budget - fixed) / rowbytes / kRouterTE * kRouterTE);
  const size_t smem = fixed + (size_t)eg * rowbytes;
  const int ngroups = (int)((T + G - 1) / G);
  const int grid = std::min(ngroups, ctx->sm_count);
  cudaError_t ce;
#define CTB_LAUNCH_ROUTER(TTV)                                                                                  \
  ce = cudaFuncSetAttribute(moe_router_kernel<TTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
  if (ce != cudaSuccess) return cuda_fail(ce, "ctb_moe_router: shared memory opt-in");                          \
  moe_router_kernel<TTV><<<grid, kRouterThreads, smem, static_cast<cudaStream_t>(stream)>>>(                    \
      (const __half*)hidden, (const __half*)W_r, topk_ids, (__half*)topk_weights, logits, (int)T, (int)H, (int)E, \
      topk, eg, tw);
  if (TT == 4) { CTB_LAUNCH_ROUTER(4) } else { CTB_LAUNCH_ROUTER(2) }
#undef CTB_LAUNCH_ROUTER
  CTB_CHECK_LAUNCH("ctb_moe_router launch");
  return CTB_OK;
}

int ctb_moe_align(ctb_ctx* ctx, void* stream, const void* topk_ids, int ids_bits, int64_t T, int64_t topk, int64_t E,
                  int tile_m, int32_t* sorted_token_ids, int32_t* sorted_expert_ids, int32_t* num_blocks,
                  int64_t capacity_blocks) {
  CTB_CHECK_CTX(ctx);
  if (T <= 0 || topk <= 0 || E <= 0 || T * topk > (1 << 24)) return fail(CTB_BAD_ARG, "ctb_moe_align: bad shape");
  if (E > kMaxExperts) return fail(CTB_UNSUPPORTED, "ctb_moe_align: at most %d experts", kMaxExperts);
  if (ids_bits != 32 && ids_bits != 64) return fail(CTB_BAD_ARG, "ctb_moe_align: ids_bits must be 32 or 64");
  if (!is_pow2(tile_m)) return fail(CTB_UNSUPPORTED_TILE, "ctb_moe_align: tile_m %d is not a power of two", tile_m);
  if (capacity_blocks < ctb_moe_max_blocks(T, topk, E, tile_m))
    return fail(CTB_BAD_ARG, "ctb_moe_align: capacity_blocks %lld < ctb_moe_max_blocks = %lld", (long long)capacity_blocks,
                (long long)ctb_moe_max_blocks(T, topk, E, tile_m));
  CTB_CHECK_DEV(topk_ids); CTB_CHECK_DEV(sorted_token_ids); CTB_CHECK_DEV(sorted_expert_ids); CTB_CHECK_DEV(num_blocks);
  return launch_align(ctx, static_cast<cudaStream_t>(stream), topk_ids, ids_bits, (int)T, (int)topk, (int)E, tile_m,
                      sorted_token_ids, sorted_expert_ids, num_blocks, (int)capacity_blocks);
}

int ctb_moe_fused_gemm(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, const void* topk_weights,
                       const int32_t* sorted_token_ids, const int32_t* sorted_expert_ids, int64_t num_slots_padded,
                       int64_t K, int64_t N, int64_t E, int64_t a_cols, int64_t c_cols, int num_token_replicas,
                       int mul_routed_weight, int tile_m, int tile_n, int tile_k) {
  CTB_CHECK_CTX(ctx);
  int r = check_tile("ctb_moe_fused_gemm", tile_m, tile_n, tile_k);
  if (r) return r;
  if (K <= 0 || N <= 0 || E <= 0 || a_cols <= 0 || c_cols <= 0 || num_token_replicas <= 0 || num_slots_padded < 0 ||
      num_slots_padded % tile_m)
    return fail(CTB_BAD_ARG, "ctb_moe_fused_gemm: bad shape");
  if (K % 8) return fail(CTB_BAD_ALIGN, "ctb_moe_fused_gemm: K must be a multiple of 8");
  if (num_slots_padded == 0) return CTB_OK;
  CTB_CHECK_DEV(A); CTB_CHECK_DEV(B); CTB_CHECK_DEV(C); CTB_CHECK_DEV(sorted_token_ids); CTB_CHECK_DEV(sorted_expert_ids);
  if (mul_routed_weight) CTB_CHECK_DEV(topk_weights);
  if ((uintptr_t)A % 16 || (uintptr_t)B % 16) return fail(CTB_BAD_ALIGN, "ctb_moe_fused_gemm: 16-byte alignment");
  const int nb = (int)(num_slots_padded / tile_m);
  return launch_gemm(ctx, static_cast<cudaStream_t>(stream), EPI_F16, (const __half*)A, K, (int)a_cols,
                     (const __half*)B, (int)K, (int)N, (int)N, (int)E, (const __half*)topk_weights, sorted_token_ids,
                     sorted_expert_ids, nullptr, nb, nb, num_token_replicas, mul_routed_weight, tile_m, (int)c_cols, C,
                     N);
}

int ctb_moe_silu_and_mul(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, int64_t n, int64_t cols,
                         int64_t lda, int64_t ldb, int64_t ldc, int tile_n) {
  CTB_CHECK_CTX(ctx);
  if (n <= 0 || cols < 0 || lda < n || ldb < n || ldc < n) return fail(CTB_BAD_ARG, "ctb_moe_silu_and_mul: bad shape");
  if (!is_pow2(tile_n) || tile_n < n)
    return fail(CTB_UNSUPPORTED_TILE, "ctb_moe_silu_and_mul: TILE_N must be a power of two >= the row count");
  if (cols == 0) return CTB_OK;
  CTB_CHECK_DEV(A); CTB_CHECK_DEV(B); CTB_CHECK_DEV(C);
  const long long tot = n * cols;
  moe_silu_and_mul_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const __half*)A, (const __half*)B, (__half*)C, (int)n, cols, lda, ldb, ldc);
  CTB_CHECK_LAUNCH("ctb_moe_silu_and_mul launch");
  return CTB_OK;
}

int ctb_moe_ffn(ctb_ctx* ctx, void* stream, const void* hidden, const void* w1, const void* w2,
                const void* topk_weights, const void* topk_ids, int ids_bits, void* out, int64_t T, int64_t H,
                int64_t I, int64_t E, int64_t topk, int tile_m, int tile_n, int tile_k) {
  CTB_CHECK_CTX(ctx);
  int r = check_tile("ctb_moe_ffn", tile_m, tile_n, tile_k);
  if (r) return r;
  if (T <= 0 || H <= 0 || I <= 0 || E <= 0 || topk <= 0 || T * topk > (1 << 24))
    return fail(CTB_BAD_ARG, "ctb_moe_ffn: bad shape");
  if (E > kMaxExperts) return fail(CTB_UNSUPPORTED, "ctb_moe_ffn: at most %d experts", kMaxExperts);
  if (H % 8 || I % 8) return fail(CTB_BAD_ALIGN, "ctb_moe_ffn: hidden and intermediate sizes must be multiples of 8");
  if (ids_bits != 32 && ids_bits != 64) return fail(CTB_BAD_ARG, "ctb_moe_ffn: ids_bits must be 32 or 64");
  CTB_CHECK_DEV(hidden); CTB_CHECK_DEV(w1); CTB_CHECK_DEV(w2); CTB_CHECK_DEV(topk_weights); CTB_CHECK_DEV(topk_ids);
  CTB_CHECK_DEV(out);
  if ((uintptr_t)hidden % 16 || (uintptr_t)w1 % 16 || (uintptr_t)w2 % 16 || (uintptr_t)out % 16)
    return fail(CTB_BAD_ALIGN, "ctb_moe_ffn: 16-byte alignment of hidden, w1, w2");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int total = (int)(T * topk);
  const int cap = (int)ctb_moe_max_blocks(T, topk, E, tile_m);
  // scratch: sorted ids | expert ids | block count | activations (I, total) f16 | per-slot outputs (H, total) f16
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  const size_t o_tok = 0, o_exp = up((size_t)cap * tile_m * 4), o_nb = o_exp + up((size_t)cap * 4), o_act = o_nb + 256,
               o_slots = o_act + up((size_t)total * I * 2), bytes = o_slots + up((size_t)total * H * 2);
  void* ws;
  r = workspace(ctx, bytes, &ws, st);
  if (r) return r;
  unsigned char* w = (unsigned char*)ws;
  int* s_tok = (int*)(w + o_tok);
  int* s_exp = (int*)(w + o_exp);
  int* s_nb = (int*)(w + o_nb);
  __half* act = (__half*)(w + o_act);
  __half* slots = (__half*)(w + o_slots);
  r = launch_align(ctx, st, topk_ids, ids_bits, (int)T, (int)topk, (int)E, tile_m, s_tok, s_exp, s_nb, cap, 0, w1,
                   warm_bytes(T * topk, 2 * I * H * E * 2));
  if (r) return r;
  // gate/up projection with the SwiGLU epilogue: act(:, id) = silu(Wg x) * (Wu x)
  r = launch_gemm(ctx, st, EPI_SWIGLU, (const __half*)hidden, H, (int)T, (const __half*)w1, (int)H, (int)(2 * I),
                  (int)I, (int)E, nullptr, s_tok, s_exp, s_nb, -1, cap, (int)topk, 0, tile_m, total, act, I);
  if (r) return r;
  // down projection scaled by the routing weight, one f16 column per slot (the reference's cache3)
  r = launch_gemm(ctx, st, EPI_F16, act, I, total, (const __half*)w2, (int)I, (int)H, (int)H, (int)E,
                  (const __half*)topk_weights, s_tok, s_exp, s_nb, -1, cap, 1, 1, tile_m, total, slots, H, (int)T,
                  (int)topk);
  if (r) return r;
  const long long n8 = T * (H / 8);
  moe_combine_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(slots, (__half*)out, (int)T, (int)H, (int)topk);
  CTB_CHECK_LAUNCH("ctb_moe_ffn combine launch");
  return CTB_OK;
}

static int check_ep(const char* who, const ctb_ep_buffers* b) {
  if (!b) return fail(CTB_BAD_ARG, "%s: null buffer table", who);
  if (b->world < 1 || b->world > CTB_EP_MAX_RANKS || b->rank < 0 || b->rank >= b->world)
    return fail(CTB_BAD_ARG, "%s: world %d / rank %d out of range (at most %d ranks)", who, b->world, b->rank,
                CTB_EP_MAX_RANKS);
  for (int q = 0; q < b->world; ++q) {
    if (!b->recv_rows[q] || !b->recv_ids[q] || !b->recv_gates[q] || !b->slot_out[q])
      return fail(CTB_BAD_ARG, "%s: null buffer of rank %d", who, q);
    if ((uintptr_t)b->recv_rows[q] % 16 || (uintptr_t)b->slot_out[q] % 16)
      return fail(CTB_BAD_ALIGN, "%s: row buffers of rank %d must be 16-byte aligned", who, q);
  }
  return CTB_OK;
}

int ctb_moe_ep_dispatch(ctb_ctx* ctx, void* stream, const ctb_ep_buffers* bufs, const void* hidden,
                        const int32_t* topk_ids, const void* topk_weights, int64_t T, int64_t H, int64_t E,
                        int64_t topk) {
  CTB_CHECK_CTX(ctx);
  int r = check_ep("ctb_moe_ep_dispatch", bufs);
  if (r) return r;
  if (T < 0 || H <= 0 || E <= 0 || topk <= 0 || T * topk > (1 << 24)) return fail(CTB_BAD_ARG, "ctb_moe_ep_dispatch: bad shape");
  if (E % bufs->world) return fail(CTB_BAD_ARG, "ctb_moe_ep_dispatch: the experts must divide evenly over the ranks");
  if (H % 8) return fail(CTB_BAD_ALIGN, "ctb_moe_ep_dispatch: H must be a multiple of 8");
  if (T == 0) return CTB_OK;
  CTB_CHECK_DEV(hidden); CTB_CHECK_DEV(topk_ids); CTB_CHECK_DEV(topk_weights);
  if ((uintptr_t)hidden % 16) return fail(CTB_BAD_ALIGN, "ctb_moe_ep_dispatch: 16-byte alignment of hidden");
  EpPtrs pp;
  for (int q = 0; q < CTB_EP_MAX_RANKS; ++q) {
    const bool on = q < bufs->world;
    pp.rows[q] = on ? (uint4*)bufs->recv_rows[q] : nullptr;
    pp.ids[q] = on ? bufs->recv_ids[q] : nullptr;
    pp.gates[q] = on ? (__half*)bufs->recv_gates[q] : nullptr;
  }
  const long long cap = T * topk;
  const int grid = (int)std::min<long long>((cap + 7) / 8, (long long)ctx->sm_count * 8);
  moe_ep_dispatch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint4*)hidden, topk_ids, (const __half*)topk_weights, pp, (int)T, (int)topk, (int)(H / 8), (int)E,
      (int)(E / bufs->world), bufs->world, bufs->rank, ctx->dev_status);
  CTB_CHECK_LAUNCH("ctb_moe_ep_dispatch launch");
  return CTB_OK;
}

int ctb_moe_ep_barrier(ctb_ctx* ctx, void* stream, const ctb_ep_buffers* bufs) {
  CTB_CHECK_CTX(ctx);
  int r = check_ep("ctb_moe_ep_barrier", bufs);
  if (r) return r;
  if (!bufs->epoch) return fail(CTB_BAD_ARG, "ctb_moe_ep_barrier: null epoch counter");
  EpFlags f;
  for (int q = 0; q < CTB_EP_MAX_RANKS; ++q) {
    f.flags[q] = q < bufs->world ? bufs->flags[q] : nullptr;
    if (q < bufs->world && !f.flags[q]) return fail(CTB_BAD_ARG, "ctb_moe_ep_barrier: null flag array of rank %d", q);
  }
  moe_ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, bufs->epoch, bufs->world, bufs->rank,
                                                                        ctx->dev_status, ctx->flag_wait_ns);
  CTB_CHECK_LAUNCH("ctb_moe_ep_barrier launch");
  return CTB_OK;
}

int ctb_moe_ep_experts(ctb_ctx* ctx, void* stream, const ctb_ep_buffers* bufs, const void* w1_local,
                       const void* w2_local, int64_t cap, int64_t H, int64_t I, int64_t E_local, int tile_m, int tile_n,
                       int tile_k) {
  CTB_CHECK_CTX(ctx);
  int r = check_ep("ctb_moe_ep_experts", bufs);
  if (r) return r;
  r = check_tile("ctb_moe_ep_experts", tile_m, tile_n, tile_k);
  if (r) return r;
  const long long R = cap * bufs->world;  // columns of the receive buffers
  if (cap <= 0) return fail(CTB_BAD_ARG, "ctb_moe_ep_experts: bad shape");
  const int me = bufs->rank;
  // every received column is one token with a single choice; id 0 = the slot went to another rank
  return moe_experts_rows(ctx, static_cast<cudaStream_t>(stream), bufs->recv_rows[me], H, bufs->recv_ids[me],
                          bufs->recv_gates[me], R, H, I, E_local, w1_local, w2_local, tile_m, bufs->slot_out[me], H,
                          bufs->slot_out, cap);
}

int ctb_moe_gather_rows(ctb_ctx* ctx, void* stream, void* dst, const void* src, const int32_t* ids, int64_t n_ids,
                        int64_t row_elems, int num_token_replicas, int64_t src_rows) {
  CTB_CHECK_CTX(ctx);
  if (n_ids < 0 || row_elems <= 0 || num_token_replicas <= 0 || src_rows < 0)
    return fail(CTB_BAD_ARG, "ctb_moe_gather_rows: bad shape");
  if (row_elems % 8) return fail(CTB_BAD_ALIGN, "ctb_moe_gather_rows: rows must be multiples of 8 f16 elements");
  if (n_ids == 0) return CTB_OK;
  CTB_CHECK_DEV(dst); CTB_CHECK_DEV(src); CTB_CHECK_DEV(ids);
  if ((uintptr_t)dst % 16 || (uintptr_t)src % 16) return fail(CTB_BAD_ALIGN, "ctb_moe_gather_rows: 16-byte alignment");
  const int vecs = (int)(row_elems / 8);
  const long long tot = n_ids * vecs;
  moe_gather_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (uint4*)dst, (const uint4*)src, ids, n_ids, vecs, num_token_replicas, src_rows);
  CTB_CHECK_LAUNCH("ctb_moe_gather_rows launch");
  return CTB_OK;
}

int ctb_moe_scatter_rows(ctb_ctx* ctx, void* stream, void* dst, const void* src, const int32_t* ids, int64_t n_ids,
                         int64_t row_elems, int64_t dst_rows) {
  CTB_CHECK_CTX(ctx);
  if (n_ids < 0 || row_elems <= 0 || dst_rows < 0) return fail(CTB_BAD_ARG, "ctb_moe_scatter_rows: bad shape");
  if (row_elems % 8) return fail(CTB_BAD_ALIGN, "ctb_moe_scatter_rows: rows must be multiples of 8 f16 elements");
  if (n_ids == 0) return CTB_OK;
  CTB_CHECK_DEV(dst); CTB_CHECK_DEV(src); CTB_CHECK_DEV(ids);
  if ((uintptr_t)dst % 16 || (uintptr_t)src % 16) return fail(CTB_BAD_ALIGN, "ctb_moe_scatter_rows: 16-byte alignment");
  const int vecs = (int)(row_elems / 8);
  const long long tot = n_ids * vecs;
  moe_scatter_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (uint4*)dst, (const uint4*)src, ids, n_ids, vecs, dst_rows);
  CTB_CHECK_LAUNCH("ctb_moe_scatter_rows launch");
  return CTB_OK;
}

int ctb_moe_combine(ctb_ctx* ctx, void* stream, const void* slots, void* out, int64_t T, int64_t H, int64_t topk) {
  CTB_CHECK_CTX(ctx);
  if (T < 0 || H <= 0 || topk <= 0) return fail(CTB_BAD_ARG, "ctb_moe_combine: bad shape");
  if (H % 8) return fail(CTB_BAD_ALIGN, "ctb_moe_combine: H must be a multiple of 8");
  if (T == 0) return CTB_OK;
  CTB_CHECK_DEV(slots); CTB_CHECK_DEV(out);
  if ((uintptr_t)slots % 16 || (uintptr_t)out % 16) return fail(CTB_BAD_ALIGN, "ctb_moe_combine: 16-byte alignment");
  const long long n8 = T * (H / 8);
  moe_combine_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const __half*)slots, (__half*)out, (int)T, (int)H, (int)topk);
  CTB_CHECK_LAUNCH("ctb_moe_combine launch");
  return CTB_OK;
}

}  // extern "C"
