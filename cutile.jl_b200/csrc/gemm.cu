// Dense and batched GEMM for sm_100a: C(M,N[,b]) = A(M,K[,b]) * B(K,N[,b]),
// Julia column-major (counterparts of matmul_kernel, examples/matmul.jl:28-60,
// and batch_matmul_kernel, examples/batchmatmul.jl:15-56).
//
// f32 inputs run as TF32 tensor-core MMAs with f32 accumulation (the reference
// converts f32 -> tf32, examples/matmul.jl:49-52; the tensor core here reads the
// raw f32 bits from shared memory and ignores the low 13 mantissa bits, i.e.
// truncation instead of the reference's round-to-nearest-even); f16 inputs run
// as f16 MMAs with f32 accumulation and an f16 result.
//
// One persistent CTA per SM, 6 warps:
//   warp 0     TMA producer: per k-block, A as 128-byte-wide boxes (M contiguous,
//              "MN-major") and B as one box (K contiguous, "K-major"), 128B swizzle
//              (32-byte-atom flavour for the tf32 A operand),
//              into a ring of kStages shared-memory stages guarded by mbarriers;
//   warp 1     MMA issuer: tcgen05.mma 128 x 256 x (32 bytes of K) from shared-memory
//              descriptors into one of two 256-column TMEM accumulators;
//              tcgen05.commit frees the stage / publishes the accumulator;
//   warps 2-5  epilogue: tcgen05.ld the finished accumulator (lane = row m) and
//              store C with coalesced 128-byte rows while the MMA warp already
//              works on the next tile in the other accumulator.
// Out-of-range parts of edge tiles are zero-filled by TMA and masked on store.
//
// Large problems run gemm_pair_kernel instead: the two CTAs of a 2-CTA cluster share one 256 x 256 tile
// (tcgen05 cta_group::2, the counterpart of the reference's num_ctas = 2 hint on this architecture,
// examples/matmul.jl:30).  Each CTA loads its own 128 rows of A and its own 128 columns of B per k-block, so an SM
// takes in 32 KB of operands per 128 x 256 x (128 bytes of K) of MMA work instead of 48 KB: operand delivery, not the
// tensor pipe, is what bounds the single-CTA kernel.  No load in this file is a cluster multicast.
#include <cuda_bf16.h>

#include <type_traits>

#include "ctx.h"
#include "ptx.cuh"

using namespace ctb;
using namespace ctb_internal;

namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kAccCols = kTileN;  // f32 accumulator columns per tile
constexpr uint32_t kTmemCols = 512;

// f32 accumulator -> result element (round to nearest even for the 16-bit types)
template <typename T>
__device__ __forceinline__ T from_f32(float v) {
  if constexpr (std::is_same<T, float>::value) return v;
  else if constexpr (std::is_same<T, __nv_bfloat16>::value) return __float2bfloat16_rn(v);
  else return __float2half_rn(v);
}

template <typename T>
struct Cfg {
  static constexpr int ES = sizeof(T);
  static constexpr int BK = 128 / ES;          // K elements per stage = one 128-byte swizzle span
  static constexpr int UK = 32 / ES;           // K per MMA instruction
  static constexpr int CHUNK_M = 128 / ES;     // M elements per A box (128 bytes)
  static constexpr int A_BOXES = kTileM / CHUNK_M;
  static constexpr int A_BOX_BYTES = BK * 128;  // BK rows of 128 bytes
  static constexpr int A_BYTES = A_BOXES * A_BOX_BYTES;
  static constexpr int B_BYTES = kTileN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr uint32_t FMT = sizeof(T) == 4 ? FMT_TF32 : std::is_same<T, __nv_bfloat16>::value ? FMT_BF16 : FMT_F16;
  // An MN-major tf32 operand must use the 128-byte swizzle with 32-byte atoms
  // (4 K-rows per swizzle period); 16-bit types use the ordinary 128-byte swizzle.
  static constexpr uint32_t A_LAYOUT = sizeof(T) == 4 ? SDESC_SW128_ATOM32 : SDESC_SW128;
  static constexpr uint32_t A_SBO = sizeof(T) == 4 ? 512 : 1024;
};

struct Params {
  int M, N, K, batch;
  long long ldc, strideC;
  int tiles_m, tiles_n, num_tiles;
  // Split-K (single-CTA kernel, few tiles): a work unit is (tile, split); split s takes the k-blocks
  // [s * nk / splits, (s + 1) * nk / splits) and leaves its f32 accumulator tile in partial[unit] (column by column,
  // 128 rows each); gemm_splitk_reduce_kernel adds the splits in ascending order.
  int splits;
  float* partial;
};

__device__ __forceinline__ void tile_coords(const Params& p, int t, int& b, int& tm, int& tn) {
  const int per_batch = p.tiles_m * p.tiles_n;
  b = t / per_batch;
  const int r = t - b * per_batch;
  // grouped order of examples/matmul.jl:13-24 (GROUP_SIZE_M = 8) for L2 reuse
  const int in_group = 8 * p.tiles_n;
  const int first = (r / in_group) * 8;
  const int gsz = min(p.tiles_m - first, 8);
  tm = first + (r % in_group) % gsz;
  tn = (r % in_group) / gsz;
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                T* __restrict__ C, const Params p, int* status) {
  using G = Cfg<T>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full[kStages], empty[kStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmapA);
    tma_prefetch_desc(&tmapB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort = &abort_s;
  const int nk = (p.K + G::BK - 1) / G::BK;
  const int units = p.num_tiles * p.splits;

  if (warp == 0) {
    // ---- TMA producer: the whole warp walks the loop, one elected lane issues
    int stage = 0;
    uint32_t phase = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      int b, tm, tn;
      tile_coords(p, u / p.splits, b, tm, tn);
      const int sp = u % p.splits, kb_lo = sp * nk / p.splits, kb_hi = (sp + 1) * nk / p.splits;
      bool ok = true;
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        ok = CTB_WARP_WAIT(&empty[stage], phase ^ 1, status, DEV_TIMEOUT_SLOT, abort);
        if (!ok) break;
        unsigned char* sa = smem + (size_t)stage * G::STAGE_BYTES;
        if (elect_one()) {
          mbar_expect_tx(&full[stage], G::STAGE_BYTES);
#pragma unroll
          for (int j = 0; j < G::A_BOXES; ++j)
            tma_load_3d(sa + j * G::A_BOX_BYTES, &tmapA, tm * kTileM + j * G::CHUNK_M, kb * G::BK, b, &full[stage]);
          tma_load_3d(sa + G::A_BYTES, &tmapB, kb * G::BK, tn * kTileN, b, &full[stage]);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) break;
    }
  } else if (warp == 1) {
    // ---- MMA issuer: the whole warp walks the loop, one elected lane issues
    constexpr uint32_t idesc = make_idesc(G::FMT, kTileM, kTileN, /*A MN-major*/ 1, /*B K-major*/ 0);
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!CTB_WARP_WAIT(&acc_empty[acc], acc_phase ^ 1, status, DEV_TIMEOUT_SLOT, abort)) break;
      tc_fence_after();
      const uint32_t d = tmem_base + acc * kAccCols;
      const int sp = u % p.splits, kb_lo = sp * nk / p.splits, kb_hi = (sp + 1) * nk / p.splits;
      bool ok = true;
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        ok = CTB_WARP_WAIT(&full[stage], phase, status, DEV_TIMEOUT_TMA, abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + (size_t)stage * G::STAGE_BYTES);
        const uint32_t sb = sa + G::A_BYTES;
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < G::BK / G::UK; ++k) {
            const uint64_t ad = make_sdesc(sa + k * G::UK * 128, G::A_BOX_BYTES, G::A_SBO, G::A_LAYOUT);
            const uint64_t bd = make_sdesc_sw128(sb + k * 32, 0, 1024);
            if constexpr (sizeof(T) == 4)
              mma_tf32_ss(d, ad, bd, idesc, ((kb - kb_lo) | k) != 0);
            else
              mma_f16_ss(d, ad, bd, idesc, ((kb - kb_lo) | k) != 0);
          }
          tc_commit(&empty[stage]);
        }
        __syncwarp();
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) break;
      if (elect_one()) tc_commit(&acc_full[acc]);
      __syncwarp();
    }
  } else {
    const int sub = warp & 3;  // TMEM lanes [32*sub, 32*sub+32) belong to this warp
    int it = 0;
    for (int u = blockIdx.x; u < units; u += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      int b, tm, tn;
      tile_coords(p, u / p.splits, b, tm, tn);
      bool ok = CTB_WARP_WAIT(&acc_full[acc], acc_phase, status, DEV_TIMEOUT_MMA, abort);
      if (!ok) break;
      tc_fence_after();
      const int m = tm * kTileM + sub * 32 + lane;
      T* crow = C + (long long)b * p.strideC + m;
      float* prow = p.partial + (long long)u * (kTileM * kTileN) + sub * 32 + lane;
      const uint32_t taddr = tmem_base + acc * kAccCols + ((uint32_t)(sub * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < kTileN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tc_wait_ld();
        const int n0 = tn * kTileN + c * 32;
        if (p.splits > 1) {
#pragma unroll
          for (int j = 0; j < 32; ++j) prow[(c * 32 + j) * kTileM] = __uint_as_float(r[j]);
        } else if (m < p.M) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (n0 + j < p.N) {
              if constexpr (sizeof(T) == 4)
                crow[(long long)(n0 + j) * p.ldc] = __uint_as_float(r[j]);
              else
                crow[(long long)(n0 + j) * p.ldc] = from_f32<T>(__uint_as_float(r[j]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Adds the splits of every tile in ascending order and writes C.  A thread takes four consecutive rows of a column
// (16-byte loads; a warp covers 128 rows = one column of the tile) and requests eight splits at a time.
template <typename T>
__global__ void __launch_bounds__(256)
    gemm_splitk_reduce_kernel(const float* __restrict__ partial, T* __restrict__ C, const Params p) {
  constexpr int kTileElems = kTileM * kTileN;
  const long long total = (long long)p.num_tiles * (kTileElems / 4);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / (kTileElems / 4)), e = (int)(i - (long long)t * (kTileElems / 4)) * 4;
    const int col = e / kTileM, row = e - col * kTileM;
    int b, tm, tn;
    tile_coords(p, t, b, tm, tn);
    const int m = tm * kTileM + row, n = tn * kTileN + col;
    if (m >= p.M || n >= p.N) continue;
    const float4* src = reinterpret_cast<const float4*>(partial + (long long)t * p.splits * kTileElems + e);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < p.splits; s0 += 8) {
      float4 v[8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        v[q] = s0 + q < p.splits ? __ldcs(src + (long long)(s0 + q) * (kTileElems / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int q = 0; q < 8; ++q) {  // ascending split order
        acc.x += v[q].x;
        acc.y += v[q].y;
        acc.z += v[q].z;
        acc.w += v[q].w;
      }
    }
    T* dst = C + (long long)b * p.strideC + (long long)n * p.ldc + m;
    const float o[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (m + q < p.M) {
        if constexpr (sizeof(T) == 4)
          dst[q] = o[q];
        else
          dst[q] = from_f32<T>(o[q]);
      }
    }
  }
}

// ---- CTA-pair kernel ---------------------------------------------------------------------------------------------
// Cluster of 2 CTAs = one 256 (M) x 256 (N) tile per step.  CTA rank r holds A rows [128 r, 128 r + 128) and
// B columns [128 r, 128 r + 128) of the tile in its shared memory and the accumulator rows [128 r, 128 r + 128) x 256
// columns in its TMEM.  Barriers: full[] lives in rank 0 and counts the bytes of both CTAs' loads; empty[] and
// acc_full[] exist in both CTAs and are arrived by rank 0's multicast commits; acc_empty[] lives in rank 0 and is
// arrived by the epilogue warps of both CTAs.
constexpr int kPairStages = 6;
constexpr int kPairTileM = 256;

template <typename T>
struct PairCfg {
  using G = Cfg<T>;
  static constexpr int B_ROWS = kTileN / 2;          // columns of the tile held by one CTA
  static constexpr int B_BYTES = B_ROWS * 128;
  static constexpr int STAGE_BYTES = G::A_BYTES + B_BYTES;  // per CTA
};

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmapA, const __grid_constant__ CUtensorMap tmapB,
                     T* __restrict__ C, const Params p, int* status) {
  using G = Cfg<T>;
  using P = PairCfg<T>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t full[kPairStages], empty[kPairStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 8);  // four epilogue warps in each of the two CTAs
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmapA);
    tma_prefetch_desc(&tmapB);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_s, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();  // the peer's barriers exist before anything is signalled on them
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  volatile int* abort = &abort_s;
  const int nk = (p.K + G::BK - 1) / G::BK;

  if (warp == 0) {
    // ---- TMA producer (both CTAs): own halves of A and B, bytes counted on rank 0's full barrier
    int stage = 0;
    uint32_t phase = 0;
    for (int t = pair; t < p.num_tiles; t += num_pairs) {
      int b, tm, tn;
      tile_coords(p, t, b, tm, tn);
      const int m0 = tm * kPairTileM + (int)rank * kTileM, n0 = tn * kTileN + (int)rank * P::B_ROWS;
      bool ok = true;
      for (int kb = 0; kb < nk; ++kb) {
        ok = CTB_WARP_WAIT(&empty[stage], phase ^ 1, status, DEV_TIMEOUT_SLOT, abort);
        if (!ok) break;
        unsigned char* sa = smem + (size_t)stage * P::STAGE_BYTES;
        if (elect_one()) {
          if (rank == 0) mbar_expect_tx(&full[stage], 2 * P::STAGE_BYTES);
          const uint32_t bar = map_to_cta(&full[stage], 0);
#pragma unroll
          for (int j = 0; j < G::A_BOXES; ++j)
            tma_load_3d_pair(sa + j * G::A_BOX_BYTES, &tmapA, m0 + j * G::CHUNK_M, kb * G::BK, b, bar);
          tma_load_3d_pair(sa + G::A_BYTES, &tmapB, kb * G::BK, n0, b, bar);
        }
        __syncwarp();
        if (++stage == kPairStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (!ok) break;
    }
  } else if (warp == 1) {
    if (rank == 0) {
      // ---- MMA issuer (rank 0 only): one instruction drives the tensor cores of both SMs
      constexpr uint32_t idesc = make_idesc(G::FMT, kPairTileM, kTileN, /*A MN-major*/ 1, /*B K-major*/ 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = pair; t < p.num_tiles; t += num_pairs, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!CTB_WARP_WAIT(&acc_empty[acc], acc_phase ^ 1, status, DEV_TIMEOUT_SLOT, abort)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * kAccCols;
        bool ok = true;
        for (int kb = 0; kb < nk; ++kb) {
          ok = CTB_WARP_WAIT(&full[stage], phase, status, DEV_TIMEOUT_TMA, abort);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * P::STAGE_BYTES);
          const uint32_t sb = sa + G::A_BYTES;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < G::BK / G::UK; ++k) {
              const uint64_t ad = make_sdesc(sa + k * G::UK * 128, G::A_BOX_BYTES, G::A_SBO, G::A_LAYOUT);
              const uint64_t bd = make_sdesc_sw128(sb + k * 32, 0, 1024);
              if constexpr (sizeof(T) == 4)
                mma_tf32_ss_pair(d, ad, bd, idesc, (kb | k) != 0);
              else
                mma_f16_ss_pair(d, ad, bd, idesc, (kb | k) != 0);
            }
            tc_commit_pair(&empty[stage], 3);
          }
          __syncwarp();
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (elect_one()) tc_commit_pair(&acc_full[acc], 3);
        __syncwarp();
      }
    }
  } else {
    const int sub = warp & 3;  // TMEM lanes [32*sub, 32*sub+32) belong to this warp
    int it = 0;
    for (int t = pair; t < p.num_tiles; t += num_pairs, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      int b, tm, tn;
      tile_coords(p, t, b, tm, tn);
      bool ok = CTB_WARP_WAIT(&acc_full[acc], acc_phase, status, DEV_TIMEOUT_MMA, abort);
      if (!ok) break;
      tc_fence_after();
      const int m = tm * kPairTileM + (int)rank * kTileM + sub * 32 + lane;
      T* crow = C + (long long)b * p.strideC + m;
      const uint32_t taddr = tmem_base + acc * kAccCols + ((uint32_t)(sub * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < kTileN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tc_wait_ld();
        const int n0 = tn * kTileN + c * 32;
        if (m < p.M) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (n0 + j < p.N) {
              if constexpr (sizeof(T) == 4)
                crow[(long long)(n0 + j) * p.ldc] = __uint_as_float(r[j]);
              else
                crow[(long long)(n0 + j) * p.ldc] = from_f32<T>(__uint_as_float(r[j]));
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(&acc_empty[acc], 0));
    }
  }
  // Neither CTA may leave (or free its TMEM) while the other can still read its shared memory, write its TMEM or
  // signal its barriers: every thread of both CTAs meets here, also after an abort.
  tc_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

// How many 2-CTA clusters of gemm_pair_kernel the device runs at once (asked once per element type).
template <typename T>
int pair_clusters(ctb_ctx* ctx, size_t smem) {
  static int cached[16] = {0};  // per device; 0 = not asked yet, -1 = unavailable
  int& c = cached[ctx->device & 15];
  if (c == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * ctx->sm_count);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<T>, &cfg);
    c = (e == cudaSuccess && n > 0) ? n : -1;
    if (e != cudaSuccess) (void)cudaGetLastError();
  }
  return c;
}

// out[i] = in[i] rounded to TF32 precision, nearest even (NaNs stay NaNs): u + 0xFFF + bit 13, low 13 bits cleared.
__global__ void __launch_bounds__(256) tf32_round_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, long long n4,
                                                         const uint32_t* __restrict__ in_tail, uint32_t* __restrict__ out_tail,
                                                         int tail) {
  auto rne = [](uint32_t u) {
    const bool nan = ((u >> 23) & 0xFFu) == 0xFFu && (u & 0x7FFFFFu) != 0;
    const uint32_t r = (u + 0xFFFu + ((u >> 13) & 1u)) & 0xFFFFE000u;
    return nan ? ((u & 0xFFFFE000u) | 0x2000u) : r;
  };
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    uint4 v = __ldcs(in + i);
    v.x = rne(v.x); v.y = rne(v.y); v.z = rne(v.z); v.w = rne(v.w);
    out[i] = v;
  }
  if (blockIdx.x == 0 && (int)threadIdx.x < tail) out_tail[threadIdx.x] = rne(in_tail[threadIdx.x]);
}

template <typename T>
int launch(ctb_ctx* ctx, cudaStream_t st, const T* A, const T* B, T* C, int M, int N, int K, int batch, long long lda,
           long long ldb, long long ldc, long long sA, long long sB, long long sC) {
  using G = Cfg<T>;
  const CUtensorMapDataType dt = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  size_t ws_used = 0;  // bytes of the context scratch taken by rounded operand copies (the split-K partials follow)
  if (sizeof(T) == 4 && ctx->tf32_rne) {
    // rounded copies with the layout of the originals (same leading dimensions and batch strides)
    // elements from the first to the last one that the arrays are known to hold
    const long long ea = (long long)(batch - 1) * sA + lda * (long long)(K - 1) + M;
    const long long eb = (long long)(batch - 1) * sB + ldb * (long long)(N - 1) + K;
    auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
    const size_t oa = 0, ob = up((size_t)ea * 4);
    ws_used = ob + up((size_t)eb * 4);
    const size_t partial_max = (size_t)ctx->sm_count * kTileM * kTileN * sizeof(float);  // split-K: at most one tile per SM
    void* ws = nullptr;
    int r = workspace(ctx, ws_used + partial_max, &ws, st);
    if (r) return r;
    float* A2 = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + oa);
    float* B2 = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + ob);
    const int rgrid = ctx->sm_count * 8;
    tf32_round_kernel<<<rgrid, 256, 0, st>>>(reinterpret_cast<const uint4*>(A), reinterpret_cast<uint4*>(A2), ea / 4,
                                            reinterpret_cast<const uint32_t*>(A) + (ea & ~3ll),
                                            reinterpret_cast<uint32_t*>(A2) + (ea & ~3ll), (int)(ea & 3));
    tf32_round_kernel<<<rgrid, 256, 0, st>>>(reinterpret_cast<const uint4*>(B), reinterpret_cast<uint4*>(B2), eb / 4,
                                            reinterpret_cast<const uint32_t*>(B) + (eb & ~3ll),
                                            reinterpret_cast<uint32_t*>(B2) + (eb & ~3ll), (int)(eb & 3));
    CTB_CHECK_LAUNCH("ctb_gemm operand rounding launch");
    A = reinterpret_cast<const T*>(A2);
    B = reinterpret_cast<const T*>(B2);
  }
  CUtensorMap ta, tb;
  {
    // A memory: [batch][K][M], M contiguous
    uint64_t dims[3] = {(uint64_t)M, (uint64_t)K, (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)lda * G::ES, (uint64_t)(batch > 1 ? sA : lda * (long long)K) * G::ES};
    uint32_t box[3] = {(uint32_t)G::CHUNK_M, (uint32_t)G::BK, 1};
    int r = make_tmap(&ta, dt, 3, A, dims, str, box,
                      sizeof(T) == 4 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B);
    if (r) return r;
  }
  {
    // B memory: [batch][N][K], K contiguous
    uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)batch};
    uint64_t str[2] = {(uint64_t)ldb * G::ES, (uint64_t)(batch > 1 ? sB : ldb * (long long)N) * G::ES};
    uint32_t box[3] = {(uint32_t)G::BK, (uint32_t)kTileN, 1};
    int r = make_tmap(&tb, dt, 3, B, dims, str, box);
    if (r) return r;
  }
  Params p;
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.ldc = ldc; p.strideC = sC;
  {
    // CTA pairs when there are enough 256 x 256 tiles to occupy at least half of the SM pairs
    const long long pairs = (long long)((M + kPairTileM - 1) / kPairTileM) * ((N + kTileN - 1) / kTileN) * batch;
    if (M >= kPairTileM && N >= kTileN && pairs * 4 >= ctx->sm_count && pairs <= INT32_MAX) {
      using P = PairCfg<T>;
      CUtensorMap tb2;
      uint64_t dims[3] = {(uint64_t)K, (uint64_t)N, (uint64_t)batch};
      uint64_t str[2] = {(uint64_t)ldb * G::ES, (uint64_t)(batch > 1 ? sB : ldb * (long long)N) * G::ES};
      uint32_t box[3] = {(uint32_t)G::BK, (uint32_t)P::B_ROWS, 1};
      int r = make_tmap(&tb2, dt, 3, B, dims, str, box);
      if (r) return r;
      p.tiles_m = (M + kPairTileM - 1) / kPairTileM;
      p.tiles_n = (N + kTileN - 1) / kTileN;
      p.num_tiles = (int)pairs;
      p.splits = 1;
      p.partial = nullptr;
      const size_t smem = (size_t)kPairStages * P::STAGE_BYTES + 1024;
      auto k = gemm_pair_kernel<T>;
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return cuda_fail(e, "ctb_gemm: shared memory opt-in");
      const int clusters = pair_clusters<T>(ctx, smem);
      if (clusters > 0) {
        const int grid = 2 * (int)std::min<long long>(pairs, clusters);
        k<<<grid, kThreads, smem, st>>>(ta, tb2, C, p, ctx->dev_status);
        CTB_CHECK_LAUNCH("ctb_gemm launch");
        return CTB_OK;
      }
    }
  }
  p.tiles_m = (M + kTileM - 1) / kTileM;
  p.tiles_n = (N + kTileN - 1) / kTileN;
  const long long nt = (long long)p.tiles_m * p.tiles_n * batch;
  if (nt > INT32_MAX) return fail(CTB_UNSUPPORTED, "ctb_gemm: too many tiles");
  p.num_tiles = (int)nt;
  // Few tiles and a long K (one rank's share of a batch-sharded problem): split K over the idle SMs, at least four
  // k-blocks per split.
  const int nk = (K + G::BK - 1) / G::BK;
  p.splits = (int)std::max<long long>(1, std::min<long long>(std::min<long long>(ctx->sm_count / nt, nk / 4), 16));
  p.partial = nullptr;
  if (p.splits > 1) {
    void* ws = nullptr;
    int r = workspace(ctx, ws_used + (size_t)nt * p.splits * kTileM * kTileN * sizeof(float), &ws, st);
    if (r) return r;
    p.partial = reinterpret_cast<float*>(static_cast<unsigned char*>(ws) + ws_used);
  }
  const size_t smem = (size_t)kStages * G::STAGE_BYTES + 1024;
  auto k = gemm_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_gemm: shared memory opt-in");
  const int grid = (int)std::min<long long>(nt * p.splits, ctx->sm_count);
  k<<<grid, kThreads, smem, st>>>(ta, tb, C, p, ctx->dev_status);
  CTB_CHECK_LAUNCH("ctb_gemm launch");
  if (p.splits > 1) {
    const long long work = nt * kTileM * kTileN / 4;
    const int rgrid = (int)std::min<long long>((work + 255) / 256, (long long)ctx->sm_count * 8);
    gemm_splitk_reduce_kernel<T><<<rgrid, 256, 0, st>>>(p.partial, C, p);
    CTB_CHECK_LAUNCH("ctb_gemm split-K reduction launch");
  }
  return CTB_OK;
}

int gemm_common(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
                int64_t batch, int64_t lda, int64_t ldb, int64_t ldc, int64_t sA, int64_t sB, int64_t sC, int dtype,
                int tm, int tn, int tk, const char* who) {
  CTB_CHECK_CTX(ctx);
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0 || M > INT32_MAX || N > INT32_MAX || K > INT32_MAX || batch > 65535)
    return fail(CTB_BAD_ARG, "%s: bad shape M=%lld N=%lld K=%lld batch=%lld", who, (long long)M, (long long)N,
                (long long)K, (long long)batch);
  if (lda < M || ldb < K || ldc < M) return fail(CTB_BAD_ARG, "%s: leading dimension too small", who);
  if (!is_pow2(tm) || !is_pow2(tn) || !is_pow2(tk))
    return fail(CTB_UNSUPPORTED_TILE, "%s: tile sizes must be powers of two (got %d,%d,%d)", who, tm, tn, tk);
  if (dtype != CTB_F32 && dtype != CTB_F16 && dtype != CTB_BF16)
    return fail(CTB_BAD_ARG, "%s: dtype must be CTB_F32, CTB_F16 or CTB_BF16", who);
  CTB_CHECK_DEV(A); CTB_CHECK_DEV(B); CTB_CHECK_DEV(C);
  const int es = dtype == CTB_F32 ? 4 : 2;
  if ((lda * es) % 16 || (ldb * es) % 16 || (sA * es) % 16 || (sB * es) % 16 || (uintptr_t)A % 16 || (uintptr_t)B % 16)
    return fail(CTB_BAD_ALIGN, "%s: A and B need 16-byte aligned bases, leading dimensions and batch strides (TMA)", who);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CTB_F32)
    return launch<float>(ctx, st, (const float*)A, (const float*)B, (float*)C, (int)M, (int)N, (int)K, (int)batch, lda,
                         ldb, ldc, sA, sB, sC);
  if (dtype == CTB_BF16)
    return launch<__nv_bfloat16>(ctx, st, (const __nv_bfloat16*)A, (const __nv_bfloat16*)B, (__nv_bfloat16*)C, (int)M, (int)N,
                                 (int)K, (int)batch, lda, ldb, ldc, sA, sB, sC);
  return launch<__half>(ctx, st, (const __half*)A, (const __half*)B, (__half*)C, (int)M, (int)N, (int)K, (int)batch,
                        lda, ldb, ldc, sA, sB, sC);
}

}  // namespace

extern "C" {

int ctb_gemm(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, int64_t M, int64_t N, int64_t K,
             int64_t lda, int64_t ldb, int64_t ldc, int dtype, int tm, int tn, int tk) {
  return gemm_common(ctx, stream, A, B, C, M, N, K, 1, lda, ldb, ldc, 0, 0, 0, dtype, tm, tn, tk, "ctb_gemm");
}

int ctb_gemm_batched(ctb_ctx* ctx, void* stream, const void* A, const void* B, void* C, int64_t M, int64_t N,
                     int64_t K, int64_t batch, int64_t lda, int64_t ldb, int64_t ldc, int64_t strideA,
                     int64_t strideB, int64_t strideC, int dtype, int tm, int tn, int tk) {
  if (batch > 1 && (strideA < lda * K || strideB < ldb * N || strideC < ldc * N))
    return fail(CTB_BAD_ARG, "ctb_gemm_batched: batch strides overlap");
  return gemm_common(ctx, stream, A, B, C, M, N, K, batch, lda, ldb, ldc, strideA, strideB, strideC, dtype, tm, tn, tk,
                     "ctb_gemm_batched");
}

}  // extern "C"
