// Flash multi-head attention forward for sm_100a (counterpart of fmha_kernel /
// cutile_fmha, examples/fmha.jl:20-139,146-168): f16 Q/K/V, head dim 64,
// online softmax in f32 (exp2 with the scale folded as qk_scale/ln2, flush to
// zero; scale applied after the row max, :107), P rounded to f16 before P*V
// (:124), approximate final divide (:132-134), causal mask with a query offset
// `input_pos`, ragged K/V length, grouped-query heads.  Like the reference (:69-76)
// the loop over K/V tiles stops at the last tile that a causal query tile can see,
// and only tiles from `mask_start` on pay for masking.
//
// One persistent CTA per SM runs TWO independent pipelines ("streams") side by side, each
// working through (128-query tile, batch*head) items.  16 warps:
//   warps 0-3   softmax of stream 0, warps 4-7 softmax of stream 1: thread = query row (TMEM
//               lane).  The 128 scores of the row are pulled into registers at once (which
//               frees S for the next Q*K^T), then row max, exp2, row sum, P written back to
//               TMEM as packed f16.  O accumulates in TMEM across tiles; it is rescaled (read,
//               multiplied, written back) only when a row's maximum has grown by more than 2^8
//               since the exponent reference was last moved, which is exact (P and the row sum
//               use the same reference) and happens at most a few times per row;
//   warps 8-11  epilogue of both streams: O / l -> f16 -> shared memory -> one tiled bulk
//               store per warp, off the softmax warps' path;
//   warps 12/13 TMA producer (Q twice buffered, K and V tiles of 128 keys x 64 through two
//               mbarrier rings, 128-byte swizzle) and MMA issuer of stream 0: S = Q*K^T
//               (tcgen05.mma 128x128x16, both operands K-major in shared memory), O += P*V
//               (128x64x16, P read from TMEM as the A operand, V MN-major in shared memory).
//               S(j+1) is issued as soon as the softmax warps have pulled S(j), also across
//               the end of an item; warps 14/15: the same for stream 1.
// TMEM: stream s owns columns 256 s .. 256 s + 255 (S 128, P 64 packed f16, O 64).
// Register budgets per role via setmaxnreg: softmax 192, the other warps 64.
// Work items are handed out heaviest first (the last query tile of a causal problem sees the
// most keys) from a global counter; a stream asks for its next item while the loads of the
// current item's last two tiles are issued, and publishes it to the other roles through a
// small ring in shared memory.
//
// What bounds the kernel is the exp2 unit: about 14.5 results per clock and SM measured (a
// 128 x 128 score tile costs each of the four schedulers about 1130 clocks when two warps
// share the unit, 1275 for a warp on its own), against 512 clocks of tensor-core time per
// tile.  A polynomial exp2 on the FMA pipe costs more per element than the unit does.
#include <cuda_bf16.h>
#include <math.h>

#include "ctx.h"
#include "ptx.cuh"

using namespace ctb;
using namespace ctb_internal;

namespace {

constexpr int kTM = 128, kTN = 128, kD = 64;
constexpr int kTileBytes = kTN * kD * 2;  // 16 KiB: one Q, K or V tile


// Development aid, compiled in with -DCTB_FMHA_TRACE only: clock64() stamps of the phases of the first score tiles
// of warp 0 of each softmax warpgroup of CTA 0 (read back with ctb_debug_fmha_trace).
#ifdef CTB_FMHA_TRACE
constexpr int kTraceTiles = 48, kTracePoints = 8;
__device__ long long g_trace[2][kTraceTiles][kTracePoints];
#define CTB_TR(k)                                                                                    \
  do {                                                                                               \
    if (blockIdx.x == 0 && w == 0 && lane == 0 && ns < kTraceTiles) g_trace[s][ns][k] = clock64();   \
  } while (0)
#else
#define CTB_TR(k) do { } while (0)
#endif

constexpr int kThreadsD = 512;
constexpr int kRing = 4;
constexpr int kQB = 2, kKS = 2, kVS = 2;                     // Q buffers, K and V stages per stream
constexpr int kStreamBytes = (kQB + kKS + kVS) * kTileBytes;  // 96 KiB
constexpr int kOutStageBytes = kTM * kD * 2;                  // 16 KiB: the epilogue warps' staging rows
constexpr uint32_t kStreamCols = 256, kOffS = 0, kOffP = 128, kOffO = 192;

struct Params {
  int seq_q, seq_kv, heads, kv_heads, group, batch;
  int input_pos, causal;
  float scale_log2;
  int q_tiles, bh_total, items;
  int* sched;  // [0] next item, [1] CTAs that have finished (the last one clears both)
};

struct Item {
  int bh, q0, kvz, Tc, mask_start;
};
__device__ __forceinline__ void decode(const Params& p, int w, Item& it) {
  const int qt = p.q_tiles - 1 - w / p.bh_total;  // heaviest (last query tiles of a causal problem) first
  it.bh = w % p.bh_total;
  it.q0 = qt * kTM;
  const int b = it.bh / p.heads, h = it.bh - b * p.heads;
  it.kvz = b * p.kv_heads + h / p.group;
  if (p.causal) {  // loop bounds of examples/fmha.jl:65-76 (0-based tile indices here)
    it.mask_start = min((p.input_pos + it.q0) / kTN, p.seq_kv / kTN);
    it.Tc = (min(p.input_pos + it.q0 + kTM, p.seq_kv) + kTN - 1) / kTN;
  } else {
    it.Tc = (p.seq_kv + kTN - 1) / kTN;
    it.mask_start = p.seq_kv / kTN;
  }
}

__device__ __forceinline__ float2 ffma2(float a0, float a1, float b, float c) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.ftz.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a0), "f"(a1), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float2 fadd2(float2 a, float b0, float b1) {
  float2 d;
  asm("{\n\t.reg .b64 ra, rb, rd;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.ftz.f32x2 rd, ra, rb;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b0), "f"(b1));
  return d;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
template <int R>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(R));
}
template <int R>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(R));
}

struct __align__(8) SBars {  // barriers of one stream
  uint64_t q_full[kQB], q_empty[kQB], k_full[kKS], k_empty[kKS], v_full[kVS], v_empty[kVS];
  uint64_t s_full, s_free, p_full, o_full, o_final, o_free, l_full, l_empty;
  uint64_t item_full[kRing], item_empty[kRing];
};

// One 32-column chunk of a score row: hidden columns (beyond `lim`) become -inf, then the running maxima.
__device__ __forceinline__ void chunk_max(uint32_t (&v)[32], int c, bool masked, int lim, float& mx0, float& mx1,
                                          float& mx2, float& mx3) {
  if (masked) {
#pragma unroll
    for (int k = 0; k < 32; ++k)
      if (c * 32 + k > lim) v[k] = 0xff800000u;
  }
#pragma unroll
  for (int k = 0; k < 32; k += 8) {
    mx0 = fmax3(mx0, __uint_as_float(v[k + 0]), __uint_as_float(v[k + 1]));
    mx1 = fmax3(mx1, __uint_as_float(v[k + 2]), __uint_as_float(v[k + 3]));
    mx2 = fmax3(mx2, __uint_as_float(v[k + 4]), __uint_as_float(v[k + 5]));
    mx3 = fmax3(mx3, __uint_as_float(v[k + 6]), __uint_as_float(v[k + 7]));
  }
}

// two f32 -> one 32-bit pair of 16-bit floats in the operands' format (round to nearest even)
template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  if constexpr (BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    return pack_f16x2(lo, hi);
  }
}

template <bool BF16>
__global__ void __launch_bounds__(kThreadsD, 1)
    fmha_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO, const Params p,
                     int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ SBars BB[2];
  __shared__ float l_smem[2][kTM];
  __shared__ int ring[2][kRing];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < 2; ++s) {
      SBars& B = BB[s];
      for (int i = 0; i < kQB; ++i) { mbar_init(&B.q_full[i], 1); mbar_init(&B.q_empty[i], 1); }
      for (int i = 0; i < kKS; ++i) { mbar_init(&B.k_full[i], 1); mbar_init(&B.k_empty[i], 1); }
      for (int i = 0; i < kVS; ++i) { mbar_init(&B.v_full[i], 1); mbar_init(&B.v_empty[i], 1); }
      mbar_init(&B.s_full, 1); mbar_init(&B.s_free, 4); mbar_init(&B.p_full, 4);
      mbar_init(&B.o_full, 1); mbar_init(&B.o_final, 1); mbar_init(&B.o_free, 4);
      mbar_init(&B.l_full, 4); mbar_init(&B.l_empty, 4);
      for (int i = 0; i < kRing; ++i) {
        mbar_init(&B.item_full[i], 1);
        mbar_init(&B.item_empty[i], 9);  // MMA warp + 4 softmax warps + 4 epilogue warps
      }
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  if (warp == 13) {
    tmem_alloc(&tmem_base_s, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  volatile int* abort = &abort_s;

  // item n of stream s, as published by its producer warp (>= p.items: the stream has ended)
  auto read_item = [&](int s, int n, bool& ok) -> int {
    const int slot = n % kRing;
    ok = CTB_WARP_WAIT(&BB[s].item_full[slot], (n / kRing) & 1, status, DEV_TIMEOUT_SLOT, abort);
    if (!ok) return p.items;
    const int idx = ring[s][slot];
    __syncwarp();
    if (lane == 0) mbar_arrive(&BB[s].item_empty[slot]);
    return idx;
  };

  if (warp >= 12) {
    reg_dec<64>();
    const int s = (warp - 12) >> 1;
    SBars& B = BB[s];
    unsigned char* sQ = smem + s * kStreamBytes;
    unsigned char* sK = sQ + kQB * kTileBytes;
    unsigned char* sV = sK + kKS * kTileBytes;
    if (((warp - 12) & 1) == 0) {
      // ---- scheduler + TMA producer of stream s (whole warp in lock step, one elected lane issues)
      auto fetch = [&]() -> int {
        int v = 0;
        if (lane == 0) v = atomicAdd(&p.sched[0], 1);
        return __shfl_sync(0xffffffffu, v, 0);
      };
      auto publish = [&](int n, int idx) -> bool {
        const int slot = n % kRing;
        if (!CTB_WARP_WAIT(&B.item_empty[slot], ((n / kRing) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort)) return false;
        if (lane == 0) {
          ring[s][slot] = idx;
          mbar_arrive(&B.item_full[slot]);
        }
        __syncwarp();
        return true;
      };
      // The next item is fetched late, when the loads of the current item's last two tiles are issued: work is
      // handed out heaviest first, and an item claimed early is an item that cannot go to a stream that runs dry.
      // (The other roles ask for item n+1 during the last score tile of item n.)
      int cur = fetch();
      bool ok = publish(0, cur);
      int g = 0;
      for (int n = 0; ok && cur < p.items; ++n) {
        Item it;
        decode(p, cur, it);
        const int qb = n % kQB;
        ok = CTB_WARP_WAIT(&B.q_empty[qb], ((n / kQB) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(&B.q_full[qb], kTileBytes);
          tma_load_3d(sQ + qb * kTileBytes, &tmQ, 0, it.q0, it.bh, &B.q_full[qb]);
        }
        __syncwarp();
        int nxt = p.items;
        for (int j = 0; j < it.Tc; ++j, ++g) {
          if (j == max(0, it.Tc - 2)) {
            nxt = fetch();
            ok = publish(n + 1, nxt);
            if (!ok) break;
          }
          const int ks = g % kKS, vs = g % kVS;
          ok = CTB_WARP_WAIT(&B.k_empty[ks], ((g / kKS) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(&B.k_full[ks], kTileBytes);
            tma_load_3d(sK + ks * kTileBytes, &tmK, 0, j * kTN, it.kvz, &B.k_full[ks]);
          }
          __syncwarp();
          ok = CTB_WARP_WAIT(&B.v_empty[vs], ((g / kVS) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(&B.v_full[vs], kTileBytes);
            tma_load_3d(sV + vs * kTileBytes, &tmV, 0, j * kTN, it.kvz, &B.v_full[vs]);
          }
          __syncwarp();
        }
        cur = nxt;
      }
    } else {
      // ---- MMA issuer of stream s (whole warp in lock step, one elected lane issues)
      constexpr uint32_t kFmt = BF16 ? FMT_BF16 : FMT_F16;
      constexpr uint32_t idesc_qk = make_idesc(kFmt, kTM, kTN, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(kFmt, kTM, kD, 0, /*V is MN-major*/ 1);
      const uint32_t tS = tmem + s * kStreamCols + kOffS, tP = tmem + s * kStreamCols + kOffP,
                     tO = tmem + s * kStreamCols + kOffO;
      bool ok = true;
      // S = Q*K^T for score tile gt of the stream (K tile landed, S free); `last` frees the Q buffer afterwards
      auto issue_qk = [&](int gt, int qb, bool last) {
        tc_fence_after();
        const int ks = gt % kKS;
        const uint32_t aQ = smem_u32(sQ + qb * kTileBytes), aK = smem_u32(sK + ks * kTileBytes);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < kD / 16; ++k)
            mma_f16_ss(tS, make_sdesc_sw128(aQ + k * 32, 0, 1024), make_sdesc_sw128(aK + k * 32, 0, 1024), idesc_qk, k != 0);
          tc_commit(&B.k_empty[ks]);
          tc_commit(&B.s_full);
          if (last) tc_commit(&B.q_empty[qb]);
        }
        __syncwarp();
      };
      int g = 0;
      Item cur, nxt;
      int idx = read_item(s, 0, ok);
      if (ok && idx < p.items) {
        decode(p, idx, cur);
        ok = CTB_WARP_WAIT(&B.q_full[0], 0, status, DEV_TIMEOUT_TMA, abort) &&
             CTB_WARP_WAIT(&B.k_full[0], 0, status, DEV_TIMEOUT_TMA, abort);
        if (ok) issue_qk(0, 0, cur.Tc == 1);
        for (int i = 0; ok; ++i) {
          bool has_next = false;
          const int qb = i % kQB, qn = (i + 1) % kQB;
          for (int j = 0; j < cur.Tc; ++j) {
            const int gj = g + j, vs = gj % kVS;
            const bool in_cur = j + 1 < cur.Tc;
            if (!in_cur) {  // the last tile of the item: which item comes next?
              const int nidx = read_item(s, i + 1, ok);
              if (!ok) break;
              has_next = nidx < p.items;
              if (has_next) decode(p, nidx, nxt);
            }
            if (in_cur || has_next) {
              // the next scores of the stream: S(gj) has been read into registers by then and can be overwritten
              // while softmax(gj) still runs.  At the end of an item they belong to the next item.
              if (!in_cur) ok = CTB_WARP_WAIT(&B.q_full[qn], ((i + 1) / kQB) & 1, status, DEV_TIMEOUT_TMA, abort);
              if (ok) ok = CTB_WARP_WAIT(&B.k_full[(gj + 1) % kKS], ((gj + 1) / kKS) & 1, status, DEV_TIMEOUT_TMA, abort) &&
                           CTB_WARP_WAIT(&B.s_free, gj & 1, status, DEV_TIMEOUT_SLOT, abort);
              if (!ok) break;
              if (in_cur) issue_qk(gj + 1, qb, j + 2 == cur.Tc);
              else issue_qk(gj + 1, qn, nxt.Tc == 1);
            }
            ok = CTB_WARP_WAIT(&B.v_full[vs], (gj / kVS) & 1, status, DEV_TIMEOUT_TMA, abort);
            // the first P*V of an item overwrites O: the epilogue must have read the previous item's
            if (ok && j == 0 && i > 0) ok = CTB_WARP_WAIT(&B.o_free, (i - 1) & 1, status, DEV_TIMEOUT_SLOT, abort);
            if (ok) ok = CTB_WARP_WAIT(&B.p_full, gj & 1, status, DEV_TIMEOUT_SLOT, abort);
            if (!ok) break;
            tc_fence_after();
            const uint32_t aV = smem_u32(sV + vs * kTileBytes);
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < kTN / 16; ++k)
                mma_f16_ts(tO, tP + k * 8, make_sdesc_sw128(aV + k * 2048, 0, 1024), idesc_pv, (j | k) != 0);
              tc_commit(&B.v_empty[vs]);
              tc_commit(&B.o_full);
              if (j == cur.Tc - 1) tc_commit(&B.o_final);
            }
            __syncwarp();
          }
          if (!ok || !has_next) break;
          g += cur.Tc;
          cur = nxt;
        }
      }
    }
  } else if (warp < 8) {
    reg_inc<192>();
    // ---- softmax of stream s: thread = query row = TMEM lane
    const int s = warp >> 2, w = warp & 3;
    SBars& B = BB[s];
    const int row = w * 32 + lane;
    const uint32_t trow = tmem + ((uint32_t)(w * 32) << 16) + s * kStreamCols;
    int ns = 0;  // score tiles of the stream so far
    bool ok = true;
    for (int n_item = 0; ok; ++n_item) {
      const int idx = read_item(s, n_item, ok);
      if (!ok || idx >= p.items) break;
      Item it;
      decode(p, idx, it);
      const int vis_last = p.causal ? min(it.q0 + row + p.input_pos, p.seq_kv - 1) : p.seq_kv - 1;  // last visible key
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < it.Tc; ++j, ++ns) {
        CTB_TR(0);
        ok = CTB_WARP_WAIT(&B.s_full, ns & 1, status, DEV_TIMEOUT_MMA, abort);
        if (!ok) break;
        tc_fence_after();
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(trow + kOffS + c * 32, sr[c]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&B.s_free);  // the next Q*K^T may overwrite S
        CTB_TR(1);
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int c = 0; c < 4; ++c) chunk_max(sr[c], c, j >= it.mask_start, vis_last - j * kTN, mx0, mx1, mx2, mx3);
        // ---- exponent reference: moved (and O, l rescaled) only when the maximum grew by more than 2^8
        const float m_true = fmaxf(m_ref, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2);
        const bool grow = m_true - m_ref > 8.0f || m_ref == -INFINITY;
        CTB_TR(2);
        if (ns > 0) {  // P*V of the previous score tile has read P (and, for a rescale, has landed in O)
          ok = CTB_WARP_WAIT(&B.o_full, (ns - 1) & 1, status, DEV_TIMEOUT_MMA, abort);
          if (!ok) break;
          tc_fence_after();
        }
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = grow ? (m_true == -INFINITY ? 0.f : m_true) : m_ref;
          const float alpha = ex2_approx_ftz(m_ref - m_new);  // 0 on an item's first tile, 1 for rows that keep their reference
          l *= alpha;
          m_ref = m_new;
          if (j > 0) {
#pragma unroll 1
            for (int cc = 0; cc < kD / 16; ++cc) {
              uint32_t o[16];
              tmem_ld16(trow + kOffO + cc * 16, o);
              tc_wait_ld();
#pragma unroll
              for (int k = 0; k < 16; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
              tmem_st16(trow + kOffO + cc * 16, o);
            }
          }
        }
        CTB_TR(3);
        CTB_TR(4);
        float2 a0 = make_float2(0.f, 0.f), a1 = make_float2(0.f, 0.f);
        const float nm = -m_ref;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int k = 0; k < 32; k += 4) {
            const float2 x0 = ffma2(__uint_as_float(sr[c][k + 0]), __uint_as_float(sr[c][k + 1]), p.scale_log2, nm);
            const float2 x1 = ffma2(__uint_as_float(sr[c][k + 2]), __uint_as_float(sr[c][k + 3]), p.scale_log2, nm);
            const float p0 = ex2_approx_ftz(x0.x), p1 = ex2_approx_ftz(x0.y);
            const float p2 = ex2_approx_ftz(x1.x), p3 = ex2_approx_ftz(x1.y);
            a0 = fadd2(a0, p0, p1);
            a1 = fadd2(a1, p2, p3);
            pk[(k >> 1) + 0] = pack16<BF16>(p0, p1);
            pk[(k >> 1) + 1] = pack16<BF16>(p2, p3);
          }
          tmem_st16(trow + kOffP + c * 16, pk);
        }
        CTB_TR(5);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&B.p_full);
        l += (a0.x + a0.y) + (a1.x + a1.y);
        CTB_TR(6);
      }
      if (!ok) break;
      // ---- the item is done: hand the row sums to the epilogue warps
      if (n_item > 0) {
        ok = CTB_WARP_WAIT(&B.l_empty, (n_item - 1) & 1, status, DEV_TIMEOUT_SLOT, abort);
        if (!ok) break;
      }
      l_smem[s][row] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&B.l_full);
    }
  } else {
    reg_dec<64>();
    // ---- epilogue of both streams: O / l -> f16 -> shared memory (this warp's 32 rows, 128-byte swizzle) -> one
    // tiled bulk store per warp; thread = query row.  Whichever stream finishes an item first is served first.
    const int w = warp & 3;
    const int row = w * 32 + lane;
    unsigned char* stage = smem + 2 * kStreamBytes + w * (32 * kD * 2);  // 4 KiB per warp, shared by both streams
    int done[2] = {0, 0};
    int cur[2];
    bool ok = true;
    cur[0] = read_item(0, 0, ok);
    if (ok) cur[1] = read_item(1, 0, ok);
    uint64_t t_idle = globaltimer_ns();
    while (ok && (cur[0] < p.items || cur[1] < p.items)) {
      bool progressed = false;
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        if (!ok || cur[s] >= p.items) continue;
        SBars& B = BB[s];
        if (!__all_sync(0xffffffffu, mbar_try_wait(&B.l_full, done[s] & 1))) continue;
        progressed = true;
        const float l = l_smem[s][row];
        __syncwarp();
        if (lane == 0) mbar_arrive(&B.l_empty);
        ok = CTB_WARP_WAIT1(&B.o_final, done[s] & 1, status, DEV_TIMEOUT_MMA, abort);
        if (!ok) break;
        tc_fence_after();
        Item it;
        decode(p, cur[s], it);
        const float inv = rcp_approx_ftz(l);
        const uint32_t tO = tmem + ((uint32_t)(w * 32) << 16) + s * kStreamCols + kOffO;
        bulk_wait_read<0>();  // the previous store of this warp has read the staging rows
        __syncwarp();
#pragma unroll
        for (int c = 0; c < kD / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tO + c * 32, r);
          tc_wait_ld();
          if (c == kD / 32 - 1) {  // everything is in registers: the next item may overwrite O
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&B.o_free);
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 v;
            v.x = pack16<BF16>(__uint_as_float(r[k * 8 + 0]) * inv, __uint_as_float(r[k * 8 + 1]) * inv);
            v.y = pack16<BF16>(__uint_as_float(r[k * 8 + 2]) * inv, __uint_as_float(r[k * 8 + 3]) * inv);
            v.z = pack16<BF16>(__uint_as_float(r[k * 8 + 4]) * inv, __uint_as_float(r[k * 8 + 5]) * inv);
            v.w = pack16<BF16>(__uint_as_float(r[k * 8 + 6]) * inv, __uint_as_float(r[k * 8 + 7]) * inv);
            // 16-byte chunk c*4+k of row `lane`, at its place in the 128-byte swizzle
            *reinterpret_cast<uint4*>(stage + lane * 128 + (((c * 4 + k) ^ (lane & 7)) << 4)) = v;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && it.q0 + w * 32 < p.seq_q) {  // rows beyond seq_q are clipped by the tensor map
          tma_store_3d(&tmO, stage, 0, it.q0 + w * 32, it.bh);
          bulk_commit();
        }
        ++done[s];
        cur[s] = read_item(s, done[s], ok);
      }
      if (progressed) {
        t_idle = globaltimer_ns();
      } else if (*abort || globaltimer_ns() - t_idle > kWaitLimitNs) {
        if (!*abort) atomicMax(status, DEV_TIMEOUT_SLOT);
        *abort = 1;
        ok = false;
      }
    }
    bulk_wait<0>();  // this warp's output stores are complete
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 13) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
  if (threadIdx.x == 0) {  // the last CTA to get here rearms the scheduler for the next launch
    __threadfence();
    if (atomicAdd(&p.sched[1], 1) == (int)gridDim.x - 1) {
      p.sched[0] = 0;
      p.sched[1] = 0;
      __threadfence();
    }
  }
}

}  // namespace

extern "C" int ctb_fmha_fwd(ctb_ctx* ctx, void* stream, const void* Q, const void* K, const void* V, void* Out,
                            int64_t d_k, int64_t d_v, int64_t seq_q, int64_t seq_kv, int64_t heads, int64_t kv_heads,
                            int64_t batch, float qk_scale, int32_t input_pos, int tile_m, int tile_n,
                            int query_group_size, int causal, int dtype) {
  CTB_CHECK_CTX(ctx);
  if (seq_q <= 0 || seq_kv <= 0 || heads <= 0 || kv_heads <= 0 || batch <= 0 || query_group_size <= 0)
    return fail(CTB_BAD_ARG, "ctb_fmha_fwd: non-positive dimension");
  if (heads != kv_heads * query_group_size)
    return fail(CTB_BAD_ARG, "ctb_fmha_fwd: heads (%lld) != kv_heads (%lld) * query_group_size (%d)", (long long)heads,
                (long long)kv_heads, query_group_size);
  if (!is_pow2(tile_m) || !is_pow2(tile_n))
    return fail(CTB_UNSUPPORTED_TILE, "ctb_fmha_fwd: tile_m/tile_n must be powers of two");
  if (dtype != CTB_F16 && dtype != CTB_BF16) return fail(CTB_UNSUPPORTED, "ctb_fmha_fwd: f16 and bf16 are implemented");
  const CUtensorMapDataType tdt = dtype == CTB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (d_k != kD || d_v != kD) return fail(CTB_UNSUPPORTED, "ctb_fmha_fwd: only head dimension 64 is implemented");
  if (input_pos < 0) return fail(CTB_BAD_ARG, "ctb_fmha_fwd: negative input_pos");
  if (seq_q > (1 << 24) || seq_kv > (1 << 24) || heads * batch > 65535 * 64)
    return fail(CTB_UNSUPPORTED, "ctb_fmha_fwd: shape too large");
  CTB_CHECK_DEV(Q); CTB_CHECK_DEV(K); CTB_CHECK_DEV(V); CTB_CHECK_DEV(Out);
  if ((uintptr_t)Q % 16 || (uintptr_t)K % 16 || (uintptr_t)V % 16 || (uintptr_t)Out % 16)
    return fail(CTB_BAD_ALIGN, "ctb_fmha_fwd: Q, K, V, Out must be 16-byte aligned");

  CUtensorMap tq, tk, tv;
  const uint32_t box[3] = {kD, kTN, 1};
  {
    uint64_t dims[3] = {kD, (uint64_t)seq_q, (uint64_t)(heads * batch)};
    uint64_t str[2] = {kD * 2, (uint64_t)seq_q * kD * 2};
    int r = make_tmap(&tq, tdt, 3, Q, dims, str, box);
    if (r) return r;
  }
  {
    uint64_t dims[3] = {kD, (uint64_t)seq_kv, (uint64_t)(kv_heads * batch)};
    uint64_t str[2] = {kD * 2, (uint64_t)seq_kv * kD * 2};
    int r = make_tmap(&tk, tdt, 3, K, dims, str, box);
    if (r) return r;
    r = make_tmap(&tv, tdt, 3, V, dims, str, box);
    if (r) return r;
  }
  Params p;
  p.seq_q = (int)seq_q; p.seq_kv = (int)seq_kv; p.heads = (int)heads; p.kv_heads = (int)kv_heads;
  p.group = query_group_size; p.batch = (int)batch; p.input_pos = input_pos; p.causal = causal ? 1 : 0;
  p.scale_log2 = qk_scale * 1.4426950408889634f;
  p.q_tiles = (int)((seq_q + kTM - 1) / kTM);
  p.bh_total = (int)(heads * batch);
  const long long items = (long long)p.q_tiles * p.bh_total;
  if (items > INT32_MAX) return fail(CTB_UNSUPPORTED, "ctb_fmha_fwd: too many work items");
  p.items = (int)items;
  p.sched = sched_slot(ctx);
  CUtensorMap to;  // output rows leave 32 at a time (one epilogue warp's share of a query tile)
  {
    const uint32_t obox[3] = {kD, 32, 1};
    uint64_t dims[3] = {kD, (uint64_t)seq_q, (uint64_t)(heads * batch)};
    uint64_t str[2] = {kD * 2, (uint64_t)seq_q * kD * 2};
    int r = make_tmap(&to, tdt, 3, Out, dims, str, obox);
    if (r) return r;
  }
  const size_t smem = (size_t)2 * kStreamBytes + kOutStageBytes + 1024;
  const int grid = std::min((p.items + 1) / 2, ctx->sm_count);  // one persistent CTA per SM, two streams each
  auto kern = dtype == CTB_BF16 ? fmha_kernel<true> : fmha_kernel<false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_fmha_fwd: shared memory opt-in");
  kern<<<grid, kThreadsD, smem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, to, p, ctx->dev_status);
  CTB_CHECK_LAUNCH("ctb_fmha_fwd launch");
  return CTB_OK;
}

#ifdef CTB_FMHA_TRACE
// Copies the phase stamps of the last launch to the host: [2 tiles][48 score tiles][8 points] of int64.
extern "C" int ctb_debug_fmha_trace(long long* host) {
  cudaError_t e = cudaMemcpyFromSymbol(host, g_trace, sizeof(g_trace));
  return e == cudaSuccess ? CTB_OK : cuda_fail(e, "ctb_debug_fmha_trace");
}
#endif
