// Flash multi-head attention forward for sm_100a (counterpart of fmha_kernel /
// cutile_fmha, examples/fmha.jl:20-139,146-168): f16 Q/K/V, head dim 64,
// online softmax in f32 (exp2 with the scale folded as qk_scale/ln2, flush to
// zero; scale applied after the row max, :107), P rounded to f16 before P*V
// (:124), approximate final divide (:132-134), causal mask with a query offset
// `input_pos`, ragged K/V length, grouped-query heads.
//
// Persistent CTAs, two per SM (so that one CTA's softmax overlaps the other's
// tensor-core work), each walking a static list of (128-query tile, batch*head)
// work items dealt heaviest first in alternating direction.  Loads of the next
// item (a second Q buffer, the K/V rings) run under the current one.  6 warps:
//   warp 0    TMA producer: Q once, then K and V tiles (128 keys x 64, 128-byte
//             swizzle) through two mbarrier rings;
//   warp 1    MMA issuer (one thread): S = Q*K^T  (tcgen05.mma 128x128x16, both
//             operands K-major in shared memory, S in TMEM columns 0..127);
//             PV = P*V (128x64x16, P read from TMEM columns 128..191 as the A
//             operand, V MN-major in shared memory, result in columns 192..255).
//             S(j+1) is issued as soon as the softmax warps have pulled S(j) into
//             registers, i.e. before P(j) is complete, so the scores of the next
//             tile are normally waiting when softmax(j) ends;
//   warps 2-5 softmax: thread = query row (TMEM lane).  The 128 scores of the row
//             are pulled into registers at once (which frees S), then row max,
//             exp2, row sum, P written back to TMEM as packed f16.  O accumulates in TMEM across
//             tiles; it is rescaled (read, multiplied, written back) only when a
//             row's maximum has grown by more than 2^8 since the exponent
//             reference was last moved, which is exact (P and the row sum use the
//             same reference) and happens at most a few times per row.
// Like the reference (:69-76) the loop stops at the last tile that a causal
// query tile can see, and only tiles from `mask_start` on pay for masking.
#include <math.h>

#include "ctx.h"
#include "ptx.cuh"

using namespace ctb;
using namespace ctb_internal;

namespace {

constexpr int kTM = 128, kTN = 128, kD = 64;
constexpr int kQBufs = 2, kKStages = 2, kVStages = 2;
constexpr int kThreads = 192;
constexpr int kTileBytes = kTN * kD * 2;  // 16 KiB: one Q, K or V tile
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColP = 128, kColO = 192;

struct Params {
  int seq_q, seq_kv, heads, kv_heads, group, batch;
  int input_pos, causal;
  float scale_log2;  // qk_scale / ln 2
  int q_tiles, bh_total, items;
};

// One work item = one (128-query tile, batch*head).  Items are numbered heaviest first (the last query tile of a
// causal problem sees the most keys) and dealt to the persistent CTAs in rounds of alternating direction, so that
// every CTA gets a mix of heavy and light items.
struct Item {
  int bh, q0, kvz, Tc, mask_start;
};
__device__ __forceinline__ bool get_item(const Params& p, int i, Item& it) {
  const int G = gridDim.x, c = blockIdx.x;
  const long long w = (long long)i * G + ((i & 1) ? G - 1 - c : c);
  if (w >= p.items) return false;
  const int qt = p.q_tiles - 1 - (int)(w / p.bh_total);
  it.bh = (int)(w % p.bh_total);
  it.q0 = qt * kTM;
  const int b = it.bh / p.heads, h = it.bh - b * p.heads;
  it.kvz = b * p.kv_heads + h / p.group;
  // loop bounds, examples/fmha.jl:65-76 (0-based tile indices here)
  if (p.causal) {
    it.mask_start = min((p.input_pos + it.q0) / kTN, p.seq_kv / kTN);
    it.Tc = (min(p.input_pos + it.q0 + kTM, p.seq_kv) + kTN - 1) / kTN;
  } else {
    it.Tc = (p.seq_kv + kTN - 1) / kTN;
    it.mask_start = p.seq_kv / kTN;
  }
  return true;
}

__global__ void __launch_bounds__(kThreads, 2)
    fmha_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, __half* __restrict__ Out, const Params p, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem;
  unsigned char* sK = sQ + kQBufs * kTileBytes;
  unsigned char* sV = sK + kKStages * kTileBytes;
  __shared__ __align__(8) uint64_t q_full[kQBufs], q_empty[kQBufs], k_full[kKStages], k_empty[kKStages],
      v_full[kVStages], v_empty[kVStages], s_full, s_free, p_full, o_full, o_free;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < kQBufs; ++s) { mbar_init(&q_full[s], 1); mbar_init(&q_empty[s], 1); }
    for (int s = 0; s < kKStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < kVStages; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    mbar_init(&s_full, 1);
    mbar_init(&s_free, 4);
    mbar_init(&p_full, 4);
    mbar_init(&o_full, 1);
    mbar_init(&o_free, 4);
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_s, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  volatile int* abort = &abort_s;

  // All three roles walk the same item sequence; g counts this CTA's K/V tiles across items and indexes the
  // K/V rings and the parity of the per-tile handshakes.
  if (warp == 0) {
    // ---- TMA producer (whole warp in lock step, one elected lane issues)
    int g = 0;
    Item it;
    for (int i = 0; get_item(p, i, it); ++i) {
      const int qb = i % kQBufs;
      if (!CTB_WARP_WAIT(&q_empty[qb], ((i / kQBufs) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort)) break;
      if (elect_one()) {
        mbar_expect_tx(&q_full[qb], kTileBytes);
        tma_load_3d(sQ + qb * kTileBytes, &tmQ, 0, it.q0, it.bh, &q_full[qb]);
      }
      __syncwarp();
      bool ok = true;
      for (int j = 0; j < it.Tc; ++j, ++g) {
        const int ks = g % kKStages, vs = g % kVStages;
        ok = CTB_WARP_WAIT(&k_empty[ks], ((g / kKStages) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(&k_full[ks], kTileBytes);
          tma_load_3d(sK + ks * kTileBytes, &tmK, 0, j * kTN, it.kvz, &k_full[ks]);
        }
        __syncwarp();
        ok = CTB_WARP_WAIT(&v_empty[vs], ((g / kVStages) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(&v_full[vs], kTileBytes);
          tma_load_3d(sV + vs * kTileBytes, &tmV, 0, j * kTN, it.kvz, &v_full[vs]);
        }
        __syncwarp();
      }
      if (!ok) break;
    }
  } else if (warp == 1) {
    // ---- MMA issuer (whole warp in lock step, one elected lane issues)
    constexpr uint32_t idesc_qk = make_idesc(FMT_F16, kTM, kTN, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(FMT_F16, kTM, kD, 0, /*V is MN-major*/ 1);
    // S = Q*K^T for global tile gt (its K tile has landed, S is free); `last` frees the Q buffer afterwards
    auto issue_qk = [&](int gt, int qb, bool last) {
      tc_fence_after();
      const int ks = gt % kKStages;
      const uint32_t aQ = smem_u32(sQ + qb * kTileBytes), aK = smem_u32(sK + ks * kTileBytes);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < kD / 16; ++k)
          mma_f16_ss(tmem + kColS, make_sdesc_sw128(aQ + k * 32, 0, 1024), make_sdesc_sw128(aK + k * 32, 0, 1024),
                     idesc_qk, k != 0);
        tc_commit(&k_empty[ks]);
        tc_commit(&s_full);
        if (last) tc_commit(&q_empty[qb]);
      }
      __syncwarp();
    };
    int g = 0;
    Item it;
    bool ok = true;
    for (int i = 0; ok && get_item(p, i, it); ++i) {
      const int qb = i % kQBufs;
      ok = CTB_WARP_WAIT(&q_full[qb], (i / kQBufs) & 1, status, DEV_TIMEOUT_TMA, abort) &&
           CTB_WARP_WAIT(&k_full[g % kKStages], (g / kKStages) & 1, status, DEV_TIMEOUT_TMA, abort);
      // the softmax warps have pulled the previous item's last scores out of S
      if (ok && g > 0) ok = CTB_WARP_WAIT(&s_free, (g - 1) & 1, status, DEV_TIMEOUT_SLOT, abort);
      if (!ok) break;
      issue_qk(g, qb, it.Tc == 1);
      for (int j = 0; j < it.Tc; ++j) {
        const int gj = g + j, vs = gj % kVStages;
        if (j + 1 < it.Tc) {
          // S(j) has been read into registers: the next scores can overwrite it while softmax(j) still runs
          ok = CTB_WARP_WAIT(&k_full[(gj + 1) % kKStages], ((gj + 1) / kKStages) & 1, status, DEV_TIMEOUT_TMA, abort) &&
               CTB_WARP_WAIT(&s_free, gj & 1, status, DEV_TIMEOUT_SLOT, abort);
          if (!ok) break;
          issue_qk(gj + 1, qb, j + 2 == it.Tc);
        }
        ok = CTB_WARP_WAIT(&v_full[vs], (gj / kVStages) & 1, status, DEV_TIMEOUT_TMA, abort);
        // the first P*V of an item overwrites O: the previous item's epilogue must have read it
        if (ok && j == 0 && i > 0) ok = CTB_WARP_WAIT(&o_free, (i - 1) & 1, status, DEV_TIMEOUT_SLOT, abort);
        if (ok) ok = CTB_WARP_WAIT(&p_full, gj & 1, status, DEV_TIMEOUT_SLOT, abort);
        if (!ok) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + vs * kTileBytes);
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < kTN / 16; ++k)
            mma_f16_ts(tmem + kColO, tmem + kColP + k * 8, make_sdesc_sw128(aV + k * 2048, 0, 1024), idesc_pv, (j | k) != 0);
          tc_commit(&v_empty[vs]);
          tc_commit(&o_full);
        }
        __syncwarp();
      }
      g += it.Tc;
    }
  } else {
    // ---- softmax + epilogue: thread = query row = TMEM lane
    const int sub = warp & 3;
    const int row = sub * 32 + lane;
    const uint32_t trow = tmem + ((uint32_t)(sub * 32) << 16);
    int g = 0;
    Item it;
    bool ok = true;
    for (int i = 0; ok && get_item(p, i, it); ++i) {
      const int qpos = it.q0 + row + p.input_pos;  // position used by the causal rule
      const int vis_last = p.causal ? min(qpos, p.seq_kv - 1) : p.seq_kv - 1;  // last visible key of this row
      float m_ref = -INFINITY;  // exponent reference (scaled, log2 domain)
      float l = 0.f;            // row sum relative to m_ref
      for (int j = 0; j < it.Tc; ++j) {
        const int gj = g + j;
        ok = CTB_WARP_WAIT(&s_full, gj & 1, status, DEV_TIMEOUT_MMA, abort);
        if (!ok) break;
        tc_fence_after();
        const bool masked = j >= it.mask_start;
        const int lim = vis_last - j * kTN;  // column i of this tile is visible iff i <= lim
        // ---- the whole score row goes to registers in one go; S is then free for the next tile's Q*K^T
        uint32_t sr[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld32(trow + kColS + c * 32, sr[c]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free);
        // ---- row maximum of the raw scores (four independent chains)
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        if (masked) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int k = 0; k < 32; k += 4) {
              mx0 = fmaxf(mx0, c * 32 + k + 0 <= lim ? __uint_as_float(sr[c][k + 0]) : -INFINITY);
              mx1 = fmaxf(mx1, c * 32 + k + 1 <= lim ? __uint_as_float(sr[c][k + 1]) : -INFINITY);
              mx2 = fmaxf(mx2, c * 32 + k + 2 <= lim ? __uint_as_float(sr[c][k + 2]) : -INFINITY);
              mx3 = fmaxf(mx3, c * 32 + k + 3 <= lim ? __uint_as_float(sr[c][k + 3]) : -INFINITY);
            }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int k = 0; k < 32; k += 4) {
              mx0 = fmaxf(mx0, __uint_as_float(sr[c][k + 0]));
              mx1 = fmaxf(mx1, __uint_as_float(sr[c][k + 1]));
              mx2 = fmaxf(mx2, __uint_as_float(sr[c][k + 2]));
              mx3 = fmaxf(mx3, __uint_as_float(sr[c][k + 3]));
            }
        }
        const float m_true = fmaxf(m_ref, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2);
        // ---- move the exponent reference (and rescale O, l) only when the maximum grew by more than 2^8
        const bool grow = m_true - m_ref > 8.0f || m_ref == -INFINITY;
        if (j > 0) {  // PV(j-1) must have consumed P(j-1) (and, for a rescale, landed in O) before P(j) is written
          ok = CTB_WARP_WAIT(&o_full, (gj - 1) & 1, status, DEV_TIMEOUT_MMA, abort);
          if (!ok) break;
          tc_fence_after();
        }
        if (__any_sync(0xffffffffu, grow)) {
          const float m_new = m_true == -INFINITY ? 0.f : m_true;  // fully masked so far: keep everything zero
          const float alpha = ex2_approx_ftz(m_ref - m_new);       // 0 on the first tile
          l *= alpha;
          m_ref = m_new;
          if (j > 0) {  // O holds the sum of the previous tiles
#pragma unroll 1
            for (int c = 0; c < kD / 16; ++c) {
              uint32_t t[16];
              tmem_ld16(trow + kColO + c * 16, t);
              tc_wait_ld();
#pragma unroll
              for (int k = 0; k < 16; ++k) t[k] = __float_as_uint(__uint_as_float(t[k]) * alpha);
              tmem_st16(trow + kColO + c * 16, t);
            }
          }
        }
        // ---- p = exp2(s*scale - m_ref), row sum, P -> TMEM as packed f16
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        const float nm = -m_ref;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
#pragma unroll
          for (int k = 0; k < 32; k += 4) {
            float p0 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c][k + 0]), p.scale_log2, nm));
            float p1 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c][k + 1]), p.scale_log2, nm));
            float p2 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c][k + 2]), p.scale_log2, nm));
            float p3 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c][k + 3]), p.scale_log2, nm));
            if (masked) {
              if (c * 32 + k + 0 > lim) p0 = 0.f;
              if (c * 32 + k + 1 > lim) p1 = 0.f;
              if (c * 32 + k + 2 > lim) p2 = 0.f;
              if (c * 32 + k + 3 > lim) p3 = 0.f;
            }
            s0 += p0; s1 += p1; s2 += p2; s3 += p3;
            pk[(k >> 1) + 0] = pack_f16x2(p0, p1);
            pk[(k >> 1) + 1] = pack_f16x2(p2, p3);
          }
          tmem_st16(trow + kColP + c * 16, pk);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full);
        l += (s0 + s1) + (s2 + s3);
      }
      if (!ok) break;
      g += it.Tc;
      // ---- epilogue of the item: O / l -> f16 -> global, then O is free for the next item
      ok = CTB_WARP_WAIT(&o_full, (g - 1) & 1, status, DEV_TIMEOUT_MMA, abort);
      if (!ok) break;
      tc_fence_after();
      const float inv = rcp_approx_ftz(l);
      const bool store = it.q0 + row < p.seq_q;
      uint4* dst = reinterpret_cast<uint4*>(Out + ((long long)it.bh * p.seq_q + it.q0 + row) * kD);
#pragma unroll
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(trow + kColO + c * 32, r);
        tc_wait_ld();
        if (c == kD / 32 - 1) {  // everything is in registers: the next item may overwrite O
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&o_free);
        }
        if (store) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 v;
            v.x = pack_f16x2(__uint_as_float(r[k * 8 + 0]) * inv, __uint_as_float(r[k * 8 + 1]) * inv);
            v.y = pack_f16x2(__uint_as_float(r[k * 8 + 2]) * inv, __uint_as_float(r[k * 8 + 3]) * inv);
            v.z = pack_f16x2(__uint_as_float(r[k * 8 + 4]) * inv, __uint_as_float(r[k * 8 + 5]) * inv);
            v.w = pack_f16x2(__uint_as_float(r[k * 8 + 6]) * inv, __uint_as_float(r[k * 8 + 7]) * inv);
            dst[c * 4 + k] = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
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
  if (dtype != CTB_F16) return fail(CTB_UNSUPPORTED, "ctb_fmha_fwd: only f16 is implemented");
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
    int r = make_tmap(&tq, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, Q, dims, str, box);
    if (r) return r;
  }
  {
    uint64_t dims[3] = {kD, (uint64_t)seq_kv, (uint64_t)(kv_heads * batch)};
    uint64_t str[2] = {kD * 2, (uint64_t)seq_kv * kD * 2};
    int r = make_tmap(&tk, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, K, dims, str, box);
    if (r) return r;
    r = make_tmap(&tv, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, V, dims, str, box);
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
  const size_t smem = (size_t)(kQBufs + kKStages + kVStages) * kTileBytes + 1024;
  cudaError_t e = cudaFuncSetAttribute(fmha_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_fmha_fwd: shared memory opt-in");
  const int grid = (int)std::min<long long>(items, 2LL * ctx->sm_count);  // two persistent CTAs per SM
  fmha_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, (__half*)Out, p,
                                                                         ctx->dev_status);
  CTB_CHECK_LAUNCH("ctb_fmha_fwd launch");
  return CTB_OK;
}
