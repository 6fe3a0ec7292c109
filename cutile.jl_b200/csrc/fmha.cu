// Flash multi-head attention forward for sm_100a (counterpart of fmha_kernel /
// cutile_fmha, examples/fmha.jl:20-139,146-168): f16 Q/K/V, head dim 64,
// online softmax in f32 (exp2 with the scale folded as qk_scale/ln2, flush to
// zero; scale applied after the row max, :107), P rounded to f16 before P*V
// (:124), approximate final divide (:132-134), causal mask with a query offset
// `input_pos`, ragged K/V length, grouped-query heads.
//
// One CTA per (128-query tile, batch*head), two CTAs resident per SM so that one
// CTA's softmax overlaps the other's tensor-core work.  6 warps:
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
// Heavier (later) query tiles are scheduled first.
#include <math.h>

#include "ctx.h"
#include "ptx.cuh"

using namespace ctb;
using namespace ctb_internal;

namespace {

constexpr int kTM = 128, kTN = 128, kD = 64;
constexpr int kKStages = 3, kVStages = 2;
constexpr int kThreads = 192;
constexpr int kTileBytes = kTN * kD * 2;  // 16 KiB: one Q, K or V tile
constexpr uint32_t kTmemCols = 256;
constexpr uint32_t kColS = 0, kColP = 128, kColO = 192;

struct Params {
  int seq_q, seq_kv, heads, kv_heads, group, batch;
  int input_pos, causal;
  float scale_log2;  // qk_scale / ln 2
  int q_tiles;
};

__global__ void __launch_bounds__(kThreads, 2)
    fmha_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, __half* __restrict__ Out, const Params p, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem;
  unsigned char* sK = smem + kTileBytes;
  unsigned char* sV = sK + kKStages * kTileBytes;
  __shared__ __align__(8) uint64_t q_full, k_full[kKStages], k_empty[kKStages], v_full[kVStages], v_empty[kVStages],
      s_full, s_free, p_full, o_full;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x;                           // batch*heads + head
  const int qt = p.q_tiles - 1 - (int)blockIdx.y;      // heavy tiles first
  const int b = bh / p.heads, h = bh - b * p.heads;
  const int kvh = h / p.group;
  const int q0 = qt * kTM;

  // loop bounds, examples/fmha.jl:65-76 (0-based tile indices here)
  int Tc, mask_start;
  if (p.causal) {
    mask_start = min((p.input_pos + q0) / kTN, p.seq_kv / kTN);
    const int m_end = p.input_pos + q0 + kTM;
    Tc = (min(m_end, p.seq_kv) + kTN - 1) / kTN;
  } else {
    Tc = (p.seq_kv + kTN - 1) / kTN;
    mask_start = p.seq_kv / kTN;
  }

  if (threadIdx.x == 0) {
    abort_s = 0;
    mbar_init(&q_full, 1);
    for (int s = 0; s < kKStages; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
    for (int s = 0; s < kVStages; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
    mbar_init(&s_full, 1);
    mbar_init(&s_free, 4);
    mbar_init(&p_full, 4);
    mbar_init(&o_full, 1);
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

  if (warp == 0) {
    // ---- TMA producer (whole warp in lock step, one elected lane issues)
    if (elect_one()) {
      mbar_expect_tx(&q_full, kTileBytes);
      tma_load_3d(sQ, &tmQ, 0, q0, bh, &q_full);
    }
    __syncwarp();
    const int kvz = b * p.kv_heads + kvh;
    for (int j = 0; j < Tc; ++j) {
      const int ks = j % kKStages, vs = j % kVStages;
      if (!CTB_WARP_WAIT(&k_empty[ks], ((j / kKStages) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort)) break;
      if (elect_one()) {
        mbar_expect_tx(&k_full[ks], kTileBytes);
        tma_load_3d(sK + ks * kTileBytes, &tmK, 0, j * kTN, kvz, &k_full[ks]);
      }
      __syncwarp();
      if (!CTB_WARP_WAIT(&v_empty[vs], ((j / kVStages) & 1) ^ 1, status, DEV_TIMEOUT_SLOT, abort)) break;
      if (elect_one()) {
        mbar_expect_tx(&v_full[vs], kTileBytes);
        tma_load_3d(sV + vs * kTileBytes, &tmV, 0, j * kTN, kvz, &v_full[vs]);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---- MMA issuer (whole warp in lock step, one elected lane issues)
    constexpr uint32_t idesc_qk = make_idesc(FMT_F16, kTM, kTN, 0, 0);
    constexpr uint32_t idesc_pv = make_idesc(FMT_F16, kTM, kD, 0, /*V is MN-major*/ 1);
    const uint32_t aQ = smem_u32(sQ);
    auto issue_qk = [&](int j) -> bool {
      const int ks = j % kKStages;
      if (j == 0 && !CTB_WARP_WAIT(&k_full[ks], 0, status, DEV_TIMEOUT_TMA, abort)) return false;  // later tiles: caller waited
      tc_fence_after();
      const uint32_t aK = smem_u32(sK + ks * kTileBytes);
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < kD / 16; ++k)
          mma_f16_ss(tmem + kColS, make_sdesc_sw128(aQ + k * 32, 0, 1024), make_sdesc_sw128(aK + k * 32, 0, 1024),
                     idesc_qk, k != 0);
        tc_commit(&k_empty[ks]);
        tc_commit(&s_full);
      }
      __syncwarp();
      return true;
    };
    bool ok = CTB_WARP_WAIT(&q_full, 0, status, DEV_TIMEOUT_TMA, abort);
    if (ok) ok = issue_qk(0);
    for (int j = 0; ok && j < Tc; ++j) {
      const int vs = j % kVStages;
      // S(j) has been read into registers: the next scores can overwrite it while softmax(j) still runs
      if (j + 1 < Tc) {
        const int ks = (j + 1) % kKStages;  // the K tile landed long ago: take that wait off the critical path
        if (!CTB_WARP_WAIT(&k_full[ks], ((j + 1) / kKStages) & 1, status, DEV_TIMEOUT_TMA, abort)) break;
        if (!CTB_WARP_WAIT(&s_free, j & 1, status, DEV_TIMEOUT_SLOT, abort)) break;
        ok = issue_qk(j + 1);
        if (!ok) break;
      }
      if (!CTB_WARP_WAIT(&v_full[vs], (j / kVStages) & 1, status, DEV_TIMEOUT_TMA, abort)) break;
      if (!CTB_WARP_WAIT(&p_full, j & 1, status, DEV_TIMEOUT_SLOT, abort)) break;
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
  } else {
    const int sub = warp & 3;
    const int row = sub * 32 + lane;          // query row inside the tile = TMEM lane
    const int qpos = q0 + row + p.input_pos;  // position used by the causal rule
    const uint32_t trow = tmem + ((uint32_t)(sub * 32) << 16);
    const int vis_last = p.causal ? min(qpos, p.seq_kv - 1) : p.seq_kv - 1;  // last visible key of this row
    float m_ref = -INFINITY;  // exponent reference (scaled, log2 domain)
    float l = 0.f;            // row sum relative to m_ref
    bool ok = true;
    for (int j = 0; j < Tc; ++j) {
      ok = mbar_wait(&s_full, j & 1, status, DEV_TIMEOUT_MMA, abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const bool masked = j >= mask_start;
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
          for (int i = 0; i < 32; i += 4) {
            mx0 = fmaxf(mx0, c * 32 + i + 0 <= lim ? __uint_as_float(sr[c][i + 0]) : -INFINITY);
            mx1 = fmaxf(mx1, c * 32 + i + 1 <= lim ? __uint_as_float(sr[c][i + 1]) : -INFINITY);
            mx2 = fmaxf(mx2, c * 32 + i + 2 <= lim ? __uint_as_float(sr[c][i + 2]) : -INFINITY);
            mx3 = fmaxf(mx3, c * 32 + i + 3 <= lim ? __uint_as_float(sr[c][i + 3]) : -INFINITY);
          }
      } else {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            mx0 = fmaxf(mx0, __uint_as_float(sr[c][i + 0]));
            mx1 = fmaxf(mx1, __uint_as_float(sr[c][i + 1]));
            mx2 = fmaxf(mx2, __uint_as_float(sr[c][i + 2]));
            mx3 = fmaxf(mx3, __uint_as_float(sr[c][i + 3]));
          }
      }
      const float m_true = fmaxf(m_ref, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2);
      // ---- move the exponent reference (and rescale O, l) only when the maximum grew by more than 2^8
      const bool grow = m_true - m_ref > 8.0f || m_ref == -INFINITY;
      if (j > 0) {  // PV(j-1) must have consumed P(j-1) (and, for a rescale, landed in O) before P(j) is written
        ok = mbar_wait(&o_full, (j - 1) & 1, status, DEV_TIMEOUT_MMA, abort);
        ok = __all_sync(0xffffffffu, ok);
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
            for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
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
        for (int i = 0; i < 32; i += 4) {
          float p0 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c][i + 0]), p.scale_log2, nm));
          float p1 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c][i + 1]), p.scale_log2, nm));
          float p2 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c][i + 2]), p.scale_log2, nm));
          float p3 = ex2_approx_ftz(fmaf(__uint_as_float(sr[c][i + 3]), p.scale_log2, nm));
          if (masked) {
            if (c * 32 + i + 0 > lim) p0 = 0.f;
            if (c * 32 + i + 1 > lim) p1 = 0.f;
            if (c * 32 + i + 2 > lim) p2 = 0.f;
            if (c * 32 + i + 3 > lim) p3 = 0.f;
          }
          s0 += p0; s1 += p1; s2 += p2; s3 += p3;
          pk[(i >> 1) + 0] = pack_f16x2(p0, p1);
          pk[(i >> 1) + 1] = pack_f16x2(p2, p3);
        }
        tmem_st16(trow + kColP + c * 16, pk);
      }
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
      l += (s0 + s1) + (s2 + s3);
    }
    if (ok) {
      ok = mbar_wait(&o_full, (Tc - 1) & 1, status, DEV_TIMEOUT_MMA, abort);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      const float inv = rcp_approx_ftz(l);
      const bool store = q0 + row < p.seq_q;
      uint4* dst = reinterpret_cast<uint4*>(Out + ((long long)bh * p.seq_q + q0 + row) * kD);
#pragma unroll
      for (int c = 0; c < kD / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(trow + kColO + c * 32, r);
        tc_wait_ld();
        if (store) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_f16x2(__uint_as_float(r[i * 8 + 0]) * inv, __uint_as_float(r[i * 8 + 1]) * inv);
            v.y = pack_f16x2(__uint_as_float(r[i * 8 + 2]) * inv, __uint_as_float(r[i * 8 + 3]) * inv);
            v.z = pack_f16x2(__uint_as_float(r[i * 8 + 4]) * inv, __uint_as_float(r[i * 8 + 5]) * inv);
            v.w = pack_f16x2(__uint_as_float(r[i * 8 + 6]) * inv, __uint_as_float(r[i * 8 + 7]) * inv);
            dst[c * 4 + i] = v;
          }
        }
      }
      tc_fence_before();
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
  const size_t smem = (size_t)(1 + kKStages + kVStages) * kTileBytes + 1024;
  cudaError_t e = cudaFuncSetAttribute(fmha_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_fmha_fwd: shared memory opt-in");
  dim3 grid((unsigned)(heads * batch), (unsigned)p.q_tiles);
  fmha_kernel<<<grid, kThreads, smem, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, (__half*)Out, p,
                                                                         ctx->dev_status);
  CTB_CHECK_LAUNCH("ctb_fmha_fwd launch");
  return CTB_OK;
}
