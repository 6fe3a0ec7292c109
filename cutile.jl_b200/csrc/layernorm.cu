// LayerNorm forward and backward for sm_100a.  All three kernels are HBM-bound.
//
// forward (counterpart of layer_norm_fwd, examples/layernorm.jl:27-68):
//   persistent CTAs; each row comes into a ring of shared-memory stages by one
//   bulk async copy, lives in registers for mean, variance of the centred
//   values (the reference's two-pass formula, :45-54) and
//   y = (x-mean)*rstd*w+b, and leaves through a bulk store.
//   Algorithmic bytes: 2*M*N*4 + 2*N*4 + 2*M*4.
// backward (layer_norm_bwd_dx_partial_dwdb, :118-171): rows of X and dY are
//   staged into shared memory by bulk async copies, dX leaves through a bulk
//   store, and dW/dB accumulate in registers.  The reference serialises the
//   partial dW/dB update behind a CAS spin-lock per group (:154-167); here a
//   thread-block cluster owns each group column of the (N, GROUP_SIZE_M)
//   partial buffers: its CTAs split the group's rows, exchange their register
//   partials through distributed shared memory and write the column once, in a
//   fixed order, so the result is deterministic and needs neither locks nor a
//   zero-fill.  Algorithmic bytes: 3*M*N*4 + 3*N*4 + 2*M*4.
// final reduce (layer_norm_bwd_dwdb, :186-205): column sums of the partials.
#include <cooperative_groups.h>

#include <algorithm>
#include <mutex>

#include "ctx.h"
#include "ptx.cuh"

namespace cg = cooperative_groups;
using namespace ctb;
using namespace ctb_internal;

namespace {

// ------------------------------------------------------------------- forward
constexpr int kFwdThreads = 256;

template <int NW>
__device__ __forceinline__ float block_sum1(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < NW; ++i) r += red[i];
  __syncthreads();
  return r;
}

// Fast path: N % 4 == 0, 16-byte aligned rows, N <= 4*kFwdThreads*NV.  Two-pass variance on centred values as the
// reference (examples/layernorm.jl:45-54); W and B stay in registers across the CTA's rows.
// Rows are moved by the bulk-copy engine: persistent CTAs, each row comes into a ring of
// shared-memory stages by one cp.async.bulk (mbarrier completion), is normalised in registers, written back into its
// stage and leaves by one bulk copy shared -> global, so the loads and stores of neighbouring rows run under the
// arithmetic of the current one and no thread waits on its own global loads.
constexpr int kFwdStages = 3;
template <int NV>
__global__ void __launch_bounds__(kFwdThreads)
    ln_fwd_staged_kernel(const float* __restrict__ X, const float* __restrict__ W, const float* __restrict__ B,
                         float* __restrict__ Y, float* __restrict__ Mean, float* __restrict__ Rstd, int N, int M,
                         long long ldx, long long ldy, float eps, int stage_bytes, int* status) {
  extern __shared__ __align__(128) unsigned char lsm[];
  __shared__ __align__(8) uint64_t full[kFwdStages];
  __shared__ float red[kFwdThreads / 32];
  const int tid = threadIdx.x;
  const int npack = N >> 2;
  const uint32_t row_bytes = (uint32_t)N * 4u;
  if (tid == 0) {
    for (int s = 0; s < kFwdStages; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  const int first = blockIdx.x, step = gridDim.x;
  const int nrows = first < M ? (M - first + step - 1) / step : 0;
  if (tid == 0) {
    for (int i = 0; i < kFwdStages && i < nrows; ++i) {
      mbar_expect_tx(&full[i], row_bytes);
      bulk_g2s(lsm + (size_t)i * stage_bytes, X + (long long)(first + i * step) * ldx, row_bytes, &full[i]);
    }
  }
  float4 w[NV], b[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int p = tid + v * kFwdThreads;
    if (p < npack) {
      w[v] = reinterpret_cast<const float4*>(W)[p];
      b[v] = reinterpret_cast<const float4*>(B)[p];
    }
  }
  const float fn = (float)N;
  bool alive = true;
  for (int i = 0; i < nrows && alive; ++i) {
    const int s = i % kFwdStages;
    const int row = first + i * step;
    float4* buf = reinterpret_cast<float4*>(lsm + (size_t)s * stage_bytes);
    if (!mbar_wait(&full[s], (i / kFwdStages) & 1, status, DEV_TIMEOUT_TMA)) alive = false;
    alive = __syncthreads_and(alive);
    if (!alive) break;
    float4 x[NV];
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int p = tid + v * kFwdThreads;
      if (p < npack) {
        x[v] = buf[p];
        sum += (x[v].x + x[v].y) + (x[v].z + x[v].w);
      }
    }
    const float mean = block_sum1<kFwdThreads / 32>(sum, red) / fn;
    float q = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      if (tid + v * kFwdThreads < npack) {
        x[v].x -= mean; x[v].y -= mean; x[v].z -= mean; x[v].w -= mean;
        q += (x[v].x * x[v].x + x[v].y * x[v].y) + (x[v].z * x[v].z + x[v].w * x[v].w);
      }
    }
    const float var = block_sum1<kFwdThreads / 32>(q, red) / fn;
    const float rstd = 1.0f / sqrtf(var + eps);
    if (tid == 0) {
      Mean[row] = mean;
      Rstd[row] = rstd;
    }
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int p = tid + v * kFwdThreads;
      if (p < npack) {
        float4 y;
        y.x = x[v].x * rstd * w[v].x + b[v].x;
        y.y = x[v].y * rstd * w[v].y + b[v].y;
        y.z = x[v].z * rstd * w[v].z + b[v].z;
        y.w = x[v].w * rstd * w[v].w + b[v].w;
        buf[p] = y;
      }
    }
    fence_proxy_async_smem();  // generic-proxy writes -> visible to the bulk store
    __syncthreads();
    if (tid == 0) {
      bulk_s2g(Y + (long long)row * ldy, buf, row_bytes);
      bulk_commit();
      // refill the stage of the PREVIOUS row: its store was committed one iteration ago
      const int nxt = i - 1 + kFwdStages;
      if (i >= 1 && nxt < nrows) {
        bulk_wait_read<1>();
        const int ps = (i - 1) % kFwdStages;
        mbar_expect_tx(&full[ps], row_bytes);
        bulk_g2s(lsm + (size_t)ps * stage_bytes, X + (long long)(first + nxt * step) * ldx, row_bytes, &full[ps]);
      }
    }
  }
  if (tid == 0) bulk_wait<0>();  // stores complete before the CTA (and its shared memory) goes away
}

// Any N, any alignment: three passes over the row (the later ones hit L1/L2).
__global__ void __launch_bounds__(kFwdThreads) ln_fwd_generic_kernel(const float* __restrict__ X,
                                                                     const float* __restrict__ W,
                                                                     const float* __restrict__ B, float* __restrict__ Y,
                                                                     float* __restrict__ Mean, float* __restrict__ Rstd,
                                                                     int N, int M, long long ldx, long long ldy,
                                                                     float eps) {
  __shared__ float red[kFwdThreads / 32];
  const int tid = threadIdx.x;
  const float fn = (float)N;
  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const float* src = X + (long long)row * ldx;
    float* dst = Y + (long long)row * ldy;
    float s = 0.f;
    for (int i = tid; i < N; i += kFwdThreads) s += src[i];
    const float mean = block_sum1<kFwdThreads / 32>(s, red) / fn;
    float q = 0.f;
    for (int i = tid; i < N; i += kFwdThreads) {
      const float c = src[i] - mean;
      q += c * c;
    }
    const float var = block_sum1<kFwdThreads / 32>(q, red) / fn;
    const float rstd = 1.0f / sqrtf(var + eps);
    if (tid == 0) {
      Mean[row] = mean;
      Rstd[row] = rstd;
    }
    for (int i = tid; i < N; i += kFwdThreads) dst[i] = (src[i] - mean) * rstd * W[i] + B[i];
  }
}

// ------------------------------------------------------------------ backward
constexpr int kBwdThreads = 512;
constexpr int kBwdWarps = kBwdThreads / 32;
constexpr int kBwdStages = 3;

// Fast path.  Grid = group_size_m * C CTAs in clusters of C; cluster g owns
// partial column g; CTA rank r of the cluster takes rows g + G*(r + C*j).
// Shared memory: kBwdStages stages of [x row | dy row]; dX overwrites the x row.
template <int NV>
__global__ void __launch_bounds__(kBwdThreads)
    ln_bwd_kernel(float* __restrict__ DX, const float* __restrict__ DY, float* __restrict__ DW, float* __restrict__ DB,
                  const float* __restrict__ X, const float* __restrict__ W, const float* __restrict__ Mean,
                  const float* __restrict__ Rstd, int N, int M, long long ldx, long long lddy, long long lddx, int G,
                  int row_stride_bytes, int* status) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[kBwdStages];
  __shared__ float red[2][kBwdWarps];
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int g = blockIdx.x / C;
  const int tid = threadIdx.x;
  const int npack = N >> 2;
  const uint32_t row_bytes = (uint32_t)N * 4u;
  const int stage_bytes = 2 * row_stride_bytes;
  const float inv_n = 1.0f / (float)N;

  if (tid == 0) {
    for (int s = 0; s < kBwdStages; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();

  const int first = g + G * rank, step = G * C;
  const int nrows = first < M ? (M - first + step - 1) / step : 0;
  auto issue = [&](int i, int s) {
    const long long row = first + (long long)i * step;
    unsigned char* base = smem + (size_t)s * stage_bytes;
    mbar_expect_tx(&full[s], 2 * row_bytes);
    bulk_g2s(base, X + row * ldx, row_bytes, &full[s]);
    bulk_g2s(base + row_stride_bytes, DY + row * lddy, row_bytes, &full[s]);
  };
  if (tid == 0)
    for (int i = 0; i < kBwdStages && i < nrows; ++i) issue(i, i);

  float4 w[NV], dw[NV], db[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int p = tid + v * kBwdThreads;
    w[v] = p < npack ? reinterpret_cast<const float4*>(W)[p] : make_float4(0.f, 0.f, 0.f, 0.f);
    dw[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    db[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  }

  float mean = 0.f, rstd = 0.f;
  if (nrows > 0) {
    mean = Mean[first];
    rstd = Rstd[first];
  }
  bool alive = true;
  for (int i = 0; i < nrows; ++i) {
    const int s = i % kBwdStages;
    const long long row = first + (long long)i * step;
    float mean_next = 0.f, rstd_next = 0.f;
    if (i + 1 < nrows) {  // issued before the wait so the latency is hidden behind it
      mean_next = Mean[row + step];
      rstd_next = Rstd[row + step];
    }
    if (!mbar_wait(&full[s], (i / kBwdStages) & 1, status, DEV_TIMEOUT_TMA)) alive = false;
    alive = __syncthreads_and(alive);
    if (!alive) break;
    float4* xs = reinterpret_cast<float4*>(smem + (size_t)s * stage_bytes);
    const float4* dys = reinterpret_cast<const float4*>(smem + (size_t)s * stage_bytes + row_stride_bytes);

    float4 xh[NV], dy[NV];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int p = tid + v * kBwdThreads;
      if (p < npack) {
        const float4 x = xs[p];
        dy[v] = dys[p];
        xh[v].x = (x.x - mean) * rstd; xh[v].y = (x.y - mean) * rstd;
        xh[v].z = (x.z - mean) * rstd; xh[v].w = (x.w - mean) * rstd;
        const float a0 = w[v].x * dy[v].x, a1 = w[v].y * dy[v].y, a2 = w[v].z * dy[v].z, a3 = w[v].w * dy[v].w;
        c1 += (xh[v].x * a0 + xh[v].y * a1) + (xh[v].z * a2 + xh[v].w * a3);
        c2 += (a0 + a1) + (a2 + a3);
      }
    }
    c1 = warp_sum(c1);
    c2 = warp_sum(c2);
    if ((tid & 31) == 0) {
      red[0][tid >> 5] = c1;
      red[1][tid >> 5] = c2;
    }
    __syncthreads();
    c1 = 0.f;
    c2 = 0.f;
#pragma unroll
    for (int k = 0; k < kBwdWarps; ++k) {
      c1 += red[0][k];
      c2 += red[1][k];
    }
    c1 *= inv_n;
    c2 *= inv_n;
#pragma unroll
    for (int v = 0; v < NV; ++v) {
      const int p = tid + v * kBwdThreads;
      if (p < npack) {
        float4 dx;
        dx.x = (w[v].x * dy[v].x - (xh[v].x * c1 + c2)) * rstd;
        dx.y = (w[v].y * dy[v].y - (xh[v].y * c1 + c2)) * rstd;
        dx.z = (w[v].z * dy[v].z - (xh[v].z * c1 + c2)) * rstd;
        dx.w = (w[v].w * dy[v].w - (xh[v].w * c1 + c2)) * rstd;
        xs[p] = dx;
        dw[v].x += dy[v].x * xh[v].x; dw[v].y += dy[v].y * xh[v].y;
        dw[v].z += dy[v].z * xh[v].z; dw[v].w += dy[v].w * xh[v].w;
        db[v].x += dy[v].x; db[v].y += dy[v].y; db[v].z += dy[v].z; db[v].w += dy[v].w;
      }
    }
    fence_proxy_async_smem();
    __syncthreads();  // also orders this row's reads of red[] before the next row's writes
    if (tid == 0) {
      bulk_s2g(DX + row * lddx, xs, row_bytes);
      bulk_commit();
      const int nxt = i - 1 + kBwdStages;
      if (i >= 1 && nxt < nrows) {
        bulk_wait_read<1>();
        issue(nxt, (i - 1) % kBwdStages);
      }
    }
    mean = mean_next;
    rstd = rstd_next;
  }

  // Exchange the register partials through (distributed) shared memory.
  if (tid == 0) bulk_wait_read<0>();
  __syncthreads();
  float4* sdw = reinterpret_cast<float4*>(smem);
  float4* sdb = reinterpret_cast<float4*>(smem + row_stride_bytes);
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int p = tid + v * kBwdThreads;
    if (p < npack) {
      sdw[p] = dw[v];
      sdb[p] = db[v];
    }
  }
  cluster.sync();
  if (alive) {
    const int per = (npack + C - 1) / C;
    const int lo = rank * per, hi = min(npack, lo + per);
    for (int p = lo + tid; p < hi; p += kBwdThreads) {
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      for (int k = 0; k < C; ++k) {  // ascending rank: fixed summation order
        const float4 u = cluster.map_shared_rank(sdw, k)[p];
        const float4 t = cluster.map_shared_rank(sdb, k)[p];
        a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
        b.x += t.x; b.y += t.y; b.z += t.z; b.w += t.w;
      }
      reinterpret_cast<float4*>(DW + (long long)g * N)[p] = a;
      reinterpret_cast<float4*>(DB + (long long)g * N)[p] = b;
    }
  }
  cluster.sync();  // peers may still be reading this CTA's shared memory
  if (tid == 0) bulk_wait<0>();
}

// Any N <= kBwdThreads*kGenCols, any alignment: one CTA per group, scalar accesses.
constexpr int kGenCols = 16;
__global__ void __launch_bounds__(kBwdThreads)
    ln_bwd_generic_kernel(float* __restrict__ DX, const float* __restrict__ DY, float* __restrict__ DW,
                          float* __restrict__ DB, const float* __restrict__ X, const float* __restrict__ W,
                          const float* __restrict__ Mean, const float* __restrict__ Rstd, int N, int M, long long ldx,
                          long long lddy, long long lddx, int G) {
  __shared__ float red[2][kBwdWarps];
  const int tid = threadIdx.x, g = blockIdx.x;
  const float inv_n = 1.0f / (float)N;
  float dw[kGenCols], db[kGenCols];
#pragma unroll
  for (int k = 0; k < kGenCols; ++k) dw[k] = db[k] = 0.f;
  for (long long row = g; row < M; row += G) {
    const float mean = Mean[row], rstd = Rstd[row];
    float xh[kGenCols], dy[kGenCols], wd[kGenCols];
    float c1 = 0.f, c2 = 0.f;
#pragma unroll
    for (int k = 0; k < kGenCols; ++k) {
      const int c = tid + k * kBwdThreads;
      if (c < N) {
        xh[k] = (X[row * ldx + c] - mean) * rstd;
        dy[k] = DY[row * lddy + c];
        wd[k] = W[c] * dy[k];
        c1 += xh[k] * wd[k];
        c2 += wd[k];
      }
    }
    c1 = warp_sum(c1);
    c2 = warp_sum(c2);
    if ((tid & 31) == 0) {
      red[0][tid >> 5] = c1;
      red[1][tid >> 5] = c2;
    }
    __syncthreads();
    c1 = c2 = 0.f;
#pragma unroll
    for (int k = 0; k < kBwdWarps; ++k) {
      c1 += red[0][k];
      c2 += red[1][k];
    }
    __syncthreads();
    c1 *= inv_n;
    c2 *= inv_n;
#pragma unroll
    for (int k = 0; k < kGenCols; ++k) {
      const int c = tid + k * kBwdThreads;
      if (c < N) {
        DX[row * lddx + c] = (wd[k] - (xh[k] * c1 + c2)) * rstd;
        dw[k] += dy[k] * xh[k];
        db[k] += dy[k];
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kGenCols; ++k) {
    const int c = tid + k * kBwdThreads;
    if (c < N) {
      DW[(long long)g * N + c] = dw[k];
      DB[(long long)g * N + c] = db[k];
    }
  }
}

// Column sums of the (N, G) partials.  Block = 32 columns x 8 group slices; each
// slice adds its groups in ascending order, then the 8 slice sums are added in
// ascending slice order: a fixed summation tree, so the result is deterministic.
constexpr int kRedCols = 32, kRedSlices = 8;
__global__ void __launch_bounds__(kRedCols * kRedSlices)
    ln_bwd_reduce_kernel(const float* __restrict__ DW, const float* __restrict__ DB, float* __restrict__ FDW,
                         float* __restrict__ FDB, int N, int G) {
  __shared__ float sw[kRedSlices][kRedCols], sb[kRedSlices][kRedCols];
  const int cx = threadIdx.x & (kRedCols - 1), sl = threadIdx.x / kRedCols;
  const int c = blockIdx.x * kRedCols + cx;
  const int per = (G + kRedSlices - 1) / kRedSlices;
  float a = 0.f, b = 0.f;
  if (c < N) {
    const int g1 = min(G, (sl + 1) * per);
#pragma unroll 4
    for (int g = sl * per; g < g1; ++g) {
      a += DW[(long long)g * N + c];
      b += DB[(long long)g * N + c];
    }
  }
  sw[sl][cx] = a;
  sb[sl][cx] = b;
  __syncthreads();
  if (sl == 0 && c < N) {
    a = 0.f;
    b = 0.f;
#pragma unroll
    for (int k = 0; k < kRedSlices; ++k) {
      a += sw[k][cx];
      b += sb[k][cx];
    }
    FDW[c] = a;
    FDB[c] = b;
  }
}

template <int NV>
int launch_bwd(ctb_ctx* ctx, cudaStream_t st, float* DX, const float* DY, float* DW, float* DB, const float* X,
               const float* W, const float* Mean, const float* Rstd, int N, int M, long long ldx, long long lddy,
               long long lddx, int G) {
  const int row_stride = (N * 4 + 127) & ~127;
  const size_t smem = (size_t)kBwdStages * 2 * row_stride;
  auto k = ln_bwd_kernel<NV>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd: shared memory opt-in");
  // Cluster size: the largest of 8,4,2,1 that keeps every CTA resident at once
  // and gives each CTA at least two rows.
  int per_sm = (int)((size_t)220 * 1024 / (smem + 1024));
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 2048 / kBwdThreads) per_sm = 2048 / kBwdThreads;
  int C = 8;
  while (C > 1 && ((long long)G * C > (long long)ctx->sm_count * per_sm || (long long)G * C * 2 > M)) C >>= 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G * C);
  cfg.blockDim = dim3(kBwdThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, k, DX, DY, DW, DB, X, W, Mean, Rstd, N, M, ldx, lddy, lddx, G, row_stride,
                         ctx->dev_status);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_dx_partial_dwdb launch");
  return CTB_OK;
}

bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

extern "C" {

int ctb_layernorm_fwd(ctb_ctx* ctx, void* stream, const float* X, const float* W, const float* B, float* Y,
                      float* Mean, float* Rstd, int64_t N, int64_t M, int64_t ldx, int64_t ldy, float eps,
                      int tile_n) {
  CTB_CHECK_CTX(ctx);
  if (N <= 0 || M < 0 || N > INT32_MAX || M > INT32_MAX)
    return fail(CTB_BAD_ARG, "ctb_layernorm_fwd: bad shape N=%lld M=%lld", (long long)N, (long long)M);
  if (ldx < N || ldy < N) return fail(CTB_BAD_ARG, "ctb_layernorm_fwd: leading dimension smaller than N");
  if (!is_pow2(tile_n)) return fail(CTB_UNSUPPORTED_TILE, "ctb_layernorm_fwd: TILE_N %d is not a power of two", tile_n);
  if (M == 0) return CTB_OK;
  CTB_CHECK_DEV(X); CTB_CHECK_DEV(W); CTB_CHECK_DEV(B); CTB_CHECK_DEV(Y); CTB_CHECK_DEV(Mean); CTB_CHECK_DEV(Rstd);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool fast = N % 4 == 0 && ldx % 4 == 0 && ldy % 4 == 0 && aligned16(X) && aligned16(Y) && aligned16(W) &&
                    aligned16(B) && N <= 4 * kFwdThreads * 8;
  const int n = (int)N, m = (int)M;
  if (fast) {
    const int nv = (n / 4 + kFwdThreads - 1) / kFwdThreads;
    const int stage_bytes = (int)(((size_t)n * 4 + 127) & ~size_t(127));
    const size_t smem = (size_t)kFwdStages * stage_bytes;
#define CTB_LN_FWD(NVV)                                                                                          \
  {                                                                                                              \
    auto k = ln_fwd_staged_kernel<NVV>;                                                                          \
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);             \
    if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_fwd: shared memory opt-in");                        \
    int per_sm = 0;                                                                                              \
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, kFwdThreads, smem);                                \
    if (per_sm < 1) per_sm = 1;                                                                                  \
    const int grid = (int)std::min<int64_t>(M, (int64_t)ctx->sm_count * per_sm);                                 \
    k<<<grid, kFwdThreads, smem, st>>>(X, W, B, Y, Mean, Rstd, n, m, ldx, ldy, eps, stage_bytes, ctx->dev_status); \
  }
    if (nv <= 1) CTB_LN_FWD(1)
    else if (nv <= 2) CTB_LN_FWD(2)
    else if (nv <= 4) CTB_LN_FWD(4)
    else CTB_LN_FWD(8)
#undef CTB_LN_FWD
  } else {
    const int grid = (int)std::min<int64_t>(M, (int64_t)ctx->sm_count * 8);
    ln_fwd_generic_kernel<<<grid, kFwdThreads, 0, st>>>(X, W, B, Y, Mean, Rstd, n, m, ldx, ldy, eps);
  }
  CTB_CHECK_LAUNCH("ctb_layernorm_fwd launch");
  return CTB_OK;
}

int ctb_layernorm_bwd_dx_partial_dwdb(ctb_ctx* ctx, void* stream, float* DX, const float* DY, float* DW, float* DB,
                                      const float* X, const float* W, const float* Mean, const float* Rstd,
                                      void* locks, int64_t N, int64_t M, int64_t ldx, int64_t lddy, int64_t lddx,
                                      int group_size_m, int tile_n) {
  (void)locks;
  CTB_CHECK_CTX(ctx);
  if (N <= 0 || M < 0 || N > INT32_MAX || M > INT32_MAX)
    return fail(CTB_BAD_ARG, "ctb_layernorm_bwd_dx_partial_dwdb: bad shape N=%lld M=%lld", (long long)N, (long long)M);
  if (ldx < N || lddy < N || lddx < N)
    return fail(CTB_BAD_ARG, "ctb_layernorm_bwd_dx_partial_dwdb: leading dimension smaller than N");
  if (group_size_m <= 0 || group_size_m > 65535)
    return fail(CTB_BAD_ARG, "ctb_layernorm_bwd_dx_partial_dwdb: GROUP_SIZE_M %d out of range", group_size_m);
  if (!is_pow2(tile_n))
    return fail(CTB_UNSUPPORTED_TILE, "ctb_layernorm_bwd_dx_partial_dwdb: TILE_N %d is not a power of two", tile_n);
  CTB_CHECK_DEV(DW); CTB_CHECK_DEV(DB);
  if (M > 0) { CTB_CHECK_DEV(DX); CTB_CHECK_DEV(DY); CTB_CHECK_DEV(X); CTB_CHECK_DEV(Mean); CTB_CHECK_DEV(Rstd); }
  CTB_CHECK_DEV(W);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int n = (int)N, m = (int)M, G = group_size_m;
  const bool fast = N % 4 == 0 && ldx % 4 == 0 && lddy % 4 == 0 && lddx % 4 == 0 && aligned16(X) && aligned16(DY) &&
                    aligned16(DX) && aligned16(W) && aligned16(DW) && aligned16(DB) && N <= 4 * kBwdThreads * 4;
  if (fast) {
    const int nv = (n / 4 + kBwdThreads - 1) / kBwdThreads;
    if (nv <= 1) return launch_bwd<1>(ctx, st, DX, DY, DW, DB, X, W, Mean, Rstd, n, m, ldx, lddy, lddx, G);
    if (nv <= 2) return launch_bwd<2>(ctx, st, DX, DY, DW, DB, X, W, Mean, Rstd, n, m, ldx, lddy, lddx, G);
    return launch_bwd<4>(ctx, st, DX, DY, DW, DB, X, W, Mean, Rstd, n, m, ldx, lddy, lddx, G);
  }
  if (N > kBwdThreads * kGenCols)
    return fail(CTB_UNSUPPORTED, "ctb_layernorm_bwd_dx_partial_dwdb: N=%lld exceeds %d", (long long)N,
                kBwdThreads * kGenCols);
  ln_bwd_generic_kernel<<<G, kBwdThreads, 0, st>>>(DX, DY, DW, DB, X, W, Mean, Rstd, n, m, ldx, lddy, lddx, G);
  CTB_CHECK_LAUNCH("ctb_layernorm_bwd_dx_partial_dwdb launch");
  return CTB_OK;
}

int ctb_layernorm_bwd_dwdb(ctb_ctx* ctx, void* stream, const float* DW, const float* DB, float* FINAL_DW,
                           float* FINAL_DB, int64_t N, int group_size_m, int tile_m, int tile_n) {
  CTB_CHECK_CTX(ctx);
  if (N <= 0 || N > INT32_MAX || group_size_m <= 0)
    return fail(CTB_BAD_ARG, "ctb_layernorm_bwd_dwdb: bad shape N=%lld groups=%d", (long long)N, group_size_m);
  if (!is_pow2(tile_m) || !is_pow2(tile_n))
    return fail(CTB_UNSUPPORTED_TILE, "ctb_layernorm_bwd_dwdb: TILE_M/TILE_N must be powers of two");
  CTB_CHECK_DEV(DW); CTB_CHECK_DEV(DB); CTB_CHECK_DEV(FINAL_DW); CTB_CHECK_DEV(FINAL_DB);
  ln_bwd_reduce_kernel<<<(int)((N + kRedCols - 1) / kRedCols), kRedCols * kRedSlices, 0,
                         static_cast<cudaStream_t>(stream)>>>(DW, DB, FINAL_DW, FINAL_DB, (int)N, group_size_m);
  CTB_CHECK_LAUNCH("ctb_layernorm_bwd_dwdb launch");
  return CTB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------- allocation-free backward
// Some hosts of this library may not allocate device memory on the path that
// runs the backward pass: a plug-in that lives inside another runtime's memory
// plan, a real-time loop that may not block in the driver, code that runs
// while a stream is being captured.  For them the partial dW/dB buffers of the
// backward pass live in a fixed array inside the library image instead of in
// memory the caller (or the library) would have to cudaMalloc.
namespace {

constexpr int kStaticGroups = 64;     // GROUP_SIZE_M of the built-in scratch
constexpr int kStaticMaxN = 8192;     // widest row the built-in scratch can hold
// [0] = partial dW, [1] = partial dB, each (N, kStaticGroups) with N <= kStaticMaxN: 4 MiB per device, held
// from the moment the library is loaded on a device until the process exits.
static __device__ __align__(256) float g_ln_static_partials[2 * kStaticGroups * kStaticMaxN];
static __device__ int g_ln_static_status;  // bounded-wait codes of the static entry point (see DevStatus)

struct StaticDev {
  bool ready;
  float* partials;  // DEVICE address of g_ln_static_partials on this device
  int* status;
  int sm_count;
};
constexpr int kMaxDevices = 64;
StaticDev g_static_dev[kMaxDevices];
std::mutex g_static_mu;

// One-time set-up per device.  In host code the name of a __device__ array is only a handle: the address a
// kernel can use has to be asked for with cudaGetSymbolAddress while that device is current.
int static_setup(int dev, StaticDev** out) {
  if (dev < 0 || dev >= kMaxDevices) return fail(CTB_UNSUPPORTED, "ctb_layernorm_bwd_static: device %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  StaticDev& d = g_static_dev[dev];
  if (!d.ready) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_ln_static_partials);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static: cudaGetSymbolAddress(partials)");
    d.partials = static_cast<float*>(p);
    e = cudaGetSymbolAddress(&p, g_ln_static_status);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static: cudaGetSymbolAddress(status)");
    d.status = static_cast<int*>(p);
    e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static: cudaDeviceGetAttribute");
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static: cudaDeviceGetAttribute");
    if (major != 10) return fail(CTB_NO_DEVICE, "ctb_layernorm_bwd_static: device %d is not sm_100", dev);
    d.ready = true;
  }
  *out = &d;
  return CTB_OK;
}

template <int NV>
int launch_bwd_static(const StaticDev& d, cudaStream_t st, float* DX, const float* DY, float* DW, float* DB,
                      const float* X, const float* W, const float* Mean, const float* Rstd, int N, int M,
                      long long ldx, long long lddy, long long lddx) {
  const int G = kStaticGroups;
  const int row_stride = (N * 4 + 127) & ~127;
  const size_t smem = (size_t)kBwdStages * 2 * row_stride;
  auto k = ln_bwd_kernel<NV>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static: shared memory opt-in");
  int per_sm = (int)((size_t)220 * 1024 / (smem + 1024));
  per_sm = std::max(1, std::min(per_sm, 2048 / kBwdThreads));
  int C = 8;
  while (C > 1 && ((long long)G * C > (long long)d.sm_count * per_sm || (long long)G * C * 2 > M)) C >>= 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(G * C);
  cfg.blockDim = dim3(kBwdThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, k, DX, DY, DW, DB, X, W, Mean, Rstd, N, M, ldx, lddy, lddx, G, row_stride, d.status);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static launch");
  return CTB_OK;
}

}  // namespace

extern "C" int ctb_layernorm_bwd_static(void* stream, float* DX, const float* DY, const float* X, const float* W,
                                        const float* Mean, const float* Rstd, float* FINAL_DW, float* FINAL_DB,
                                        int64_t N, int64_t M, int64_t ldx, int64_t lddy, int64_t lddx) {
  if (N <= 0 || M <= 0 || M > INT32_MAX)
    return fail(CTB_BAD_ARG, "ctb_layernorm_bwd_static: bad shape N=%lld M=%lld", (long long)N, (long long)M);
  if (N > kStaticMaxN)
    return fail(CTB_UNSUPPORTED, "ctb_layernorm_bwd_static: N=%lld exceeds the built-in scratch (at most %d columns); "
                "use ctb_layernorm_bwd_dx_partial_dwdb with caller-provided partial buffers", (long long)N, kStaticMaxN);
  if (ldx < N || lddy < N || lddx < N) return fail(CTB_BAD_ARG, "ctb_layernorm_bwd_static: leading dimension smaller than N");
  if (N % 4 || ldx % 4 || lddy % 4 || lddx % 4 || !aligned16(X) || !aligned16(DY) || !aligned16(DX) || !aligned16(W))
    return fail(CTB_BAD_ALIGN, "ctb_layernorm_bwd_static: N and the leading dimensions must be multiples of 4 and "
                "X, DY, DX, W 16-byte aligned");
  CTB_CHECK_DEV(DX); CTB_CHECK_DEV(DY); CTB_CHECK_DEV(X); CTB_CHECK_DEV(W); CTB_CHECK_DEV(Mean); CTB_CHECK_DEV(Rstd);
  CTB_CHECK_DEV(FINAL_DW); CTB_CHECK_DEV(FINAL_DB);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static: cudaGetDevice");
  StaticDev* d = nullptr;
  int r = static_setup(dev, &d);
  if (r) return r;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* DW = d->partials;
  float* DB = d->partials + (size_t)kStaticGroups * kStaticMaxN;
  const int n = (int)N, m = (int)M;
  const int nv = (n / 4 + kBwdThreads - 1) / kBwdThreads;
  if (nv <= 1) r = launch_bwd_static<1>(*d, st, DX, DY, DW, DB, X, W, Mean, Rstd, n, m, ldx, lddy, lddx);
  else if (nv <= 2) r = launch_bwd_static<2>(*d, st, DX, DY, DW, DB, X, W, Mean, Rstd, n, m, ldx, lddy, lddx);
  else r = launch_bwd_static<4>(*d, st, DX, DY, DW, DB, X, W, Mean, Rstd, n, m, ldx, lddy, lddx);
  if (r) return r;
  ln_bwd_reduce_kernel<<<(n + kRedCols - 1) / kRedCols, kRedCols * kRedSlices, 0, st>>>(DW, DB, FINAL_DW, FINAL_DB, n,
                                                                                      kStaticGroups);
  CTB_CHECK_LAUNCH("ctb_layernorm_bwd_static reduce launch");
  return CTB_OK;
}

// Reads and clears the status word of the allocation-free entry point on the current device (the word lives in the
// library image next to the scratch; its address comes from the same one-time cudaGetSymbolAddress set-up).
extern "C" int ctb_layernorm_bwd_static_status(void* stream) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static_status: cudaGetDevice");
  StaticDev* d = nullptr;
  int r = static_setup(dev, &d);
  if (r) return r;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int v = 0;
  e = cudaMemcpyAsync(&v, d->status, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static_status");
  if (v == 0) return CTB_OK;
  e = cudaMemsetAsync(d->status, 0, sizeof(int), st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_layernorm_bwd_static_status: clearing the word");
  return fail(CTB_TIMEOUT, "ctb_layernorm_bwd_static: a kernel gave up a bounded wait (device code %d); DX, FINAL_DW "
              "and FINAL_DB of the calls since the last check are not valid", v);
}
