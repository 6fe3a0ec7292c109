// Row softmax for sm_100a.
//
// variant 0 ("single tile per row", the counterpart of softmax_tma_kernel,
//   examples/softmax.jl:18-42): persistent CTAs; each row is staged into shared
//   memory by one bulk async copy (cp.async.bulk + mbarrier) through a ring of
//   stages, normalised in registers, written back into the stage and stored
//   with a bulk copy shared->global, so loads and stores of neighbouring rows
//   overlap the arithmetic of the current one.
// variant 1 ("chunked", the counterpart of softmax_chunked_kernel, :48-100):
//   rows that fit the registers of a CTA and are 16-byte aligned take the
//   variant-0 kernel (one HBM read, one write; a chunk-by-chunk running
//   (max, sum) over bulk-copied chunks was measured 1.5x slower there because
//   it evaluates two exponentials per element).  Longer rows that fit shared
//   memory (up to 200 KB) are kept there whole: a running (max, sum) over the
//   chunks as they land, then a second pass that scales and stores (still one
//   HBM read, one write; for these rows the passes over shared memory cost
//   more than the second exponential).  Anything else: a running (max, sum)
//   per thread over chunks with 128-bit loads, re-read once.
//
// Both compute in f32 (examples/softmax.jl:32-35,92).  exp(x - max) is evaluated
// as ex2.approx((x - max)*log2(e)) (relative error about 2^-22 plus the rounding
// of the product) and the division as a multiplication by the exactly
// rounded reciprocal of the row sum, so that the kernel stays HBM-bound
// (2*M*N*sizeof(T) bytes per call) instead of instruction-bound.
#include <float.h>

#include <algorithm>

#include "ctx.h"
#include "ptx.cuh"

using namespace ctb;
using namespace ctb_internal;

namespace {

constexpr float kLog2e = 1.4426950408889634f;
// exp(x - m).  The subtraction comes first so that x == m gives exactly 1 and huge
// magnitudes cannot turn the rounding error of m*log2(e) into a wrong exponent.
__device__ __forceinline__ float exp_sub(float x, float m) { return ex2_approx_ftz((x - m) * kLog2e); }

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

struct __align__(8) Vec4h {
  __half2 a, b;
};

template <typename T>
struct Pack;  // 4 consecutive elements moved as one 16-byte (f32) or 8-byte (f16) access
template <>
struct Pack<float> {
  using type = float4;
  static __device__ __forceinline__ void unpack(const float4& v, float* f) {
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  }
  static __device__ __forceinline__ float4 pack(const float* f) { return make_float4(f[0], f[1], f[2], f[3]); }
};
template <>
struct Pack<__half> {
  using type = Vec4h;
  static __device__ __forceinline__ void unpack(const Vec4h& v, float* f) {
    float2 x = __half22float2(v.a), y = __half22float2(v.b);
    f[0] = x.x; f[1] = x.y; f[2] = y.x; f[3] = y.y;
  }
  static __device__ __forceinline__ Vec4h pack(const float* f) {
    Vec4h v;
    v.a = __floats2half2_rn(f[0], f[1]);
    v.b = __floats2half2_rn(f[2], f[3]);
    return v;
  }
};

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = red[0];
#pragma unroll
  for (int i = 1; i < kWarps; ++i) r = fmaxf(r, red[i]);
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < kWarps; ++i) r += red[i];  // fixed order: deterministic
  __syncthreads();
  return r;
}

// ------------------------------------------------------------------ variant 0
// MAXV: packs of 4 elements kept in registers per thread (N <= 4*kThreads*MAXV).
template <typename T, int MAXV, int STAGES>
__global__ void __launch_bounds__(kThreads) softmax_staged_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                                  int N, int M, long long ld_out, long long ld_in,
                                                                  int stage_bytes, int* status) {
  using P = typename Pack<T>::type;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[STAGES];
  __shared__ float red[kWarps];
  const int tid = threadIdx.x;
  const uint32_t row_bytes = (uint32_t)N * sizeof(T);
  const int npack = N / 4;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&full[s], 1);
    fence_mbar_init();
  }
  __syncthreads();

  const int first = blockIdx.x, step = gridDim.x;
  const int nrows = first < M ? (M - first + step - 1) / step : 0;

  // prologue: fill the ring
  if (tid == 0) {
    for (int i = 0; i < STAGES && i < nrows; ++i) {
      mbar_expect_tx(&full[i], row_bytes);
      bulk_g2s(smem + (size_t)i * stage_bytes, in + (long long)(first + i * step) * ld_in, row_bytes, &full[i]);
    }
  }

  bool alive = true;
  for (int i = 0; i < nrows && alive; ++i) {
    const int s = i % STAGES;
    const uint32_t parity = (i / STAGES) & 1;
    P* buf = reinterpret_cast<P*>(smem + (size_t)s * stage_bytes);
    if (!mbar_wait(&full[s], parity, status, DEV_TIMEOUT_TMA)) alive = false;
    alive = __syncthreads_and(alive);
    if (!alive) break;

    float x[MAXV][4];
    float mx = -FLT_MAX;
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int p = tid + v * kThreads;
      if (p < npack) {
        Pack<T>::unpack(buf[p], x[v]);
        mx = fmaxf(mx, fmaxf(fmaxf(x[v][0], x[v][1]), fmaxf(x[v][2], x[v][3])));
      }
    }
    mx = block_max(mx, red);
    float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      if (tid + v * kThreads < npack) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          x[v][k] = exp_sub(x[v][k], mx);
          s4[k] += x[v][k];
        }
      }
    }
    const float inv = 1.0f / block_sum((s4[0] + s4[1]) + (s4[2] + s4[3]), red);
#pragma unroll
    for (int v = 0; v < MAXV; ++v) {
      const int p = tid + v * kThreads;
      if (p < npack) {
#pragma unroll
        for (int k = 0; k < 4; ++k) x[v][k] *= inv;
        buf[p] = Pack<T>::pack(x[v]);
      }
    }
    fence_proxy_async_smem();  // generic-proxy writes -> visible to the bulk store
    __syncthreads();
    if (tid == 0) {
      bulk_s2g(out + (long long)(first + i * step) * ld_out, buf, row_bytes);
      bulk_commit();
      // Refill the stage used by the PREVIOUS row: its store was committed one
      // iteration ago, so waiting for "all but the newest group" has read it.
      const int nxt = i - 1 + STAGES;
      if (i >= 1 && nxt < nrows) {
        bulk_wait_read<1>();
        const int ps = (i - 1) % STAGES;
        mbar_expect_tx(&full[ps], row_bytes);
        bulk_g2s(smem + (size_t)ps * stage_bytes, in + (long long)(first + nxt * step) * ld_in, row_bytes, &full[ps]);
      }
    }
  }
  if (tid == 0) bulk_wait<0>();  // stores complete before the CTA (and its smem) goes away
}

// ------------------------------------------------------------------ variant 1, rows that fit shared memory
// Rows too long for the registers of a CTA but not for its shared memory (up to about 200 KB): one CTA per SM keeps
// the whole row on chip, so HBM is still read once and written once.  The row arrives as kRowChunks bulk copies, each
// with its own mbarrier; the threads look for the maximum of a chunk as soon as it has landed, under the copies of
// the chunks behind it and sum the exponentials in the same pass (online, rescaling when the maximum grows).  A second
// pass evaluates the exponentials again, scales and stores to global memory; a chunk's part of the buffer is refilled
// with the next row's chunk as soon as it was read.
constexpr int kRowThreads = 512;
constexpr int kRowChunks = 8;
template <typename T>
__global__ void __launch_bounds__(kRowThreads) softmax_row_smem_kernel(T* __restrict__ out, const T* __restrict__ in, int N,
                                                                       int M, long long ld_out, long long ld_in, int* status) {
  using P = typename Pack<T>::type;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ __align__(8) uint64_t full[kRowChunks];
  __shared__ float red[kRowThreads / 32];
  const int tid = threadIdx.x;
  const int npack = N / 4;
  // chunk boundaries in packs, multiples of 4 packs (16 bytes for f16, 64 for f32)
  const int per = ((npack + kRowChunks - 1) / kRowChunks + 3) & ~3;
  if (tid == 0) {
    for (int c = 0; c < kRowChunks; ++c) mbar_init(&full[c], 1);
    fence_mbar_init();
  }
  __syncthreads();
  P* buf = reinterpret_cast<P*>(smem);
  auto block_reduce = [&](float v, bool is_max) {
    v = is_max ? warp_max(v) : warp_sum(v);
    if ((tid & 31) == 0) red[tid >> 5] = v;
    __syncthreads();
    float r = red[0];
    for (int i = 1; i < kRowThreads / 32; ++i) r = is_max ? fmaxf(r, red[i]) : r + red[i];  // fixed order
    __syncthreads();
    return r;
  };
  // thread 0 issues the bulk copies of chunk c of `row` (the buffer region of the chunk must be free)
  auto load_chunk = [&](int row, int c) {
    const int p0 = c * per, p1 = min(npack, p0 + per);
    if (p1 <= p0) return;
    const uint32_t bytes = (uint32_t)(p1 - p0) * 4 * sizeof(T);
    mbar_expect_tx(&full[c], bytes);
    bulk_g2s(buf + p0, in + (long long)row * ld_in + (long long)p0 * 4, bytes, &full[c]);
  };
  if (tid == 0 && (int)blockIdx.x < M)
    for (int c = 0; c < kRowChunks; ++c) load_chunk(blockIdx.x, c);
  bool alive = true;
  int it = 0;
  for (int row = blockIdx.x; row < M && alive; row += gridDim.x, ++it) {
    // One pass over the chunks as they land: running maximum and sum of exponentials per thread, the sum rescaled
    // when the maximum grows (the chunk loop of the reference, examples/softmax.jl:48-100), then combined over the CTA
    // in a fixed order.
    float m = -FLT_MAX, l = 0.f;
    for (int c = 0; c < kRowChunks; ++c) {
      const int p0 = c * per, p1 = min(npack, p0 + per);
      if (p1 <= p0) break;
      if (!mbar_wait(&full[c], it & 1, status, DEV_TIMEOUT_TMA)) alive = false;
      for (int p = p0 + tid; p < p1; p += kRowThreads) {
        float f[4];
        Pack<T>::unpack(buf[p], f);
        const float cm = fmaxf(fmaxf(f[0], f[1]), fmaxf(f[2], f[3]));
        if (cm > m) {
          l *= exp_sub(m, cm);
          m = cm;
        }
        l += (exp_sub(f[0], m) + exp_sub(f[1], m)) + (exp_sub(f[2], m) + exp_sub(f[3], m));
      }
    }
    alive = __syncthreads_and(alive);
    if (!alive) break;
    const float mx = block_reduce(m, true);
    const float inv = 1.0f / block_reduce(l * exp_sub(m, mx), false);
    // Scale and store chunk by chunk, from registers straight to global memory (16 bytes per thread, neighbouring
    // threads neighbouring addresses); as soon as every thread has read a chunk's part of the buffer, the same part
    // takes the next row's chunk, so that the next row streams in under the rest of this one.
    const int next = row + gridDim.x;
    P* dst = reinterpret_cast<P*>(out + (long long)row * ld_out);
    for (int c = 0; c < kRowChunks; ++c) {
      const int p0 = c * per, p1 = min(npack, p0 + per);
      if (p1 <= p0) break;
      for (int p = p0 + tid; p < p1; p += kRowThreads) {
        float f[4];
        Pack<T>::unpack(buf[p], f);
#pragma unroll
        for (int k = 0; k < 4; ++k) f[k] = exp_sub(f[k], mx) * inv;
        const P v = Pack<T>::pack(f);
        if constexpr (sizeof(P) == 16) __stcs(reinterpret_cast<float4*>(dst + p), *reinterpret_cast<const float4*>(&v));
        else __stcs(reinterpret_cast<uint2*>(dst + p), *reinterpret_cast<const uint2*>(&v));
      }
      __syncthreads();  // all reads of the chunk are done before the bulk copy overwrites it
      if (tid == 0 && next < M) load_chunk(next, c);
    }
  }
}

// ------------------------------------------------------------------ variant 1, any row
// VEC = elements per load (4 => Pack<T>, 1 => scalar).  CACHE = register-resident
// packs per thread; rows with more are re-read from global for the final pass.
template <typename T, int VEC, int CACHE>
__global__ void __launch_bounds__(kThreads) softmax_online_kernel(T* __restrict__ out, const T* __restrict__ in,
                                                                  int N, int M, long long ld_out, long long ld_in) {
  __shared__ float red[kWarps];
  const int tid = threadIdx.x;
  const int nvec = (N + VEC - 1) / VEC;  // VEC==4 only when N % 4 == 0
  const int nstep = (nvec + kThreads - 1) / kThreads;

  for (int row = blockIdx.x; row < M; row += gridDim.x) {
    const T* src = in + (long long)row * ld_in;
    T* dst = out + (long long)row * ld_out;
    float cache[CACHE][VEC];
    float m = -FLT_MAX, l = 0.f;

    auto load = [&](int i, float* f) -> bool {
      const int p = tid + i * kThreads;
      if (p >= nvec) return false;
      if constexpr (VEC == 4) {
        Pack<T>::unpack(reinterpret_cast<const typename Pack<T>::type*>(src)[p], f);
      } else {
        f[0] = (float)src[p];
      }
      return true;
    };
    auto update = [&](const float* f) {
      float cm = f[0];
#pragma unroll
      for (int k = 1; k < VEC; ++k) cm = fmaxf(cm, f[k]);
      if (cm > m) {
        l *= exp_sub(m, cm);
        m = cm;
      }
#pragma unroll
      for (int k = 0; k < VEC; ++k) l += exp_sub(f[k], m);
    };

#pragma unroll
    for (int i = 0; i < CACHE; ++i)
      if (i < nstep && load(i, cache[i])) update(cache[i]);
    for (int i = CACHE; i < nstep; ++i) {
      float f[VEC];
      if (load(i, f)) update(f);
    }
    const float mg = block_max(m, red);
    const float inv = 1.0f / block_sum(l * exp_sub(m, mg), red);  // threads with no data: l = 0

    auto store = [&](int i, float* f) {
      const int p = tid + i * kThreads;
#pragma unroll
      for (int k = 0; k < VEC; ++k) f[k] = exp_sub(f[k], mg) * inv;
      if constexpr (VEC == 4) {
        reinterpret_cast<typename Pack<T>::type*>(dst)[p] = Pack<T>::pack(f);
      } else {
        dst[p] = (T)f[0];
      }
    };
#pragma unroll
    for (int i = 0; i < CACHE; ++i)
      if (i < nstep && tid + i * kThreads < nvec) store(i, cache[i]);
    for (int i = CACHE; i < nstep; ++i) {
      float f[VEC];
      if (load(i, f)) store(i, f);
    }
  }
}

template <typename T>
int launch(ctb_ctx* ctx, cudaStream_t st, T* out, const T* in, int N, int M, long long ldo, long long ldi,
           int variant, int tile_size) {
  const bool vec_ok = (N % 4 == 0) && (ldo % 4 == 0) && (ldi % 4 == 0) &&
                      ((uintptr_t)out % (4 * sizeof(T)) == 0) && ((uintptr_t)in % (4 * sizeof(T)) == 0);
  const size_t row_bytes = (size_t)N * sizeof(T);
  const bool bulk_ok = row_bytes % 16 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)in % 16 == 0 &&
                       (ldo * sizeof(T)) % 16 == 0 && (ldi * sizeof(T)) % 16 == 0;
  constexpr int STAGES = 3, MAXV = 8;
  const bool fits = N <= 4 * kThreads * MAXV;
  if (variant == 0 && !bulk_ok)
    return fail(CTB_BAD_ALIGN,
                "ctb_softmax variant 0: rows must start on 16-byte boundaries and N*elemsize be a multiple of 16");
  if (variant == 0 && !fits)
    return fail(CTB_UNSUPPORTED, "ctb_softmax variant 0: N=%d exceeds the single-tile limit %d; use variant 1", N,
                4 * kThreads * MAXV);
  if (bulk_ok && fits) {
    // Both variants: a row that fits the registers of one CTA is read once and written once whatever the chunk
    // size asks for; the chunk loop of the reference (examples/softmax.jl:48-100) only matters for longer rows.
    const int stage_bytes = (int)((row_bytes + 127) & ~size_t(127));
    const size_t smem = (size_t)STAGES * stage_bytes;
    auto k = softmax_staged_kernel<T, MAXV, STAGES>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_softmax: shared memory opt-in");
    int per_sm = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, kThreads, smem);
    if (per_sm < 1) per_sm = 1;
    const int grid = min(M, ctx->sm_count * per_sm);
    k<<<grid, kThreads, smem, st>>>(out, in, N, M, ldo, ldi, stage_bytes, ctx->dev_status);
  } else if (bulk_ok && row_bytes <= 200 * 1024) {
    const size_t smem = (row_bytes + 127) & ~size_t(127);
    auto k = softmax_row_smem_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_softmax: shared memory opt-in");
    const int per_sm = std::max(1, (int)((size_t)220 * 1024 / (smem + 2048)));
    const int grid = min(M, ctx->sm_count * std::min(per_sm, 4));
    k<<<grid, kRowThreads, smem, st>>>(out, in, N, M, ldo, ldi, ctx->dev_status);
  } else {
    int per_sm = 8;
    const int grid = min(M, ctx->sm_count * per_sm);
    if (vec_ok)
      softmax_online_kernel<T, 4, 8><<<grid, kThreads, 0, st>>>(out, in, N, M, ldo, ldi);
    else
      softmax_online_kernel<T, 1, 8><<<grid, kThreads, 0, st>>>(out, in, N, M, ldo, ldi);
  }
  CTB_CHECK_LAUNCH("ctb_softmax launch");
  return CTB_OK;
}

}  // namespace

extern "C" int ctb_softmax(ctb_ctx* ctx, void* stream, void* output, const void* input, int64_t N, int64_t M,
                           int64_t ld_out, int64_t ld_in, int variant, int tile_size, int dtype) {
  CTB_CHECK_CTX(ctx);
  if (N <= 0 || M < 0 || N > INT32_MAX || M > INT32_MAX)
    return fail(CTB_BAD_ARG, "ctb_softmax: bad shape N=%lld M=%lld", (long long)N, (long long)M);
  if (ld_out < N || ld_in < N) return fail(CTB_BAD_ARG, "ctb_softmax: leading dimension smaller than N");
  if (variant != 0 && variant != 1) return fail(CTB_BAD_ARG, "ctb_softmax: variant must be 0 or 1");
  if (!is_pow2(tile_size)) return fail(CTB_UNSUPPORTED_TILE, "ctb_softmax: tile_size %d is not a power of two", tile_size);
  if (variant == 0 && tile_size < N)
    return fail(CTB_UNSUPPORTED_TILE, "ctb_softmax variant 0: tile_size %d must cover the row (N=%lld)", tile_size,
                (long long)N);
  if (M == 0) return CTB_OK;
  CTB_CHECK_DEV(output);
  CTB_CHECK_DEV(input);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CTB_F32)
    return launch<float>(ctx, st, (float*)output, (const float*)input, (int)N, (int)M, ld_out, ld_in, variant, tile_size);
  if (dtype == CTB_F16)
    return launch<__half>(ctx, st, (__half*)output, (const __half*)input, (int)N, (int)M, ld_out, ld_in, variant, tile_size);
  return fail(CTB_BAD_ARG, "ctb_softmax: dtype must be CTB_F32 or CTB_F16");
}
