// Element-wise addition and matrix transpose for sm_100a (counterparts of vec_add_kernel_1d / _2d / _1d_gather,
// examples/vadd.jl:10-45, and transpose_kernel, examples/transpose.jl:11-19).  Both are bound by HBM bandwidth:
// 3 * n * sizeof(T) bytes for the addition (examples/vadd.jl:131-136), 2 * m * n * sizeof(T) for the transpose
// (examples/transpose.jl:62-66).  128-bit coalesced accesses, grids sized in multiples of the SM count.
#include <cuda_fp16.h>

#include "ctx.h"

using namespace ctb_internal;

namespace {

template <typename T>
struct Vec16;  // 16 bytes of T
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ uint4 add(uint4 a, uint4 b) {
    float4 x = *reinterpret_cast<float4*>(&a), y = *reinterpret_cast<float4*>(&b);
    float4 z = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
    return *reinterpret_cast<uint4*>(&z);
  }
  static __device__ __forceinline__ float add1(float a, float b) { return a + b; }
};
template <>
struct Vec16<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ uint4 add(uint4 a, uint4 b) {
    uint4 z;
    const __half2* x = reinterpret_cast<const __half2*>(&a);
    const __half2* y = reinterpret_cast<const __half2*>(&b);
    __half2* o = reinterpret_cast<__half2*>(&z);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = __hadd2(x[i], y[i]);
    return z;
  }
  static __device__ __forceinline__ __half add1(__half a, __half b) { return __hadd(a, b); }
};

// c = a + b over `rows` rows of `n` contiguous elements (row strides in elements).  A CTA walks whole rows when they
// are long, or the flat array when the rows are dense (ld == n), four 16-byte vectors per thread and trip.
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) vadd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ c,
                                                   long long n, long long rows, long long lda, long long ldb, long long ldc) {
  constexpr int V = Vec16<T>::N;
  const long long per_row = VEC ? n / V : n;  // work units per row
  const long long total = per_row * rows;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long r = i / per_row, k = i - r * per_row;
    if (VEC) {
      const uint4 x = __ldcs(reinterpret_cast<const uint4*>(a + r * lda) + k);
      const uint4 y = __ldcs(reinterpret_cast<const uint4*>(b + r * ldb) + k);
      __stcs(reinterpret_cast<uint4*>(c + r * ldc) + k, Vec16<T>::add(x, y));
    } else {
      c[r * ldc + k] = Vec16<T>::add1(a[r * lda + k], b[r * ldb + k]);
    }
  }
}

// y(n, m) = transpose of x(m, n), both with the first dimension contiguous.  64 x 64 tiles through shared memory:
// 16-byte loads along m, 16-byte stores along n.
constexpr int kTT = 64;
template <typename T>
__global__ void __launch_bounds__(256) transpose_kernel(const T* __restrict__ x, T* __restrict__ y, int m, int n, long long ldx,
                                                        long long ldy, int tiles_m, long long tiles) {
  __shared__ T tile[kTT][kTT + 16 / sizeof(T) + 1];
  constexpr int V = 16 / sizeof(T);
  const bool vec_in = (ldx % V == 0) && ((uintptr_t)x % 16 == 0), vec_out = (ldy % V == 0) && ((uintptr_t)y % 16 == 0);
  for (long long t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int tm = (int)(t % tiles_m), tn = (int)(t / tiles_m);
    const int m0 = tm * kTT, n0 = tn * kTT;
    // load: column j of x (fixed n index) is contiguous along m
    for (int i = threadIdx.x; i < kTT * (kTT / V); i += 256) {
      const int j = i / (kTT / V), v = i - j * (kTT / V);
      const int mm = m0 + v * V, nn = n0 + j;
      if (nn < n) {
        if (vec_in && mm + V <= m) {
          const uint4 q = __ldcs(reinterpret_cast<const uint4*>(x + (long long)nn * ldx + mm));
          const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
          for (int k = 0; k < V; ++k) tile[v * V + k][j] = e[k];
        } else {
          for (int k = 0; k < V; ++k)
            if (mm + k < m) tile[v * V + k][j] = x[(long long)nn * ldx + mm + k];
        }
      }
    }
    __syncthreads();
    // store: column i of y (fixed m index) is contiguous along n
    for (int i = threadIdx.x; i < kTT * (kTT / V); i += 256) {
      const int r = i / (kTT / V), v = i - r * (kTT / V);
      const int mm = m0 + r, nn = n0 + v * V;
      if (mm < m) {
        if (vec_out && nn + V <= n) {
          uint4 q;
          T* e = reinterpret_cast<T*>(&q);
#pragma unroll
          for (int k = 0; k < V; ++k) e[k] = tile[r][v * V + k];
          __stcs(reinterpret_cast<uint4*>(y + (long long)mm * ldy + nn), q);
        } else {
          for (int k = 0; k < V; ++k)
            if (nn + k < n) y[(long long)mm * ldy + nn + k] = tile[r][v * V + k];
        }
      }
    }
    __syncthreads();
  }
}

}  // namespace

extern "C" {

int ctb_vadd(ctb_ctx* ctx, void* stream, const void* a, const void* b, void* c, int64_t n, int64_t rows, int64_t lda,
             int64_t ldb, int64_t ldc, int tile_x, int tile_y, int use_gather, int dtype) {
  CTB_CHECK_CTX(ctx);
  (void)use_gather;  // the gather/scatter formulation of the reference addresses the same contiguous elements
  if (n < 0 || rows < 0) return fail(CTB_BAD_ARG, "ctb_vadd: negative size");
  if (!is_pow2(tile_x) || !is_pow2(tile_y)) return fail(CTB_UNSUPPORTED_TILE, "ctb_vadd: tile sizes must be powers of two");
  if (rows > 1 && (lda < n || ldb < n || ldc < n)) return fail(CTB_BAD_ARG, "ctb_vadd: leading dimension smaller than the row length");
  if (dtype != CTB_F32 && dtype != CTB_F16) return fail(CTB_UNSUPPORTED, "ctb_vadd: element type must be f32 or f16");
  if (n == 0 || rows == 0) return CTB_OK;
  CTB_CHECK_DEV(a); CTB_CHECK_DEV(b); CTB_CHECK_DEV(c);
  if (rows > 1 && lda == n && ldb == n && ldc == n) {  // dense: one long row
    n *= rows;
    rows = 1;
  }
  const int es = dtype == CTB_F32 ? 4 : 2, V = 16 / es;
  const bool vec = n % V == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)b % 16 == 0 && (uintptr_t)c % 16 == 0 &&
                   (rows == 1 || (lda % V == 0 && ldb % V == 0 && ldc % V == 0));
  const long long units = (vec ? n / V : n) * rows;
  const int grid = (int)std::max<long long>(1, std::min<long long>((units + 255) / 256, (long long)ctx->sm_count * 16));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define CTB_VADD(T, VECV) vadd_kernel<T, VECV><<<grid, 256, 0, st>>>((const T*)a, (const T*)b, (T*)c, n, rows, lda, ldb, ldc)
  if (dtype == CTB_F32) { if (vec) CTB_VADD(float, true); else CTB_VADD(float, false); }
  else { if (vec) CTB_VADD(__half, true); else CTB_VADD(__half, false); }
#undef CTB_VADD
  CTB_CHECK_LAUNCH("ctb_vadd launch");
  return CTB_OK;
}

int ctb_transpose(ctb_ctx* ctx, void* stream, const void* x, void* y, int64_t m, int64_t n, int64_t ldx, int64_t ldy, int tm,
                  int tn, int dtype) {
  CTB_CHECK_CTX(ctx);
  if (m < 0 || n < 0 || m > INT32_MAX || n > INT32_MAX) return fail(CTB_BAD_ARG, "ctb_transpose: bad shape");
  if (!is_pow2(tm) || !is_pow2(tn)) return fail(CTB_UNSUPPORTED_TILE, "ctb_transpose: tile sizes must be powers of two");
  if (ldx < m || ldy < n) return fail(CTB_BAD_ARG, "ctb_transpose: leading dimension smaller than the column length");
  if (dtype != CTB_F32 && dtype != CTB_F16) return fail(CTB_UNSUPPORTED, "ctb_transpose: element type must be f32 or f16");
  if (m == 0 || n == 0) return CTB_OK;
  CTB_CHECK_DEV(x); CTB_CHECK_DEV(y);
  const int tiles_m = (int)((m + kTT - 1) / kTT);
  const long long tiles = (long long)tiles_m * ((n + kTT - 1) / kTT);
  const int grid = (int)std::max<long long>(1, std::min<long long>(tiles, (long long)ctx->sm_count * 8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == CTB_F32)
    transpose_kernel<float><<<grid, 256, 0, st>>>((const float*)x, (float*)y, (int)m, (int)n, ldx, ldy, tiles_m, tiles);
  else
    transpose_kernel<__half><<<grid, 256, 0, st>>>((const __half*)x, (__half*)y, (int)m, (int)n, ldx, ldy, tiles_m, tiles);
  CTB_CHECK_LAUNCH("ctb_transpose launch");
  return CTB_OK;
}

}  // extern "C"
