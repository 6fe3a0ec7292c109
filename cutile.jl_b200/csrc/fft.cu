// Batched complex-to-complex FFT of length N = F0 * F1 * F2 as three DFT-matrix stages with twiddle factors between
// them (counterpart of fft_kernel, examples/fft.jl:22-126; the caller passes the DFT matrices and twiddles it built
// with make_twiddles, examples/fft.jl:128-176, and the kernel uses exactly those values).
//
// One CTA transforms one batch item.  With the input index n = n2 + F2 * n1 + F1F2 * n0 and the output index
// k = k0 + F0 * k1 + F0F1 * k2 (the reference's reshapes and permutes written out):
//   stage 0: line j = n2 + F2 * n1:   a(j, k0)  = T0[j + F1F2 * k0] * sum_n0 x[j + F1F2 * n0] * W0(n0, k0)
//   stage 1: line r = k0 + F0 * n2:   b(r, k1)  = T1[n2 + F2 * k1]  * sum_n1 a(n2 + F2 * n1, k0) * W1(n1, k1)
//   stage 2: line t = k0 + F0 * k1:   y[t + F0F1 * k2]              = sum_n2 b(k0 + F0 * n2, k1) * W2(n2, k2)
// A thread owns whole lines: it reads the F inputs of a line into registers and produces its F outputs with f32 FMAs
// (the DFT matrix is broadcast from shared memory), so the input is read from global memory once, coalesced, the two
// intermediate arrays live in shared memory (padded by one element per 16 so that both the line-major writes and the
// element-major reads are free of bank conflicts), and the output is written once, coalesced.  Algorithmic bytes:
// 2 * batch * N * 8 (examples/fft.jl reports time only; it calls this a latency benchmark, :249-252).
#include <algorithm>
#include <type_traits>

#include "ctx.h"

using namespace ctb_internal;

namespace {

constexpr int kMaxFactor = 32;
constexpr int kMaxN = 8192;

__device__ __forceinline__ int pad16(int p) { return p + (p >> 4); }

__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(fmaf(a.x, b.x, -a.y * b.y), fmaf(a.x, b.y, a.y * b.x));
}

template <class Fn>
__device__ __forceinline__ void with_factor(int f, Fn fn) {
  switch (f) {
    case 1: fn(std::integral_constant<int, 1>{}); break;
    case 2: fn(std::integral_constant<int, 2>{}); break;
    case 4: fn(std::integral_constant<int, 4>{}); break;
    case 8: fn(std::integral_constant<int, 8>{}); break;
    case 16: fn(std::integral_constant<int, 16>{}); break;
    default: fn(std::integral_constant<int, 32>{}); break;
  }
}

// out(line, k) = sum_n in(line, n) * W(n, k) for the lines of this thread; Ws[k * F + n] = W(n, k).  The inputs of a
// line stay in registers; the outputs are produced a few at a time (four independent FMA chains each) so that the
// register count does not grow with F * F.
template <int F, class In, class Out>
__device__ __forceinline__ void dft_lines(const float2* __restrict__ Ws, int lines, In in, Out out) {
  for (int line = threadIdx.x; line < lines; line += blockDim.x) {
    float2 x[F];
#pragma unroll
    for (int n = 0; n < F; ++n) x[n] = in(line, n);
#pragma unroll 4
    for (int k = 0; k < F; ++k) {
      float rr = 0.f, ii = 0.f, ri = 0.f, ir = 0.f;
#pragma unroll
      for (int n = 0; n < F; ++n) {
        const float2 w = Ws[k * F + n];
        rr = fmaf(x[n].x, w.x, rr);
        ii = fmaf(x[n].y, w.y, ii);
        ri = fmaf(x[n].x, w.y, ri);
        ir = fmaf(x[n].y, w.x, ir);
      }
      out(line, k, make_float2(rr - ii, ri + ir));
    }
  }
}

// Copies a (2, F, F) DFT matrix into shared memory: the complex element W(i, j) sits at i + F * j in both, which is
// the Ws[k * F + n] = W(n, k) that dft_lines reads.
__device__ __forceinline__ void load_dft(float2* Ws, const float2* __restrict__ W, int F) {
  for (int e = threadIdx.x; e < F * F; e += blockDim.x) Ws[e] = __ldg(W + e);
}

__global__ void __launch_bounds__(256)
fft_kernel(const float2* __restrict__ x, float2* __restrict__ y, const float2* __restrict__ W0, const float2* __restrict__ W1,
           const float2* __restrict__ W2, const float2* __restrict__ T0, const float2* __restrict__ T1, int F0, int F1, int F2) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int N = F0 * F1 * F2, F1F2 = F1 * F2, F0F2 = F0 * F2, F0F1 = F0 * F1;
  const int padded = pad16(N - 1) + 1;
  float2* A = reinterpret_cast<float2*>(smem_raw);
  float2* B = A + padded;
  float2* Ws0 = B + padded;
  float2* Ws1 = Ws0 + F0 * F0;
  float2* Ws2 = Ws1 + F1 * F1;
  load_dft(Ws0, W0, F0);
  load_dft(Ws1, W1, F1);
  load_dft(Ws2, W2, F2);
  __syncthreads();

  const float2* __restrict__ xb = x + (size_t)blockIdx.x * N;
  float2* __restrict__ yb = y + (size_t)blockIdx.x * N;

  with_factor(F0, [&](auto f) {
    constexpr int F = decltype(f)::value;
    dft_lines<F>(
        Ws0, F1F2, [&](int j, int n0) { return __ldcs(xb + j + F1F2 * n0); },
        [&](int j, int k0, float2 v) { A[pad16(F * j + k0)] = cmul(v, __ldg(T0 + j + F1F2 * k0)); });
  });
  __syncthreads();
  with_factor(F1, [&](auto f) {
    constexpr int F = decltype(f)::value;
    dft_lines<F>(
        Ws1, F0F2, [&](int r, int n1) { return A[pad16(r + F0F2 * n1)]; },
        [&](int r, int k1, float2 v) { B[pad16(F * r + k1)] = cmul(v, __ldg(T1 + r / F0 + F2 * k1)); });
  });
  __syncthreads();
  with_factor(F2, [&](auto f) {
    constexpr int F = decltype(f)::value;
    dft_lines<F>(
        Ws2, F0F1,
        [&](int t, int n2) {
          const int k1 = t / F0, k0 = t - k1 * F0;
          return B[pad16(k1 + F1 * k0 + F0F1 * n2)];
        },
        [&](int t, int k2, float2 v) { __stcs(yb + t + F0F1 * k2, v); });
  });
}

size_t fft_smem_bytes(int N, int F0, int F1, int F2) {
  const size_t padded = (size_t)(N - 1) + ((N - 1) >> 4) + 1;
  return (2 * padded + (size_t)F0 * F0 + (size_t)F1 * F1 + (size_t)F2 * F2) * sizeof(float2);
}

}  // namespace

extern "C" int ctb_fft(ctb_ctx* ctx, void* stream, const void* x, void* y, const void* W0, const void* W1, const void* W2,
                       const void* T0, const void* T1, int64_t N, int F0, int F1, int F2, int64_t batch, int BS, int D) {
  CTB_CHECK_CTX(ctx);
  for (int f : {F0, F1, F2})
    if (f < 1 || !is_pow2(f)) return fail(CTB_UNSUPPORTED_TILE, "ctb_fft: factors must be powers of two (got %d)", f);
  for (int f : {F0, F1, F2})
    if (f > kMaxFactor) return fail(CTB_UNSUPPORTED, "ctb_fft: factors up to %d are implemented (got %d)", kMaxFactor, f);
  if (N != (int64_t)F0 * F1 * F2) return fail(CTB_BAD_ARG, "ctb_fft: N must equal F0 * F1 * F2");
  if (N > kMaxN) return fail(CTB_UNSUPPORTED, "ctb_fft: N up to %d is implemented", kMaxN);
  if (batch < 0 || BS < 1 || batch % BS != 0) return fail(CTB_BAD_ARG, "ctb_fft: batch must be a non-negative multiple of BS");
  if (!is_pow2(BS)) return fail(CTB_UNSUPPORTED_TILE, "ctb_fft: BS must be a power of two");
  if (D < 2 || !is_pow2(D) || (2 * N) % D != 0)
    return fail(CTB_BAD_ARG, "ctb_fft: 2 * N must be divisible by atom_packing_dim (a power of two >= 2)");
  if (batch > INT32_MAX) return fail(CTB_BAD_ARG, "ctb_fft: batch too large");
  if (batch == 0) return CTB_OK;
  CTB_CHECK_DEV(x); CTB_CHECK_DEV(y); CTB_CHECK_DEV(W0); CTB_CHECK_DEV(W1); CTB_CHECK_DEV(W2); CTB_CHECK_DEV(T0); CTB_CHECK_DEV(T1);
  for (const void* p : {x, (const void*)y, W0, W1, W2, T0, T1})
    if ((uintptr_t)p % 8 != 0) return fail(CTB_BAD_ALIGN, "ctb_fft: arrays must be 8-byte aligned");
  const size_t smem = fft_smem_bytes((int)N, F0, F1, F2);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(fft_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_fft: shared memory attribute");
  }
  const int lines = (int)(N / std::min(F0, std::min(F1, F2)));
  const int threads = std::min(256, std::max(32, (lines + 31) / 32 * 32));
  fft_kernel<<<(unsigned)batch, threads, smem, static_cast<cudaStream_t>(stream)>>>(
      (const float2*)x, (float2*)y, (const float2*)W0, (const float2*)W1, (const float2*)W2, (const float2*)T0, (const float2*)T1,
      F0, F1, F2);
  CTB_CHECK_LAUNCH("ctb_fft launch");
  return CTB_OK;
}
