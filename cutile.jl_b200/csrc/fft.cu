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
// (the DFT matrix is broadcast from shared memory; packed two-wide FMAs), so the input is read from global memory once, coalesced, the two
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

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {  // (a.x * b.x + c.x, a.y * b.y + c.y), one instruction
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}

// out(line, k) = tw(line, k) * sum_n in(line, n) * W(n, k) for the lines of this thread.  The DFT matrix sits in
// shared memory as two planes, Wre[n * F + k] and Wim[n * F + k].  The inputs of a line stay in registers (each part
// duplicated into a register pair); the outputs are produced four at a time with packed two-wide FMAs - a pair of
// neighbouring outputs per instruction, eight independent chains - from two 16-byte broadcast loads per input, and
// the twiddle factors of the next four are fetched (global memory, read-only path) before the current four are
// computed.  F = 32 takes the scalar form.  (Measured no faster: two lines per thread with 128 threads, which halves
// the shared-memory reads of the matrix - 21.5 us against 16.3 us per 256 x 4096 points; the stages are bound by
// latency with 16 warps per SM, not by the FMA or shared-memory throughput.)
template <int F, class In, class Tw, class Out>
__device__ __forceinline__ void dft_lines(const float* __restrict__ Wre, const float* __restrict__ Wim, int lines, In in,
                                          Tw tw, Out out) {
  constexpr int KG = F < 4 ? F : 4;
  for (int line = threadIdx.x; line < lines; line += blockDim.x) {
    float2 x[F], t_next[KG];
#pragma unroll
    for (int n = 0; n < F; ++n) x[n] = in(line, n);
#pragma unroll
    for (int i = 0; i < KG; ++i) t_next[i] = tw(line, i);
#pragma unroll 1
    for (int k0 = 0; k0 < F; k0 += KG) {
      float2 t[KG], res[KG];
#pragma unroll
      for (int i = 0; i < KG; ++i) t[i] = t_next[i];
      if (k0 + KG < F) {
#pragma unroll
        for (int i = 0; i < KG; ++i) t_next[i] = tw(line, k0 + KG + i);
      }
      if constexpr (KG == 4 && F <= 16) {
        float2 rr[2], ii[2], ri[2], ir[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) rr[h] = ii[h] = ri[h] = ir[h] = make_float2(0.f, 0.f);
#pragma unroll
        for (int n = 0; n < F; ++n) {
          const float4 wr = *reinterpret_cast<const float4*>(Wre + n * F + k0);
          const float4 wi = *reinterpret_cast<const float4*>(Wim + n * F + k0);
          const float2 xr = make_float2(x[n].x, x[n].x), xi = make_float2(x[n].y, x[n].y);
          const float2 wr2[2] = {make_float2(wr.x, wr.y), make_float2(wr.z, wr.w)};
          const float2 wi2[2] = {make_float2(wi.x, wi.y), make_float2(wi.z, wi.w)};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            rr[h] = fma2(xr, wr2[h], rr[h]);
            ii[h] = fma2(xi, wi2[h], ii[h]);
            ri[h] = fma2(xr, wi2[h], ri[h]);
            ir[h] = fma2(xi, wr2[h], ir[h]);
          }
        }
        res[0] = make_float2(rr[0].x - ii[0].x, ri[0].x + ir[0].x);
        res[1] = make_float2(rr[0].y - ii[0].y, ri[0].y + ir[0].y);
        res[2] = make_float2(rr[1].x - ii[1].x, ri[1].x + ir[1].x);
        res[3] = make_float2(rr[1].y - ii[1].y, ri[1].y + ir[1].y);
      } else {
#pragma unroll
        for (int i = 0; i < KG; ++i) {
          const int k = k0 + i;
          float rr = 0.f, ii = 0.f, ri = 0.f, ir = 0.f;
#pragma unroll
          for (int n = 0; n < F; ++n) {
            const float wr = Wre[n * F + k], wi = Wim[n * F + k];
            rr = fmaf(x[n].x, wr, rr);
            ii = fmaf(x[n].y, wi, ii);
            ri = fmaf(x[n].x, wi, ri);
            ir = fmaf(x[n].y, wr, ir);
          }
          res[i] = make_float2(rr - ii, ri + ir);
        }
      }
#pragma unroll
      for (int i = 0; i < KG; ++i) out(line, k0 + i, cmul(res[i], t[i]));
    }
  }
}

// Splits a (2, F, F) DFT matrix (complex element W(i, j) at i + F * j) into the planes Wre[n * F + k] = Re W(n, k)
// and Wim[n * F + k] = Im W(n, k), Wim directly behind Wre.
__device__ __forceinline__ void load_dft(float* Wre, const float2* __restrict__ W, int F) {
  float* Wim = Wre + F * F;
  for (int e = threadIdx.x; e < F * F; e += blockDim.x) {
    const int n = e / F, k = e - n * F;
    const float2 w = __ldg(W + n + F * k);
    Wre[e] = w.x;
    Wim[e] = w.y;
  }
}

__global__ void __launch_bounds__(256, 2)
fft_kernel(const float2* __restrict__ x, float2* __restrict__ y, const float2* __restrict__ W0, const float2* __restrict__ W1,
           const float2* __restrict__ W2, const float2* __restrict__ T0, const float2* __restrict__ T1, int F0, int F1, int F2) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int N = F0 * F1 * F2, F1F2 = F1 * F2, F0F2 = F0 * F2, F0F1 = F0 * F1;
  const int padded = (pad16(N - 1) + 2) & ~1;  // elements per intermediate array, even: every region starts on 16 bytes
  float2* A = reinterpret_cast<float2*>(smem_raw);
  float2* B = A + padded;
  float* Ws0 = reinterpret_cast<float*>(B + padded);  // 16-byte aligned planes (read with 16-byte loads)
  float* Ws1 = Ws0 + ((2 * F0 * F0 + 3) & ~3);
  float* Ws2 = Ws1 + ((2 * F1 * F1 + 3) & ~3);
  load_dft(Ws0, W0, F0);
  load_dft(Ws1, W1, F1);
  load_dft(Ws2, W2, F2);
  __syncthreads();

  const float2* __restrict__ xb = x + (size_t)blockIdx.x * N;
  float2* __restrict__ yb = y + (size_t)blockIdx.x * N;

  with_factor(F0, [&](auto f) {
    constexpr int F = decltype(f)::value;
    dft_lines<F>(
        Ws0, Ws0 + F * F, F1F2, [&](int j, int n0) { return __ldcs(xb + j + F1F2 * n0); },
        [&](int j, int k0) { return __ldg(T0 + j + F1F2 * k0); },
        [&](int j, int k0, float2 v) { A[pad16(F * j + k0)] = v; });
  });
  __syncthreads();
  with_factor(F1, [&](auto f) {
    constexpr int F = decltype(f)::value;
    dft_lines<F>(
        Ws1, Ws1 + F * F, F0F2, [&](int r, int n1) { return A[pad16(r + F0F2 * n1)]; },
        [&](int r, int k1) { return __ldg(T1 + r / F0 + F2 * k1); },
        [&](int r, int k1, float2 v) { B[pad16(F * r + k1)] = v; });
  });
  __syncthreads();
  with_factor(F2, [&](auto f) {
    constexpr int F = decltype(f)::value;
    dft_lines<F>(
        Ws2, Ws2 + F * F, F0F1,
        [&](int t, int n2) {
          const int k1 = t / F0, k0 = t - k1 * F0;
          return B[pad16(k1 + F1 * k0 + F0F1 * n2)];
        },
        [&](int, int) { return make_float2(1.f, 0.f); },
        [&](int t, int k2, float2 v) { __stcs(yb + t + F0F1 * k2, v); });
  });
}

size_t fft_smem_bytes(int N, int F0, int F1, int F2) {
  const size_t padded = ((size_t)(N - 1) + ((N - 1) >> 4) + 2) & ~(size_t)1;
  return (2 * padded + (size_t)F0 * F0 + (size_t)F1 * F1 + (size_t)F2 * F2 + 4) * sizeof(float2);
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
