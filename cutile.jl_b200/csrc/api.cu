// Context, error reporting, scratch and tensor-map helpers of libcutile_b200.
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "ctx.h"

namespace ctb_internal {

static thread_local char g_err[512] = "";

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof g_err, fmt, ap);
  va_end(ap);
  return status;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(CTB_CUDA_ERROR, "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
}

bool is_pow2(long long v) { return v > 0 && (v & (v - 1)) == 0; }

bool is_device_ptr(const void* p) {
  if (!p) return false;
  cudaPointerAttributes a;
  cudaError_t e = cudaPointerGetAttributes(&a, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

int workspace(ctb_ctx* ctx, size_t bytes, void** out, cudaStream_t stream) {
  if (bytes > ctx->workspace_bytes) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) cudaGetLastError();
    if (cap != cudaStreamCaptureStatusNone)
      return fail(CTB_UNSUPPORTED, "the context's scratch would have to grow to %zu bytes while the stream is being "
                  "captured; call ctb_reserve_workspace before the capture", bytes);
    if (ctx->workspace) {
      cudaError_t e = cudaDeviceSynchronize();
      if (e != cudaSuccess) return cuda_fail(e, "workspace: synchronize before regrow");
      cudaFree(ctx->workspace);
      ctx->workspace = nullptr;
      ctx->workspace_bytes = 0;
    }
    size_t want = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    cudaError_t e = cudaMalloc(&ctx->workspace, want);
    if (e != cudaSuccess) return cuda_fail(e, "workspace: cudaMalloc");
    ctx->workspace_bytes = want;
  }
  *out = ctx->workspace;
  return CTB_OK;
}

int* sched_slot(ctb_ctx* ctx) {
  const unsigned n = __atomic_fetch_add(&ctx->sched_next, 1u, __ATOMIC_RELAXED);
  return ctx->sched_pool + 2 * (n % kSchedSlots);
}

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    else
      cudaGetLastError();
  });
  return fn;
}

int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return fail(CTB_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gdim[5], gstr[5];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = enc(out, dt, rank, const_cast<void*>(base), gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(CTB_BAD_ALIGN,
                "tensor map rejected (CUresult %d): base %p must be 16-byte aligned and strides multiples of 16 bytes",
                (int)r, base);
  return CTB_OK;
}

}  // namespace ctb_internal

using namespace ctb_internal;

extern "C" {

int ctb_create(ctb_ctx** out, int device) {
  if (!out) return fail(CTB_BAD_ARG, "ctb_create: null output pointer");
  *out = nullptr;
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n == 0) {
    cudaGetLastError();
    return fail(CTB_NO_DEVICE, "ctb_create: no CUDA device (%s); this library has no CPU path",
                e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  }
  if (device < 0 || device >= n) return fail(CTB_BAD_ARG, "ctb_create: device %d out of range [0,%d)", device, n);
  cudaDeviceProp p;
  e = cudaGetDeviceProperties(&p, device);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_create: cudaGetDeviceProperties");
  if (p.major != 10)
    return fail(CTB_NO_DEVICE, "ctb_create: device %d is sm_%d%d; the kernels are built for sm_100a only", device,
                p.major, p.minor);
  e = cudaSetDevice(device);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_create: cudaSetDevice");
  ctb_ctx* c = new ctb_ctx();
  c->device = device;
  c->sm_count = p.multiProcessorCount;
  c->cc_major = p.major;
  c->cc_minor = p.minor;
  c->workspace = nullptr;
  c->workspace_bytes = 0;
  c->sched_pool = nullptr;
  c->sched_next = 0;
  c->flag_wait_ns = 2000000000ull;
  c->tf32_rne = 0;
  c->comm = nullptr;
  e = cudaMalloc(&c->dev_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->dev_status, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaMalloc(&c->sched_pool, 2 * kSchedSlots * sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->sched_pool, 0, 2 * kSchedSlots * sizeof(int));
  if (e != cudaSuccess) {
    delete c;
    return cuda_fail(e, "ctb_create: status word");
  }
  *out = c;
  return CTB_OK;
}

void ctb_destroy(ctb_ctx* ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  comm_release(ctx);
  if (ctx->workspace) cudaFree(ctx->workspace);
  if (ctx->dev_status) cudaFree(ctx->dev_status);
  if (ctx->sched_pool) cudaFree(ctx->sched_pool);
  delete ctx;
}

const char* ctb_last_error(void) { return g_err; }

const char* ctb_status_string(int s) {
  switch (s) {
    case CTB_OK: return "OK";
    case CTB_BAD_ARG: return "BAD_ARG";
    case CTB_BAD_ALIGN: return "BAD_ALIGN";
    case CTB_UNSUPPORTED_TILE: return "UNSUPPORTED_TILE";
    case CTB_UNSUPPORTED: return "UNSUPPORTED";
    case CTB_CUDA_ERROR: return "CUDA_ERROR";
    case CTB_NCCL_ERROR: return "NCCL_ERROR";
    case CTB_TIMEOUT: return "TIMEOUT";
    case CTB_NO_DEVICE: return "NO_DEVICE";
  }
  return "UNKNOWN";
}

int ctb_version_info(char* buf, size_t n) {
  if (!buf || n == 0) return fail(CTB_BAD_ARG, "ctb_version_info: empty buffer");
  int rt = 0, drv = 0;
  cudaRuntimeGetVersion(&rt);
  if (cudaDriverGetVersion(&drv) != cudaSuccess) {
    cudaGetLastError();
    drv = 0;
  }
  snprintf(buf, n, "libcutile_b200 0.1.0; target sm_100a; CUDA runtime %d.%d; driver API %d.%d", rt / 1000,
           (rt % 1000) / 10, drv / 1000, (drv % 1000) / 10);
  return CTB_OK;
}

int ctb_validate_hints(int num_ctas, int occupancy, int opt_level, int num_worker_warps) {
  // the reference's validate_hint (src/language/types.jl:864-882); CTB_HINT_UNSET = the keyword was not given
  if (num_ctas != CTB_HINT_UNSET) {
    if (num_ctas < 1 || num_ctas > 16) return fail(CTB_BAD_ARG, "num_ctas must be between 1 and 16, got %d", num_ctas);
    if (!is_pow2(num_ctas)) return fail(CTB_BAD_ARG, "num_ctas must be a power of 2, got %d", num_ctas);
  }
  if (occupancy != CTB_HINT_UNSET && (occupancy < 1 || occupancy > 32))
    return fail(CTB_BAD_ARG, "occupancy must be between 1 and 32, got %d", occupancy);
  if (opt_level != CTB_HINT_UNSET && (opt_level < 0 || opt_level > 3))
    return fail(CTB_BAD_ARG, "opt_level must be between 0 and 3, got %d", opt_level);
  if (num_worker_warps != CTB_HINT_UNSET && num_worker_warps != 4 && num_worker_warps != 8)
    return fail(CTB_BAD_ARG, "num_worker_warps must be either 4 or 8, got %d", num_worker_warps);
  return CTB_OK;
}

int ctb_set_flag_wait_limit(ctb_ctx* ctx, uint64_t nanoseconds) {
  CTB_CHECK_CTX(ctx);
  if (nanoseconds < 1000ull || nanoseconds > 10000000000ull)
    return fail(CTB_BAD_ARG, "ctb_set_flag_wait_limit: the limit must lie between 1 microsecond and 10 seconds");
  ctx->flag_wait_ns = nanoseconds;
  return CTB_OK;
}

int ctb_set_tf32_rounding(ctb_ctx* ctx, int nearest_even) {
  CTB_CHECK_CTX(ctx);
  if (nearest_even != 0 && nearest_even != 1) return fail(CTB_BAD_ARG, "ctb_set_tf32_rounding: mode must be 0 or 1");
  ctx->tf32_rne = nearest_even;
  return CTB_OK;
}

int ctb_check_device_status(ctb_ctx* ctx, void* stream) {
  CTB_CHECK_CTX(ctx);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_check_device_status");
  if (v == 0) return CTB_OK;
  cudaMemsetAsync(ctx->dev_status, 0, sizeof(int), s);
  cudaStreamSynchronize(s);
  if (v == 4) return fail(CTB_BAD_ARG, "a kernel read an out-of-range index from an index array");
  return fail(CTB_TIMEOUT, "a kernel gave up a bounded wait (device code %d: 1=TMA bytes, 2=MMA commit, 3=pipeline slot)",
              v);
}

}  // extern "C"
