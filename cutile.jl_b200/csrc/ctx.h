// Library-internal context, error reporting and argument checks shared by the
// per-kernel translation units.  Nothing here is part of the C ABI.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/cutile_b200.h"

struct ctb_ctx {
  int device;
  int sm_count;
  int cc_major, cc_minor;
  int* dev_status;        // one int in device memory; kernels atomicMax error codes into it
  void* workspace;        // grown on demand (ctb_internal::workspace)
  size_t workspace_bytes;
  // Work counters of kernels that hand out work items dynamically: kSchedSlots pairs of ints, zero between
  // launches (the last CTA of a launch clears its pair).  Launches take the pairs in turn, so that launches
  // that overlap on the device (different streams) do not share one.
  int* sched_pool;
  unsigned sched_next;
  void* comm;             // ctb_internal::Comm* once an NCCL communicator is attached (multi.cu)
  unsigned long long flag_wait_ns;  // how long a kernel waits for another rank's flag before it gives up
  int tf32_rne;           // 1: f32 GEMM operands are rounded to TF32 (nearest even) by a pass of their own first
};

namespace ctb_internal {

int fail(int status, const char* fmt, ...);  // sets the thread-local message, returns status
int cuda_fail(cudaError_t e, const char* what);
bool is_pow2(long long v);
// True when p looks like device (or managed) memory of the current context.
bool is_device_ptr(const void* p);
// Returns ctx scratch of at least `bytes`.  Growing it frees and reallocates (after a device synchronise), which is
// refused while `stream` is being captured; ctb_reserve_workspace sizes it up front.
int workspace(ctb_ctx* ctx, size_t bytes, void** out, cudaStream_t stream);
// Destroys the NCCL communicator attached to the context, if any (multi.cu).
void comm_release(ctb_ctx* ctx);
// Expert phase shared by the expert-parallel MoE paths (defined with the MoE kernels).
size_t moe_experts_rows_workspace(int64_t R, int64_t I, int64_t E_local, int tile_m);
int moe_experts_rows(ctb_ctx* ctx, cudaStream_t st, const void* rows, int64_t ld_rows, const int32_t* ids,
                     const void* gates, int64_t R, int64_t H, int64_t I, int64_t E_local, const void* w1_local,
                     const void* w2_local, int tile_m, void* C, int64_t ldc, void* const* c_peer, int64_t c_split);
constexpr int kSchedSlots = 256;
// The next pair of work counters of the context (see ctb_ctx::sched_pool).
int* sched_slot(ctb_ctx* ctx);

// cuTensorMapEncodeTiled, resolved through the runtime so that the library has
// no link-time dependency on libcuda and loads on machines without a driver.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled();

// rank-`rank` tiled map, zero fill.  dims/box in elements (innermost first),
// strides in bytes for dims 1..rank-1.
int make_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box,
              CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B);

#define CTB_CHECK_CTX(ctx)                                                              \
  do {                                                                                  \
    if (!(ctx)) return ctb_internal::fail(CTB_BAD_ARG, "%s: null context", __func__);   \
  } while (0)

#define CTB_CHECK_DEV(p)                                                                          \
  do {                                                                                            \
    if (!ctb_internal::is_device_ptr(p))                                                          \
      return ctb_internal::fail(CTB_BAD_ARG, "%s: argument %s is not a device pointer", __func__, #p); \
  } while (0)

#define CTB_CHECK_LAUNCH(what)                                     \
  do {                                                             \
    cudaError_t e__ = cudaGetLastError();                          \
    if (e__ != cudaSuccess) return ctb_internal::cuda_fail(e__, what); \
  } while (0)

}  // namespace ctb_internal
