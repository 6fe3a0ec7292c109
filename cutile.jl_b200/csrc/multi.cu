// Multi-GPU side of libcutile_b200: groups of per-device contexts, NCCL communicators owned by the
// library, batch-sharded launches of the batched GEMM and of FMHA, and the expert-parallel MoE FFN
// with its token exchange either as NCCL send/receive pairs or as stores into peer memory.
//
// The reference is single-GPU (its MoE host wrapper, examples/moe.jl:218-257, runs on one device and
// one stream); the partitioning is that of the benchmark configuration: batched GEMM and FMHA split
// by batch with no communication, MoE expert-parallel with experts [r*E/N, (r+1)*E/N) on rank r and
// the tokens sharded by rank.
//
// NCCL is loaded at run time (dlopen of libnccl.so.2): a host process that already carries an NCCL
// (a Python process with torch, a Julia process with NCCL.jl) then shares that copy, and the library
// itself links against nothing but the CUDA runtime.  Only the public entry points are used.
#include <dlfcn.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "ctx.h"
#include "ptx.cuh"

using namespace ctb;
using namespace ctb_internal;

// ------------------------------------------------------------------ NCCL, resolved at run time
namespace {

typedef struct ncclComm* ncclComm_t;
struct NcclUniqueId {
  char internal[CTB_UNIQUE_ID_BYTES];
};
enum { kNcclSuccess = 0, kNcclInt32 = 2, kNcclUint8 = 1, kNcclFloat16 = 6 };

struct NcclApi {
  void* handle = nullptr;
  int (*GetVersion)(int*) = nullptr;
  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*Send)(const void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  char why[200] = "";
};

NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) {
      snprintf(api.why, sizeof api.why, "libnccl.so.2 could not be loaded (%s)", dlerror());
      return;
    }
    bool ok = true;
    auto sym = [&](const char* name) {
      void* p = dlsym(api.handle, name);
      if (!p) {
        ok = false;
        snprintf(api.why, sizeof api.why, "NCCL symbol %s is missing", name);
      }
      return p;
    };
    api.GetVersion = reinterpret_cast<int (*)(int*)>(sym("ncclGetVersion"));
    api.GetUniqueId = reinterpret_cast<int (*)(NcclUniqueId*)>(sym("ncclGetUniqueId"));
    api.CommInitAll = reinterpret_cast<int (*)(ncclComm_t*, int, const int*)>(sym("ncclCommInitAll"));
    api.CommInitRank = reinterpret_cast<int (*)(ncclComm_t*, int, NcclUniqueId, int)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<int (*)(ncclComm_t)>(sym("ncclCommDestroy"));
    api.CommAbort = reinterpret_cast<int (*)(ncclComm_t)>(sym("ncclCommAbort"));
    api.GroupStart = reinterpret_cast<int (*)()>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<int (*)()>(sym("ncclGroupEnd"));
    api.Send = reinterpret_cast<int (*)(const void*, size_t, int, int, ncclComm_t, cudaStream_t)>(sym("ncclSend"));
    api.Recv = reinterpret_cast<int (*)(void*, size_t, int, int, ncclComm_t, cudaStream_t)>(sym("ncclRecv"));
    api.GetErrorString = reinterpret_cast<const char* (*)(int)>(sym("ncclGetErrorString"));
    if (!ok) {
      dlclose(api.handle);
      api.handle = nullptr;
    }
  });
  return &api;
}

int nccl_fail(int code, const char* what) {
  NcclApi* a = nccl_api();
  return fail(CTB_NCCL_ERROR, "%s: %s", what, (a->handle && a->GetErrorString) ? a->GetErrorString(code) : "NCCL error");
}
#define CTB_NCCL(call, what)                         \
  do {                                               \
    const int rc__ = (call);                         \
    if (rc__ != kNcclSuccess) return nccl_fail(rc__, what); \
  } while (0)

struct Comm {
  ncclComm_t comm;
  int rank, world;
};

int need_nccl(NcclApi** out) {
  NcclApi* a = nccl_api();
  if (!a->handle) return fail(CTB_NCCL_ERROR, "NCCL is not available: %s", a->why);
  *out = a;
  return CTB_OK;
}

}  // namespace

struct ctb_group {
  std::vector<ctb_ctx*> ctx;
  std::vector<int> devices;
};

// Releases what ctb_destroy cannot know about.  Called from ctb_destroy.
namespace ctb_internal {
void comm_release(ctb_ctx* ctx) {
  if (!ctx->comm) return;
  Comm* c = static_cast<Comm*>(ctx->comm);
  NcclApi* a = nccl_api();
  if (a->handle && c->comm) a->CommDestroy(c->comm);
  delete c;
  ctx->comm = nullptr;
}
}  // namespace ctb_internal

extern "C" {

int ctb_create_multi(ctb_group** out, const int* devices, int ndev) {
  if (!out) return fail(CTB_BAD_ARG, "ctb_create_multi: null output pointer");
  *out = nullptr;
  if (!devices || ndev < 1 || ndev > CTB_EP_MAX_RANKS)
    return fail(CTB_BAD_ARG, "ctb_create_multi: need a list of 1..%d devices (got %d)", CTB_EP_MAX_RANKS, ndev);
  for (int i = 0; i < ndev; ++i)
    for (int j = 0; j < i; ++j)
      if (devices[i] == devices[j]) return fail(CTB_BAD_ARG, "ctb_create_multi: device %d is listed twice", devices[i]);
  int prev = 0;
  cudaGetDevice(&prev);
  ctb_group* g = new ctb_group();
  int r = CTB_OK;
  for (int i = 0; i < ndev && r == CTB_OK; ++i) {
    ctb_ctx* c = nullptr;
    r = ctb_create(&c, devices[i]);
    if (r == CTB_OK) {
      g->ctx.push_back(c);
      g->devices.push_back(devices[i]);
    }
  }
  // every device can read and write every other device's memory (kernels of this library store into peer buffers)
  for (int i = 0; i < ndev && r == CTB_OK; ++i) {
    cudaSetDevice(devices[i]);
    for (int j = 0; j < ndev && r == CTB_OK; ++j) {
      if (i == j) continue;
      int can = 0;
      cudaError_t e = cudaDeviceCanAccessPeer(&can, devices[i], devices[j]);
      if (e != cudaSuccess || !can) {
        cudaGetLastError();
        r = fail(CTB_UNSUPPORTED, "ctb_create_multi: device %d cannot access device %d's memory", devices[i], devices[j]);
        break;
      }
      e = cudaDeviceEnablePeerAccess(devices[j], 0);
      if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
      else if (e != cudaSuccess) r = cuda_fail(e, "ctb_create_multi: cudaDeviceEnablePeerAccess");
    }
  }
  if (r == CTB_OK && ndev > 1) {
    NcclApi* a = nullptr;
    r = need_nccl(&a);
    if (r == CTB_OK) {
      std::vector<ncclComm_t> comms(ndev, nullptr);
      const int rc = a->CommInitAll(comms.data(), ndev, devices);
      if (rc != kNcclSuccess) r = nccl_fail(rc, "ctb_create_multi: ncclCommInitAll");
      else
        for (int i = 0; i < ndev; ++i) g->ctx[i]->comm = new Comm{comms[i], i, ndev};
    }
  }
  cudaSetDevice(prev);
  if (r != CTB_OK) {
    ctb_destroy_multi(g);
    return r;
  }
  *out = g;
  return CTB_OK;
}

void ctb_destroy_multi(ctb_group* g) {
  if (!g) return;
  for (ctb_ctx* c : g->ctx) ctb_destroy(c);
  delete g;
}

int ctb_group_size(const ctb_group* g) { return g ? (int)g->ctx.size() : 0; }

ctb_ctx* ctb_group_ctx(ctb_group* g, int i) {
  if (!g || i < 0 || i >= (int)g->ctx.size()) {
    fail(CTB_BAD_ARG, "ctb_group_ctx: index %d out of range", i);
    return nullptr;
  }
  return g->ctx[i];
}

int ctb_comm_unique_id(void* id) {
  if (!id) return fail(CTB_BAD_ARG, "ctb_comm_unique_id: null buffer");
  NcclApi* a = nullptr;
  int r = need_nccl(&a);
  if (r) return r;
  NcclUniqueId u;
  CTB_NCCL(a->GetUniqueId(&u), "ctb_comm_unique_id: ncclGetUniqueId");
  memcpy(id, &u, sizeof u);
  return CTB_OK;
}

int ctb_comm_init_rank(ctb_ctx* ctx, const void* id, int rank, int world) {
  CTB_CHECK_CTX(ctx);
  if (!id) return fail(CTB_BAD_ARG, "ctb_comm_init_rank: null id");
  if (world < 1 || world > CTB_EP_MAX_RANKS || rank < 0 || rank >= world)
    return fail(CTB_BAD_ARG, "ctb_comm_init_rank: rank %d / world %d out of range (at most %d ranks)", rank, world,
                CTB_EP_MAX_RANKS);
  if (ctx->comm) return fail(CTB_BAD_ARG, "ctb_comm_init_rank: the context already has a communicator");
  NcclApi* a = nullptr;
  int r = need_nccl(&a);
  if (r) return r;
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_comm_init_rank: cudaSetDevice");
  NcclUniqueId u;
  memcpy(&u, id, sizeof u);
  ncclComm_t c = nullptr;
  CTB_NCCL(a->CommInitRank(&c, world, u, rank), "ctb_comm_init_rank: ncclCommInitRank");
  ctx->comm = new Comm{c, rank, world};
  return CTB_OK;
}

int ctb_comm_abort(ctb_ctx* ctx) {
  CTB_CHECK_CTX(ctx);
  if (!ctx->comm) return CTB_OK;
  Comm* c = static_cast<Comm*>(ctx->comm);
  NcclApi* a = nccl_api();
  int rc = kNcclSuccess;
  if (a->handle && c->comm) rc = a->CommAbort(c->comm);
  delete c;
  ctx->comm = nullptr;
  if (rc != kNcclSuccess) return nccl_fail(rc, "ctb_comm_abort: ncclCommAbort");
  return CTB_OK;
}

int ctb_comm_info(ctb_ctx* ctx, int* rank, int* world, int* nccl_version) {
  CTB_CHECK_CTX(ctx);
  Comm* c = static_cast<Comm*>(ctx->comm);
  if (rank) *rank = c ? c->rank : 0;
  if (world) *world = c ? c->world : 1;
  if (nccl_version) {
    *nccl_version = 0;
    NcclApi* a = nccl_api();
    if (a->handle) a->GetVersion(nccl_version);
  }
  return CTB_OK;
}

// ------------------------------------------------------------------ batch-sharded launches (no communication)
int ctb_gemm_batched_sharded(ctb_group* g, void* const* streams, const void* const* A, const void* const* B,
                             void* const* C, int64_t M, int64_t N, int64_t K, const int64_t* batch_per_dev, int64_t lda,
                             int64_t ldb, int64_t ldc, int64_t strideA, int64_t strideB, int64_t strideC, int dtype,
                             int tm, int tn, int tk) {
  if (!g) return fail(CTB_BAD_ARG, "ctb_gemm_batched_sharded: null group");
  if (!streams || !A || !B || !C || !batch_per_dev) return fail(CTB_BAD_ARG, "ctb_gemm_batched_sharded: null argument table");
  int prev = 0;
  cudaGetDevice(&prev);
  int r = CTB_OK;
  for (size_t i = 0; i < g->ctx.size() && r == CTB_OK; ++i) {
    if (batch_per_dev[i] < 0) r = fail(CTB_BAD_ARG, "ctb_gemm_batched_sharded: negative batch count for device %zu", i);
    if (batch_per_dev[i] <= 0) continue;
    cudaSetDevice(g->devices[i]);
    r = ctb_gemm_batched(g->ctx[i], streams[i], A[i], B[i], C[i], M, N, K, batch_per_dev[i], lda, ldb, ldc, strideA,
                         strideB, strideC, dtype, tm, tn, tk);
  }
  cudaSetDevice(prev);
  return r;
}

int ctb_fmha_fwd_sharded(ctb_group* g, void* const* streams, const void* const* Q, const void* const* K,
                         const void* const* V, void* const* Out, int64_t d_k, int64_t d_v, int64_t seq_q,
                         int64_t seq_kv, int64_t heads, int64_t kv_heads, const int64_t* batch_per_dev, float qk_scale,
                         int32_t input_pos, int tile_m, int tile_n, int query_group_size, int causal, int dtype) {
  if (!g) return fail(CTB_BAD_ARG, "ctb_fmha_fwd_sharded: null group");
  if (!streams || !Q || !K || !V || !Out || !batch_per_dev) return fail(CTB_BAD_ARG, "ctb_fmha_fwd_sharded: null argument table");
  int prev = 0;
  cudaGetDevice(&prev);
  int r = CTB_OK;
  for (size_t i = 0; i < g->ctx.size() && r == CTB_OK; ++i) {
    if (batch_per_dev[i] < 0) r = fail(CTB_BAD_ARG, "ctb_fmha_fwd_sharded: negative batch count for device %zu", i);
    if (batch_per_dev[i] <= 0) continue;
    cudaSetDevice(g->devices[i]);
    r = ctb_fmha_fwd(g->ctx[i], streams[i], Q[i], K[i], V[i], Out[i], d_k, d_v, seq_q, seq_kv, heads, kv_heads,
                     batch_per_dev[i], qk_scale, input_pos, tile_m, tile_n, query_group_size, causal, dtype);
  }
  cudaSetDevice(prev);
  return r;
}

}  // extern "C"

// ------------------------------------------------------------------ expert-parallel MoE
namespace {

// Per-rank state of the expert-parallel MoE: ONE device allocation that peers map (by pointer inside one process,
// by a CUDA IPC handle across processes), plus local staging for the NCCL exchange.
//   shared block: recv_rows (N*cap, H) f16 | recv_ids (N*cap) i32 | recv_gates (N*cap) f16 | slot_out (cap, H) f16 |
//                 flags (N) u32 | epoch u32
//   local block:  send_rows (cap, H) | send_ids (cap) | send_gates (cap) | order (cap) | back_rows (cap, H) |
//                 y_rows (N*cap, H) | counters
struct EpLayout {
  size_t recv_rows, recv_ids, recv_gates, slot_out, flags, epoch, bytes;
};
EpLayout ep_layout(int world, int64_t cap, int64_t H) {
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  EpLayout L;
  const size_t R = (size_t)world * cap;
  L.recv_rows = 0;
  L.recv_ids = up(R * H * 2);
  L.recv_gates = L.recv_ids + up(R * 4);
  L.slot_out = L.recv_gates + up(R * 2);
  L.flags = L.slot_out + up((size_t)cap * H * 2);
  L.epoch = L.flags + 256;
  L.bytes = L.epoch + 256;
  return L;
}

}  // namespace

struct ctb_ep {
  ctb_ctx* ctx;
  int world, rank;
  int64_t T, H, topk, cap;
  EpLayout L;
  unsigned char* shared;                         // this rank's shared block
  unsigned char* peer[CTB_EP_MAX_RANKS];         // every rank's shared block as seen from this device
  bool peer_ipc[CTB_EP_MAX_RANKS];               // opened with cudaIpcOpenMemHandle (must be closed)
  ctb_ep_buffers table;
  // NCCL mode
  unsigned char* local;
  __half *send_rows, *back_rows, *y_rows;
  int *send_ids, *order, *dest, *pos;            // dest/pos: destination rank of a slot and its place among that rank's
  int* counters;                                 // [0..8) send counts, [16..24) received counts
  __half* send_gates;
  int* host_counts;                              // pinned: [0..N) send counts, [N..2N) receive counts
};

namespace {

void ep_fill_table(ctb_ep* ep) {
  ctb_ep_buffers& t = ep->table;
  memset(&t, 0, sizeof t);
  t.world = ep->world;
  t.rank = ep->rank;
  for (int q = 0; q < ep->world; ++q) {
    unsigned char* b = ep->peer[q];
    if (!b) continue;
    t.recv_rows[q] = b + ep->L.recv_rows;
    t.recv_ids[q] = reinterpret_cast<int32_t*>(b + ep->L.recv_ids);
    t.recv_gates[q] = b + ep->L.recv_gates;
    t.slot_out[q] = b + ep->L.slot_out;
    t.flags[q] = reinterpret_cast<uint32_t*>(b + ep->L.flags);
  }
  t.epoch = reinterpret_cast<uint32_t*>(ep->shared + ep->L.epoch);
}

int ep_connected(const ctb_ep* ep, const char* who) {
  for (int q = 0; q < ep->world; ++q)
    if (!ep->peer[q]) return fail(CTB_BAD_ARG, "%s: the buffers of rank %d have not been imported", who, q);
  return CTB_OK;
}

// counts[d] = local slots whose expert lives on rank d; pos[slot] = the slot's position among those of its rank.
// One CTA: the slots of a rank are few thousand at most.
__global__ void ep_count_kernel(const int* __restrict__ topk_ids, int T, int topk, int E, int El, int world,
                                int* __restrict__ counts, int* __restrict__ dest, int* __restrict__ pos, int* status) {
  __shared__ int c[CTB_EP_MAX_RANKS];
  if (threadIdx.x < CTB_EP_MAX_RANKS) c[threadIdx.x] = 0;
  __syncthreads();
  const int cap = T * topk;
  for (int s = threadIdx.x; s < cap; s += blockDim.x) {
    const int t = s / topk, k = s - t * topk;
    const int e = topk_ids[(long long)k * T + t];
    int d = -1;
    if (e >= 1 && e <= E) d = (e - 1) / El;
    else atomicMax(status, DEV_BAD_INDEX);
    dest[s] = d;
    pos[s] = d >= 0 ? atomicAdd(&c[d], 1) : 0;
  }
  __syncthreads();
  if (threadIdx.x < world) counts[threadIdx.x] = c[threadIdx.x];
}

struct EpOffsets {
  int off[CTB_EP_MAX_RANKS];
};
// One warp per slot: its token row goes to row off[dest] + pos of the send buffer, with the local expert id (1-based
// on the owner), the gate and, in `order`, the flat slot id (1-based) the result has to come back to.
__global__ void ep_pack_kernel(const uint4* __restrict__ X, const int* __restrict__ topk_ids,
                               const __half* __restrict__ topk_w, const int* __restrict__ dest,
                               const int* __restrict__ pos, EpOffsets so, uint4* __restrict__ send_rows,
                               int* __restrict__ send_ids, __half* __restrict__ send_gates, int* __restrict__ order, int T,
                               int topk, int vecs, int El) {
  const int lane = threadIdx.x & 31;
  const int cap = T * topk;
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  for (int s = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); s < cap; s += nwarps) {
    const int d = dest[s];
    if (d < 0) continue;
    const int t = s / topk, k = s - t * topk;
    const int r = so.off[d] + pos[s];
    if (lane == 0) {
      send_ids[r] = topk_ids[(long long)k * T + t] - d * El;
      send_gates[r] = topk_w[(long long)k * T + t];
      order[r] = s + 1;
    }
    const uint4* src = X + (long long)t * vecs;
    uint4* dst = send_rows + (long long)r * vecs;
    for (int v = lane; v < vecs; v += 32) dst[v] = src[v];
  }
}

}  // namespace

extern "C" {

int ctb_ep_create(ctb_ctx* ctx, int world, int rank, int64_t T_local, int64_t H, int64_t topk, ctb_ep** out) {
  CTB_CHECK_CTX(ctx);
  if (!out) return fail(CTB_BAD_ARG, "ctb_ep_create: null output pointer");
  *out = nullptr;
  if (world < 1 || world > CTB_EP_MAX_RANKS || rank < 0 || rank >= world)
    return fail(CTB_BAD_ARG, "ctb_ep_create: rank %d / world %d out of range (at most %d ranks)", rank, world,
                CTB_EP_MAX_RANKS);
  if (T_local <= 0 || H <= 0 || topk <= 0 || T_local * topk * world > (1 << 24) || H % 8)
    return fail(CTB_BAD_ARG, "ctb_ep_create: bad shape (T_local %lld, H %lld, topk %lld)", (long long)T_local,
                (long long)H, (long long)topk);
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_ep_create: cudaSetDevice");
  ctb_ep* ep = new ctb_ep();
  memset(ep, 0, sizeof *ep);
  ep->ctx = ctx;
  ep->world = world;
  ep->rank = rank;
  ep->T = T_local;
  ep->H = H;
  ep->topk = topk;
  ep->cap = T_local * topk;
  ep->L = ep_layout(world, ep->cap, H);
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  const size_t cap = (size_t)ep->cap, R = cap * world;
  const size_t o_send = 0, o_sids = o_send + up(cap * H * 2), o_sg = o_sids + up(cap * 4), o_ord = o_sg + up(cap * 2),
               o_back = o_ord + up(cap * 4), o_y = o_back + up(cap * H * 2), o_dest = o_y + up(R * H * 2),
               o_pos = o_dest + up(cap * 4), o_cnt = o_pos + up(cap * 4), local_bytes = o_cnt + 256;
  e = cudaMalloc(&ep->shared, ep->L.bytes);
  if (e == cudaSuccess) e = cudaMemset(ep->shared, 0, ep->L.bytes);  // flags and epoch start at zero
  if (e == cudaSuccess) e = cudaMalloc(&ep->local, local_bytes);
  if (e == cudaSuccess) e = cudaMallocHost(&ep->host_counts, 2 * CTB_EP_MAX_RANKS * sizeof(int));
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    ctb_ep_destroy(ep);
    return cuda_fail(e, "ctb_ep_create: allocation");
  }
  ep->send_rows = reinterpret_cast<__half*>(ep->local + o_send);
  ep->send_ids = reinterpret_cast<int*>(ep->local + o_sids);
  ep->send_gates = reinterpret_cast<__half*>(ep->local + o_sg);
  ep->order = reinterpret_cast<int*>(ep->local + o_ord);
  ep->back_rows = reinterpret_cast<__half*>(ep->local + o_back);
  ep->y_rows = reinterpret_cast<__half*>(ep->local + o_y);
  ep->dest = reinterpret_cast<int*>(ep->local + o_dest);
  ep->pos = reinterpret_cast<int*>(ep->local + o_pos);
  ep->counters = reinterpret_cast<int*>(ep->local + o_cnt);
  ep->peer[rank] = ep->shared;
  ep_fill_table(ep);
  *out = ep;
  return CTB_OK;
}

void ctb_ep_destroy(ctb_ep* ep) {
  if (!ep) return;
  cudaSetDevice(ep->ctx->device);
  for (int q = 0; q < ep->world; ++q)
    if (ep->peer_ipc[q] && ep->peer[q]) cudaIpcCloseMemHandle(ep->peer[q]);
  if (ep->shared) cudaFree(ep->shared);
  if (ep->local) cudaFree(ep->local);
  if (ep->host_counts) cudaFreeHost(ep->host_counts);
  cudaGetLastError();
  delete ep;
}

int ctb_ep_export(ctb_ep* ep, void* handle) {
  if (!ep || !handle) return fail(CTB_BAD_ARG, "ctb_ep_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == CTB_EP_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t h;
  cudaSetDevice(ep->ctx->device);
  cudaError_t e = cudaIpcGetMemHandle(&h, ep->shared);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_ep_export: cudaIpcGetMemHandle");
  memcpy(handle, &h, sizeof h);
  return CTB_OK;
}

int ctb_ep_import(ctb_ep* ep, int peer, const void* handle) {
  if (!ep || !handle) return fail(CTB_BAD_ARG, "ctb_ep_import: null argument");
  if (peer < 0 || peer >= ep->world) return fail(CTB_BAD_ARG, "ctb_ep_import: rank %d out of range", peer);
  if (peer == ep->rank) return CTB_OK;
  if (ep->peer[peer]) return fail(CTB_BAD_ARG, "ctb_ep_import: rank %d has been imported already", peer);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  cudaSetDevice(ep->ctx->device);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return cuda_fail(e, "ctb_ep_import: cudaIpcOpenMemHandle");
  ep->peer[peer] = static_cast<unsigned char*>(p);
  ep->peer_ipc[peer] = true;
  ep_fill_table(ep);
  return CTB_OK;
}

int ctb_ep_connect_local(ctb_ep* const* eps, int n) {
  if (!eps || n < 1) return fail(CTB_BAD_ARG, "ctb_ep_connect_local: empty list");
  for (int i = 0; i < n; ++i) {
    if (!eps[i]) return fail(CTB_BAD_ARG, "ctb_ep_connect_local: null entry %d", i);
    if (eps[i]->world != n || eps[i]->rank != i)
      return fail(CTB_BAD_ARG, "ctb_ep_connect_local: entry %d is rank %d of %d, expected rank %d of %d", i, eps[i]->rank,
                  eps[i]->world, i, n);
    if (eps[i]->cap != eps[0]->cap || eps[i]->H != eps[0]->H)
      return fail(CTB_BAD_ARG, "ctb_ep_connect_local: entry %d was created for another shape", i);
  }
  for (int i = 0; i < n; ++i) {
    for (int q = 0; q < n; ++q) eps[i]->peer[q] = eps[q]->shared;  // peer access was enabled by ctb_create_multi
    ep_fill_table(eps[i]);
  }
  return CTB_OK;
}

const ctb_ep_buffers* ctb_ep_table(const ctb_ep* ep) { return ep ? &ep->table : nullptr; }

}  // extern "C"

namespace {

struct EpCall {
  ctb_ep* ep;
  cudaStream_t st;
  const void *hidden, *w1, *w2, *gates;
  const int32_t* ids;
  void* out;
};

int ep_check_call(const char* who, const EpCall& c, int64_t T, int64_t H, int64_t I, int64_t E, int64_t topk, int tile_m,
                  int tile_n, int tile_k) {
  if (!c.ep) return fail(CTB_BAD_ARG, "%s: null expert-parallel state", who);
  if (T != c.ep->T || H != c.ep->H || topk != c.ep->topk)
    return fail(CTB_BAD_ARG, "%s: shape (T %lld, H %lld, topk %lld) differs from the one the buffers were created for "
                "(T %lld, H %lld, topk %lld)", who, (long long)T, (long long)H, (long long)topk, (long long)c.ep->T,
                (long long)c.ep->H, (long long)c.ep->topk);
  if (I <= 0 || E <= 0 || E % c.ep->world)
    return fail(CTB_BAD_ARG, "%s: the %lld experts must divide evenly over the %d ranks", who, (long long)E, c.ep->world);
  if (!is_pow2(tile_m) || !is_pow2(tile_n) || !is_pow2(tile_k))
    return fail(CTB_UNSUPPORTED_TILE, "%s: tile sizes must be powers of two", who);
  if (!is_device_ptr(c.hidden) || !is_device_ptr(c.w1) || !is_device_ptr(c.w2) || !is_device_ptr(c.gates) ||
      !is_device_ptr(c.ids) || !is_device_ptr(c.out))
    return fail(CTB_BAD_ARG, "%s: every array must be a device pointer", who);
  return ep_connected(c.ep, who);
}

// Peer-memory mode: dispatch kernel -> barrier -> expert phase (epilogue stores into the senders' buffers) ->
// barrier -> sum over top-k.  Nothing but kernel launches: no host synchronisation, capturable in a CUDA graph.
int ep_step_peer(const EpCall& c, int64_t T, int64_t H, int64_t I, int64_t E, int64_t topk, int tile_m, int tile_n,
                 int tile_k) {
  ctb_ep* ep = c.ep;
  int r = ctb_moe_ep_dispatch(ep->ctx, c.st, &ep->table, c.hidden, c.ids, c.gates, T, H, E, topk);
  if (r) return r;
  r = ctb_moe_ep_barrier(ep->ctx, c.st, &ep->table);
  if (r) return r;
  r = ctb_moe_ep_experts(ep->ctx, c.st, &ep->table, c.w1, c.w2, ep->cap, H, I, E / ep->world, tile_m, tile_n, tile_k);
  if (r) return r;
  r = ctb_moe_ep_barrier(ep->ctx, c.st, &ep->table);
  if (r) return r;
  return ctb_moe_combine(ep->ctx, c.st, ep->table.slot_out[ep->rank], c.out, T, H, topk);
}

// NCCL mode for `n` ranks driven by this thread (1 in a process-per-GPU job, all of them in a single-process group).
// Rows are packed by destination rank, the per-pair counts cross first (one host synchronisation: ncclSend/ncclRecv
// take their sizes from the host), then rows with their expert ids and gates, the expert phase runs on what
// arrived, and the weighted outputs go back the same way.
int ep_step_nccl(EpCall* calls, int n, int64_t T, int64_t H, int64_t I, int64_t E, int64_t topk, int tile_m) {
  NcclApi* a = nullptr;
  int r = need_nccl(&a);
  if (r) return r;
  const int world = calls[0].ep->world;
  const int El = (int)(E / world);
  const int vecs = (int)(H / 8);
  for (int i = 0; i < n; ++i)
    if (!calls[i].ep->ctx->comm) return fail(CTB_NCCL_ERROR, "ctb_moe_ffn_ep: rank %d has no NCCL communicator", calls[i].ep->rank);
  // ---- 1. destinations and per-destination counts; counts cross
  for (int i = 0; i < n; ++i) {
    ctb_ep* ep = calls[i].ep;
    cudaSetDevice(ep->ctx->device);
    ep_count_kernel<<<1, 1024, 0, calls[i].st>>>(calls[i].ids, (int)T, (int)topk, (int)E, El, world, ep->counters, ep->dest, ep->pos,
                                                 ep->ctx->dev_status);
    CTB_CHECK_LAUNCH("ctb_moe_ffn_ep: count launch");
  }
  CTB_NCCL(a->GroupStart(), "ncclGroupStart");
  for (int i = 0; i < n; ++i) {
    ctb_ep* ep = calls[i].ep;
    Comm* cm = static_cast<Comm*>(ep->ctx->comm);
    for (int q = 0; q < world; ++q) {
      CTB_NCCL(a->Send(ep->counters + q, 1, kNcclInt32, q, cm->comm, calls[i].st), "ncclSend(counts)");
      CTB_NCCL(a->Recv(ep->counters + 2 * CTB_EP_MAX_RANKS + q, 1, kNcclInt32, q, cm->comm, calls[i].st), "ncclRecv(counts)");
    }
  }
  CTB_NCCL(a->GroupEnd(), "ncclGroupEnd(counts)");
  for (int i = 0; i < n; ++i) {
    ctb_ep* ep = calls[i].ep;
    cudaSetDevice(ep->ctx->device);
    cudaError_t e = cudaMemcpyAsync(ep->host_counts, ep->counters, CTB_EP_MAX_RANKS * sizeof(int), cudaMemcpyDeviceToHost, calls[i].st);
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(ep->host_counts + CTB_EP_MAX_RANKS, ep->counters + 2 * CTB_EP_MAX_RANKS, CTB_EP_MAX_RANKS * sizeof(int),
                          cudaMemcpyDeviceToHost, calls[i].st);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_moe_ffn_ep: copying the counts");
  }
  for (int i = 0; i < n; ++i) {
    cudaSetDevice(calls[i].ep->ctx->device);
    cudaError_t e = cudaStreamSynchronize(calls[i].st);
    if (e != cudaSuccess) return cuda_fail(e, "ctb_moe_ffn_ep: waiting for the counts");
  }
  // ---- 2. pack by destination, rows cross with ids and gates
  std::vector<EpOffsets> soff(n), roff(n);
  std::vector<int> rtot(n);
  for (int i = 0; i < n; ++i) {
    ctb_ep* ep = calls[i].ep;
    int s = 0, rr = 0;
    for (int q = 0; q < world; ++q) {
      soff[i].off[q] = s;
      roff[i].off[q] = rr;
      s += ep->host_counts[q];
      rr += ep->host_counts[CTB_EP_MAX_RANKS + q];
    }
    for (int q = world; q < CTB_EP_MAX_RANKS; ++q) soff[i].off[q] = roff[i].off[q] = 0;
    rtot[i] = rr;
    if (s > ep->cap || rr > ep->cap * world) return fail(CTB_BAD_ARG, "ctb_moe_ffn_ep: counts out of range (an expert id is invalid)");
    cudaSetDevice(ep->ctx->device);
    const int grid = (int)std::min<int64_t>((ep->cap + 7) / 8, (int64_t)ep->ctx->sm_count * 8);
    ep_pack_kernel<<<grid, 256, 0, calls[i].st>>>((const uint4*)calls[i].hidden, calls[i].ids, (const __half*)calls[i].gates, ep->dest,
                                                  ep->pos, soff[i], (uint4*)ep->send_rows, ep->send_ids, ep->send_gates, ep->order,
                                                  (int)T, (int)topk, vecs, El);
    CTB_CHECK_LAUNCH("ctb_moe_ffn_ep: pack launch");
  }
  // received rows land in the shared block's receive buffers (compact: R_i rows)
  CTB_NCCL(a->GroupStart(), "ncclGroupStart");
  for (int i = 0; i < n; ++i) {
    ctb_ep* ep = calls[i].ep;
    Comm* cm = static_cast<Comm*>(ep->ctx->comm);
    __half* rrows = reinterpret_cast<__half*>(ep->shared + ep->L.recv_rows);
    int* rids = reinterpret_cast<int*>(ep->shared + ep->L.recv_ids);
    __half* rg = reinterpret_cast<__half*>(ep->shared + ep->L.recv_gates);
    for (int q = 0; q < world; ++q) {
      const size_t sc = ep->host_counts[q], rc = ep->host_counts[CTB_EP_MAX_RANKS + q];
      if (sc) {
        CTB_NCCL(a->Send(ep->send_rows + (size_t)soff[i].off[q] * H, sc * H, kNcclFloat16, q, cm->comm, calls[i].st), "ncclSend(rows)");
        CTB_NCCL(a->Send(ep->send_ids + soff[i].off[q], sc, kNcclInt32, q, cm->comm, calls[i].st), "ncclSend(ids)");
        CTB_NCCL(a->Send(ep->send_gates + soff[i].off[q], sc, kNcclFloat16, q, cm->comm, calls[i].st), "ncclSend(gates)");
      }
      if (rc) {
        CTB_NCCL(a->Recv(rrows + (size_t)roff[i].off[q] * H, rc * H, kNcclFloat16, q, cm->comm, calls[i].st), "ncclRecv(rows)");
        CTB_NCCL(a->Recv(rids + roff[i].off[q], rc, kNcclInt32, q, cm->comm, calls[i].st), "ncclRecv(ids)");
        CTB_NCCL(a->Recv(rg + roff[i].off[q], rc, kNcclFloat16, q, cm->comm, calls[i].st), "ncclRecv(gates)");
      }
    }
  }
  CTB_NCCL(a->GroupEnd(), "ncclGroupEnd(rows)");
  // ---- 3. expert phase on what arrived
  for (int i = 0; i < n; ++i) {
    ctb_ep* ep = calls[i].ep;
    if (rtot[i] == 0) continue;
    cudaSetDevice(ep->ctx->device);
    r = moe_experts_rows(ep->ctx, calls[i].st, ep->shared + ep->L.recv_rows, H,
                         reinterpret_cast<const int32_t*>(ep->shared + ep->L.recv_ids), ep->shared + ep->L.recv_gates,
                         rtot[i], H, I, El, calls[i].w1, calls[i].w2, tile_m, ep->y_rows, H, nullptr, 0);
    if (r) return r;
  }
  // ---- 4. outputs go back to the ranks that sent the rows
  CTB_NCCL(a->GroupStart(), "ncclGroupStart");
  for (int i = 0; i < n; ++i) {
    ctb_ep* ep = calls[i].ep;
    Comm* cm = static_cast<Comm*>(ep->ctx->comm);
    for (int q = 0; q < world; ++q) {
      const size_t sc = ep->host_counts[q], rc = ep->host_counts[CTB_EP_MAX_RANKS + q];
      if (rc) CTB_NCCL(a->Send(ep->y_rows + (size_t)roff[i].off[q] * H, rc * H, kNcclFloat16, q, cm->comm, calls[i].st), "ncclSend(outputs)");
      if (sc) CTB_NCCL(a->Recv(ep->back_rows + (size_t)soff[i].off[q] * H, sc * H, kNcclFloat16, q, cm->comm, calls[i].st), "ncclRecv(outputs)");
    }
  }
  CTB_NCCL(a->GroupEnd(), "ncclGroupEnd(outputs)");
  // ---- 5. back into flat slot order, sum over top-k
  for (int i = 0; i < n; ++i) {
    ctb_ep* ep = calls[i].ep;
    cudaSetDevice(ep->ctx->device);
    void* slot_out = ep->shared + ep->L.slot_out;
    r = ctb_moe_scatter_rows(ep->ctx, calls[i].st, slot_out, ep->back_rows, ep->order, ep->cap, H, ep->cap);
    if (r) return r;
    r = ctb_moe_combine(ep->ctx, calls[i].st, slot_out, calls[i].out, T, H, topk);
    if (r) return r;
  }
  return CTB_OK;
}

}  // namespace

extern "C" {

int ctb_moe_ffn_ep(ctb_ep* ep, void* stream, const void* hidden, const void* w1_local, const void* w2_local,
                   const void* topk_weights, const int32_t* topk_ids, void* out, int64_t T_local, int64_t H, int64_t I,
                   int64_t E, int64_t topk, int tile_m, int tile_n, int tile_k, int a2a_mode) {
  EpCall c{ep, static_cast<cudaStream_t>(stream), hidden, w1_local, w2_local, topk_weights, topk_ids, out};
  int r = ep_check_call("ctb_moe_ffn_ep", c, T_local, H, I, E, topk, tile_m, tile_n, tile_k);
  if (r) return r;
  if (a2a_mode == CTB_A2A_PEER) return ep_step_peer(c, T_local, H, I, E, topk, tile_m, tile_n, tile_k);
  if (a2a_mode == CTB_A2A_NCCL) {
    int prev = 0;
    cudaGetDevice(&prev);
    r = ep_step_nccl(&c, 1, T_local, H, I, E, topk, tile_m);
    cudaSetDevice(prev);
    return r;
  }
  return fail(CTB_BAD_ARG, "ctb_moe_ffn_ep: a2a_mode must be CTB_A2A_NCCL (0) or CTB_A2A_PEER (1)");
}

int ctb_moe_ffn_ep_group(ctb_group* g, ctb_ep* const* eps, void* const* streams, const void* const* hidden,
                         const void* const* w1_local, const void* const* w2_local, const void* const* topk_weights,
                         const int32_t* const* topk_ids, void* const* out, int64_t T_local, int64_t H, int64_t I,
                         int64_t E, int64_t topk, int tile_m, int tile_n, int tile_k, int a2a_mode) {
  if (!g) return fail(CTB_BAD_ARG, "ctb_moe_ffn_ep_group: null group");
  if (!eps || !streams || !hidden || !w1_local || !w2_local || !topk_weights || !topk_ids || !out)
    return fail(CTB_BAD_ARG, "ctb_moe_ffn_ep_group: null argument table");
  const int n = (int)g->ctx.size();
  std::vector<EpCall> calls(n);
  for (int i = 0; i < n; ++i) {
    calls[i] = EpCall{eps[i], static_cast<cudaStream_t>(streams[i]), hidden[i], w1_local[i], w2_local[i], topk_weights[i],
                      topk_ids[i], out[i]};
    int r = ep_check_call("ctb_moe_ffn_ep_group", calls[i], T_local, H, I, E, topk, tile_m, tile_n, tile_k);
    if (r) return r;
    if (eps[i]->ctx != g->ctx[i] || eps[i]->world != n || eps[i]->rank != i)
      return fail(CTB_BAD_ARG, "ctb_moe_ffn_ep_group: entry %d does not belong to device %d of the group", i, i);
  }
  int prev = 0;
  cudaGetDevice(&prev);
  int r = CTB_OK;
  if (a2a_mode == CTB_A2A_PEER) {
    // the launches of one rank never wait for the host, so the ranks can be enqueued one after the other
    for (int i = 0; i < n && r == CTB_OK; ++i) {
      cudaSetDevice(g->devices[i]);
      r = ep_step_peer(calls[i], T_local, H, I, E, topk, tile_m, tile_n, tile_k);
    }
  } else if (a2a_mode == CTB_A2A_NCCL) {
    r = ep_step_nccl(calls.data(), n, T_local, H, I, E, topk, tile_m);
  } else {
    r = fail(CTB_BAD_ARG, "ctb_moe_ffn_ep_group: a2a_mode must be CTB_A2A_NCCL (0) or CTB_A2A_PEER (1)");
  }
  cudaSetDevice(prev);
  return r;
}

// ------------------------------------------------------------------ scratch sizing
size_t ctb_workspace_bytes(int op, const int64_t* dims, int ndims) {
  auto up = [](size_t v) { return (v + 255) & ~size_t(255); };
  if (!dims) return 0;
  if (op == CTB_OP_MOE_FFN && ndims >= 6) {  // T, H, I, E, topk, tile_m
    const int64_t T = dims[0], H = dims[1], I = dims[2], E = dims[3], topk = dims[4], tile_m = dims[5];
    if (T <= 0 || H <= 0 || I <= 0 || E <= 0 || topk <= 0 || tile_m <= 0) return 0;
    const size_t total = (size_t)(T * topk), cap = (size_t)ctb_moe_max_blocks(T, topk, E, (int)tile_m);
    return up(cap * tile_m * 4) + up(cap * 4) + 256 + up(total * I * 2) + up(total * H * 2);
  }
  if (op == CTB_OP_MOE_EP && ndims >= 6) {  // T_local, H, I, E_local, topk, tile_m, [world]
    const int64_t world = ndims >= 7 ? dims[6] : 1;
    if (dims[0] <= 0 || dims[2] <= 0 || dims[3] <= 0 || dims[4] <= 0 || dims[5] <= 0 || world <= 0) return 0;
    return moe_experts_rows_workspace(dims[0] * dims[4] * world, dims[2], dims[3], (int)dims[5]);
  }
  return 0;
}

int ctb_reserve_workspace(ctb_ctx* ctx, void* stream, size_t bytes) {
  CTB_CHECK_CTX(ctx);
  void* ws = nullptr;
  return bytes ? workspace(ctx, bytes, &ws, static_cast<cudaStream_t>(stream)) : CTB_OK;
}

}  // extern "C"
