// Data-parallel gradient exchange behind the C ABI: one NCCL communicator per context and the
// gradient mean of the step (ferrotensor-trainer/src/distributed.rs:107-185 averages the
// gradients of all ranks before the optimizer runs, ferrotensor-trainer/src/lib.rs:318-328
// calls it from Trainer::apply_gradients; there the exchange goes through files in a shared
// directory with a `max_wait`, here through NCCL over NVLink with host-side time limits).
//
// NCCL is bound at run time (dlopen of libnccl.so.2, or the path in FT_NCCL_LIB), so the
// library loads, and single-rank users run, on a machine without it.  Communicators are
// created non-blocking: every NCCL call returns at once and its progress is polled with a
// deadline, so a rank that never joins ends in FT_ERR_COMM on the host instead of a hung call.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <chrono>
#include <mutex>
#include <thread>

#include "ft_common.cuh"

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetVersion)(int*) = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
  ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
  ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                            cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  char why[256] = "";
};

NcclApi g_api;
std::once_flag g_api_once;

template <typename F>
bool bind(void* h, const char* name, F& fn) {
  fn = (F)dlsym(h, name);
  return fn != nullptr;
}

void load_api() {
  const char* names[3] = {getenv("FT_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
  for (const char* n : names) {
    if (!n || !*n) continue;
    g_api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
    if (g_api.handle) break;
    snprintf(g_api.why, sizeof(g_api.why), "%s", dlerror());
  }
  if (!g_api.handle) return;
  void* h = g_api.handle;
  bool ok = bind(h, "ncclGetVersion", g_api.GetVersion) & bind(h, "ncclGetUniqueId", g_api.GetUniqueId) &
            bind(h, "ncclCommInitRankConfig", g_api.CommInitRankConfig) &
            bind(h, "ncclCommGetAsyncError", g_api.CommGetAsyncError) &
            bind(h, "ncclCommAbort", g_api.CommAbort) & bind(h, "ncclCommDestroy", g_api.CommDestroy) &
            bind(h, "ncclAllReduce", g_api.AllReduce) & bind(h, "ncclGetErrorString", g_api.GetErrorString);
  if (!ok) {
    snprintf(g_api.why, sizeof(g_api.why), "the NCCL library lacks a required entry point");
    g_api.handle = nullptr;
  }
}

// NULL (with ft_last_error set) when NCCL cannot be bound
NcclApi* nccl() {
  std::call_once(g_api_once, load_api);
  if (!g_api.handle) {
    ft_set_error("NCCL is not available: %s", g_api.why[0] ? g_api.why : "library not found");
    return nullptr;
  }
  return &g_api;
}

using Clock = std::chrono::steady_clock;

}  // namespace

struct FtComm {
  FtContext* ctx = nullptr;
  int world = 1, rank = 0;
  int timeout_ms = 0;
  ncclComm_t comm = nullptr;
  bool broken = false;        // aborted after an error or a timeout: every later call fails
  cudaEvent_t done = nullptr; // recorded after the last collective enqueued
  bool pending = false;
};

namespace {

int comm_fail(FtComm* c, const char* what, ncclResult_t r) {
  NcclApi* api = &g_api;
  ft_set_error("%s: NCCL error %d (%s), rank %d of %d", what, (int)r,
               api->GetErrorString ? api->GetErrorString(r) : "?", c->rank, c->world);
  if (c->comm) {
    api->CommAbort(c->comm);
    c->comm = nullptr;
  }
  c->broken = true;
  return FT_ERR_COMM;
}

// Waits until the communicator's asynchronous state leaves ncclInProgress or the deadline passes.
int comm_settle(FtComm* c, const char* what, ncclResult_t first) {
  NcclApi* api = &g_api;
  ncclResult_t state = first;
  const auto deadline = Clock::now() + std::chrono::milliseconds(c->timeout_ms);
  while (state == ncclInProgress) {
    ncclResult_t q = api->CommGetAsyncError(c->comm, &state);
    if (q != ncclSuccess) return comm_fail(c, what, q);
    if (state != ncclInProgress) break;
    if (Clock::now() > deadline) {
      ft_set_error("%s: timed out after %d ms waiting for the other ranks (rank %d of %d)", what,
                   c->timeout_ms, c->rank, c->world);
      api->CommAbort(c->comm);
      c->comm = nullptr;
      c->broken = true;
      return FT_ERR_COMM;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  if (state != ncclSuccess) return comm_fail(c, what, state);
  return FT_OK;
}

}  // namespace

extern "C" int ft_comm_unique_id(void* id_out) {
  FT_REQUIRE(id_out, "ft_comm_unique_id: id_out is NULL");
  static_assert(sizeof(ncclUniqueId) == FT_COMM_ID_BYTES, "FT_COMM_ID_BYTES must match ncclUniqueId");
  NcclApi* api = nccl();
  if (!api) return FT_ERR_COMM;
  ncclUniqueId id;
  ncclResult_t r = api->GetUniqueId(&id);
  if (r != ncclSuccess) {
    ft_set_error("ft_comm_unique_id: NCCL error %d (%s)", (int)r, api->GetErrorString(r));
    return FT_ERR_COMM;
  }
  memcpy(id_out, &id, sizeof(id));
  return FT_OK;
}

extern "C" int ft_comm_create(FtContext* ctx, int world_size, int rank, const void* id,
                              int timeout_ms, FtComm** out) {
  FT_REQUIRE(ctx && out, "ft_comm_create: NULL argument");
  // the reference's FileGradSyncConfig::new rejects the same two cases with these words
  FT_REQUIRE(world_size >= 1, "world_size must be >= 1");
  FT_REQUIRE(rank >= 0 && rank < world_size, "rank %d is out of range for world_size %d", rank,
             world_size);
  FT_REQUIRE(timeout_ms > 0, "ft_comm_create: timeout_ms must be positive");
  FtComm* c = new FtComm();
  c->ctx = ctx;
  c->world = world_size;
  c->rank = rank;
  c->timeout_ms = timeout_ms;
  if (world_size == 1) {   // nothing to exchange: no NCCL needed
    *out = c;
    return FT_OK;
  }
  if (!id) {
    delete c;
    ft_set_error("ft_comm_create: id is NULL");
    return FT_ERR_INVALID;
  }
  NcclApi* api = nccl();
  if (!api) {
    delete c;
    return FT_ERR_COMM;
  }
  int prev = -1;
  cudaError_t ce = cudaGetDevice(&prev);
  if (ce == cudaSuccess && prev != ctx->device) ce = cudaSetDevice(ctx->device);
  if (ce == cudaSuccess) ce = cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming);
  if (ce != cudaSuccess) {
    delete c;
    return ft_cuda_fail(ce, "ft_comm_create", __FILE__, __LINE__);
  }
  ncclUniqueId uid;
  memcpy(&uid, id, sizeof(uid));
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  ncclResult_t r = api->CommInitRankConfig(&c->comm, world_size, uid, rank, &cfg);
  int rc = FT_OK;
  if (r != ncclSuccess && r != ncclInProgress) rc = comm_fail(c, "ft_comm_create", r);
  else rc = comm_settle(c, "ft_comm_create", ncclInProgress);
  if (prev >= 0 && prev != ctx->device) cudaSetDevice(prev);
  if (rc != FT_OK) {
    if (c->done) cudaEventDestroy(c->done);
    delete c;
    return rc;
  }
  *out = c;
  return FT_OK;
}

extern "C" int ft_comm_destroy(FtComm* c) {
  if (!c) return FT_OK;
  if (c->comm) {
    // the stream's collectives must have finished before the communicator goes away
    cudaStreamSynchronize(c->ctx->stream);
    g_api.CommDestroy(c->comm);
  }
  if (c->done) cudaEventDestroy(c->done);
  delete c;
  return FT_OK;
}

extern "C" int ft_comm_info(FtComm* c, int* world_size, int* rank) {
  FT_REQUIRE(c && world_size && rank, "ft_comm_info: NULL argument");
  *world_size = c->world;
  *rank = c->rank;
  return FT_OK;
}

// Sum over ranks, in place, enqueued on the context's stream.
int ft_comm_allreduce_f32(FtComm* c, float* buf, size_t n) {
  FT_REQUIRE(c && (buf || n == 0), "ft_comm_allreduce: NULL argument");
  if (c->broken) {
    ft_set_error("ft_comm_allreduce: the communicator was aborted by an earlier failure");
    return FT_ERR_COMM;
  }
  if (c->world == 1 || n == 0) return FT_OK;
  ncclResult_t r = g_api.AllReduce(buf, buf, n, ncclFloat, ncclSum, c->comm, c->ctx->stream);
  if (r != ncclSuccess && r != ncclInProgress) return comm_fail(c, "ft_comm_allreduce", r);
  FT_TRY(comm_settle(c, "ft_comm_allreduce", r));
  c->ctx->launches++;
  FT_CUDA(cudaEventRecord(c->done, c->ctx->stream));
  c->pending = true;
  return FT_OK;
}

extern "C" int ft_comm_allreduce_sum(FtComm* c, float* buf, size_t n) {
  return ft_comm_allreduce_f32(c, buf, n);
}

extern "C" int ft_comm_wait(FtComm* c, int timeout_ms) {
  FT_REQUIRE(c, "ft_comm_wait: comm is NULL");
  if (c->broken) {
    ft_set_error("ft_comm_wait: the communicator was aborted by an earlier failure");
    return FT_ERR_COMM;
  }
  if (!c->pending) return FT_OK;
  const int limit = timeout_ms > 0 ? timeout_ms : c->timeout_ms;
  const auto deadline = Clock::now() + std::chrono::milliseconds(limit);
  for (;;) {
    cudaError_t e = cudaEventQuery(c->done);
    if (e == cudaSuccess) break;
    if (e != cudaErrorNotReady) return ft_cuda_fail(e, "ft_comm_wait", __FILE__, __LINE__);
    ncclResult_t state = ncclSuccess;
    ncclResult_t q = g_api.CommGetAsyncError(c->comm, &state);
    if (q != ncclSuccess) return comm_fail(c, "ft_comm_wait", q);
    if (state != ncclSuccess && state != ncclInProgress) return comm_fail(c, "ft_comm_wait", state);
    if (Clock::now() > deadline) {
      // a peer never entered the collective: aborting the communicator ends the waiting kernel
      ft_set_error("ft_comm_wait: the collective did not finish within %d ms (rank %d of %d)", limit,
                   c->rank, c->world);
      g_api.CommAbort(c->comm);
      c->comm = nullptr;
      c->broken = true;
      return FT_ERR_COMM;
    }
    std::this_thread::sleep_for(std::chrono::microseconds(100));
  }
  c->pending = false;
  return FT_OK;
}

int ft_comm_world(const FtComm* c) { return c ? c->world : 1; }
FtContext* ft_comm_ctx(const FtComm* c) { return c ? c->ctx : nullptr; }
