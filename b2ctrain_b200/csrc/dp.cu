// Data parallelism over the GPUs of one node: the communicator, the dense gradient all-reduce, the stream-ordered
// barrier and the peer mappings the sharded update kernel (optim.cu) reads and writes through.
//
// The reference has no multi-GPU code; its step shards by view (src/train/trainer.cpp:464-529 touches shared state only
// in optimizer_step). NCCL is resolved at run time from libnccl.so.2 so that single-GPU users of the library do not
// need it; whichever NCCL the process has already loaded (a host framework's copy, say) is the one that is used.
#include "dp.cuh"
#include <dlfcn.h>
#include <nccl.h>
#include <cstring>

namespace b2k {
namespace {

struct Nccl {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*Broadcast)(const void*, void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  bool ok = false;
};

Nccl& nccl() {
  static Nccl n;
  if (n.lib) return n;
  for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
    n.lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (n.lib) break;
  }
  if (!n.lib) return n;
  n.GetUniqueId = (decltype(n.GetUniqueId))dlsym(n.lib, "ncclGetUniqueId");
  n.CommInitRank = (decltype(n.CommInitRank))dlsym(n.lib, "ncclCommInitRank");
  n.CommDestroy = (decltype(n.CommDestroy))dlsym(n.lib, "ncclCommDestroy");
  n.AllReduce = (decltype(n.AllReduce))dlsym(n.lib, "ncclAllReduce");
  n.AllGather = (decltype(n.AllGather))dlsym(n.lib, "ncclAllGather");
  n.Broadcast = (decltype(n.Broadcast))dlsym(n.lib, "ncclBroadcast");
  n.GroupStart = (decltype(n.GroupStart))dlsym(n.lib, "ncclGroupStart");
  n.GroupEnd = (decltype(n.GroupEnd))dlsym(n.lib, "ncclGroupEnd");
  n.ok = n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.AllReduce && n.AllGather && n.Broadcast && n.GroupStart && n.GroupEnd;
  return n;
}

// NCCL failures travel as B2K_ERR_CUDA with the NCCL code offset into a range no CUDA error uses.
int nccl_status(ncclResult_t r) {
  if (r == ncclSuccess) return B2K_OK;
  g_last_cuda_error = 100000 + (int)r;
  return B2K_ERR_CUDA;
}
#define B2K_NCCL(expr) do { const int st_ = nccl_status(expr); if (st_) return st_; } while (0)

}  // namespace
}  // namespace b2k

using namespace b2k;

static_assert(B2K_DP_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "the rendezvous id is NCCL's");
static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle_buf holds 64 bytes per rank");

extern "C" int b2k_dp_unique_id(uint8_t* id) {
  B2K_REQUIRE(id);
  Nccl& n = nccl();
  if (!n.ok) return B2K_ERR_UNSUPPORTED;
  ncclUniqueId u;
  B2K_NCCL(n.GetUniqueId(&u));
  std::memcpy(id, u.internal, B2K_DP_ID_BYTES);
  return B2K_OK;
}

extern "C" int b2k_dp_init(B2kDp** out, const uint8_t* id, int32_t rank, int32_t world) {
  B2K_REQUIRE(out && id && world >= 1 && world <= B2K_DP_MAX_RANKS && rank >= 0 && rank < world);
  Nccl& n = nccl();
  if (!n.ok) return B2K_ERR_UNSUPPORTED;
  B2kDp* dp = new B2kDp();
  dp->rank = rank; dp->world = world;
  cudaError_t e = cudaGetDevice(&dp->device);
  if (e == cudaSuccess) e = cudaMalloc(&dp->barrier_word, 4 * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMemset(dp->barrier_word, 0, 4 * sizeof(uint32_t));
  if (e == cudaSuccess) e = cudaMalloc(&dp->handle_buf, (size_t)world * 64);
  if (e != cudaSuccess) { g_last_cuda_error = (int)e; delete dp; return B2K_ERR_CUDA; }
  ncclUniqueId u;
  std::memcpy(u.internal, id, B2K_DP_ID_BYTES);
  ncclComm_t comm = nullptr;
  const int st = nccl_status(n.CommInitRank(&comm, world, u, rank));
  if (st) { cudaFree(dp->barrier_word); cudaFree(dp->handle_buf); delete dp; return st; }
  dp->comm = comm;
  *out = dp;
  return B2K_OK;
}

extern "C" int b2k_dp_destroy(B2kDp* dp) {
  if (!dp) return B2K_OK;
  cudaDeviceSynchronize();
  for (int i = 0; i < dp->n_opened; i++) cudaIpcCloseMemHandle(dp->opened[i]);
  if (dp->comm) nccl().CommDestroy((ncclComm_t)dp->comm);
  cudaFree(dp->barrier_word); cudaFree(dp->handle_buf);
  delete dp;
  return B2K_OK;
}

extern "C" int b2k_dp_allreduce_grads(B2kDp* dp, float* grad, uint64_t count, b2k_stream_t s) {
  B2K_REQUIRE(dp && dp->comm && (grad || count == 0));
  if (count == 0 || dp->world == 1) return B2K_OK;
  B2K_NCCL(nccl().AllReduce(grad, grad, (size_t)count, ncclFloat32, ncclSum, (ncclComm_t)dp->comm, (cudaStream_t)s));
  return B2K_OK;
}

extern "C" int b2k_dp_allreduce_stat(B2kDp* dp, float* stat, uint64_t count, int32_t op, b2k_stream_t s) {
  B2K_REQUIRE(dp && dp->comm && (stat || count == 0) && (op == 0 || op == 1));
  if (count == 0 || dp->world == 1) return B2K_OK;
  B2K_NCCL(nccl().AllReduce(stat, stat, (size_t)count, ncclFloat32, op == 0 ? ncclSum : ncclMax, (ncclComm_t)dp->comm, (cudaStream_t)s));
  return B2K_OK;
}

extern "C" int b2k_dp_barrier(B2kDp* dp, b2k_stream_t s) {
  B2K_REQUIRE(dp && dp->comm);
  if (dp->world == 1) return B2K_OK;
  B2K_NCCL(nccl().AllReduce(dp->barrier_word, dp->barrier_word, 1, ncclUint32, ncclSum, (ncclComm_t)dp->comm, (cudaStream_t)s));
  return B2K_OK;
}

extern "C" int b2k_dp_share(B2kDp* dp, void* base, void** peers, b2k_stream_t stream) {
  B2K_REQUIRE(dp && dp->comm && base && peers);
  cudaStream_t s = (cudaStream_t)stream;
  if (dp->world == 1) { peers[0] = base; return B2K_OK; }
  if (dp->n_opened + dp->world > (int)(sizeof(dp->opened) / sizeof(dp->opened[0]))) return B2K_ERR_CAPACITY;
  cudaIpcMemHandle_t mine;
  B2K_CUDA(cudaIpcGetMemHandle(&mine, base));
  B2K_CUDA(cudaMemcpyAsync(dp->handle_buf + (size_t)dp->rank * 64, &mine, 64, cudaMemcpyHostToDevice, s));
  B2K_NCCL(nccl().AllGather(dp->handle_buf + (size_t)dp->rank * 64, dp->handle_buf, 64, ncclChar, (ncclComm_t)dp->comm, s));
  cudaIpcMemHandle_t all[B2K_DP_MAX_RANKS];
  B2K_CUDA(cudaMemcpyAsync(all, dp->handle_buf, (size_t)dp->world * 64, cudaMemcpyDeviceToHost, s));
  B2K_CUDA(cudaStreamSynchronize(s));
  for (int r = 0; r < dp->world; r++) {
    if (r == dp->rank) { peers[r] = base; continue; }
    void* p = nullptr;
    B2K_CUDA(cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess));
    dp->opened[dp->n_opened++] = p;
    peers[r] = p;
  }
  return B2K_OK;
}

extern "C" int b2k_dp_release_shares(B2kDp* dp, b2k_stream_t stream) {
  B2K_REQUIRE(dp);
  B2K_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  for (int i = 0; i < dp->n_opened; i++) cudaIpcCloseMemHandle(dp->opened[i]);
  dp->n_opened = 0;
  return B2K_OK;
}

extern "C" int b2k_dp_gather_slices(B2kDp* dp, void* base, uint64_t elem_bytes, int32_t lanes, uint64_t lane_stride, int32_t n, b2k_stream_t stream) {
  B2K_REQUIRE(dp && dp->comm && base && elem_bytes > 0 && lanes >= 0 && n >= 0 && lane_stride >= (uint64_t)n);
  if (dp->world == 1 || n == 0 || lanes == 0) return B2K_OK;
  Nccl& nc = nccl();
  B2K_NCCL(nc.GroupStart());
  for (int r = 0; r < dp->world; r++) {
    int32_t first = 0, count = 0;
    b2k_dp_slice(n, r, dp->world, &first, &count);
    if (count == 0) continue;
    for (int l = 0; l < lanes; l++) {
      char* p = (char*)base + ((uint64_t)l * lane_stride + (uint64_t)first) * elem_bytes;
      const int st = nccl_status(nc.Broadcast(p, p, (size_t)count * elem_bytes, ncclChar, r, (ncclComm_t)dp->comm, (cudaStream_t)stream));
      if (st) { nc.GroupEnd(); return st; }
    }
  }
  B2K_NCCL(nc.GroupEnd());
  return B2K_OK;
}

extern "C" int b2k_dp_slice(int32_t n, int32_t rank, int32_t world, int32_t* first, int32_t* count) {
  B2K_REQUIRE(first && count && n >= 0 && world >= 1 && rank >= 0 && rank < world);
  const long long per = (((long long)n + world - 1) / world + 127) / 128 * 128;   // whole update blocks per rank
  const long long a = per * rank < n ? per * rank : n, b = per * (rank + 1) < n ? per * (rank + 1) : n;
  *first = (int32_t)a; *count = (int32_t)(b - a);
  return B2K_OK;
}
