// Multi-GPU plumbing: NCCL (resolved at run time with dlopen, so the library
// loads on hosts without NCCL) for the column-parallel all-gather and the
// row-parallel all-reduce.  One context = one rank = one GPU.
#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>

#include "tl_common.cuh"

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api;
  tried = true;
  const char* override_path = std::getenv("TL_NCCL_LIB");
  const char* names[] = {override_path, "libnccl.so.2", "libnccl.so"};
  for (const char* nm : names) {
    if (!nm || !*nm) continue;
    api.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) break;
  }
  if (!api.handle) return api;
#define TL_SYM(field, name) *(void**)(&api.field) = dlsym(api.handle, name)
  TL_SYM(GetUniqueId, "ncclGetUniqueId");
  TL_SYM(CommInitRank, "ncclCommInitRank");
  TL_SYM(CommDestroy, "ncclCommDestroy");
  TL_SYM(AllReduce, "ncclAllReduce");
  TL_SYM(AllGather, "ncclAllGather");
  TL_SYM(GetErrorString, "ncclGetErrorString");
#undef TL_SYM
  api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.AllGather && api.GetErrorString;
  return api;
}

ncclDataType_t nccl_dtype(int32_t dt) { return dt == TL_F32 ? ncclFloat32 : dt == TL_F16 ? ncclFloat16 : ncclBfloat16; }

// [world][m][n_local] -> [m][world*n_local]
template <typename T>
__global__ void interleave_cols_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t m, int64_t n_local, int world) {
  const int64_t total = m * n_local * world;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t c = i % n_local, rm = i / n_local, r = rm % m, w = rm / m;
    out[r * (n_local * world) + w * n_local + c] = in[i];
  }
}

}  // namespace

#define TL_NCCL(ctx, expr)                                                                      \
  do {                                                                                          \
    ncclResult_t _r = (expr);                                                                   \
    if (_r != ncclSuccess)                                                                      \
      return tl_set_error((ctx), TL_ERR_NCCL, "%s: %s failed: %s", __func__, #expr, nccl().GetErrorString(_r)); \
  } while (0)

extern "C" {

int32_t tl_comm_unique_id(void* out_id128) {
  if (!out_id128) return tl_set_error(nullptr, TL_ERR_INVALID_ARG, "tl_comm_unique_id: null pointer");
  if (!nccl().ok) return tl_set_error(nullptr, TL_ERR_NCCL, "tl_comm_unique_id: NCCL library not found (set TL_NCCL_LIB)");
  static_assert(sizeof(ncclUniqueId) == TL_COMM_ID_BYTES, "NCCL unique id size");
  ncclUniqueId id;
  TL_NCCL(nullptr, nccl().GetUniqueId(&id));
  std::memcpy(out_id128, &id, sizeof(id));
  return TL_OK;
}

int32_t tl_comm_init(tl_ctx* ctx, int32_t rank, int32_t world, const void* id128) {
  TL_CHECK_CTX(ctx);
  if (world < 1 || rank < 0 || rank >= world)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_comm_init: rank %d outside world %d", rank, world);
  if (ctx->nccl_comm) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_comm_init: communicator already initialised");
  ctx->rank = rank;
  ctx->world = world;
  if (world == 1) return TL_OK;  // single rank: collectives are identities
  if (!id128) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_comm_init: null id");
  if (!nccl().ok) return tl_set_error(ctx, TL_ERR_NCCL, "tl_comm_init: NCCL library not found (set TL_NCCL_LIB)");
  DeviceGuard guard(ctx->device);
  ncclUniqueId id;
  std::memcpy(&id, id128, sizeof(id));
  ncclComm_t comm = nullptr;
  TL_NCCL(ctx, nccl().CommInitRank(&comm, world, id, rank));
  ctx->nccl_comm = comm;
  return TL_OK;
}

int32_t tl_comm_destroy(tl_ctx* ctx) {
  TL_CHECK_CTX(ctx);
  if (ctx->nccl_comm) {
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    nccl().CommDestroy((ncclComm_t)ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
  }
  ctx->rank = 0;
  ctx->world = 1;
  return TL_OK;
}

int32_t tl_allgather_cols(tl_ctx* ctx, const void* local, void* out, int64_t m, int64_t n_local, int32_t dtype) {
  TL_CHECK_CTX(ctx);
  if (!local || !out) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_allgather_cols: null pointer");
  if (m < 0 || n_local < 0 || !tl_dtype_valid(dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_allgather_cols: bad shape or dtype");
  const size_t esz = tl_dtype_size(dtype);
  const size_t count = size_t(m) * n_local;
  if (count == 0) return TL_OK;
  DeviceGuard guard(ctx->device);
  if (ctx->world == 1) {
    if (local != out) TL_CUDA(ctx, cudaMemcpyAsync(out, local, count * esz, cudaMemcpyDeviceToDevice, ctx->stream));
    return TL_OK;
  }
  if (!ctx->nccl_comm) return tl_set_error(ctx, TL_ERR_NCCL, "tl_allgather_cols: communicator not initialised");
  if (m == 1) {
    TL_NCCL(ctx, nccl().AllGather(local, out, count, nccl_dtype(dtype), (ncclComm_t)ctx->nccl_comm, ctx->stream));
    return TL_OK;
  }
  void* stage = nullptr;
  int32_t rc = tl_ensure_scratch(ctx, count * esz * ctx->world, &stage);
  if (rc != TL_OK) return rc;
  TL_NCCL(ctx, nccl().AllGather(local, stage, count, nccl_dtype(dtype), (ncclComm_t)ctx->nccl_comm, ctx->stream));
  const int64_t total = int64_t(count) * ctx->world;
  const int block = 256;
  const int grid = int(std::min<int64_t>((total + block - 1) / block, int64_t(ctx->sm_count) * 8));
  if (esz == 4) interleave_cols_kernel<uint32_t><<<grid, block, 0, ctx->stream>>>((const uint32_t*)stage, (uint32_t*)out, m, n_local, ctx->world);
  else interleave_cols_kernel<uint16_t><<<grid, block, 0, ctx->stream>>>((const uint16_t*)stage, (uint16_t*)out, m, n_local, ctx->world);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_allreduce_sum(tl_ctx* ctx, void* buf, int64_t count, int32_t dtype) {
  TL_CHECK_CTX(ctx);
  if (!buf) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_allreduce_sum: null pointer");
  if (count < 0 || !tl_dtype_valid(dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_allreduce_sum: bad count or dtype");
  if (count == 0 || ctx->world == 1) return TL_OK;
  if (!ctx->nccl_comm) return tl_set_error(ctx, TL_ERR_NCCL, "tl_allreduce_sum: communicator not initialised");
  DeviceGuard guard(ctx->device);
  TL_NCCL(ctx, nccl().AllReduce(buf, buf, size_t(count), nccl_dtype(dtype), ncclSum, (ncclComm_t)ctx->nccl_comm, ctx->stream));
  return TL_OK;
}

}  // extern "C"
