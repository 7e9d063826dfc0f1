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

// ---------------------------------------------------------------------------
// One-shot all-reduce over peer-mapped memory (push model).
//
// Exchange buffer of a rank (cudaMalloc, exported with cudaIpcGetMemHandle):
//   slots  [2 halves][kMaxPeers ranks][max_bytes]   slot (h, r) is WRITTEN BY RANK r
//   flags  u32 [2][kMaxPeers][kP2PCtas]              likewise
//   epochs u32 [kP2PCtas]                            owner-only per-CTA call counter; it lives on
//                                                    the device so that a replayed graph keeps counting
// CTA c of every rank owns slice c of the message.  It pushes its slice into slot (e&1, rank)
// of EVERY rank with plain stores (posted writes over NVLink: one-way latency, no read round
// trip), then one release-store per peer publishes epoch e in flags[e&1][rank][c].  It waits
// (bounded) until all ranks' flags for (e&1, c) reach e and sums the world slots -- all local
// memory now -- in rank order, so every rank computes the same bits.  Calls alternate halves:
// a rank can be at most one call ahead of a peer, and then it writes the other half.
// CTAs never wait on CTAs of the same GPU.
// ---------------------------------------------------------------------------
namespace {
constexpr int kP2PCtas = 8;
constexpr int kP2PThreads = 512;

struct P2PArgs {
  void* base[tl_ctx::kMaxPeers];  // every rank's exchange buffer as mapped HERE (own = local)
  int rank, world;
  size_t max_bytes;
  int64_t count;
  const void* src;
  void* dst;
  int* status;
  int spin_limit;  // polls of one wait before it gives up (the context's wait_limit_polls)
  int dst_dtype;   // f32 exchange only: the type the sums are stored as (one rounding)
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <typename T> __device__ __forceinline__ void add8(float (&acc)[8], const uint4& v);
template <> __device__ __forceinline__ void add8<float>(float (&)[8], const uint4&) {}  // f32 takes the float4 path
template <> __device__ __forceinline__ void add8<__half>(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
    acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
  }
}
template <> __device__ __forceinline__ void add8<__nv_bfloat16>(float (&acc)[8], const uint4& v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc[2 * i] += __uint_as_float(w[i] << 16); acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ uint8_t* p2p_slot(void* base, size_t max_bytes, int half, int r) {
  return reinterpret_cast<uint8_t*>(base) + (size_t(half) * tl_ctx::kMaxPeers + r) * max_bytes;
}
__device__ __forceinline__ uint32_t* p2p_flags(void* base, size_t max_bytes) {
  return reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(base) + 2 * size_t(tl_ctx::kMaxPeers) * max_bytes);
}

// T = element type (2 or 4 bytes); 16-byte vectors; f32 accumulation in rank order.
template <typename T>
__global__ void __launch_bounds__(kP2PThreads) p2p_allreduce_kernel(P2PArgs a) {
  __shared__ int ok_flag;
  const int cta = blockIdx.x, tid = threadIdx.x;
  // the next kernel in the stream (a GEMV that first prefetches weights) may start right away;
  // this kernel itself must see its predecessor's output before it reads src
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  uint32_t* my_flags = p2p_flags(a.base[a.rank], a.max_bytes);
  uint32_t* epochs = my_flags + 2 * tl_ctx::kMaxPeers * kP2PCtas;
  const uint32_t epoch = epochs[cta] + 1;  // every thread reads it before thread 0 bumps it below
  const int half = epoch & 1;
  const size_t bytes = size_t(a.count) * sizeof(T);
  const size_t vecs = (bytes + 15) / 16;  // slots are padded: whole 16-byte vectors
  const size_t per = (vecs + kP2PCtas - 1) / kP2PCtas;
  const size_t v0 = size_t(cta) * per, v1 = v0 + per < vecs ? v0 + per : vecs;
  // 1. push this CTA's slice into slot (half, rank) of every rank
  for (size_t i = v0 + tid; i < v1; i += blockDim.x) {
    uint4 v;
    if ((i + 1) * 16 <= bytes) v = reinterpret_cast<const uint4*>(a.src)[i];
    else {  // ragged tail: zero padded
      v = make_uint4(0, 0, 0, 0);
      uint8_t* zb = reinterpret_cast<uint8_t*>(&v);
      const uint8_t* sb = reinterpret_cast<const uint8_t*>(a.src) + i * 16;
      for (size_t b = 0; b < bytes - i * 16; ++b) zb[b] = sb[b];
    }
    for (int r = 0; r < a.world; ++r) reinterpret_cast<uint4*>(p2p_slot(a.base[r], a.max_bytes, half, a.rank))[i] = v;
  }
  __syncthreads();  // all pushes of the CTA happen-before the release stores below
  // 2. publish: one release store per rank (system scope, cumulative over the barrier)
  if (tid == 0) { epochs[cta] = epoch; ok_flag = 1; }
  if (tid < a.world)
    st_release_sys(p2p_flags(a.base[tid], a.max_bytes) + (half * tl_ctx::kMaxPeers + a.rank) * kP2PCtas + cta, epoch);
  __syncthreads();
  // 3. wait (bounded) for every rank's slice to have landed here
  if (tid < a.world) {
    const uint32_t* f = my_flags + (half * tl_ctx::kMaxPeers + tid) * kP2PCtas + cta;
    int spins = 0;
    while (int32_t(ld_acquire_sys(f) - epoch) < 0) {
      if (++spins > a.spin_limit) { ok_flag = 0; atomicExch(a.status, TL_ERR_TIMEOUT); break; }
    }
  }
  __syncthreads();
  if (!ok_flag) return;
  // 4. sum the world slots (local memory) in rank order: identical bits on every rank
  uint4* d4 = reinterpret_cast<uint4*>(a.dst);
  for (size_t i = v0 + tid; i < v1; i += blockDim.x) {
    uint4 out;
    if (sizeof(T) == 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < a.world; ++r) {
        const uint4 u = __ldcv(reinterpret_cast<const uint4*>(p2p_slot(a.base[a.rank], a.max_bytes, half, r)) + i);
        const float4 v = *reinterpret_cast<const float4*>(&u);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      out = *reinterpret_cast<uint4*>(&acc);
      if (a.dst_dtype != TL_F32) {
        // f32 partial sums, 16-bit result: the sum is rounded ONCE, so the sharded product is as
        // accurate as the unsharded one (16-bit partials lose up to half an ulp of each partial)
        const float o[4] = {acc.x, acc.y, acc.z, acc.w};
        const int64_t e0 = int64_t(i) * 4;
        if (e0 + 4 <= a.count) {
          uint32_t w0, w1;
          if (a.dst_dtype == TL_F16) {
            const __half2 h0 = __floats2half2_rn(o[0], o[1]), h1 = __floats2half2_rn(o[2], o[3]);
            w0 = *reinterpret_cast<const uint32_t*>(&h0); w1 = *reinterpret_cast<const uint32_t*>(&h1);
          } else {
            const __nv_bfloat162 h0 = __floats2bfloat162_rn(o[0], o[1]), h1 = __floats2bfloat162_rn(o[2], o[3]);
            w0 = *reinterpret_cast<const uint32_t*>(&h0); w1 = *reinterpret_cast<const uint32_t*>(&h1);
          }
          reinterpret_cast<uint2*>(a.dst)[i] = make_uint2(w0, w1);
        } else {
          for (int j = 0; e0 + j < a.count; ++j) tl_store_out(a.dst, a.dst_dtype, e0 + j, o[j]);
        }
        continue;
      }
    } else {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int r = 0; r < a.world; ++r)
        add8<T>(acc, __ldcv(reinterpret_cast<const uint4*>(p2p_slot(a.base[a.rank], a.max_bytes, half, r)) + i));
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (DT<T>::id == TL_F16) {
          const __half2 h = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        } else {
          const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
          w[j] = *reinterpret_cast<const uint32_t*>(&h);
        }
      }
      out = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if ((i + 1) * 16 <= bytes) d4[i] = out;
    else {  // the last vector extends past count: dst must not be overrun
      const uint8_t* ob = reinterpret_cast<const uint8_t*>(&out);
      uint8_t* db = reinterpret_cast<uint8_t*>(a.dst) + i * 16;
      for (size_t b = 0; b < bytes - i * 16; ++b) db[b] = ob[b];
    }
  }
}

static_assert(kP2PCtas == 8, "tl_p2p_fused_offset assumes 8 CTAs' worth of flags and epochs");
size_t p2p_total_bytes(size_t max_bytes) { return tl_p2p_total_bytes(max_bytes); }
}  // namespace

extern "C" {

int32_t tl_p2p_create(tl_ctx* ctx, size_t max_bytes, void* out_handle64) {
  TL_CHECK_CTX(ctx);
  if (!out_handle64 || max_bytes == 0) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_p2p_create: bad argument");
  if (ctx->p2p_local) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_p2p_create: exchange buffer already exists");
  static_assert(sizeof(cudaIpcMemHandle_t) == TL_P2P_HANDLE_BYTES, "IPC handle size");
  DeviceGuard guard(ctx->device);
  max_bytes = (max_bytes + 255) & ~size_t(255);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, p2p_total_bytes(max_bytes));
  if (e != cudaSuccess) {
    cudaGetLastError();
    return tl_set_error(ctx, TL_ERR_OOM, "tl_p2p_create: %s", cudaGetErrorString(e));
  }
  TL_CUDA(ctx, cudaMemset(p, 0, p2p_total_bytes(max_bytes)));
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    cudaGetLastError();
    return tl_set_error(ctx, TL_ERR_CUDA, "tl_p2p_create: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  std::memcpy(out_handle64, &h, sizeof(h));
  ctx->p2p_local = p;
  ctx->p2p_max_bytes = max_bytes;
  return TL_OK;
}

int32_t tl_p2p_attach(tl_ctx* ctx, const void* handles) {
  TL_CHECK_CTX(ctx);
  if (!handles || !ctx->p2p_local) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_p2p_attach: call tl_p2p_create first");
  if (ctx->world > tl_ctx::kMaxPeers) return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "tl_p2p_attach: at most %d ranks", tl_ctx::kMaxPeers);
  DeviceGuard guard(ctx->device);
  for (int r = 0; r < ctx->world; ++r) {
    if (r == ctx->rank) { ctx->p2p_peer[r] = ctx->p2p_local; continue; }
    cudaIpcMemHandle_t h;
    std::memcpy(&h, reinterpret_cast<const uint8_t*>(handles) + size_t(r) * TL_P2P_HANDLE_BYTES, sizeof(h));
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return tl_set_error(ctx, TL_ERR_CUDA, "tl_p2p_attach: cannot map rank %d's buffer: %s", r, cudaGetErrorString(e));
    }
    ctx->p2p_peer[r] = p;
  }
  ctx->p2p_attached = true;
  return TL_OK;
}

int32_t tl_p2p_attach_loopback(tl_ctx* ctx, int32_t world) {
  TL_CHECK_CTX(ctx);
  if (!ctx->p2p_local) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_p2p_attach_loopback: call tl_p2p_create first");
  if (ctx->nccl_comm || ctx->p2p_attached)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_p2p_attach_loopback: the context already has peers");
  if (world < 1 || world > tl_ctx::kMaxPeers)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_p2p_attach_loopback: world %d outside [1,%d]", world, tl_ctx::kMaxPeers);
  for (int r = 0; r < world; ++r) ctx->p2p_peer[r] = ctx->p2p_local;  // every "peer" is this rank's own buffer
  ctx->rank = 0;
  ctx->world = world;
  ctx->p2p_attached = true;
  return TL_OK;
}

int32_t tl_p2p_reset(tl_ctx* ctx) {
  TL_CHECK_CTX(ctx);
  if (!ctx->p2p_local) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "tl_p2p_reset: no exchange buffer");
  DeviceGuard guard(ctx->device);
  TL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  // flags, per-CTA epochs, and the fused kernel's tile epochs and arrival counters: everything but the slots
  const size_t flags_off = 2 * size_t(tl_ctx::kMaxPeers) * ctx->p2p_max_bytes;
  TL_CUDA(ctx, cudaMemset(reinterpret_cast<uint8_t*>(ctx->p2p_local) + flags_off, 0,
                          tl_p2p_fused_slots_offset(ctx->p2p_max_bytes) - flags_off));
  // the push words AND its slots: their data carries epochs, which restart from zero
  TL_CUDA(ctx, cudaMemset(reinterpret_cast<uint8_t*>(ctx->p2p_local) + tl_p2p_push_words_offset(ctx->p2p_max_bytes), 0,
                          tl_p2p_total_bytes(ctx->p2p_max_bytes) - tl_p2p_push_words_offset(ctx->p2p_max_bytes)));
  TL_CUDA(ctx, cudaMemset(ctx->dev_status, 0, sizeof(int)));
  ctx->fused_tiles = 0;
  ctx->push_pending = false;
  return TL_OK;
}

static int32_t p2p_allreduce_impl(tl_ctx* ctx, const char* who, const void* src, int32_t dtype, void* dst, int32_t dst_dtype,
                                  int64_t count) {
  TL_CHECK_CTX(ctx);
  if (!src || !dst) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: null pointer", who);
  if (count < 0 || !tl_dtype_valid(dtype) || !tl_dtype_valid(dst_dtype)) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: bad count or dtype", who);
  if (dst_dtype != dtype && dtype != TL_F32)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "%s: a result type other than the exchange type needs f32 partial sums", who);
  if (count == 0) return TL_OK;
  const size_t bytes = size_t(count) * tl_dtype_size(dtype);
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: pointers must be 16-byte aligned", who);
  if (ctx->world == 1) {
    DeviceGuard guard(ctx->device);
    if (dst_dtype != dtype) return tl_unary_op(ctx, 0, src, dtype, dst, dst_dtype, count);  // the cast alone
    if (src != dst) TL_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return TL_OK;
  }
  if (!ctx->p2p_attached) return tl_set_error(ctx, TL_ERR_INVALID_ARG, "%s: peers not attached", who);
  if (((bytes + 15) & ~size_t(15)) > ctx->p2p_max_bytes)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "%s: %zu bytes exceed the exchange buffer (%zu)", who, bytes, ctx->p2p_max_bytes);
  DeviceGuard guard(ctx->device);
  P2PArgs a{};
  for (int r = 0; r < ctx->world; ++r) a.base[r] = ctx->p2p_peer[r];
  a.rank = ctx->rank; a.world = ctx->world; a.max_bytes = ctx->p2p_max_bytes; a.count = count;
  a.src = src; a.dst = dst; a.status = ctx->dev_status; a.spin_limit = ctx->wait_limit_polls;
  a.dst_dtype = dtype == TL_F32 ? dst_dtype : TL_F32;  // read by the f32 instantiation only
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(kP2PCtas);
  cfg.blockDim = dim3(kP2PThreads);
  cfg.stream = ctx->stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (dtype == TL_F32) cudaLaunchKernelEx(&cfg, p2p_allreduce_kernel<float>, a);
  else if (dtype == TL_F16) cudaLaunchKernelEx(&cfg, p2p_allreduce_kernel<__half>, a);
  else cudaLaunchKernelEx(&cfg, p2p_allreduce_kernel<__nv_bfloat16>, a);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES]++;
  return TL_OK;
}

int32_t tl_allreduce_sum_p2p(tl_ctx* ctx, const void* src, void* dst, int64_t count, int32_t dtype) {
  return p2p_allreduce_impl(ctx, "tl_allreduce_sum_p2p", src, dtype, dst, dtype, count);
}

int32_t tl_allreduce_sum_p2p_f32_to(tl_ctx* ctx, const float* src, void* dst, int32_t dst_dtype, int64_t count) {
  return p2p_allreduce_impl(ctx, "tl_allreduce_sum_p2p_f32_to", src, TL_F32, dst, dst_dtype, count);
}

}  // extern "C"
