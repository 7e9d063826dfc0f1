// Streaming small-batch (m = 1..16) weight-only int8 matmul: kernel id 8 "stream" of family
// TL_FAMILY_QGEMV.  Same arithmetic contract as the other small-batch kernels
// (src/backend/webgpu/matmul/gemv.ts:311-466 in the reference): out[m,n] = epi(alpha * a . W^T).
//
// What it is built around (measured on B200): a read-only stream of cp.async.bulk copies of
// >= 2 KB row pieces, issued by several lanes, reaches 7.0 TB/s with 64-96 KB in flight per SM,
// needs all SMs, and costs neither registers nor issue slots of the warps that compute.  And:
// between two dependent launches HBM idles for 2-3 us (the finishing kernel only drains, the
// next one may not start), which is a quarter of a 60 MB matrix's streaming time.
//
//   * Persistent grid, one CTA per SM, sized (<= 113 KB shared memory, <= 88 registers) so that
//     TWO launches are resident on every SM: the running one and, under programmatic dependent
//     launch, its successor.
//   * Warp roles.  Producer warps stream the weight through a ring of shared-memory stages
//     (stage = 16 rows x up to 32 k blocks of 64 bytes, one bulk copy per row piece, rows padded
//     by 64 bytes so that fragment reads are bank-conflict free).  Consumer warps turn stages into
//     mma.sync.m16n8k16 products (weights = A operand, batch = B operand; the k blocks of a stage
//     are dealt to the warps round-robin) and keep f32 accumulators per row tile.  One epilogue
//     warp sums the consumers' partial fragments of a finished tile (double-buffered in shared
//     memory), applies scale + epilogue and stores, so the consumers never stop for a tile end.
//   * Work split.  The weight is a flat sequence of k blocks (tile-major); CTA c takes the
//     contiguous share [T*c/G, T*(c+1)/G), so every SM streams the same number of bytes whatever
//     N is.  A row tile whose k range is shared by several CTAs is finished by the last one to
//     arrive: every sharer parks its f32 partial tile in a fixed scratch slot and bumps the
//     tile's counter; the last arriver adds the parts IN CTA ORDER (results do not depend on
//     arrival order), applies the epilogue and clears the counter.  Nobody waits on anybody.
//   * Drain-timed ring fill.  The successor's producers do not fill their ring at once: lane 0
//     watches a counter that the running launch's producers bump when they have issued their
//     last stage, and fills only then.  The successor's first 96 KB per SM therefore travel
//     exactly while the predecessor drains, and HBM never idles across the launch boundary.  The
//     counter is advisory (results never depend on it): the watcher also leaves when the
//     consumers of its own CTA pass griddepcontrol.wait, and after a bounded number of polls.
//
// Every wait is bounded; a wait that runs out records a code in the context's status word,
// raises the CTA's abort flag and the roles return.
//
// Standing (B200, 14336 x 4096, graph-replayed over rotating weight copies): results match the
// other kernels, the successor launch is resident beside the running one and fills its ring during
// the drain as designed, and with the MMA work taken out the consumer phase streams at 6.3 TB/s.
// With the real work it is SLOWER than the ring kernel (18-20 us against 12.7 us per launch at
// m = 1): a stage (32 KB) takes eight consumer warps 0.7 us from "full" to "all arrived", the ring
// holds three stages, so a slot is reused every 0.7 + 0.4 (issue) + 1.8 us (HBM under load) and the
// 64 KB in flight per SM cover only two thirds of the bandwidth-latency product; the register file
// of two resident launches (80 registers x 12 warps each) leaves no room for more consumer warps
// (16 lean warps at 48 registers measured slower still), and asking L2 for stages ahead of the ring
// did not shorten the cycle.  The kernel stays a tuning candidate (never the default choice).
#include <algorithm>

#include "tl_common.cuh"
#include "tl_mma_frag.cuh"
#include "tl_tma.cuh"

namespace {

constexpr int kStream = 8;
constexpr int kStreamMaxItems = 4;
constexpr int kStreamMaxStages = 8;
constexpr int kStreamMaxProducers = 2;
constexpr int kPfSlots = 8;
constexpr int kPfPollLimit = 1 << 16;

struct StreamArgs {
  const void* a;                          // activations [m, k]
  const uint8_t* w[kStreamMaxItems];      // packed weights [n_i, k]
  const void* scales[kStreamMaxItems];
  void* out[kStreamMaxItems];             // [m, n_i]
  int32_t n[kStreamMaxItems];
  int32_t tile_start[kStreamMaxItems + 1];  // flat 16-row tile ranges of the items
  EpiParams epi[kStreamMaxItems];
  int32_t m, k, kb_per_tile;              // kb_per_tile = k / 64
  int32_t group, groups_per_row, scales_dtype, out_dtype;
  float wscale;                           // 1/127 for the snorm convention, 1 for direct
  int64_t total_kb;                       // tiles * kb_per_tile
  int32_t skb, nstages, producers;
  int32_t l2_ahead;                       // stages the producers ask L2 for beyond the ring (0 = off)
  uint32_t row_stride;                    // bytes between rows of a stage: skb * 64 + 64
  float* partial;                         // [grid][2][NT * 128] f32 partial tiles of shared row tiles
  unsigned* counters;                     // [grid], all zero between launches
  int* status;
  uint32_t* pf_flags;                     // [kPfSlots] drain counters (advisory)
  int32_t pf_slot, pf_prev, pf_thresh;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void l2_prefetch_bulk(const void* gptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gptr), "r"(bytes) : "memory");
}

// The CTA whose share [T*c/G, T*(c+1)/G) holds k block b.
__device__ __forceinline__ int stream_owner(int64_t b, int64_t total, int grid) {
  const int64_t c = ((b + 1) * grid + total - 1) / total - 1;
  return int(c < grid - 1 ? c : grid - 1);
}

// Walks a CTA's share stage by stage; every role runs the same walk.  The share is walked
// rotated by one tile: first its LAST row tile, then the rest from the start.  The tiles a CTA
// shares with its neighbours (the first and the last of its share) are therefore the first two
// it works on, for every CTA, so the hand-over of shared tiles (scratch, fence, counter) overlaps
// the stream instead of sitting in the kernel's tail.
struct StreamWalk {
  int64_t cur, end, b0, split;  // [split, b1) is walked first, then [b0, split)
  int32_t tile, kb0, kb_per_tile, skb;
  bool second;
  __device__ StreamWalk(int64_t b0_, int64_t b1, int32_t kbt, int32_t skb_) : end(b1), b0(b0_), kb_per_tile(kbt), skb(skb_) {
    const int64_t last_tile_start = ((b1 - 1) / kbt) * kbt;
    split = last_tile_start > b0_ ? last_tile_start : b0_;
    second = split == b0_;  // a share inside one tile has no second part
    cur = split;
    tile = int32_t(cur / kbt);
    kb0 = int32_t(cur - int64_t(tile) * kbt);
    if (b1 <= b0_) { cur = end; second = true; }
  }
  __device__ bool done() const { return cur >= end && second; }
  __device__ int count() const {  // k blocks of the current stage
    const int64_t left = end - cur;
    int n = kb_per_tile - kb0;
    if (n > skb) n = skb;
    return left < n ? int(left) : n;
  }
  // true when the stage just consumed was this CTA's last of its tile
  __device__ bool advance(int n) {
    cur += n;
    kb0 += n;
    const bool tile_end = kb0 == kb_per_tile || cur >= end;
    if (kb0 == kb_per_tile) { kb0 = 0; ++tile; }
    if (cur >= end && !second) {
      second = true;
      cur = b0;
      end = split;
      tile = int32_t(cur / kb_per_tile);
      kb0 = int32_t(cur - int64_t(tile) * kb_per_tile);
    }
    return tile_end;
  }
};

template <typename AT, int NT, bool GROUPED, int C, int JMAX>
__global__ void __launch_bounds__((C + 4) * 32, 2) qgemv_stream_kernel(const __grid_constant__ StreamArgs p) {
  extern __shared__ __align__(128) uint8_t stream_smem[];
  __shared__ uint64_t full_bar[kStreamMaxStages], empty_bar[kStreamMaxStages], red_full[2], red_empty[2];
  __shared__ int abort_flag, released;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t stage_bytes = 16u * p.row_stride;
  float* red = reinterpret_cast<float*>(stream_smem + size_t(p.nstages) * stage_bytes);  // [2][C][NT][4][32]
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.nstages; ++s) {
      mbar_init(&full_bar[s], p.producers);
      mbar_init(&empty_bar[s], C);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&red_full[b], C);
      mbar_init(&red_empty[b], 1);
    }
    abort_flag = 0;
    released = 0;
    mbar_fence_init();
  }
  __syncthreads();
  const int grid = int(gridDim.x), cta = int(blockIdx.x);
  const int64_t b0 = p.total_kb * cta / grid, b1 = p.total_kb * (cta + 1) / grid;
  const int ep_warp = C + p.producers;

  if (warp >= C && warp < ep_warp) {
    // ------------------------------ producers ------------------------------
    const int pw = warp - C;
    const int rows_mine = 16 / p.producers;  // rows pw, pw + producers, ...
    if (p.pf_flags != nullptr) {
      if (pw == 0 && lane == 0) {
        if (cta == 0) *reinterpret_cast<volatile uint32_t*>(p.pf_flags + ((p.pf_slot + kPfSlots / 2) & (kPfSlots - 1))) = 0u;
        const volatile uint32_t* flag = p.pf_flags + p.pf_prev;
        const volatile int* rel = &released;
        for (int it = 0; it < kPfPollLimit; ++it) {
          if (*flag >= uint32_t(p.pf_thresh) || *rel != 0) break;
          __nanosleep(100);
        }
        *reinterpret_cast<volatile int*>(&released) = 2;  // lets the other producer warps go
      } else if (lane == 0) {
        const volatile int* rel = &released;
        for (int it = 0; it < kPfPollLimit; ++it) {
          if (*rel != 0) break;
          __nanosleep(100);
        }
      }
      __syncwarp();
    }
    StreamWalk wk(b0, b1, p.kb_per_tile, p.skb);
    // A second cursor runs nstages + l2_ahead stages ahead and only asks L2 for the pieces
    // (cp.async.bulk.prefetch.L2, fire and forget): the HBM latency (about 1.8 us under load) is then
    // covered by L2 capacity instead of shared memory, and the ring's loads hit L2.
    StreamWalk wa(b0, b1, p.kb_per_tile, p.skb);
    auto ask_l2 = [&]() {
      if (wa.done()) return;
      const int n = wa.count();
      if (lane < rows_mine) {
        const int r = pw + lane * p.producers;
        const int t = wa.tile;
        const int it = (t >= p.tile_start[1]) + (t >= p.tile_start[2]) + (t >= p.tile_start[3]);
        int64_t row = int64_t(t - p.tile_start[it]) * 16 + r;
        if (row > p.n[it] - 1) row = p.n[it] - 1;
        l2_prefetch_bulk(p.w[it] + row * p.k + int64_t(wa.kb0) * 64, uint32_t(n) * 64u);
      }
      wa.advance(n);
    };
    if (p.l2_ahead > 0) {
      for (int i = 0; i < p.nstages && !wa.done(); ++i) wa.advance(wa.count());  // the ring's first fill needs no hint
      for (int i = 0; i < p.l2_ahead; ++i) ask_l2();
    }
    for (int i = 0; !wk.done(); ++i) {
      const int s = i % p.nstages, n = wk.count();
      if (i >= p.nstages && !mbar_wait(&empty_bar[s], ((i / p.nstages) - 1) & 1, &abort_flag)) {
        if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_EMPTY); }
        return;
      }
      const uint32_t piece = uint32_t(n) * 64u;
      if (lane == 0) mbar_expect_tx(&full_bar[s], piece * uint32_t(rows_mine));
      __syncwarp();
      if (lane < rows_mine) {
        const int r = pw + lane * p.producers;
        const int t = wk.tile;
        const int it = (t >= p.tile_start[1]) + (t >= p.tile_start[2]) + (t >= p.tile_start[3]);
        int64_t row = int64_t(t - p.tile_start[it]) * 16 + r;
        if (row > p.n[it] - 1) row = p.n[it] - 1;
        bulk_load(smem_u32(stream_smem) + uint32_t(s) * stage_bytes + uint32_t(r) * p.row_stride,
                  p.w[it] + row * p.k + int64_t(wk.kb0) * 64, piece, &full_bar[s]);
      }
      wk.advance(n);
      if (p.l2_ahead > 0) ask_l2();
    }
    if (p.pf_flags != nullptr && pw == 0 && lane == 0) atomicAdd(p.pf_flags + p.pf_slot, 1u);
    return;
  }

  // everything below reads the predecessor's output or writes global memory
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (warp == 0 && lane == 0) atomicCAS(&released, 0, 1);

  if (warp == ep_warp) {
    // ------------------------------ epilogue warp ------------------------------
    // Lane (g, tt) owns weight rows g and g+8 of a tile (fragment slots 0,1 and 2,3) for batch
    // columns 2tt, 2tt+1 of every token tile.
    // (The per-row values of a tile are requested one tile AHEAD: they are cold misses that take
    // as long as a tile takes to stream, and this warp has nothing to overlap them with otherwise.)
    StreamWalk wk(b0, b1, p.kb_per_tile, p.skb);
    const int g = lane >> 2, tt = lane & 3;
    int tile_i = 0;
    float sc_next[2] = {0.f, 0.f}, bias_next[2] = {0.f, 0.f};
    auto request_rows = [&](int t) {
      const int it = (t >= p.tile_start[1]) + (t >= p.tile_start[2]) + (t >= p.tile_start[3]);
      const int64_t tile_row = int64_t(t - p.tile_start[it]) * 16;
      const bool fast_bias = p.epi[it].fast != 0 && p.epi[it].fast_bias != nullptr;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t row = min(tile_row + g + 8 * h, int64_t(p.n[it]) - 1);
        sc_next[h] = GROUPED ? p.wscale : p.wscale * tl_load_scale(p.scales[it], p.scales_dtype, row);
        bias_next[h] = fast_bias ? __ldg(p.epi[it].fast_bias + row) : 0.f;
      }
    };
    if (!wk.done()) request_rows(wk.tile);
    while (!wk.done()) {
      const int t = wk.tile;
      const int64_t t_lo = int64_t(t) * p.kb_per_tile, t_hi = t_lo + p.kb_per_tile;
      bool tile_end = false;
      while (!tile_end) tile_end = wk.advance(wk.count());
      const int it = (t >= p.tile_start[1]) + (t >= p.tile_start[2]) + (t >= p.tile_start[3]);
      const int64_t tile_row = int64_t(t - p.tile_start[it]) * 16;
      const int n_it = p.n[it];
      const EpiParams& epi = p.epi[it];
      const bool fast = epi.fast != 0;
      const float sc[2] = {sc_next[0], sc_next[1]}, bias[2] = {bias_next[0], bias_next[1]};
      if (!wk.done()) request_rows(wk.tile);
      const int buf = tile_i & 1;
      if (!mbar_wait(&red_full[buf], (tile_i >> 1) & 1, &abort_flag)) {
        if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_FULL); }
        return;
      }
      float v[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float sum = 0.f;
#pragma unroll
          for (int w = 0; w < C; ++w) sum += red[(((buf * C + w) * NT + nt) * 4 + i) * 32 + lane];
          v[nt][i] = sum;
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_empty[buf]);
      ++tile_i;
      const bool whole = b0 <= t_lo && b1 >= t_hi;
      bool finish = true;
      if (!whole) {
        // shared row tile: park the partial, count, and let the last arriver add the parts in CTA order
        const int c_lo = stream_owner(t_lo, p.total_kb, grid), c_hi = stream_owner(t_hi - 1, p.total_kb, grid);
        float* mine = p.partial + (size_t(2 * cta + (cta == c_lo ? 1 : 0)) * NT * 128);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) __stcg(mine + (nt * 4 + i) * 32 + lane, v[nt][i]);
        __threadfence();
        __syncwarp();
        unsigned prev = 0;
        if (lane == 0) prev = atomicAdd(p.counters + c_lo, 1u);
        prev = __shfl_sync(0xffffffffu, prev, 0);
        finish = prev == unsigned(c_hi - c_lo);
        if (finish) {
          __threadfence();
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) v[nt][i] = 0.f;
          for (int cc = c_lo; cc <= c_hi; ++cc) {
            const float* part = p.partial + (size_t(2 * cc + (cc == c_lo ? 1 : 0)) * NT * 128);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
              for (int i = 0; i < 4; ++i) v[nt][i] += __ldcg(part + (nt * 4 + i) * 32 + lane);
          }
          __syncwarp();
          if (lane == 0) p.counters[c_lo] = 0u;
        }
      }
      if (finish) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int h = i >> 1;
            const int64_t row = tile_row + g + 8 * h;
            const int col = 8 * nt + 2 * tt + (i & 1);
            float r;
            if (fast) {
              r = (v[nt][i] * sc[h]) * epi.alpha + bias[h];  // tl_apply_epilogue's order: scale, alpha, bias, unary
              if (epi.fast_unary) r = tl_unary(epi.fast_unary, r);
            } else {
              r = (row < n_it && col < p.m) ? tl_apply_epilogue(epi, v[nt][i] * sc[h], col, row, n_it) : 0.f;
            }
            v[nt][i] = r;
          }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int64_t row = tile_row + g + 8 * (i >> 1);
            const int col = 8 * nt + 2 * tt + (i & 1);
            if (row < n_it && col < p.m) tl_store_out(p.out[it], p.out_dtype, int64_t(col) * n_it + row, v[nt][i]);
          }
      }
    }
    return;
  }

  if (warp > ep_warp) return;

  // ------------------------------ consumers ------------------------------
  const int g = lane >> 2, t4 = lane & 3;
  const AT* a = reinterpret_cast<const AT*>(p.a);
  const AT* a_col[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) a_col[nt] = a + int64_t(min(g + 8 * nt, p.m - 1)) * p.k + 16 * t4;
  float total[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) total[nt][e] = 0.f;
  const uint32_t ring = smem_u32(stream_smem);
  const uint32_t frag_off = uint32_t(g) * p.row_stride + 16u * uint32_t(t4);
  StreamWalk wk(b0, b1, p.kb_per_tile, p.skb);
  int tile_i = 0;
  for (int i = 0; !wk.done(); ++i) {
    const int s = i % p.nstages, n = wk.count(), kb0 = wk.kb0;
    int j0 = (warp - kb0) % C;
    if (j0 < 0) j0 += C;
    // This warp's activation fragments (and group scales) of the stage are requested before the
    // wait for the stage's weights, so that their latency hides behind it.  Nothing below is
    // conditional on how many of the JMAX k blocks exist: a missing one reads a valid address and
    // multiplies zero weights, so the compiler is free to interleave the blocks' MMA chains.
    uint4 bx[JMAX][NT][2];
    float s_lo[JMAX], s_hi[JMAX];
    if (GROUPED) {
      const int tt = wk.tile;
      const int it = (tt >= p.tile_start[1]) + (tt >= p.tile_start[2]) + (tt >= p.tile_start[3]);
      const int64_t tile_row = int64_t(tt - p.tile_start[it]) * 16;
      const int64_t r_lo = min(tile_row + g, int64_t(p.n[it]) - 1), r_hi = min(tile_row + g + 8, int64_t(p.n[it]) - 1);
#pragma unroll
      for (int jj = 0; jj < JMAX; ++jj) {
        const int j = j0 + jj * C;
        const int gi = ((kb0 + (j < n ? j : 0)) * 64) / p.group;
        s_lo[jj] = tl_load_scale(p.scales[it], p.scales_dtype, r_lo * p.groups_per_row + gi);
        s_hi[jj] = tl_load_scale(p.scales[it], p.scales_dtype, r_hi * p.groups_per_row + gi);
      }
    }
    constexpr bool kAhead = C <= 8;  // 16 lean consumer warps (48 registers) load fragments right before use instead
    if (kAhead) {
#pragma unroll
      for (int jj = 0; jj < JMAX; ++jj) {
        const int j = j0 + jj * C;
        const int kb = kb0 + (j < n ? j : 0);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4* src = reinterpret_cast<const uint4*>(a_col[nt] + int64_t(kb) * 64);
          bx[jj][nt][0] = __ldg(src);
          bx[jj][nt][1] = __ldg(src + 1);
        }
      }
    }
    if (!mbar_wait(&full_bar[s], (i / p.nstages) & 1, &abort_flag)) {
      if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_FULL); }
      return;
    }
    const uint32_t sbase = ring + uint32_t(s) * stage_bytes + frag_off;
    if (!kAhead) {
      // lean path (16 consumer warps, 48 registers): one k block at a time, fragments loaded right
      // before use; latency is covered by the other warps
#pragma unroll
      for (int jj = 0; jj < JMAX; ++jj) {
        const int j = j0 + jj * C;
        const bool ok = j < n;
        const int kb = kb0 + (ok ? j : 0);
        uint4 x[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint4* src = reinterpret_cast<const uint4*>(a_col[nt] + int64_t(kb) * 64);
          x[nt][0] = __ldg(src);
          x[nt][1] = __ldg(src + 1);
        }
        uint4 wl = lds128(sbase + uint32_t(ok ? j : 0) * 64u);
        uint4 wh = lds128(sbase + uint32_t(ok ? j : 0) * 64u + 8u * p.row_stride);
        if (!ok) { wl = make_uint4(0, 0, 0, 0); wh = make_uint4(0, 0, 0, 0); }
        float c[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) c[nt][e] = GROUPED ? 0.f : total[nt][e];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint32_t wlo = q == 0 ? wl.x : q == 1 ? wl.y : q == 2 ? wl.z : wl.w;
          const uint32_t whi = q == 0 ? wh.x : q == 1 ? wh.y : q == 2 ? wh.z : wh.w;
          uint32_t a0, a1, a2, a3;
          MmaOps<AT>::cvt(wlo, a0, a2);
          MmaOps<AT>::cvt(whi, a1, a3);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 v = x[nt][q >> 1];
            const uint32_t x0 = (q & 1) ? v.z : v.x, x1 = (q & 1) ? v.w : v.y;
            MmaOps<AT>::mma_free(c[nt], a0, a1, a2, a3, x0, x1);
          }
        }
        if (GROUPED) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            total[nt][0] = fmaf(s_lo[jj], c[nt][0], total[nt][0]);
            total[nt][1] = fmaf(s_lo[jj], c[nt][1], total[nt][1]);
            total[nt][2] = fmaf(s_hi[jj], c[nt][2], total[nt][2]);
            total[nt][3] = fmaf(s_hi[jj], c[nt][3], total[nt][3]);
          }
        } else {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) total[nt][e] = c[nt][e];
        }
      }
    }
    // two k blocks at a time, q outer and k block inner: consecutive MMAs belong to different
    // accumulator chains (a dependent m16n8k16 chain issues every 20 cycles, two chains every 10)
#pragma unroll
    for (int j2 = 0; kAhead && j2 < JMAX; j2 += 2) {
      uint4 wl[2], wh[2];
      float c[2][NT][4];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) c[u][nt][e] = 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int j = j0 + (j2 + u) * C;
        const bool ok = j2 + u < JMAX && j < n;
        wl[u] = lds128(sbase + uint32_t(ok ? j : 0) * 64u);
        wh[u] = lds128(sbase + uint32_t(ok ? j : 0) * 64u + 8u * p.row_stride);
        if (!ok) { wl[u] = make_uint4(0, 0, 0, 0); wh[u] = make_uint4(0, 0, 0, 0); }  // int8 zeros
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          if (j2 + u >= JMAX) continue;
          const uint32_t wlo = q == 0 ? wl[u].x : q == 1 ? wl[u].y : q == 2 ? wl[u].z : wl[u].w;
          const uint32_t whi = q == 0 ? wh[u].x : q == 1 ? wh[u].y : q == 2 ? wh[u].z : wh[u].w;
          uint32_t a0, a1, a2, a3;
          MmaOps<AT>::cvt(wlo, a0, a2);  // row g   : k slots (2t,2t+1) and (2t+8,2t+9)
          MmaOps<AT>::cvt(whi, a1, a3);  // row g+8
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const uint4 v = bx[j2 + u][nt][q >> 1];
            const uint32_t x0 = (q & 1) ? v.z : v.x, x1 = (q & 1) ? v.w : v.y;
            MmaOps<AT>::mma_free(c[u][nt], a0, a1, a2, a3, x0, x1);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (j2 + u >= JMAX) continue;
        if (GROUPED) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            total[nt][0] = fmaf(s_lo[j2 + u], c[u][nt][0], total[nt][0]);
            total[nt][1] = fmaf(s_lo[j2 + u], c[u][nt][1], total[nt][1]);
            total[nt][2] = fmaf(s_hi[j2 + u], c[u][nt][2], total[nt][2]);
            total[nt][3] = fmaf(s_hi[j2 + u], c[u][nt][3], total[nt][3]);
          }
        } else {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) total[nt][e] += c[u][nt][e];
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[s]);  // this warp no longer reads the stage
    if (wk.advance(n)) {
      // tile finished (for this CTA): hand the fragment sums to the epilogue warp
      const int buf = tile_i & 1;
      if (tile_i >= 2 && !mbar_wait(&red_empty[buf], ((tile_i >> 1) - 1) & 1, &abort_flag)) {
        if (lane == 0 && !abort_flag) { abort_flag = 1; atomicExch(p.status, TL_DEV_TIMEOUT_EMPTY); }
        return;
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          red[(((buf * C + warp) * NT + nt) * 4 + e) * 32 + lane] = total[nt][e];
          total[nt][e] = 0.f;
        }
      __syncwarp();
      if (lane == 0) mbar_arrive(&red_full[buf]);
      ++tile_i;
    }
  }
}

template <typename AT, int NT, bool GROUPED>
cudaError_t stream_launch_j(int cwarps, int jmax, int grid, int block, size_t smem, cudaStream_t s, const StreamArgs& p) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#define TL_STREAM_GO(C_, J_)                                                                          \
  do {                                                                                               \
    auto kern = qgemv_stream_kernel<AT, NT, GROUPED, C_, J_>;                                         \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));              \
    return cudaLaunchKernelEx(&cfg, kern, p);                                                        \
  } while (0)
  if (cwarps == 16) {
    if (jmax <= 1) TL_STREAM_GO(16, 1);
    TL_STREAM_GO(16, 2);
  }
  if (jmax <= 2) TL_STREAM_GO(8, 2);
  TL_STREAM_GO(8, 4);
#undef TL_STREAM_GO
}

template <typename AT>
cudaError_t stream_launch(bool two, bool grouped, int cwarps, int jmax, int grid, int block, size_t smem, cudaStream_t s, const StreamArgs& p) {
  if (two) return grouped ? stream_launch_j<AT, 2, true>(cwarps, jmax, grid, block, smem, s, p) : stream_launch_j<AT, 2, false>(cwarps, jmax, grid, block, smem, s, p);
  return grouped ? stream_launch_j<AT, 1, true>(cwarps, jmax, grid, block, smem, s, p) : stream_launch_j<AT, 1, false>(cwarps, jmax, grid, block, smem, s, p);
}

}  // namespace

bool tl_qgemv_stream_applicable(const tl_variant& v, int64_t m, int64_t k, int32_t a_dtype, const tl_quant_desc& q) {
  return v.kernel == kStream && m >= 1 && m <= 16 && (a_dtype == TL_F16 || a_dtype == TL_BF16) && k % 64 == 0 && k >= 64 &&
         q.group_size % 64 == 0 && (v.p0 == 8 || v.p0 == 16) && v.p1 >= 2 && v.p1 <= kStreamMaxStages && ((v.p2 & 3) == 1 || (v.p2 & 3) == 2) && (v.p2 >> 2) <= 16 &&
         v.p3 >= 8 && v.p3 <= 32 && v.p3 % 2 == 0;
}

// Geometry of a stream launch: grid, block, dynamic shared memory.
void tl_qgemv_stream_geometry(tl_ctx* ctx, const tl_variant& v, int32_t m, int64_t tiles, int64_t k, int* grid, int* block,
                              size_t* smem) {
  const int nt = m > 8 ? 2 : 1;
  const int64_t total_kb = tiles * (k / 64);
  *grid = int(std::max<int64_t>(1, std::min<int64_t>(ctx->sm_count, total_kb / 8)));
  *block = (v.p0 + (v.p2 & 3) + 1) * 32;
  *smem = size_t(v.p1) * 16 * (size_t(v.p3) * 64 + 64) + size_t(2) * v.p0 * nt * 4 * 32 * sizeof(float);
}

// One launch over up to four matrices that read the same activations (items of one tl_qgemv_nt_batched
// call, or the single matrix of tl_qgemv_nt).
int32_t tl_launch_qgemv_stream(tl_ctx* ctx, const tl_variant& v, const void* a, int32_t a_dtype, int32_t n_items,
                               const void* const* packed, const void* const* scales, void* const* out, const int64_t* n,
                               const EpiParams* epi, int32_t out_dtype, int32_t m, int64_t k, const tl_quant_desc& q,
                               tl_plan_receipt* receipt) {
  if (!tl_qgemv_stream_applicable(v, m, k, a_dtype, q) || n_items < 1 || n_items > kStreamMaxItems)
    return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "qgemv: variant stream cannot run m=%d k=%lld G=%d %s", m, (long long)k,
                        q.group_size, tl_dtype_name(a_dtype));
  StreamArgs p{};
  int64_t tiles = 0;
  for (int i = 0; i < kStreamMaxItems; ++i) {
    p.tile_start[i] = int32_t(tiles);
    if (i >= n_items) continue;
    p.w[i] = reinterpret_cast<const uint8_t*>(packed[i]);
    p.scales[i] = scales[i];
    p.out[i] = out[i];
    p.n[i] = int32_t(n[i]);
    p.epi[i] = epi[i];
    tiles += (n[i] + 15) / 16;
    if ((reinterpret_cast<uintptr_t>(packed[i]) & 15))
      return tl_set_error(ctx, TL_ERR_INVALID_ARG, "qgemv: stream needs 16-byte aligned weight pointers");
  }
  p.tile_start[kStreamMaxItems] = int32_t(tiles);
  if (reinterpret_cast<uintptr_t>(a) & 15)
    return tl_set_error(ctx, TL_ERR_INVALID_ARG, "qgemv: stream needs 16-byte aligned activation pointers");
  int grid = 0, block = 0;
  size_t smem = 0;
  tl_qgemv_stream_geometry(ctx, v, m, tiles, k, &grid, &block, &smem);
  if (receipt) {
    receipt->choice = v;
    receipt->grid[0] = grid; receipt->grid[1] = 1; receipt->grid[2] = 1;
    receipt->block = block; receipt->split_k = 1;
    return TL_OK;
  }
  const int nt = m > 8 ? 2 : 1;
  if (!ctx->stream_scratch) {
    // partial tiles [SMs][2][2 * 128] f32 + one counter per CTA; never grows, so captured graphs stay valid
    const size_t bytes = size_t(ctx->sm_count) * 2 * 2 * 128 * sizeof(float) + size_t(ctx->sm_count) * sizeof(unsigned);
    if (ctx->capturing)
      return tl_set_error(ctx, TL_ERR_UNSUPPORTED, "qgemv: the stream kernel's scratch must exist before graph capture; run the call once first");
    TL_CUDA(ctx, cudaMalloc(&ctx->stream_scratch, bytes));
    TL_CUDA(ctx, cudaMemset(ctx->stream_scratch, 0, bytes));
  }
  p.a = a;
  p.m = m; p.k = int32_t(k); p.kb_per_tile = int32_t(k / 64);
  p.group = q.group_size; p.groups_per_row = int32_t(k / q.group_size);
  p.scales_dtype = q.scales_dtype; p.out_dtype = out_dtype;
  p.wscale = q.scale_convention == TL_SCALE_SNORM127 ? 1.0f / 127.0f : 1.0f;
  p.total_kb = tiles * p.kb_per_tile;
  p.skb = v.p3; p.nstages = v.p1; p.producers = v.p2 & 3; p.l2_ahead = v.p2 >> 2;
  p.row_stride = uint32_t(v.p3) * 64u + 64u;
  p.partial = reinterpret_cast<float*>(ctx->stream_scratch);
  p.counters = reinterpret_cast<unsigned*>(reinterpret_cast<uint8_t*>(ctx->stream_scratch) + size_t(ctx->sm_count) * 2 * 2 * 128 * sizeof(float));
  p.status = ctx->dev_status;
  p.pf_flags = ctx->pf_flags;
  p.pf_slot = ctx->pf_next & (kPfSlots - 1);
  p.pf_prev = (ctx->pf_next + kPfSlots - 1) & (kPfSlots - 1);
  p.pf_thresh = (ctx->pf_last_grid + 1) / 2;
  ctx->pf_next++;
  ctx->pf_last_grid = grid;
  const bool grouped = q.group_size != k;
  const int jmax = (v.p3 + v.p0 - 1) / v.p0;
  cudaError_t e = a_dtype == TL_F16 ? stream_launch<__half>(nt == 2, grouped, v.p0, jmax, grid, block, smem, ctx->stream, p)
                                    : stream_launch<__nv_bfloat16>(nt == 2, grouped, v.p0, jmax, grid, block, smem, ctx->stream, p);
  TL_CUDA(ctx, e);
  TL_CUDA(ctx, cudaGetLastError());
  ctx->counters[TL_COUNTER_KERNEL_LAUNCHES] += 1;
  return TL_OK;
}

