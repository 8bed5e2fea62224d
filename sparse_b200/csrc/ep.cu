// Expert-parallel dispatch and combine over NVLink peer memory.
//
// Replaces the reference's five `all_to_all_single` calls per layer, the two
// host syncs between them and the local re-sort of received rows
// (utils/eval_core.py:14865-15060, 13240-13253).  One process per GPU; every
// rank maps the receive buffers of all ranks (CUDA IPC) and moves rows with
// plain peer stores and loads inside its own kernels:
//
//   publish   each rank writes its per-expert item counts into every rank's
//             counts matrix [ep][E]                                  (peer stores)
//   barrier   flag exchange in peer memory, bounded wait
//   plan      from the counts matrix every rank derives, without talking again,
//             where each (source rank, expert) segment lives in the owner's
//             receive buffer: the buffer is laid out expert-major, then source
//             rank, then the source's stable item order, so rows ARRIVE
//             expert-sorted and the owner needs no second sort; also the
//             owner's row-tile table for the grouped GEMM
//   dispatch  one warp per item copies the token's activation row and route
//             weight straight into its final row of the owner's buffer
//   barrier   rows have landed
//   (grouped GEMM on the owner, on its own rows)
//   barrier   outputs are complete
//   combine   each token reads its K output rows from the owners' buffers and
//             adds them in ascending expert id (bf16-sequential), plus the
//             shared expert's row
//
// No host synchronisation and no size negotiation: the receive buffers are
// sized for the worst case (every item of every rank to one owner).
// Wire bytes per remote (token, expert) pair: H*2 out, H*2 back, 2 for the
// route weight.
//
// The barrier's spin is bounded (2 s); on expiry it writes `status` = 3 and
// returns.  Ranks are separate processes on separate GPUs; two ranks of this
// barrier must never share one GPU.
#include <string.h>

#include <atomic>

#include "sb_common.cuh"

namespace sb {

// CTAs of the dispatch kernel per SM (sb_set_tuning("dispatch_ctas", 1..8)).
static std::atomic<int> g_dispatch_ctas{1};
int32_t set_ep_tuning(const char *key, int value) {
  if (strcmp(key, "dispatch_ctas") == 0) {
    if (value < 1 || value > 8) return fail(SB_E_INVALID_ARG, "sb_set_tuning: dispatch_ctas must be in [1,8]");
    g_dispatch_ctas.store(value);
    return SB_OK;
  }
  return SB_E_UNSUPPORTED;
}
static int dispatch_ctas_per_sm() { return g_dispatch_ctas.load(std::memory_order_relaxed); }

namespace {

constexpr int kMaxRanks = 16;
constexpr int kMaxExperts = 256;
constexpr int kMaxK = 8;
constexpr unsigned long long kBarrierLimitNs = 2000000000ull;

struct PeerPtrs { void *p[kMaxRanks]; };

__device__ __forceinline__ unsigned long long gtimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// counts_all on every rank: [ep][E]; this rank fills row `rank` everywhere.
// Items of an expert that this rank executes itself out of a cache slot
// (`local_map[e]` >= 0) take no part in the exchange: their count is published as 0.
__device__ __forceinline__ void publish_body(const int32_t *__restrict__ local_offsets, int E, int rank, int ep,
                                             const PeerPtrs &counts_all,
                                             const int32_t *__restrict__ local_map = nullptr) {
  for (int i = threadIdx.x; i < E * ep; i += blockDim.x) {
    int p = i / E, e = i - p * E;
    int32_t *dst = static_cast<int32_t *>(counts_all.p[p]) + (size_t)rank * E + e;
    const bool kept = local_map != nullptr && local_map[e] >= 0;
    *dst = kept ? 0 : local_offsets[e + 1] - local_offsets[e];
  }
}

__global__ void ep_publish_kernel(const int32_t *__restrict__ local_offsets, int E, int rank, int ep,
                                  PeerPtrs counts_all) {
  publish_body(local_offsets, E, rank, ep, counts_all);
}

// Thread p < ep tells peer p "this rank reached `epoch`" and waits for peer p's
// flag to reach it; the wait is bounded.
__device__ __forceinline__ void barrier_body(const PeerPtrs &flags, int rank, int ep, uint32_t epoch,
                                             int32_t *__restrict__ status,
                                             unsigned long long limit_ns = kBarrierLimitNs) {
  const int p = threadIdx.x;
  if (p >= ep) return;
  __threadfence_system();
  uint32_t *remote = static_cast<uint32_t *>(flags.p[p]) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
  const uint32_t *mine = static_cast<const uint32_t *>(flags.p[rank]) + p;
  const unsigned long long t0 = gtimer_ns();
  for (;;) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int32_t)(v - epoch) >= 0) break;
    if (gtimer_ns() - t0 > limit_ns) {
      if (status) atomicExch(status, 3);
      break;
    }
    __nanosleep(100);
  }
  __threadfence_system();
}

// The epoch of a barrier that takes it from this rank's device counter: every
// rank runs the same sequence of barriers, so the counters advance in step and
// a captured CUDA graph can be replayed (no epoch baked into the launch).
__device__ __forceinline__ uint32_t next_epoch(uint32_t *counter) {
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) { s_epoch = *counter + 1u; *counter = s_epoch; }
  __syncthreads();
  return s_epoch;
}

__global__ void ep_barrier_kernel(PeerPtrs flags, int rank, int ep, uint32_t epoch, uint32_t *epoch_counter,
                                  int32_t *__restrict__ status, unsigned long long limit_ns) {
  if (epoch_counter != nullptr) epoch = next_epoch(epoch_counter);
  barrier_body(flags, rank, ep, epoch, status, limit_ns);
}

// One CTA.  Reads the complete counts matrix of this rank and writes
//   dst_base[e]  first row, in the destination's receive buffer, of THIS rank's items of expert e
//   recv_offsets[E+1], tile table: this rank's receive-side expert segments
// `owner` is the destination table [ep][E]: owner[s][e] = rank that executes
// expert e for tokens on rank s (one row repeated for plain ownership, different
// rows when hot experts are replicated and sources are spread over the replicas).
__device__ __forceinline__ void plan_body(const volatile int32_t *counts_all,
                                          const int32_t *__restrict__ owner, int E, int rank, int ep,
                                          int tile_cap, int tile_rows, int32_t *__restrict__ dst_base,
                                          int32_t *__restrict__ recv_offsets, int32_t *__restrict__ tile_table,
                                          int *plan_smem) {
  int *tot = plan_smem;                    // [ep][E] rows of expert e arriving at rank d
  int *seg = tot + ep * E;                 // [ep][E] first row of expert e in rank d's buffer
  int *my_off = seg + ep * E;              // [E+1]
  int *tile_start = my_off + (E + 1);      // [E+1]
  for (int i = threadIdx.x; i < ep * E; i += blockDim.x) {
    const int d = i / E, e = i - d * E;
    int t = 0;
    for (int s = 0; s < ep; ++s)
      if (owner[(size_t)s * E + e] == d) t += counts_all[(size_t)s * E + e];
    tot[i] = t;
  }
  __syncthreads();
  if (threadIdx.x < ep) {
    const int d = threadIdx.x;
    int run = 0;
    for (int e = 0; e < E; ++e) { seg[d * E + e] = run; run += tot[d * E + e]; }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ts = 0;
    for (int e = 0; e < E; ++e) {
      my_off[e] = seg[rank * E + e];
      tile_start[e] = ts;
      ts += (tot[rank * E + e] + tile_rows - 1) / tile_rows;
    }
    const int last = E > 0 ? seg[rank * E + E - 1] + tot[rank * E + E - 1] : 0;
    my_off[E] = last; tile_start[E] = ts;
    tile_table[0] = ts < tile_cap ? ts : tile_cap;
    tile_table[1] = last;
    tile_table[2] = tile_rows; tile_table[3] = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int d = owner[(size_t)rank * E + e];
    int before = 0;
    for (int s = 0; s < rank; ++s)
      if (owner[(size_t)s * E + e] == d) before += counts_all[(size_t)s * E + e];
    dst_base[e] = seg[d * E + e] + before;
  }
  for (int e = threadIdx.x; e <= E; e += blockDim.x) recv_offsets[e] = my_off[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int n = tot[rank * E + e];
    const int nt = tile_start[e + 1] - tile_start[e];
    for (int m = 0; m < nt; ++m) {
      const int ti = tile_start[e] + m;
      if (ti >= tile_cap) break;
      int32_t *ent = tile_table + kTileHeaderInts + (size_t)ti * kTileEntryInts;
      const int rb = seg[rank * E + e] + m * tile_rows;
      const int re = min(seg[rank * E + e] + n, rb + tile_rows);
      ent[0] = e; ent[1] = rb; ent[2] = re; ent[3] = 0;
    }
  }
}

__global__ void __launch_bounds__(256)
ep_plan_kernel(const int32_t *__restrict__ counts_all, const int32_t *__restrict__ owner, int E,
               int rank, int ep, int tile_cap, int tile_rows, int32_t *__restrict__ dst_base,
               int32_t *__restrict__ recv_offsets, int32_t *__restrict__ tile_table) {
  extern __shared__ int plan_smem[];
  plan_body(counts_all, owner, E, rank, ep, tile_cap, tile_rows, dst_base, recv_offsets, tile_table, plan_smem);
}

// One warp per item: activation row and route weight to the owner's buffer.
__device__ __forceinline__ void dispatch_body(const uint4 *__restrict__ x, const int32_t *__restrict__ item_expert,
                                              const __nv_bfloat16 *__restrict__ item_scale,
                                              const int32_t *__restrict__ slot_of_item,
                                              const int32_t *__restrict__ local_offsets,
                                              const volatile int32_t *dst_base, const int32_t *__restrict__ owner,
                                              int n_items, int items_per_row, int vec_per_row, int recv_cap,
                                              const PeerPtrs &recv_rows, const PeerPtrs &recv_scale,
                                              int32_t *__restrict__ item_rank, int32_t *__restrict__ item_row,
                                              int first_warp, int warps_total, int rank = 0,
                                              const PeerPtrs *recv_meta = nullptr,
                                              const int32_t *__restrict__ local_map = nullptr) {
  const int lane = threadIdx.x & 31;
  for (int i = first_warp; i < n_items; i += warps_total) {
    const int e = item_expert[i];
    const int slot = slot_of_item[i];
    if (e < 0 || slot < 0) {
      if (lane == 0) { item_rank[i] = -1; item_row[i] = -1; }
      continue;
    }
    if (local_map != nullptr && local_map[e] >= 0) {
      // executed here out of a cache slot: the result lands in row i of this rank's own return buffer
      if (lane == 0) { item_rank[i] = rank; item_row[i] = i; }
      continue;
    }
    const int d = owner[e];
    const int row = dst_base[e] + (slot - local_offsets[e]);
    if (row >= recv_cap) {             // cannot happen with worst-case sizing; never write past the buffer
      if (lane == 0) { item_rank[i] = -1; item_row[i] = -1; }
      continue;
    }
    const uint4 *s = x + (size_t)(i / items_per_row) * vec_per_row;
    uint4 *dp = static_cast<uint4 *>(recv_rows.p[d]) + (size_t)row * vec_per_row;
    // eight 16-byte loads in flight per lane, then the eight peer stores: a 4 KB row is
    // one batch, so few warps keep the link busy and the GEMM that runs beside this
    // kernel keeps its issue slots
    for (int v0 = 0; v0 < vec_per_row; v0 += 256) {
      uint4 t[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int v = v0 + j * 32 + lane;
        if (v < vec_per_row) t[j] = __ldg(s + v);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int v = v0 + j * 32 + lane;
        if (v < vec_per_row) dp[v] = t[j];
      }
    }
    if (lane == 0) {
      static_cast<__nv_bfloat16 *>(recv_scale.p[d])[row] = item_scale[i];
      // return address of the row: sender rank and the sender's item index
      if (recv_meta != nullptr) static_cast<int32_t *>(recv_meta->p[d])[row] = (rank << 24) | i;
      // with return addresses the result comes back into row i of this rank's
      // return buffer: that is the row the local combine reads (-1 above = skip)
      item_rank[i] = d; item_row[i] = recv_meta != nullptr ? i : row;
    }
  }
}

__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const uint4 *__restrict__ x, const int32_t *__restrict__ item_expert,
                   const __nv_bfloat16 *__restrict__ item_scale,
                   const int32_t *__restrict__ slot_of_item, const int32_t *__restrict__ local_offsets,
                   const int32_t *__restrict__ dst_base, const int32_t *__restrict__ owner,
                   int n_items, int items_per_row, int vec_per_row, int recv_cap, PeerPtrs recv_rows,
                   PeerPtrs recv_scale, int32_t *__restrict__ item_rank, int32_t *__restrict__ item_row,
                   int rank, int with_meta, PeerPtrs recv_meta) {
  dispatch_body(x, item_expert, item_scale, slot_of_item, local_offsets, dst_base, owner, n_items, items_per_row,
                vec_per_row, recv_cap, recv_rows, recv_scale, item_rank, item_row,
                blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), gridDim.x * (blockDim.x >> 5), rank,
                with_meta ? &recv_meta : nullptr);
}

// For every received row: the address of its row in the sender's return buffer,
// as seen from this GPU (what the scatter epilogue of the down GEMM stores to).
__device__ __forceinline__ void resolve_body(const volatile int32_t *recv_meta, int total, const PeerPtrs &ret,
                                             int ep, int ret_rows, size_t row_bytes,
                                             unsigned long long *__restrict__ row_dst, int first, int stride) {
  for (int r = first; r < total; r += stride) {
    const int m = recv_meta[r];
    const int s = (m >> 24) & 0xff, i = m & 0xffffff;
    unsigned long long d = 0ull;
    if (s < ep && i < ret_rows)
      d = reinterpret_cast<unsigned long long>(static_cast<char *>(ret.p[s]) + (size_t)i * row_bytes);
    row_dst[r] = d;
  }
}

__global__ void __launch_bounds__(256)
ep_resolve_return_kernel(const int32_t *__restrict__ recv_meta, const int32_t *__restrict__ recv_offsets, int E,
                         PeerPtrs ret, int ep, int ret_rows, size_t row_bytes,
                         unsigned long long *__restrict__ row_dst) {
  resolve_body(recv_meta, recv_offsets[E], ret, ep, ret_rows, row_bytes, row_dst,
               blockIdx.x * blockDim.x + threadIdx.x, gridDim.x * blockDim.x);
}

// The whole send side of a decode-sized step in ONE single-CTA launch: counts
// out, barrier, plan, rows out, barrier ("rows landed").  A few dozen rows are
// a few hundred KB; the launches this saves cost more than the copy.
__global__ void __launch_bounds__(256)
ep_exchange_dispatch_kernel(const int32_t *__restrict__ local_offsets, PeerPtrs counts_all, PeerPtrs flags,
                            uint32_t *epoch_counter, const int32_t *__restrict__ owner, int E, int rank, int ep,
                            int tile_cap, int tile_rows, int32_t *dst_base, int32_t *__restrict__ recv_offsets,
                            int32_t *__restrict__ tile_table, const uint4 *__restrict__ x,
                            const int32_t *__restrict__ item_expert, const __nv_bfloat16 *__restrict__ item_scale,
                            const int32_t *__restrict__ slot_of_item, int n_items, int items_per_row,
                            int vec_per_row, int recv_cap, PeerPtrs recv_rows, PeerPtrs recv_scale,
                            int32_t *__restrict__ item_rank, int32_t *__restrict__ item_row,
                            int32_t *__restrict__ status, int with_meta, PeerPtrs recv_meta, PeerPtrs ret,
                            int ret_rows, unsigned long long *__restrict__ row_dst,
                            const int32_t *__restrict__ local_map, const int32_t *__restrict__ item_of_slot,
                            unsigned long long *__restrict__ local_dst) {
  extern __shared__ int plan_smem[];
  publish_body(local_offsets, E, rank, ep, counts_all, local_map);
  if (local_map != nullptr && local_dst != nullptr) {
    // return address of every locally sorted row (row s of the local sort is item item_of_slot[s])
    char *mine = static_cast<char *>(ret.p[rank]);
    for (int s = threadIdx.x; s < n_items; s += blockDim.x) {
      const int it = item_of_slot[s];
      local_dst[s] = (it >= 0 && it < ret_rows)
                         ? reinterpret_cast<unsigned long long>(mine + (size_t)it * vec_per_row * 16) : 0ull;
    }
  }
  __threadfence_system();
  uint32_t epoch = next_epoch(epoch_counter);
  barrier_body(flags, rank, ep, epoch, status);
  __syncthreads();
  plan_body(static_cast<const int32_t *>(counts_all.p[rank]), owner, E, rank, ep, tile_cap, tile_rows, dst_base,
            recv_offsets, tile_table, plan_smem);
  __syncthreads();                      // dst_base (global, written by this CTA) is visible to all its threads
  dispatch_body(x, item_expert, item_scale, slot_of_item, local_offsets, dst_base, owner + (size_t)rank * E,
                n_items, items_per_row, vec_per_row, recv_cap, recv_rows, recv_scale, item_rank, item_row,
                threadIdx.x >> 5, blockDim.x >> 5, rank, with_meta ? &recv_meta : nullptr, local_map);
  __threadfence_system();
  epoch = next_epoch(epoch_counter);
  barrier_body(flags, rank, ep, epoch, status);
  if (with_meta) {
    // every rank's rows and return addresses have landed: resolve them
    __syncthreads();
    resolve_body(static_cast<const int32_t *>(recv_meta.p[rank]),
                 *reinterpret_cast<const volatile int32_t *>(recv_offsets + E), ret, ep, ret_rows,
                 (size_t)vec_per_row * 16, row_dst, threadIdx.x, blockDim.x);
  }
}

// One warp per received row: the finished expert output row goes to the address
// its sender asked for (a row of the sender's return buffer; a peer store when
// the sender is another GPU).  512 contiguous bytes per warp store.
__global__ void __launch_bounds__(256)
ep_return_rows_kernel(const uint4 *__restrict__ y, const unsigned long long *__restrict__ row_dst,
                      const int32_t *__restrict__ recv_offsets, int E, int vec_per_row) {
  const int total = recv_offsets[E];
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * (blockDim.x >> 5);
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < total; r += warps_total) {
    uint4 *dst = reinterpret_cast<uint4 *>(row_dst[r]);
    if (dst == nullptr) continue;
    const uint4 *src = y + (size_t)r * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) dst[v] = __ldg(src + v);
  }
}

__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
  return pack_bf16x2(__fadd_rn(bf16_lo(a), bf16_lo(b)), __fadd_rn(bf16_hi(a), bf16_hi(b)));
}
__device__ __forceinline__ uint4 add8(uint4 a, uint4 b) {
  return make_uint4(add2(a.x, b.x), add2(a.y, b.y), add2(a.z, b.z), add2(a.w, b.w));
}

// One warp per token; rows come from the owners' output buffers.  Lanes 0..K-1
// read the token's K (expert, owner rank, row) records and rank them by expert
// id; then every lane fetches its 16-byte pieces of all K rows before the
// first add, so the peer loads of a token are in flight together.
__global__ void __launch_bounds__(256)
ep_combine_kernel(PeerPtrs y_rows, const int32_t *__restrict__ item_rank,
                  const int32_t *__restrict__ item_row, const int32_t *__restrict__ idx,
                  const uint4 *__restrict__ shared_out, int T, int vec_per_row, int K,
                  uint4 *__restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int warps_total = gridDim.x * (blockDim.x >> 5);
  for (int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < T; t += warps_total) {
    int e = 0x7fffffff;
    unsigned long long ptr = 0;
    if (lane < K) {
      const int i = t * K + lane;
      e = idx[i];
      const int d = item_rank[i], r = item_row[i];
      if (d >= 0) ptr = reinterpret_cast<unsigned long long>(static_cast<const uint4 *>(y_rows.p[d]) +
                                                               (size_t)r * vec_per_row);
    }
    int pos = 0;                                      // position of this lane's row in expert-id order
    for (int j = 0; j < K; ++j) {
      const int ej = __shfl_sync(0xffffffffu, e, j);
      pos += (ej < e || (ej == e && j < lane)) ? 1 : 0;
    }
    unsigned long long src[kMaxK];                    // row pointers in expert-id order, 0 = no row
#pragma unroll
    for (int k = 0; k < kMaxK; ++k) {
      const unsigned who = __ballot_sync(0xffffffffu, lane < K && pos == k);
      const unsigned long long p = __shfl_sync(0xffffffffu, ptr, who ? __ffs(who) - 1 : 0);
      src[k] = who ? p : 0ull;
    }
    for (int v = lane; v < vec_per_row; v += 32) {
      uint4 val[kMaxK];
#pragma unroll
      for (int k = 0; k < kMaxK; ++k) {
        val[k] = make_uint4(0, 0, 0, 0);
        if (src[k] != 0ull) val[k] = reinterpret_cast<const uint4 *>(src[k])[v];
      }
      uint4 sh = make_uint4(0, 0, 0, 0);
      if (shared_out != nullptr) sh = __ldg(shared_out + (size_t)t * vec_per_row + v);
      uint4 acc = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int k = 0; k < kMaxK; ++k)
        if (src[k] != 0ull) acc = add8(acc, val[k]);
      if (shared_out != nullptr) acc = add8(acc, sh);
      out[(size_t)t * vec_per_row + v] = acc;
    }
  }
}

int32_t fill_peers(PeerPtrs *pp, void *const *ptrs, int ep, const char *what) {
  if (ep < 1 || ep > kMaxRanks) return fail(SB_E_INVALID_ARG, "%s: ep=%d outside [1,%d]", what, ep, kMaxRanks);
  for (int i = 0; i < kMaxRanks; ++i) pp->p[i] = nullptr;
  for (int i = 0; i < ep; ++i) {
    if (!ptrs || !ptrs[i]) return fail(SB_E_INVALID_ARG, "%s: null peer pointer %d", what, i);
    pp->p[i] = ptrs[i];
  }
  return SB_OK;
}

}  // namespace
}  // namespace sb

using namespace sb;

extern "C" {

int32_t sb_peer_alloc(size_t bytes, void **out_ptr) {
  if (!out_ptr || bytes == 0) return fail(SB_E_INVALID_ARG, "sb_peer_alloc: bad arguments");
  void *p = nullptr;
  SB_CUDA_CHECK(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) { cudaFree(p); return fail(SB_E_CUDA, "sb_peer_alloc: memset: %s", cudaGetErrorString(e)); }
  SB_CUDA_CHECK(cudaDeviceSynchronize());
  *out_ptr = p;
  return SB_OK;
}

int32_t sb_peer_free(void *ptr) {
  if (ptr) SB_CUDA_CHECK(cudaFree(ptr));
  return SB_OK;
}

int32_t sb_ipc_export(const void *ptr, void *handle64) {
  if (!ptr || !handle64) return fail(SB_E_INVALID_ARG, "sb_ipc_export: null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  SB_CUDA_CHECK(cudaIpcGetMemHandle(&h, const_cast<void *>(ptr)));
  memcpy(handle64, &h, 64);
  return SB_OK;
}

int32_t sb_ipc_import(const void *handle64, void **out_ptr) {
  if (!handle64 || !out_ptr) return fail(SB_E_INVALID_ARG, "sb_ipc_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void *p = nullptr;
  SB_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out_ptr = p;
  return SB_OK;
}

int32_t sb_ipc_close(void *ptr) {
  if (ptr) SB_CUDA_CHECK(cudaIpcCloseMemHandle(ptr));
  return SB_OK;
}

int32_t sb_ep_publish_counts(const int32_t *local_offsets, int32_t E, int32_t rank, int32_t ep,
                             void *const *peer_counts, void *stream) {
  if (!local_offsets || E < 1 || E > kMaxExperts || rank < 0 || rank >= ep)
    return fail(SB_E_INVALID_ARG, "sb_ep_publish_counts: bad arguments (E=%d rank=%d ep=%d)", E, rank, ep);
  PeerPtrs pc;
  int32_t rc = fill_peers(&pc, peer_counts, ep, "sb_ep_publish_counts");
  if (rc != SB_OK) return rc;
  ep_publish_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(local_offsets, E, rank, ep, pc);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_ep_barrier(void *const *peer_flags, int32_t rank, int32_t ep, uint32_t epoch,
                      int32_t *status, void *stream) {
  if (rank < 0 || rank >= ep) return fail(SB_E_INVALID_ARG, "sb_ep_barrier: rank=%d ep=%d", rank, ep);
  PeerPtrs pf;
  int32_t rc = fill_peers(&pf, peer_flags, ep, "sb_ep_barrier");
  if (rc != SB_OK) return rc;
  ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, rank, ep, epoch, nullptr, status,
                                                                      kBarrierLimitNs);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_ep_barrier_timed(void *const *peer_flags, int32_t rank, int32_t ep, uint32_t *epoch_counter,
                            uint64_t limit_ns, int32_t *status, void *stream) {
  if (rank < 0 || rank >= ep || !epoch_counter || limit_ns == 0)
    return fail(SB_E_INVALID_ARG, "sb_ep_barrier_timed: rank=%d ep=%d limit=%llu ns", rank, ep,
                (unsigned long long)limit_ns);
  PeerPtrs pf;
  int32_t rc = fill_peers(&pf, peer_flags, ep, "sb_ep_barrier_timed");
  if (rc != SB_OK) return rc;
  ep_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pf, rank, ep, 0u, epoch_counter, status,
                                                                      (unsigned long long)limit_ns);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_ep_barrier_seq(void *const *peer_flags, int32_t rank, int32_t ep, uint32_t *epoch_counter,
                          int32_t *status, void *stream) {
  return sb_ep_barrier_timed(peer_flags, rank, ep, epoch_counter, kBarrierLimitNs, status, stream);
}

int32_t sb_ep_exchange_dispatch(const int32_t *local_offsets, void *const *peer_counts, void *const *peer_flags,
                                uint32_t *epoch_counter, const int32_t *owner, int32_t E, int32_t rank,
                                int32_t ep, int32_t recv_cap, int32_t *dst_base, int32_t *recv_offsets,
                                int32_t *tile_table, const void *x, const int32_t *item_expert,
                                const void *item_scale, const int32_t *slot_of_item, int32_t n_items,
                                int32_t items_per_row, int32_t H, void *const *peer_rows,
                                void *const *peer_scale, int32_t *item_rank, int32_t *item_row,
                                void *const *peer_meta, void *const *peer_ret, int32_t ret_rows,
                                uint64_t *row_dst, int32_t *status, void *stream) {
  return sb_ep_exchange_dispatch_local(local_offsets, peer_counts, peer_flags, epoch_counter, owner, E, rank, ep,
                                       recv_cap, dst_base, recv_offsets, tile_table, x, item_expert, item_scale,
                                       slot_of_item, n_items, items_per_row, H, peer_rows, peer_scale, item_rank,
                                       item_row, peer_meta, peer_ret, ret_rows, row_dst, nullptr, nullptr, nullptr,
                                       status, stream);
}

int32_t sb_ep_exchange_dispatch_local(const int32_t *local_offsets, void *const *peer_counts,
                                      void *const *peer_flags, uint32_t *epoch_counter, const int32_t *owner,
                                      int32_t E, int32_t rank, int32_t ep, int32_t recv_cap, int32_t *dst_base,
                                      int32_t *recv_offsets, int32_t *tile_table, const void *x,
                                      const int32_t *item_expert, const void *item_scale,
                                      const int32_t *slot_of_item, int32_t n_items, int32_t items_per_row,
                                      int32_t H, void *const *peer_rows, void *const *peer_scale,
                                      int32_t *item_rank, int32_t *item_row, void *const *peer_meta,
                                      void *const *peer_ret, int32_t ret_rows, uint64_t *row_dst,
                                      const int32_t *local_map, const int32_t *item_of_slot, uint64_t *local_dst,
                                      int32_t *status, void *stream) {
  if (local_map != nullptr && (!peer_meta || !item_of_slot || !local_dst))
    return fail(SB_E_INVALID_ARG, "sb_ep_exchange_dispatch_local: local_map needs return addresses, item_of_slot "
                                  "and local_dst");
  if (!local_offsets || !epoch_counter || !owner || !dst_base || !recv_offsets || !tile_table || E < 1 ||
      E > kMaxExperts || rank < 0 || rank >= ep || ep > kMaxRanks || recv_cap < 0)
    return fail(SB_E_INVALID_ARG, "sb_ep_exchange_dispatch: bad arguments (E=%d rank=%d ep=%d)", E, rank, ep);
  if (n_items < 0 || H % 8 != 0 || items_per_row < 1)
    return fail(SB_E_INVALID_ARG, "sb_ep_exchange_dispatch: bad arguments (n_items=%d H=%d)", n_items, H);
  if (n_items > 0 && (!x || !item_expert || !item_scale || !slot_of_item || !item_rank || !item_row))
    return fail(SB_E_INVALID_ARG, "sb_ep_exchange_dispatch: null pointer");
  PeerPtrs pc, pf, pr, ps;
  int32_t rc;
  if ((rc = fill_peers(&pc, peer_counts, ep, "sb_ep_exchange_dispatch")) != SB_OK) return rc;
  if ((rc = fill_peers(&pf, peer_flags, ep, "sb_ep_exchange_dispatch")) != SB_OK) return rc;
  if ((rc = fill_peers(&pr, peer_rows, ep, "sb_ep_exchange_dispatch")) != SB_OK) return rc;
  if ((rc = fill_peers(&ps, peer_scale, ep, "sb_ep_exchange_dispatch")) != SB_OK) return rc;
  PeerPtrs pm, pt;
  for (int i = 0; i < kMaxRanks; ++i) { pm.p[i] = nullptr; pt.p[i] = nullptr; }
  const int with_meta = peer_meta != nullptr ? 1 : 0;
  if (with_meta) {
    if (!peer_ret || !row_dst || ret_rows < 0 || n_items >= (1 << 24))
      return fail(SB_E_INVALID_ARG, "sb_ep_exchange_dispatch: return-address arguments go together");
    if ((rc = fill_peers(&pm, peer_meta, ep, "sb_ep_exchange_dispatch")) != SB_OK) return rc;
    if ((rc = fill_peers(&pt, peer_ret, ep, "sb_ep_exchange_dispatch")) != SB_OK) return rc;
  }
  const int tile_cap = recv_cap / SB_TILE_M + E;
  const size_t smem = ((size_t)2 * ep * E + 2 * (size_t)(E + 1)) * sizeof(int);
  if (smem > 48 * 1024)
    SB_CUDA_CHECK(cudaFuncSetAttribute(ep_exchange_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem));
  ep_exchange_dispatch_kernel<<<1, 256, smem, static_cast<cudaStream_t>(stream)>>>(
      local_offsets, pc, pf, epoch_counter, owner, E, rank, ep, tile_cap, sb_tile_rows(), dst_base, recv_offsets,
      tile_table, static_cast<const uint4 *>(x), item_expert, static_cast<const __nv_bfloat16 *>(item_scale),
      slot_of_item, n_items, items_per_row, H / 8, recv_cap, pr, ps, item_rank, item_row, status, with_meta, pm,
      pt, ret_rows, reinterpret_cast<unsigned long long *>(row_dst), local_map, item_of_slot,
      reinterpret_cast<unsigned long long *>(local_dst));
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_ep_plan(const int32_t *counts_all, const int32_t *owner, int32_t E, int32_t rank,
                   int32_t ep, int32_t recv_cap, int32_t *dst_base, int32_t *recv_offsets,
                   int32_t *tile_table, void *stream) {
  if (!counts_all || !owner || !dst_base || !recv_offsets || !tile_table || E < 1 || E > kMaxExperts ||
      rank < 0 || rank >= ep || ep > kMaxRanks || recv_cap < 0)
    return fail(SB_E_INVALID_ARG, "sb_ep_plan: bad arguments (E=%d rank=%d ep=%d)", E, rank, ep);
  const int tile_cap = recv_cap / SB_TILE_M + E;
  const size_t smem = ((size_t)2 * ep * E + 2 * (size_t)(E + 1)) * sizeof(int);
  if (smem > 48 * 1024)
    SB_CUDA_CHECK(cudaFuncSetAttribute(ep_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  ep_plan_kernel<<<1, 256, smem, static_cast<cudaStream_t>(stream)>>>(counts_all, owner, E, rank, ep, tile_cap,
                                                                   sb_tile_rows(), dst_base, recv_offsets,
                                                                   tile_table);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_ep_dispatch(const void *x, const int32_t *item_expert, const void *item_scale,
                       const int32_t *slot_of_item, const int32_t *local_offsets,
                       const int32_t *dst_base, const int32_t *owner, int32_t n_items,
                       int32_t items_per_row, int32_t H, int32_t ep, int32_t recv_cap,
                       void *const *peer_rows, void *const *peer_scale, int32_t *item_rank,
                       int32_t *item_row, int32_t rank, void *const *peer_meta, void *stream) {
  if (n_items < 0 || H <= 0 || H % 8 != 0 || items_per_row < 1 || n_items >= (1 << 24) || rank < 0 || rank >= ep)
    return fail(SB_E_INVALID_ARG, "sb_ep_dispatch: bad shape (n=%d H=%d rank=%d)", n_items, H, rank);
  if (n_items == 0) return SB_OK;
  if (!x || !item_expert || !item_scale || !slot_of_item || !local_offsets || !dst_base || !owner ||
      !item_rank || !item_row)
    return fail(SB_E_INVALID_ARG, "sb_ep_dispatch: null pointer");
  PeerPtrs pr, ps, pm;
  int32_t rc;
  if ((rc = fill_peers(&pr, peer_rows, ep, "sb_ep_dispatch")) != SB_OK) return rc;
  if ((rc = fill_peers(&ps, peer_scale, ep, "sb_ep_dispatch")) != SB_OK) return rc;
  for (int i = 0; i < kMaxRanks; ++i) pm.p[i] = nullptr;
  if (peer_meta != nullptr && (rc = fill_peers(&pm, peer_meta, ep, "sb_ep_dispatch")) != SB_OK) return rc;
  int blocks = (n_items + 7) / 8;
  const int max_blocks = sb_device_sm_count() * dispatch_ctas_per_sm();
  if (blocks > max_blocks) blocks = max_blocks;
  ep_dispatch_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4 *>(x), item_expert, static_cast<const __nv_bfloat16 *>(item_scale),
      slot_of_item, local_offsets, dst_base, owner, n_items, items_per_row, H / 8, recv_cap, pr, ps,
      item_rank, item_row, rank, peer_meta != nullptr ? 1 : 0, pm);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_ep_resolve_return(const int32_t *recv_meta, const int32_t *recv_offsets, int32_t E,
                             void *const *peer_ret, int32_t ep, int32_t ret_rows, int32_t H, int32_t recv_cap,
                             uint64_t *row_dst, void *stream) {
  if (!recv_meta || !recv_offsets || !row_dst || E < 1 || E > kMaxExperts || ret_rows < 0 || H <= 0 ||
      recv_cap < 0)
    return fail(SB_E_INVALID_ARG, "sb_ep_resolve_return: bad arguments");
  PeerPtrs pr;
  int32_t rc = fill_peers(&pr, peer_ret, ep, "sb_ep_resolve_return");
  if (rc != SB_OK) return rc;
  int blocks = (recv_cap + 255) / 256;
  const int max_blocks = sb_device_sm_count() * 4;
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks < 1) blocks = 1;
  ep_resolve_return_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      recv_meta, recv_offsets, E, pr, ep, ret_rows, (size_t)H * 2,
      reinterpret_cast<unsigned long long *>(row_dst));
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_ep_return_rows(const void *y, const uint64_t *row_dst, const int32_t *recv_offsets, int32_t E,
                          int32_t H, int32_t recv_cap, void *stream) {
  if (!y || !row_dst || !recv_offsets || E < 1 || E > kMaxExperts || H <= 0 || H % 8 != 0 || recv_cap < 0)
    return fail(SB_E_INVALID_ARG, "sb_ep_return_rows: bad arguments");
  int blocks = (recv_cap + 7) / 8;
  const int max_blocks = sb_device_sm_count() * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks < 1) blocks = 1;
  ep_return_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4 *>(y), reinterpret_cast<const unsigned long long *>(row_dst), recv_offsets, E, H / 8);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

int32_t sb_ep_combine(void *const *peer_y, const int32_t *item_rank, const int32_t *item_row,
                      const int32_t *idx, const void *shared_out, int32_t T, int32_t H, int32_t K,
                      int32_t ep, void *out, void *stream) {
  if (T < 0 || H <= 0 || H % 8 != 0 || K < 1 || K > kMaxK)
    return fail(SB_E_INVALID_ARG, "sb_ep_combine: bad shape (T=%d H=%d K=%d)", T, H, K);
  if (T == 0) return SB_OK;
  if (!item_rank || !item_row || !idx || !out) return fail(SB_E_INVALID_ARG, "sb_ep_combine: null pointer");
  PeerPtrs py;
  int32_t rc = fill_peers(&py, peer_y, ep, "sb_ep_combine");
  if (rc != SB_OK) return rc;
  int blocks = (T + 7) / 8;                  // 8 warps per CTA, one token per warp
  const int max_blocks = sb_device_sm_count() * 8;
  if (blocks > max_blocks) blocks = max_blocks;
  const int threads = 256;
  ep_combine_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      py, item_rank, item_row, idx, static_cast<const uint4 *>(shared_out), T, H / 8, K,
      static_cast<uint4 *>(out));
  SB_LAUNCH_CHECK();
  return SB_OK;
}

}  // extern "C"
