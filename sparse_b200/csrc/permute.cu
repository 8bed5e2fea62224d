// Expert-sorted token permutation: a stable counting sort of the flat
// (token, slot) items by expert id, the gather of activation rows into that
// order, and the row-tile table for the grouped GEMM.
//
// Replaces expand/argsort/gather/bincount of the reference's dispatch
// (utils/eval_core.py:14873-14882) and the re-sort by expert in the local
// executor (utils/eval_core.py:13240-13253).  Integer work is exact: the slot of
// an item is (number of items of smaller expert id) + (number of earlier items
// of the same expert), which is what a stable sort by expert id yields.
//
// Four launches: count (per 128-item chunk histogram) -> scan (per-expert
// prefix over chunks, expert offsets, tile table) -> scatter (ranks inside a
// chunk by warp match) -> gather (one warp per output row, 16-byte vectors).
// The gather is the only HBM-heavy part: it reads T*H*2 bytes (re-reads of a
// row hit L2) and writes n_items*H*2.
#include <atomic>

#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kChunk = 128;          // items per warp-chunk
constexpr int kWarpsPerBlock = 8;
constexpr int kMaxExperts = 256;

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
permute_count_kernel(const int32_t *__restrict__ item_expert, int n_items, int E, int nchunks,
                     int32_t *__restrict__ counts) {
  __shared__ int hist[kWarpsPerBlock][kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * kWarpsPerBlock + warp;
  for (int e = lane; e < E; e += 32) hist[warp][e] = 0;
  __syncwarp();
  if (chunk < nchunks) {
#pragma unroll
    for (int r = 0; r < kChunk / 32; ++r) {
      int i = chunk * kChunk + r * 32 + lane;
      if (i < n_items) {
        int e = item_expert[i];
        if (e >= 0 && e < E) atomicAdd(&hist[warp][e], 1);
      }
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) counts[(size_t)chunk * E + e] = hist[warp][e];
  }
}

// One CTA.  counts[c][e] becomes the number of items of expert e in chunks < c.
__global__ void __launch_bounds__(1024)
permute_scan_kernel(int32_t *__restrict__ counts, int nchunks, int E, int tile_cap, int tile_rows,
                    int32_t *__restrict__ expert_offsets, int32_t *__restrict__ tile_table) {
  __shared__ int total[kMaxExperts];
  __shared__ int offs[kMaxExperts + 1];
  __shared__ int tile_start[kMaxExperts + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < E; e += 32) {
    int running = 0;
    for (int c0 = 0; c0 < nchunks; c0 += 32) {
      int c = c0 + lane;
      int v = (c < nchunks) ? counts[(size_t)c * E + e] : 0;
      int incl = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int o = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += o;
      }
      if (c < nchunks) counts[(size_t)c * E + e] = running + incl - v;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) total[e] = running;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, ts = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = o; tile_start[e] = ts;
      o += total[e];
      ts += (total[e] + tile_rows - 1) / tile_rows;
    }
    offs[E] = o; tile_start[E] = ts;
    tile_table[0] = ts < tile_cap ? ts : tile_cap;
    tile_table[1] = o;          // total rows
    tile_table[2] = tile_rows; tile_table[3] = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) expert_offsets[e] = offs[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int nt = tile_start[e + 1] - tile_start[e];
    for (int m = 0; m < nt; ++m) {
      int ti = tile_start[e] + m;
      if (ti >= tile_cap) break;
      int32_t *ent = tile_table + kTileHeaderInts + (size_t)ti * kTileEntryInts;
      int rb = offs[e] + m * tile_rows;
      int re = offs[e + 1] < rb + tile_rows ? offs[e + 1] : rb + tile_rows;
      ent[0] = e; ent[1] = rb; ent[2] = re; ent[3] = 0;
    }
  }
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
permute_scatter_kernel(const int32_t *__restrict__ item_expert,
                       const __nv_bfloat16 *__restrict__ item_scale, int n_items, int E,
                       int nchunks, const int32_t *__restrict__ chunk_base,
                       const int32_t *__restrict__ expert_offsets,
                       int32_t *__restrict__ slot_of_item, int32_t *__restrict__ item_of_slot,
                       __nv_bfloat16 *__restrict__ slot_scale) {
  __shared__ int base[kWarpsPerBlock][kMaxExperts];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * kWarpsPerBlock + warp;
  if (chunk >= nchunks) return;
  for (int e = lane; e < E; e += 32)
    base[warp][e] = expert_offsets[e] + chunk_base[(size_t)chunk * E + e];
  __syncwarp();
#pragma unroll
  for (int r = 0; r < kChunk / 32; ++r) {
    int i = chunk * kChunk + r * 32 + lane;
    int e = -1;
    if (i < n_items) { e = item_expert[i]; if (e < 0 || e >= E) e = -1; }
    unsigned peers = __match_any_sync(0xffffffffu, e);
    int rank = __popc(peers & ((1u << lane) - 1u));
    int slot = -1;
    if (e >= 0) slot = base[warp][e] + rank;
    __syncwarp();
    if (e >= 0 && rank == 0) base[warp][e] += __popc(peers);
    __syncwarp();
    if (i < n_items) {
      slot_of_item[i] = slot;
      if (slot >= 0) {
        item_of_slot[slot] = i;
        if (slot_scale != nullptr) slot_scale[slot] = item_scale[i];
      }
    }
  }
}

// Count, scan and scatter in ONE CTA for up to kFusedMaxItems items (a 4096-token
// batch with top-4 routing is 16384): each of the 32 warps owns a contiguous
// range of items, histograms it in shared memory, the per-expert prefix over the
// warps gives every range its base, and the same warp then ranks its items in
// order.  Same result as the three-kernel path, two launches and their
// scheduling gaps fewer; the workspace is not touched.
constexpr int kFusedMaxItems = 32768;

__global__ void __launch_bounds__(1024)
permute_fused_kernel(const int32_t *__restrict__ item_expert, const __nv_bfloat16 *__restrict__ item_scale,
                     int n_items, int E, int tile_cap, int tile_rows, int32_t *__restrict__ expert_offsets,
                     int32_t *__restrict__ slot_of_item, int32_t *__restrict__ item_of_slot,
                     __nv_bfloat16 *__restrict__ slot_scale, int32_t *__restrict__ tile_table) {
  extern __shared__ int fused_smem[];
  int *hist = fused_smem;                    // [nw][E] counts, then bases
  const int nw = blockDim.x >> 5;            // warps in this CTA (1..32, fewer for few items)
  int *offs = hist + nw * E;                 // [E+1]
  int *tile_start = offs + (E + 1);          // [E+1]
  int *tot = tile_start + (E + 1);           // [E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_warp = ((n_items + nw - 1) / nw + 31) & ~31;     // items per warp, multiple of 32
  const int begin = warp * per_warp;
  const int end = min(n_items, begin + per_warp);
  for (int i = threadIdx.x; i < nw * E; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (int i = begin + lane; i < end; i += 32) {
    const int e = item_expert[i];
    if (e >= 0 && e < E) atomicAdd(&hist[warp * E + e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < nw; ++w) { const int c = hist[w * E + e]; hist[w * E + e] = run; run += c; }
    tot[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, ts = 0;
    for (int e = 0; e < E; ++e) {
      offs[e] = o; tile_start[e] = ts;
      o += tot[e];
      ts += (tot[e] + tile_rows - 1) / tile_rows;
    }
    offs[E] = o; tile_start[E] = ts;
    tile_table[0] = ts < tile_cap ? ts : tile_cap;
    tile_table[1] = o;
    tile_table[2] = tile_rows; tile_table[3] = 0;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) expert_offsets[e] = offs[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int nt = tile_start[e + 1] - tile_start[e];
    for (int m = 0; m < nt; ++m) {
      const int ti = tile_start[e] + m;
      if (ti >= tile_cap) break;
      int32_t *ent = tile_table + kTileHeaderInts + (size_t)ti * kTileEntryInts;
      const int rb = offs[e] + m * tile_rows;
      const int re = offs[e + 1] < rb + tile_rows ? offs[e + 1] : rb + tile_rows;
      ent[0] = e; ent[1] = rb; ent[2] = re; ent[3] = 0;
    }
  }
  // scatter: hist[warp][e] is now the number of items of e in earlier warps.
  // Items are fetched eight rounds ahead so the loads overlap instead of each
  // round waiting for its own.
  constexpr int kBatch = 8;
  for (int b0 = begin; b0 < end; b0 += 32 * kBatch) {
    int ev[kBatch];
    __nv_bfloat16 sv[kBatch];
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
      const int i = b0 + r * 32 + lane;
      ev[r] = -1;
      if (i < end) {
        ev[r] = item_expert[i];
        if (slot_scale != nullptr) sv[r] = item_scale[i];
      }
    }
#pragma unroll
    for (int r = 0; r < kBatch; ++r) {
      const int i = b0 + r * 32 + lane;
      int e = ev[r];
      if (e < 0 || e >= E) e = -1;
      const unsigned peers = __match_any_sync(0xffffffffu, e);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      int slot = -1;
      if (e >= 0) slot = offs[e] + hist[warp * E + e] + rank;
      __syncwarp();
      if (e >= 0 && rank == 0) hist[warp * E + e] += __popc(peers);
      __syncwarp();
      if (i < end) {
        slot_of_item[i] = slot;
        if (slot >= 0) {
          item_of_slot[slot] = i;
          if (slot_scale != nullptr) slot_scale[slot] = sv[r];
        }
      }
    }
  }
}

// One warp per output row.
__global__ void __launch_bounds__(256)
permute_gather_kernel(const uint4 *__restrict__ x, const int32_t *__restrict__ item_of_slot,
                      const int32_t *__restrict__ expert_offsets, int E, int items_per_row,
                      int vec_per_row, uint4 *__restrict__ out_rows) {
  const int lane = threadIdx.x & 31;
  const int n_rows = expert_offsets[E];
  const int warps_total = gridDim.x * (blockDim.x >> 5);
  for (int slot = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); slot < n_rows;
       slot += warps_total) {
    int src = item_of_slot[slot] / items_per_row;
    const uint4 *s = x + (size_t)src * vec_per_row;
    uint4 *d = out_rows + (size_t)slot * vec_per_row;
    for (int v = lane; v < vec_per_row; v += 32) d[v] = __ldg(s + v);
  }
}

}  // namespace

static inline int num_chunks(int n_items) { return (n_items + kChunk - 1) / kChunk; }

int32_t launch_permute(const void *x, const int32_t *item_expert, const void *item_scale,
                       int n_items, int items_per_row, int H, int E, void *ws, size_t ws_bytes,
                       void *out_rows, int32_t *expert_offsets, int32_t *slot_of_item,
                       int32_t *item_of_slot, void *slot_scale, int32_t *tile_table,
                       cudaStream_t stream) {
  if (n_items < 0 || items_per_row < 1 || H <= 0 || H % 8 != 0 || E < 1 || E > kMaxExperts)
    return fail(SB_E_INVALID_ARG, "sb_permute: need H%%8==0, 1<=E<=256, items_per_row>=1 (n=%d H=%d E=%d)",
                n_items, H, E);
  if (!expert_offsets || !tile_table || !ws)
    return fail(SB_E_INVALID_ARG, "sb_permute: null pointer");
  // out_rows == NULL: sort only, no row gather (x may then be NULL as well)
  if (n_items > 0 && (!item_expert || !slot_of_item || !item_of_slot || (out_rows && !x)))
    return fail(SB_E_INVALID_ARG, "sb_permute: null pointer");
  if ((slot_scale != nullptr) != (item_scale != nullptr))
    return fail(SB_E_INVALID_ARG, "sb_permute: item_scale and slot_scale go together");
  if (ws_bytes < sb_permute_workspace_bytes(n_items, E))
    return fail(SB_E_WORKSPACE, "sb_permute: workspace %zu < %zu bytes", ws_bytes,
                sb_permute_workspace_bytes(n_items, E));
  if (!aligned(x, 16) || !aligned(out_rows, 16))
    return fail(SB_E_INVALID_ARG, "sb_permute: rows must be 16-byte aligned");
  const int nchunks = num_chunks(n_items);
  int32_t *counts = static_cast<int32_t *>(ws);
  const int tile_cap = n_items / SB_TILE_M + E;
  if (n_items > 0 && n_items <= kFusedMaxItems) {
    // one warp per 512 items: a decode step's handful of items is one warp's work
    // At most 16 warps: measured on B200, 16384 items take the same 25 us with 16
    // warps as with 32, and a 512-thread CTA still finds room on an SM that a
    // GEMM CTA of another stream occupies (44 us there; a 1024-thread CTA waits
    // for the GEMM to leave, 125 us).
    int nw = (n_items + 511) / 512;
    nw = nw < 1 ? 1 : (nw > 16 ? 16 : nw);
    const size_t smem = ((size_t)nw * E + 2 * (size_t)(E + 1) + E) * sizeof(int);
    if (smem > 48 * 1024)
      SB_CUDA_CHECK(cudaFuncSetAttribute(permute_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
    permute_fused_kernel<<<1, nw * 32, smem, stream>>>(
        item_expert, static_cast<const __nv_bfloat16 *>(item_scale), n_items, E, tile_cap, sb_tile_rows(),
        expert_offsets, slot_of_item, item_of_slot, static_cast<__nv_bfloat16 *>(slot_scale), tile_table);
    SB_LAUNCH_CHECK();
    if (out_rows != nullptr) {
      int gblocks = (n_items + 7) / 8;
      const int max_blocks = sb_device_sm_count() * 8;
      if (gblocks > max_blocks) gblocks = max_blocks;
      permute_gather_kernel<<<gblocks, 256, 0, stream>>>(
          static_cast<const uint4 *>(x), item_of_slot, expert_offsets, E, items_per_row, H / 8,
          static_cast<uint4 *>(out_rows));
      SB_LAUNCH_CHECK();
    }
    return SB_OK;
  }
  if (nchunks > 0) {
    int blocks = (nchunks + kWarpsPerBlock - 1) / kWarpsPerBlock;
    permute_count_kernel<<<blocks, kWarpsPerBlock * 32, 0, stream>>>(item_expert, n_items, E,
                                                                    nchunks, counts);
    SB_LAUNCH_CHECK();
  }
  permute_scan_kernel<<<1, 1024, 0, stream>>>(counts, nchunks, E, tile_cap, sb_tile_rows(), expert_offsets,
                                              tile_table);
  SB_LAUNCH_CHECK();
  if (nchunks > 0) {
    int blocks = (nchunks + kWarpsPerBlock - 1) / kWarpsPerBlock;
    permute_scatter_kernel<<<blocks, kWarpsPerBlock * 32, 0, stream>>>(
        item_expert, static_cast<const __nv_bfloat16 *>(item_scale), n_items, E, nchunks, counts,
        expert_offsets, slot_of_item, item_of_slot, static_cast<__nv_bfloat16 *>(slot_scale));
    SB_LAUNCH_CHECK();
    if (out_rows != nullptr) {
      int rows_per_block = 8;
      int gblocks = (n_items + rows_per_block - 1) / rows_per_block;
      int max_blocks = sb_device_sm_count() * 8;
      if (gblocks > max_blocks) gblocks = max_blocks;
      permute_gather_kernel<<<gblocks, 256, 0, stream>>>(
          static_cast<const uint4 *>(x), item_of_slot, expert_offsets, E, items_per_row, H / 8,
          static_cast<uint4 *>(out_rows));
      SB_LAUNCH_CHECK();
    }
  }
  return SB_OK;
}

}  // namespace sb

// ---- sb_permute_noalloc: the same sort with library-owned scratch -----------------
//
// Scratch for the per-chunk histograms of sb_permute, reserved in the library's
// own device image instead of being passed in.  512 KiB; every GPU that loads
// the library carries it until the process exits.
constexpr int kStaticScratchInts = 131072;
static __device__ __align__(256) int32_t g_permute_scratch[kStaticScratchInts];

// Device address of g_permute_scratch per device ordinal (0 = not looked up yet).
// In host code the symbol's name is only a handle; the address a kernel can use
// has to be asked for, with that device current.
// Two host threads making the first call on a device both store the same value;
// the atomic makes that a defined (relaxed) access instead of a data race.
static std::atomic<int32_t *> g_permute_scratch_addr[64];

extern "C" int32_t sb_permute_noalloc(const void *x, const int32_t *item_expert,
                                      const void *item_scale, int32_t n_items,
                                      int32_t items_per_row, int32_t H, int32_t E, void *out_rows,
                                      int32_t *expert_offsets, int32_t *slot_of_item,
                                      int32_t *item_of_slot, void *slot_scale,
                                      int32_t *tile_table, void *stream) {
  if (n_items < 0 || E < 1 || E > sb::kMaxExperts)
    return sb::fail(SB_E_INVALID_ARG, "sb_permute_noalloc: need n_items>=0 and 1<=E<=256 (n=%d E=%d)",
                    n_items, E);
  const size_t need_ints = (size_t)sb::num_chunks(n_items) * (size_t)E;
  if (need_ints > (size_t)kStaticScratchInts)
    return sb::fail(SB_E_WORKSPACE,
                    "sb_permute_noalloc: %d items over %d experts need %zu scratch ints, the built-in "
                    "scratch holds %d (ceil(n_items/128)*E must not exceed it); use sb_permute with a "
                    "caller-provided workspace",
                    n_items, E, need_ints, kStaticScratchInts);
  int dev = -1;
  SB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return sb::fail(SB_E_UNSUPPORTED, "sb_permute_noalloc: device ordinal %d", dev);
  int32_t *scratch = g_permute_scratch_addr[dev].load(std::memory_order_relaxed);
  if (scratch == nullptr) {
    int32_t *p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_permute_scratch);
    if (e != cudaSuccess || p == nullptr)
      return sb::fail(SB_E_CUDA, "sb_permute_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                      cudaGetErrorString(e));
    g_permute_scratch_addr[dev].store(p, std::memory_order_relaxed);
    scratch = p;
  }
  // Nothing in the scratch has to start at zero: the count pass overwrites every
  // histogram cell the later passes read, so stale contents of an earlier call
  // are never observed.
  return sb::launch_permute(x, item_expert, item_scale, n_items, items_per_row, H, E,
                            scratch,
                            (size_t)kStaticScratchInts * sizeof(int32_t), out_rows, expert_offsets,
                            slot_of_item, item_of_slot, slot_scale, tile_table,
                            static_cast<cudaStream_t>(stream));
}

extern "C" size_t sb_permute_workspace_bytes(int32_t n_items, int32_t E) {
  size_t n = (size_t)sb::num_chunks(n_items < 0 ? 0 : n_items) * (size_t)(E < 1 ? 1 : E) * sizeof(int32_t);
  return n < 256 ? 256 : ((n + 255) / 256) * 256;
}

extern "C" size_t sb_tile_table_ints(int32_t n_items, int32_t E) {
  size_t tiles = (size_t)(n_items < 0 ? 0 : n_items) / SB_TILE_M + (size_t)(E < 1 ? 1 : E);
  return sb::kTileHeaderInts + tiles * sb::kTileEntryInts;
}
