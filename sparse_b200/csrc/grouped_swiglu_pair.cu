// Grouped bf16 SwiGLU expert MLP on CTA pairs (tcgen05 cta_group::2).
//
// Arithmetic and rounding points of the reference's expert forward
// (utils/eval_core.py:11787-11790, route weight at 11765): fp32 accumulation,
// bf16 rounding after gate, up, silu, product, down and the route-weight
// scaling.  Mapping onto the machine, chosen for ragged expert groups:
//
//  * operands are swapped: the WEIGHT rows fill the 256-row M dimension of the
//    MMA (always full), the TOKENS of one expert are the N dimension, which the
//    tensor core accepts in steps of 16 up to 256.  A group of 3 tokens costs a
//    16-wide MMA, not a 128-row tile of padding.
//  * two CTAs of a cluster work on one 256 x N tile (`cta_group::2`): each CTA
//    loads 128 weight rows and half of the token rows per 64-deep K step
//    (32 KB instead of 48 KB per CTA for the same flops), the tensor cores read
//    the token half of the peer through distributed shared memory.  That cuts
//    L2->SM traffic by a third, which is what capped the single-CTA kernel.
//  * up to six 36 KB stages (one K step of a full tile, or two K steps of a tile
//    of at most 32 tokens); TMEM holds two 128-lane x 256-column accumulators per
//    CTA.  A launch may ask for fewer stages so that a CTA of another kernel
//    (the router) fits on the SM beside it.
//  * tile walk: by default table order with a fixed stride over the CTA pairs.
//    Two alternatives sit behind sb_set_tuning("sched"): every CTA ranks the
//    table's row chunks by the size of their expert (largest first, an expert's
//    chunks together) and the pairs deal the ranked tiles out boustrophedon
//    (pair 0..P-1, then P-1..0, ...), optionally with odd pairs walking
//    backwards.  Measured on B200 with a Zipf(1.2) batch (tile cost varies 16x)
//    all three take the same time within 3 %: the kernel is bound by operand
//    traffic into the SMs, not by the tail of the walk; the backward walk also
//    re-reads 190 MB of hot experts' weights from DRAM, so table order stays.
//  * pass 1 reads the gate/up slab with gate and up rows interleaved
//    (row 2j = gate_j, row 2j+1 = up_j), so the two values a SwiGLU output
//    needs sit in adjacent TMEM lanes = adjacent threads: one shuffle, no
//    shared-memory exchange.
//  * TMA loads are plain 2-D/3-D tile loads (`.cta_group::2`, no multicast);
//    both CTAs signal the leader CTA's "full" barrier; the leader's MMA thread
//    frees a stage in both CTAs and publishes a finished accumulator to both
//    CTAs' epilogue warps with `tcgen05.commit ... multicast::cluster`.
//
// Roles per CTA (320 threads): warp 0 lane 0 = TMA producer, warp 1 = TMEM
// owner (and, in the leader CTA, lane 0 = MMA issuer), warps 2-9 = epilogue.
// All mbarrier waits are bounded (2 s); on expiry the CTA sets an abort flag,
// reports through `status`, drains, joins the cluster barrier, frees TMEM.
// A chunk whose expert has no resident weight slot raises status 2 and is
// skipped by all three roles: nothing is computed with another expert's weights.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>
#include <mutex>

#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kTileW = 256;          // weight rows per CTA pair (MMA M)
constexpr int kRowsPerCta = 128;
constexpr int kMaxN = 256;           // tokens per tile (MMA N), multiple of 16
constexpr int kBlockK = 64;
constexpr int kStages = 6;           // most the shared memory holds
constexpr int kDefaultStages = 5;    // measured on B200: a sixth stage gains nothing (the operand fetch is bandwidth-, not latency-bound)
constexpr int kThreads = 320;         // producer warp, MMA warp, 8 epilogue warps
constexpr int kEpiWarps = 8;
constexpr uint32_t kABytes = kRowsPerCta * kBlockK * 2;      // 16 KB
constexpr uint32_t kLightTokBytes = 16 * kBlockK * 2;         // 2 KB: a 16-row token box of one K step
// A stage holds one K step of a full tile (A 16 KB + B up to 16 KB) or, for a
// light tile (at most 16 tokens per CTA), TWO K steps (A, A', then the two
// 2 KB token boxes): half as many barrier round trips per weight byte, twice
// the bytes in flight, which is what bounds a tile that is pure weight traffic.
constexpr uint32_t kStageBytes = 2 * kABytes + 2 * kLightTokBytes;   // one K step per stage (36 KB)
constexpr uint32_t kSlabBytes = 2 * kABytes;                        // A + B of one K step of a full tile
constexpr uint32_t kStageBytes2 = 2 * kSlabBytes;                   // two K steps per stage (64 KB)
constexpr int kStages2 = 3;                                         // most of those the shared memory holds
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kScatterTileBytes = 16 * kRowsPerCta * 2;    // 16 tokens x this CTA's 128 output columns, bf16
constexpr int kMaxSched = 768;          // row chunks that can be ranked (larger tables are walked in table order)
constexpr uint32_t kTailBytes = 256 + 2 * kScatterTileBytes + kMaxSched * 2;   // barriers, scatter staging, chunk order
// `tail` = false: a launch that neither scatters rows nor ranks chunks needs only
// the barriers behind its stages.
__host__ __device__ constexpr uint32_t smem_bytes(int stages, uint32_t stage_bytes = kStageBytes, bool tail = true) {
  return (uint32_t)stages * stage_bytes + 1024 + (tail ? kTailBytes : 256u);
}
static_assert(smem_bytes(kStages) <= 232448 && smem_bytes(kStages2, kStageBytes2) <= 232448, "shared memory of a CTA");
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
constexpr int kSlotSkip = -2;
// kModePlain: the down pass of a launch without route weights and without row
// destinations (the shared expert's): bf16 rounding and plain stores only, held
// to 96 registers like the gate/up instance so that a router CTA fits beside it.
constexpr int kModeSwiglu = 0, kModeScale = 1, kModePlain = 2;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long gtime_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// arrive on a barrier given by its shared::cluster address (may live in the peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done;
}
// The slow half of a bounded wait, kept out of line so that the single-thread
// producer and MMA loops stay short: spin, watch the abort flag, give up after
// kWaitLimitNs.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  const unsigned long long t0 = gtime_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (gtime_ns() - t0 > kWaitLimitNs) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, abort_flag);
}
// Tile loads of a CTA pair: destination in this CTA, completion bytes counted on
// the barrier at `bar_cluster_addr` (the leader CTA's).
__device__ __forceinline__ void tma_pair_load_2d(uint32_t dst, const CUtensorMap *tm, uint32_t bar_cluster_addr,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_pair_load_3d(uint32_t dst, const CUtensorMap *tm, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// completion of all MMAs issued so far -> one arrival on the barrier at this
// shared-memory offset in BOTH CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3) : "memory");
}
// The four 16-deep MMAs of one 64-deep K step.  Descriptor start addresses are in
// 16-byte units, so the k-th MMA reads 32 bytes (2 units) further along the
// 128-byte swizzle row.  `accumulate` == 0 makes the first one overwrite D.
__device__ __forceinline__ void tc_mma_pair_bf16_x4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                                    uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 a, b;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 t, 0, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "add.u64 a, %1, 2;\n\tadd.u64 b, %2, 2;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.u64 a, %1, 4;\n\tadd.u64 b, %2, 4;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %3, t;\n\t"
      "add.u64 a, %1, 6;\n\tadd.u64 b, %2, 6;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], a, b, %3, t;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// D=f32, A=B=bf16, K-major both, M=256 (pair), N given
__device__ __forceinline__ uint32_t idesc_m256(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTileW >> 4) << 24);
}

struct Chunk { int slot, tok_begin, tok_end; bool absent; };

__device__ __forceinline__ Chunk read_chunk(const int32_t *tile_table, int dense_rows,
                                            const int32_t *slot_of_expert, int c, int skip_rows_upto,
                                            int dense_chunk, int n_slots) {
  Chunk t;
  t.absent = false;
  if (tile_table == nullptr) {
    t.slot = 0;
    t.tok_begin = c * dense_chunk;
    t.tok_end = min(dense_rows, t.tok_begin + dense_chunk);
  } else {
    const int4 e = __ldg(reinterpret_cast<const int4 *>(tile_table + kTileHeaderInts) + c);
    t.slot = slot_of_expert ? __ldg(slot_of_expert + e.x) : e.x;
    t.tok_begin = e.y;
    t.tok_end = e.z;
    if (e.z - e.y <= skip_rows_upto) {
      t.slot = kSlotSkip;                                        // light group: the streaming kernels' work
    } else if (t.slot != kSlotSkip && (t.slot < 0 || t.slot >= n_slots)) {
      t.absent = true;                                           // no resident weights: status 2, nothing computed
      t.slot = kSlotSkip;
    }
  }
  if (t.tok_end <= t.tok_begin) t.slot = kSlotSkip;
  return t;
}

// Which tile a CTA pair works on in its j-th round.  Mode 0: table order, fixed
// stride.  Mode 1: chunks ranked by size (`order`), ranked tiles dealt out
// boustrophedon.  Mode 2: as 1, odd pairs walk their rounds backwards.
// All roles of both CTAs of a pair evaluate the same function: no hand-off.
struct Sched {
  int total, n_pairs, pair, n_wtiles, rounds, mode, n_chunks, group;
  const uint16_t *order;
  __device__ __forceinline__ bool tile(int j, int &c, int &wt) const {
    int t;
    if (mode == 0) {
      t = pair + j * n_pairs;
      if (group > 1) {
        // Raster blocks of `group` chunks x all weight tiles, chunk index fastest:
        // the pairs that run at the same time then share weight tiles as well as
        // token chunks, instead of all reading one or two token chunks.
        if (t >= total) return false;
        const int per_block = group * n_wtiles;
        const int blk = t / per_block, in = t - blk * per_block;
        const int c0 = blk * group;
        const int g = min(group, n_chunks - c0);          // the last block may be narrower
        wt = in / g;
        c = c0 + (in - wt * g);
        return true;
      }
    } else {
      const int jj = (mode == 2 && (pair & 1)) ? rounds - 1 - j : j;
      t = jj * n_pairs + ((jj & 1) ? n_pairs - 1 - pair : pair);
    }
    if (t >= total) return false;
    const int r = t / n_wtiles;
    wt = t - r * n_wtiles;
    c = mode == 0 ? r : (int)order[r];
    return true;
  }
};

// The gate/up instance is held to 96 registers per thread (the "two CTAs per SM"
// of its launch bounds says only that): with 320 threads that leaves an SM the
// 32 K registers a router CTA needs beside it.
template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, MODE == kModeScale ? 1 : 2)
pair_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                 const __grid_constant__ CUtensorMap tm_x64, const __grid_constant__ CUtensorMap tm_x16,
                 const int32_t *__restrict__ tile_table, int dense_rows,
                 const int32_t *__restrict__ slot_of_expert, const __nv_bfloat16 *__restrict__ row_scale,
                 __nv_bfloat16 *__restrict__ out, int ld_out, int w_rows, int num_kb, int n_slots,
                 int32_t *__restrict__ status, int skip_rows_upto, int dense_chunk, int light_max,
                 const unsigned long long *__restrict__ row_dst, int n_stages, int sched_mode, int dense_group,
                 uint32_t stage_bytes) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char *smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t stage_bytes_all = (uint32_t)n_stages * stage_bytes;
  const int slabs = stage_bytes == kStageBytes2 ? 2 : 1;            // K steps of a full tile per stage
  const uint32_t bar_full = smem_base + stage_bytes_all;            // kStages  (used in the leader CTA)
  const uint32_t bar_empty = bar_full + 8 * kStages;               // kStages  (both CTAs)
  const uint32_t bar_tfull = bar_empty + 8 * kStages;              // 2        (both CTAs)
  const uint32_t bar_tempty = bar_tfull + 16;                      // 2        (leader CTA)
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem_al + stage_bytes_all + 8 * (2 * kStages + 4));
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
  unsigned char *scatter_stage = smem_al + stage_bytes_all + 256;
  uint16_t *order = reinterpret_cast<uint16_t *>(scatter_stage + 2 * kScatterTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();               // 0 = leader
  const int n_wtiles = (w_rows + kTileW - 1) / kTileW;
  const int n_chunks = tile_table ? __ldg(tile_table) : (dense_rows + dense_chunk - 1) / dense_chunk;
  Sched sch;
  sch.pair = blockIdx.x >> 1;
  sch.n_pairs = gridDim.x >> 1;
  sch.n_wtiles = n_wtiles;
  sch.total = n_chunks * n_wtiles;
  sch.rounds = (sch.total + sch.n_pairs - 1) / sch.n_pairs;
  sch.mode = (tile_table != nullptr && n_chunks <= kMaxSched) ? sched_mode : 0;
  sch.n_chunks = n_chunks;
  sch.group = tile_table == nullptr ? dense_group : 1;
  sch.order = order;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, 2 * kEpiWarps); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  if (sch.mode != 0) {
    // Rank the chunks by the row count of their EXPERT, largest first, ties (the
    // chunks of one expert, and experts of equal size) in table order.  An
    // expert's chunks stay together, so its weights are still in L2 when its
    // last, partial chunk runs (ranking by chunk size alone sent those tails to
    // the end of the walk and cost a third more DRAM reads).  Every CTA computes
    // the same ranking; the keys sit in the scatter staging area, which no
    // epilogue warp touches before the barrier below.
    uint16_t *key_expert = reinterpret_cast<uint16_t *>(scatter_stage);
    uint16_t *key_rows = key_expert + kMaxSched;
    uint32_t *key_total = reinterpret_cast<uint32_t *>(key_rows + kMaxSched);
    for (int i = threadIdx.x; i < n_chunks; i += kThreads) {
      const int4 e = __ldg(reinterpret_cast<const int4 *>(tile_table + kTileHeaderInts) + i);
      key_expert[i] = (uint16_t)e.x;
      key_rows[i] = (uint16_t)min(max(e.z - e.y, 0), 65535);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_chunks; i += kThreads) {
      const uint16_t ex = key_expert[i];
      uint32_t tot = 0;
      for (int j = i; j >= 0 && key_expert[j] == ex; --j) tot += key_rows[j];
      for (int j = i + 1; j < n_chunks && key_expert[j] == ex; ++j) tot += key_rows[j];
      key_total[i] = tot;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_chunks; i += kThreads) {
      const uint32_t k = key_total[i];
      int rank = 0;
      for (int j = 0; j < n_chunks; ++j) {
        const uint32_t kj = key_total[j];
        rank += (kj > k || (kj == k && j < i)) ? 1 : 0;
      }
      order[rank] = (uint16_t)i;
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();            // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      const uint32_t full_leader0 = map_to_cta(bar_full, 0);
      for (int j = 0; ok && j < sch.rounds; ++j) {
        int c, wt;
        if (!sch.tile(j, c, wt)) continue;
        const Chunk ch = read_chunk(tile_table, dense_rows, slot_of_expert, c, skip_rows_upto, dense_chunk, n_slots);
        if (ch.absent && cta == 0 && wt == 0 && status) atomicExch(status, 2);
        if (ch.slot == kSlotSkip) continue;
        const int n = ((ch.tok_end - ch.tok_begin) + 15) & ~15;
        const int tok0 = ch.tok_begin + (int)cta * (n >> 1);       // this CTA's half of the tokens
        const int wrow = wt * kTileW + (int)cta * kRowsPerCta;
        // small groups fetch a small token box: a 3-token expert moves 2 KB of
        // activations per K step, not 16 KB
        const int half = n >> 1;
        const CUtensorMap *tok_map = half <= 16 ? &tm_x16 : (half <= 64 ? &tm_x64 : &tm_x);
        const uint32_t tok_bytes = (half <= 16 ? 16u : (half <= 64 ? 64u : 128u)) * kBlockK * 2;
        const bool light = half <= light_max;
        if (!light) {
          // one K step per stage; the loop is kept short: a lone thread has nothing
          // to hide its instruction latencies behind, and it must turn a stage round
          // faster than the tensor cores consume one
          const uint32_t tx = 2 * (kABytes + tok_bytes);
          for (int kb = 0; kb < num_kb; kb += slabs) {
            if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
            const uint32_t sa = smem_base + stage * stage_bytes;
            const bool two = slabs == 2 && kb + 1 < num_kb;
            if (cta == 0) mbar_expect_tx(bar_full + 8 * stage, two ? 2 * tx : tx);
            tma_pair_load_3d(sa, &tm_w, full_leader0 + 8 * stage, kb * kBlockK, wrow, ch.slot);
            tma_pair_load_2d(sa + kABytes, tok_map, full_leader0 + 8 * stage, kb * kBlockK, tok0);
            if (two) {
              tma_pair_load_3d(sa + kSlabBytes, &tm_w, full_leader0 + 8 * stage, (kb + 1) * kBlockK, wrow, ch.slot);
              tma_pair_load_2d(sa + kSlabBytes + kABytes, tok_map, full_leader0 + 8 * stage, (kb + 1) * kBlockK, tok0);
            }
            if (++stage == n_stages) { stage = 0; phase ^= 1u; }
          }
          continue;
        }
        for (int kb = 0; kb < num_kb; kb += 2) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t full_leader = full_leader0 + 8 * stage;
          const uint32_t sa = smem_base + stage * stage_bytes;
          const int steps = kb + 1 < num_kb ? 2 : 1;
          if (cta == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * steps * (kABytes + tok_bytes));
          for (int q = 0; q < steps; ++q)
            tma_pair_load_3d(sa + q * kABytes, &tm_w, full_leader, (kb + q) * kBlockK, wrow, ch.slot);
          for (int q = 0; q < steps; ++q)
            tma_pair_load_2d(sa + 2 * kABytes + q * kLightTokBytes, tok_map, full_leader, (kb + q) * kBlockK, tok0);
          if (++stage == n_stages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (cta == 0 && lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      const uint64_t desc_fixed = umma_desc_sw128(0);     // everything but the start address (shared memory is below 256 KB)
      for (int j = 0; ok && j < sch.rounds; ++j) {
        int c, wt;
        if (!sch.tile(j, c, wt)) continue;
        const Chunk ch = read_chunk(tile_table, dense_rows, slot_of_expert, c, skip_rows_upto, dense_chunk, n_slots);
        if (ch.slot == kSlotSkip) continue;
        const int n = ((ch.tok_end - ch.tok_begin) + 15) & ~15;
        const uint32_t idesc = idesc_m256(n);
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * kMaxN;
        const bool light = (n >> 1) <= light_max;
        if (!light) {
          for (int kb = 0; kb < num_kb; kb += slabs) {
            if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint64_t adesc = desc_fixed | (uint64_t)((smem_base + stage * stage_bytes) >> 4);
            tc_mma_pair_bf16_x4(d_tmem, adesc, adesc + (kABytes >> 4), idesc, (uint32_t)kb);
            if (slabs == 2 && kb + 1 < num_kb)
              tc_mma_pair_bf16_x4(d_tmem, adesc + (kSlabBytes >> 4), adesc + ((kSlabBytes + kABytes) >> 4), idesc, 1u);
            tc_commit_pair(bar_empty + 8 * stage);
            if (++stage == n_stages) { stage = 0; phase ^= 1u; }
          }
        } else {
          for (int kb = 0; kb < num_kb; kb += 2) {
            if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t sa = smem_base + stage * stage_bytes;
            const int steps = kb + 1 < num_kb ? 2 : 1;
            for (int q = 0; q < steps; ++q) {
              const uint64_t adesc = umma_desc_sw128(sa + q * kABytes);
              const uint64_t bdesc = umma_desc_sw128(sa + 2 * kABytes + q * kLightTokBytes);
              tc_mma_pair_bf16_x4(d_tmem, adesc, bdesc, idesc, (uint32_t)(kb | q));
            }
            tc_commit_pair(bar_empty + 8 * stage);
            if (++stage == n_stages) { stage = 0; phase ^= 1u; }
          }
        }
        if (!ok) break;
        tc_commit_pair(bar_tfull + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9, both CTAs) ----------------
    // Two warps share each quarter of the TMEM lanes (a warp may only read lanes
    // 32*(warp%4)..+31) and take alternate 32-token chunks, so every scheduler has
    // two epilogue warps to hide the latency of the dependent math chains.
    const int lane_group = warp & 3;
    const int half = (warp - 2) >> 2;
    const int wl = lane_group * 32 + lane;              // weight row inside this CTA's 128
    const uint32_t tempty_leader0 = map_to_cta(bar_tempty, 0);
    int acc = 0; uint32_t acc_phase = 0;
    for (int j = 0; j < sch.rounds; ++j) {
      int c, wt;
      if (!sch.tile(j, c, wt)) continue;
      const Chunk ch = read_chunk(tile_table, dense_rows, slot_of_expert, c, skip_rows_upto, dense_chunk, n_slots);
      if (ch.slot == kSlotSkip) continue;
      bool ready = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag);
      if (MODE == kModeScale && row_dst != nullptr) {
        // The four warps of a half meet at named barriers while they stage rows:
        // they go on together or leave together, whichever warp saw the abort.
        uint32_t all_ready;
        asm volatile(
            "{\n\t.reg .pred p, q;\n\t"
            "setp.ne.u32 q, %1, 0;\n\t"
            "bar.red.and.pred p, %2, %3, q;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(all_ready) : "r"((uint32_t)ready), "r"(1 + half), "r"(128) : "memory");
        ready = all_ready != 0;
      }
      if (!ready) break;
      tc_fence_after();
      const int n_tok = ch.tok_end - ch.tok_begin;
      const uint32_t taddr = tmem_base + (uint32_t)acc * kMaxN + ((uint32_t)(lane_group * 32) << 16);
      const int wrow = wt * kTileW + (int)cta * kRowsPerCta + wl;      // row of the weight matrix
      if (MODE == kModeSwiglu) {
        // rows are interleaved: even = gate_j, odd = up_j, j = wrow / 2
        const int feat = wrow >> 1;
        const bool odd = (wl & 1) != 0;
        const bool feat_ok = feat < ld_out;
#pragma unroll 1
        for (int c0 = half * 32; c0 < n_tok; c0 += 64) {
          uint32_t v[32];
          tc_ld32(taddr + c0, v);
          tc_wait_ld();
          // The even lane (gate row) finishes the even tokens of the chunk, the odd
          // lane (up row) the odd ones: each sends the partner the value it will
          // not use itself.  One shuffle per token pair, no divergent branch.
          // all the arithmetic first, in one straight run of independent chains,
          // then the guarded stores: a branch per element would serialise the chains
          __nv_bfloat16 hv[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float keep = round_bf16(__uint_as_float(odd ? v[2 * i + 1] : v[2 * i]));
            const float give = round_bf16(__uint_as_float(odd ? v[2 * i] : v[2 * i + 1]));
            const float got = __shfl_xor_sync(0xffffffffu, give, 1);
            const float g = odd ? got : keep, u = odd ? keep : got;
            const float s = round_bf16(__fdividef(g, 1.0f + __expf(-g)));
            hv[i] = __float2bfloat16_rn(s * u);
          }
          __nv_bfloat16 *obase = out + (size_t)(ch.tok_begin + c0 + (odd ? 1 : 0)) * ld_out + feat;
          const int left = feat_ok ? n_tok - c0 - (odd ? 1 : 0) : 0;     // tokens 2i < left are this lane's to write
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (2 * i < left) obase[(size_t)(2 * i) * ld_out] = hv[i];
        }
      } else {
        const bool col_ok = wrow < ld_out;
#pragma unroll 1
        for (int c0 = half * 32; c0 < n_tok; c0 += 64) {
          uint32_t v[32];
          tc_ld32(taddr + c0, v);
          tc_wait_ld();
          // This lane's route weight of token c0+lane, packed with its right
          // neighbour's: pair k = (weights of tokens 2k, 2k+1), handed round by one
          // shuffle per pair.  The product of two bf16 values is exact in fp32, so
          // the packed bf16 multiply (one rounding) gives the bits of the fp32
          // multiply followed by the rounding to bf16.
          __nv_bfloat16 my_scale_b = __float2bfloat16_rn(1.0f);
          if (MODE != kModePlain && row_scale != nullptr && c0 + lane < n_tok)
            my_scale_b = row_scale[ch.tok_begin + c0 + lane];
          const uint32_t my_bits = (uint32_t)__bfloat16_as_ushort(my_scale_b);
          const uint32_t scale_pair = my_bits | (__shfl_down_sync(0xffffffffu, my_bits, 1) << 16);
          if (MODE == kModePlain || row_dst == nullptr) {
            uint32_t yv[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const __nv_bfloat162 a = __floats2bfloat162_rn(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
              __nv_bfloat162 y = a;
              if (MODE != kModePlain) {
                const uint32_t sp = __shfl_sync(0xffffffffu, scale_pair, 2 * k);
                y = __hmul2(a, *reinterpret_cast<const __nv_bfloat162 *>(&sp));
              }
              yv[k] = *reinterpret_cast<const uint32_t *>(&y);
            }
            unsigned short *obase = reinterpret_cast<unsigned short *>(out) + (size_t)(ch.tok_begin + c0) * ld_out + wrow;
            const int left = col_ok ? n_tok - c0 : 0;
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              if (2 * k < left) obase[(size_t)(2 * k) * ld_out] = (unsigned short)(yv[k] & 0xffffu);
              if (2 * k + 1 < left) obase[(size_t)(2 * k + 1) * ld_out] = (unsigned short)(yv[k] >> 16);
            }
          } else {
            // Scatter: every row goes straight to the address its sender asked for
            // (a row of the sender's return buffer, possibly on another GPU), so
            // the transfer back overlaps the GEMM instead of following it.  The four
            // warps that share this token chunk first put their 32-column pieces
            // side by side in shared memory, so that what leaves the SM are
            // 256-byte row segments, not 64-byte ones.
            unsigned long long my_dst = 0ull;
            if (c0 + lane < n_tok) my_dst = row_dst[ch.tok_begin + c0 + lane];
            __nv_bfloat16 *stg = reinterpret_cast<__nv_bfloat16 *>(scatter_stage + half * kScatterTileBytes);
            const int col0 = wt * kTileW + (int)cta * kRowsPerCta;       // first output column of this CTA
#pragma unroll
            for (int sub = 0; sub < 2; ++sub) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const uint32_t sp = __shfl_sync(0xffffffffu, scale_pair, sub * 16 + 2 * k);
                const __nv_bfloat162 a = __floats2bfloat162_rn(__uint_as_float(v[sub * 16 + 2 * k]),
                                                               __uint_as_float(v[sub * 16 + 2 * k + 1]));
                const __nv_bfloat162 y = __hmul2(a, *reinterpret_cast<const __nv_bfloat162 *>(&sp));
                stg[(2 * k) * kRowsPerCta + wl] = y.x;
                stg[(2 * k + 1) * kRowsPerCta + wl] = y.y;
              }
              asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(128) : "memory");
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int tj = lane_group * 4 + q;
                const unsigned long long d = __shfl_sync(0xffffffffu, my_dst, sub * 16 + tj);
                const uint2 piece = *reinterpret_cast<const uint2 *>(stg + tj * kRowsPerCta + lane * 4);
                if (d != 0ull && col0 + lane * 4 + 3 < ld_out)
                  *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(d) + col0 + lane * 4) = piece;
              }
              asm volatile("bar.sync %0, %1;" ::"r"(1 + half), "r"(128) : "memory");
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && status) atomicExch(status, 1);
    const unsigned long long t0 = gtime_ns();
    while (gtime_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();            // neither CTA leaves while the other may still touch its shared memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

// Tuning knobs behind sb_set_tuning (process-wide, read at launch time).
std::atomic<int> g_sched_mode{0};      // 0 table order / fixed stride, 1 ranked boustrophedon, 2 odd pairs backwards
std::atomic<int> g_kslabs{2};          // K steps of a full tile per pipeline stage when the caller leaves the depth open
std::atomic<int> g_dense_group{1};     // dense passes: row chunks per raster block (1 = chunk-major walk)
int sched_mode() { return g_sched_mode.load(std::memory_order_relaxed); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int32_t encode_map(CUtensorMap *tm, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, const char *what,
                   uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(SB_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {(cuuint32_t)kBlockK, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const cuuint32_t rank = d2 > 0 ? 3 : 2;
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void *>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(SB_E_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d", what, (int)r);
  return SB_OK;
}

// A tensor map depends only on (base, extents, box): a serving loop calls with
// the same few buffers every step, so each host thread remembers the last maps
// it encoded instead of asking the driver seven times per call.  The map holds
// no reference to the memory; a reused address with the same extents gives the
// same bytes.
struct MapKey {
  const void *base; uint64_t d0, d1, d2; uint32_t box_rows;
  bool operator==(const MapKey &o) const {
    return base == o.base && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && box_rows == o.box_rows;
  }
};
constexpr int kMapCacheSize = 64;
struct MapCache {
  MapKey key[kMapCacheSize];
  CUtensorMap map[kMapCacheSize];
  int used = 0, next = 0;
};

int32_t make_map(CUtensorMap *tm, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, const char *what,
                 uint32_t box_rows = kRowsPerCta) {
  static thread_local MapCache cache;
  const MapKey k = {base, d0, d1, d2, box_rows};
  for (int i = 0; i < cache.used; ++i)
    if (cache.key[i] == k) { *tm = cache.map[i]; return SB_OK; }
  int32_t rc = encode_map(tm, base, d0, d1, d2, what, box_rows);
  if (rc != SB_OK) return rc;
  const int slot = cache.used < kMapCacheSize ? cache.used++ : (cache.next++ % kMapCacheSize);
  cache.key[slot] = k;
  cache.map[slot] = *tm;
  return SB_OK;
}

// Shared-memory opt-in and carve-out preference of both kernel instances, once
// per device (the attributes are per device and per function).
int32_t prepare_device() {
  static std::mutex mu;
  static bool done[64];
  int dev = -1;
  SB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(SB_E_CUDA, "sb_grouped_swiglu: device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (done[dev]) return SB_OK;
  SB_CUDA_CHECK(cudaFuncSetAttribute(pair_gemm_kernel<kModeSwiglu>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem_bytes(kStages)));
  SB_CUDA_CHECK(cudaFuncSetAttribute(pair_gemm_kernel<kModeScale>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem_bytes(kStages)));
  SB_CUDA_CHECK(cudaFuncSetAttribute(pair_gemm_kernel<kModePlain>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem_bytes(kStages)));
  // the largest shared-memory split, so that small kernels of other streams
  // (router, sort, gather) can share an SM with a resident GEMM CTA
  SB_CUDA_CHECK(cudaFuncSetAttribute(pair_gemm_kernel<kModeSwiglu>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     (int)cudaSharedmemCarveoutMaxShared));
  SB_CUDA_CHECK(cudaFuncSetAttribute(pair_gemm_kernel<kModeScale>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     (int)cudaSharedmemCarveoutMaxShared));
  SB_CUDA_CHECK(cudaFuncSetAttribute(pair_gemm_kernel<kModePlain>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                     (int)cudaSharedmemCarveoutMaxShared));
  done[dev] = true;
  return SB_OK;
}

// Rows per chunk of a dense (single-slot) pass: the multiple of 16 in [192, 256]
// that needs the fewest rounds over `pairs` CTA pairs; among equals the widest.
// A tile's MMA time does not depend on its token extent (measured on B200: the
// same with 64, 128 or 256 tokens), so a round costs the same whatever the chunk
// width and only the number of rounds counts.
int dense_chunk_rows(int rows, int n_wtiles, int pairs) {
  int best = kMaxN;
  long best_rounds = -1;
  for (int c = kMaxN; c >= 192; c -= 16) {
    const long chunks = (rows + c - 1) / c;
    const long rounds = (chunks * n_wtiles + pairs - 1) / pairs;
    if (best_rounds < 0 || rounds < best_rounds) { best_rounds = rounds; best = c; }
  }
  return best;
}

template <int MODE>
int32_t launch_pass(const CUtensorMap &tm_w, const CUtensorMap *tm_x, const int32_t *tile_table, int dense_rows,
                    const int32_t *slot_of_expert, const void *row_scale, void *out, int ld_out, int w_rows,
                    int num_kb, int n_slots, int32_t *status, int grid, int skip_rows_upto,
                    const unsigned long long *row_dst, int n_stages, uint32_t stage_bytes, cudaStream_t stream) {
  const int n_wtiles = (w_rows + kTileW - 1) / kTileW;
  const int dense_chunk = tile_table == nullptr ? dense_chunk_rows(dense_rows, n_wtiles, grid / 2) : kMaxN;
  const int light_rows_per_cta = 16;      // tiles with at most this many tokens per CTA take two K steps per 36 KB stage
  auto kern = pair_gemm_kernel<MODE>;
  const int mode_now = sched_mode();
  const bool tail = row_dst != nullptr || (tile_table != nullptr && mode_now != 0);
  kern<<<grid, kThreads, smem_bytes(n_stages, stage_bytes, tail), stream>>>(tm_w, tm_x[0], tm_x[1], tm_x[2], tile_table, dense_rows,
                                                        slot_of_expert,
                                                        static_cast<const __nv_bfloat16 *>(row_scale),
                                                        static_cast<__nv_bfloat16 *>(out), ld_out, w_rows, num_kb,
                                                        n_slots, status, skip_rows_upto, dense_chunk, light_rows_per_cta,
                                                        row_dst, n_stages, mode_now,
                                                        g_dense_group.load(std::memory_order_relaxed), stage_bytes);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

}  // namespace

int32_t set_gemm_tuning(const char *key, int value) {
  if (strcmp(key, "sched") == 0) {
    if (value < 0 || value > 2) return fail(SB_E_INVALID_ARG, "sb_set_tuning: sched must be 0, 1 or 2");
    g_sched_mode.store(value);
    return SB_OK;
  }
  if (strcmp(key, "dense_group") == 0) {
    if (value < 1 || value > 64) return fail(SB_E_INVALID_ARG, "sb_set_tuning: dense_group must be in [1,64]");
    g_dense_group.store(value);
    return SB_OK;
  }
  if (strcmp(key, "kslabs") == 0) {
    if (value != 1 && value != 2) return fail(SB_E_INVALID_ARG, "sb_set_tuning: kslabs must be 1 or 2");
    g_kslabs.store(value);
    return SB_OK;
  }
  return SB_E_UNSUPPORTED;      // not a GEMM key
}

// w13 must be in the INTERLEAVED row order (row 2j = gate_j, row 2j+1 = up_j);
// tile_table must have been built with 256-row tiles.  Tile entries of at most
// `skip_rows_upto` rows are left to the caller (0 = none); `max_pairs` > 0
// limits the grid to that many CTA pairs.  With `row_dst` (one device address per
// row, 0 = drop) the down pass writes each result row to that address instead
// of `out`.  `passes`: 1 = gate/up + SwiGLU only, 2 = down only (hbuf already
// holds the intermediate rows), 3 = both.  `stages` in [2, 6] is the depth of
// the shared-memory pipeline (0 = 5, which leaves room on the SM for a router CTA).
int32_t launch_grouped_swiglu_pair(const void *rows, const int32_t *tile_table, int dense_rows, const void *w13,
                                   const void *w2, const int32_t *slot_of_expert, const void *row_scale,
                                   int R_cap, int H, int I, int S, void *hbuf, void *out, int32_t *status,
                                   int skip_rows_upto, int max_pairs, const unsigned long long *row_dst,
                                   cudaStream_t stream, int passes, int stages) {
  if (H < kBlockK || I < kBlockK || H % kBlockK != 0 || I % kBlockK != 0)
    return fail(SB_E_UNSUPPORTED, "sb_grouped_swiglu: H and I must be multiples of %d (H=%d I=%d)", kBlockK, H, I);
  if (R_cap <= 0 || S < 1) return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: R_cap=%d S=%d", R_cap, S);
  if (tile_table == nullptr && (dense_rows < 0 || dense_rows > R_cap))
    return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: dense_rows=%d outside [0,%d]", dense_rows, R_cap);
  if (tile_table == nullptr && dense_rows == 0) return SB_OK;
  if (!rows || !w13 || !w2 || !hbuf || (!out && !row_dst)) return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: null pointer");
  if (!aligned(rows, 128) || !aligned(w13, 128) || !aligned(w2, 128) || !aligned(hbuf, 128) || (out && !aligned(out, 16)))
    return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: operands must be 128-byte aligned");
  // Depth left open: three 64 KB stages of two K steps each (half the barrier
  // round trips per K step).  A caller that names a depth gets 36 KB stages of
  // one K step, e.g. five of them to leave room on the SM for a router CTA.
  uint32_t stage_bytes = kStageBytes;
  // -1: the launch should leave room on every SM for one router CTA.  Three
  // 64 KB stages without the scatter/ranking tail do (193 KB + the router's
  // 30 KB); with one K step per stage it is five 36 KB stages.
  if (stages == -1) stages = g_kslabs.load(std::memory_order_relaxed) == 2 ? 0 : kDefaultStages;
  if (stages == 0) {
    if (g_kslabs.load(std::memory_order_relaxed) == 2) { stages = kStages2; stage_bytes = kStageBytes2; }
    else stages = kDefaultStages;
  }
  if (stages < 2 || stages > kStages) return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: stages=%d outside [2,%d]", stages, kStages);
  int32_t rc = prepare_device();
  if (rc != SB_OK) return rc;
  CUtensorMap tm_x[3], tm_w13, tm_h[3], tm_w2;
  const uint32_t boxes[3] = {128, 64, 16};
  for (int b = 0; b < 3; ++b) {
    if ((passes & 1) && (rc = make_map(&tm_x[b], rows, (uint64_t)H, (uint64_t)R_cap, 0, "rows", boxes[b])) != SB_OK) return rc;
    if ((passes & 2) && (rc = make_map(&tm_h[b], hbuf, (uint64_t)I, (uint64_t)R_cap, 0, "hbuf", boxes[b])) != SB_OK) return rc;
  }
  if ((passes & 1) && (rc = make_map(&tm_w13, w13, (uint64_t)H, (uint64_t)2 * I, (uint64_t)S, "w13")) != SB_OK) return rc;
  if ((passes & 2) && (rc = make_map(&tm_w2, w2, (uint64_t)I, (uint64_t)H, (uint64_t)S, "w2")) != SB_OK) return rc;
  int grid = (sb_device_sm_count() / 2) * 2;
  if (grid <= 0) return fail(SB_E_CUDA, "sb_grouped_swiglu: no CUDA device");
  if (max_pairs > 0 && 2 * max_pairs < grid) grid = 2 * max_pairs;     // leave the other SMs to a concurrent launch
  if (passes & 1) {
    rc = launch_pass<kModeSwiglu>(tm_w13, tm_x, tile_table, dense_rows, slot_of_expert, nullptr, hbuf, I, 2 * I,
                                  H / kBlockK, S, status, grid, skip_rows_upto, nullptr, stages, stage_bytes, stream);
    if (rc != SB_OK) return rc;
  }
  if (!(passes & 2)) return SB_OK;
  if (row_scale == nullptr && row_dst == nullptr)
    return launch_pass<kModePlain>(tm_w2, tm_h, tile_table, dense_rows, slot_of_expert, nullptr, out, H, H,
                                   I / kBlockK, S, status, grid, skip_rows_upto, nullptr, stages, stage_bytes, stream);
  return launch_pass<kModeScale>(tm_w2, tm_h, tile_table, dense_rows, slot_of_expert, row_scale, out, H, H,
                                 I / kBlockK, S, status, grid, skip_rows_upto, row_dst, stages, stage_bytes, stream);
}

}  // namespace sb
