// Grouped bf16 SwiGLU expert MLP on Blackwell tensor cores.
//
// Replaces the per-expert Python loop of three `F.linear` calls plus the route
// weight scaling in the reference (utils/eval_core.py:11767-11793, 11765; the
// loop around it at 14690-14721 and 13240-13357) and the shared expert MLP
// (utils/eval_core.py:9455-9463).
//
// Two launches of one persistent, warp-specialised kernel template:
//   pass 1  h   = bf16( bf16(silu(bf16(x.Wg^T))) * bf16(x.Wu^T) )     [R, I]
//   pass 2  out = bf16( bf16(h.Wd^T) * row_scale )                     [R, H]
// Rounding points are those of the reference's bf16 ops, so the only numeric
// difference left is the fp32 summation order inside the tensor core.
//
// Kernel shape (per CTA, one CTA per SM):
//   - tile 128 rows x 256 accumulator columns x 64 K per stage, 4 stages of
//     48 KB shared memory filled by TMA (`cp.async.bulk.tensor`, 128-byte
//     swizzle, no multicast), completion on mbarriers;
//   - pass 1 loads 128 gate rows and 128 up rows of the same intermediate
//     columns as one 256-wide B operand, so silu(gate)*up is formed in the
//     epilogue without a second pass over memory;
//   - one thread issues `tcgen05.mma.cta_group::1.kind::f16` (M128 N256 K16)
//     into TMEM; two 256-column accumulators (all 512 TMEM columns) let the
//     epilogue of tile i overlap the main loop of tile i+1;
//   - warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner, warps 2-5 =
//     epilogue (`tcgen05.ld` 32 lanes x 32 columns, math, 64-byte stores).
// Row tiles come from the table sb_permute writes (expert, row_begin,
// row_end); rows of a tile past row_end are computed and discarded.  Weights
// live in slabs [slot][rows][K]; one 3-D tensor map addresses every slot, so a
// cache slot swap needs no re-encoding.
//
// Every wait on an mbarrier is bounded (about two seconds of %globaltimer);
// on expiry the CTA raises a flag in shared memory, reports through `status`,
// lets in-flight copies drain, frees its TMEM and returns.
#include <cuda.h>

#include <mutex>

#include "sb_common.cuh"

namespace sb {
namespace {

constexpr int kBlockM = SB_TILE_M;    // 128
constexpr int kBlockN = 256;
constexpr int kBlockK = 64;           // 128 bytes of bf16: one swizzle atom
constexpr int kStages = 4;
constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr uint32_t kABytes = kBlockM * kBlockK * 2;     // 16 KB
constexpr uint32_t kBBytes = kBlockN * kBlockK * 2;     // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;     // 48 KB
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;

// slot_of_expert value meaning "leave this expert's tiles to another launch"
// (readiness-ordered execution runs the grouped GEMM once per readiness class).
constexpr int kSlotSkip = -2;

constexpr int kModeSwiglu = 0;
constexpr int kModeScale = 1;

// ---- PTX wrappers ---------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done;
}
// Bounded wait.  Returns false if the CTA is aborting (this wait or another one
// ran out of time); the caller must then leave its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tm, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *tm, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(tm), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                            uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp gets lane
// (taddr.lane + i), columns taddr.col .. +31.
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
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile written by TMA
// with the 128-byte swizzle: rows are 128 bytes apart, groups of 8 rows are
// 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;                 // leading byte offset: unused with swizzle
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
  d |= (uint64_t)1 << 46;                 // descriptor version
  d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
  return d;
}
// Instruction descriptor: D=f32, A=B=bf16, both K-major, N=256, M=128.
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) |
                            ((uint32_t)(kBlockN >> 3) << 17) | ((uint32_t)(kBlockM >> 4) << 24);

struct TileInfo { int slot, row_begin, row_end; };

__device__ __forceinline__ TileInfo read_tile(const int32_t *tile_table, int dense_rows,
                                              const int32_t *slot_of_expert, int m_tile) {
  TileInfo t;
  if (tile_table == nullptr) {
    t.slot = 0;
    t.row_begin = m_tile * kBlockM;
    t.row_end = min(dense_rows, t.row_begin + kBlockM);
  } else {
    const int4 e = __ldg(reinterpret_cast<const int4 *>(tile_table + kTileHeaderInts) + m_tile);
    t.slot = slot_of_expert ? __ldg(slot_of_expert + e.x) : e.x;
    t.row_begin = e.y;
    t.row_end = e.z;
  }
  return t;
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                    const int32_t *__restrict__ tile_table, int dense_rows,
                    const int32_t *__restrict__ slot_of_expert,
                    const __nv_bfloat16 *__restrict__ row_scale, __nv_bfloat16 *__restrict__ out,
                    int ld_out, int n_out_cols, int num_kb, int up_row_offset, int n_slots,
                    int32_t *__restrict__ status) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char *smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem_al + kStages * kStageBytes);
  const uint32_t bar_full = smem_base + kStages * kStageBytes;          // kStages barriers
  const uint32_t bar_empty = bar_full + 8 * kStages;                    // kStages
  const uint32_t bar_tfull = bar_empty + 8 * kStages;                   // 2
  const uint32_t bar_tempty = bar_tfull + 16;                           // 2
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 4);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int kOutTileCols = (MODE == kModeSwiglu) ? kBlockN / 2 : kBlockN;
  const int n_ntiles = (n_out_cols + kOutTileCols - 1) / kOutTileCols;
  const int n_mtiles = tile_table ? __ldg(tile_table) : (dense_rows + kBlockM - 1) / kBlockM;
  const int total_tiles = n_mtiles * n_ntiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(bar_tfull + 8 * b, 1); mbar_init(bar_tempty + 8 * b, kEpiThreads); }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int m_tile = tile / n_ntiles, n_tile = tile - m_tile * n_ntiles;
        TileInfo ti = read_tile(tile_table, dense_rows, slot_of_expert, m_tile);
        if (ti.slot == kSlotSkip) continue;           // not part of this launch
        if (ti.slot < 0 || ti.slot >= n_slots) {      // expert not resident: caller error
          if (status) atomicExch(status, 2);
          ti.slot = 0;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag)) { ok = false; break; }
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb_ = sa + kABytes;
          mbar_expect_tx(full, kStageBytes);
          tma_load_2d(sa, &tm_a, full, kb * kBlockK, ti.row_begin);
          if (MODE == kModeSwiglu) {
            tma_load_3d(sb_, &tm_b, full, kb * kBlockK, n_tile * (kBlockN / 2), ti.slot);
            tma_load_3d(sb_ + kBBytes / 2, &tm_b, full, kb * kBlockK,
                        up_row_offset + n_tile * (kBlockN / 2), ti.slot);
          } else {
            tma_load_3d(sb_, &tm_b, full, kb * kBlockK, n_tile * kBlockN, ti.slot);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if (read_tile(tile_table, dense_rows, slot_of_expert, tile / n_ntiles).slot == kSlotSkip) continue;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * kBlockN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint64_t adesc = umma_desc_sw128(sa);
          const uint64_t bdesc = umma_desc_sw128(sa + kABytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            // advance 32 bytes (16 bf16) along K inside the swizzle atom
            tc_mma_bf16(d_tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), kIdesc,
                        (kb | k) != 0 ? 1u : 0u);
          }
          tc_commit(bar_empty + 8 * stage);     // frees the stage when these MMAs retire
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(bar_tfull + 8 * acc);         // accumulator complete
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int lane_group = warp & 3;            // TMEM lanes this warp may read
    const int row_in_tile = lane_group * 32 + lane;
    int acc = 0; uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int m_tile = tile / n_ntiles, n_tile = tile - m_tile * n_ntiles;
      const TileInfo ti = read_tile(tile_table, dense_rows, slot_of_expert, m_tile);
      if (ti.slot == kSlotSkip) continue;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) break;
      tc_fence_after();
      const int row = ti.row_begin + row_in_tile;
      const bool row_ok = row < ti.row_end;
      const uint32_t taddr = tmem_base + (uint32_t)acc * kBlockN + ((uint32_t)(lane_group * 32) << 16);
      __nv_bfloat16 *orow = out + (size_t)row * ld_out + (size_t)n_tile * kOutTileCols;
      if (MODE == kModeSwiglu) {
#pragma unroll 1
        for (int c = 0; c < kOutTileCols / 32; ++c) {
          uint32_t g[32], u[32];
          tc_ld32(taddr + c * 32, g);
          tc_ld32(taddr + kBlockN / 2 + c * 32, u);
          tc_wait_ld();
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float h2[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const float gv = round_bf16(__uint_as_float(g[2 * i + j]));
              const float uv = round_bf16(__uint_as_float(u[2 * i + j]));
              const float sv = round_bf16(gv / (1.0f + expf(-gv)));
              h2[j] = sv * uv;
            }
            packed[i] = pack_bf16x2(h2[0], h2[1]);
          }
          if (row_ok && n_tile * kOutTileCols + c * 32 < n_out_cols) {
            uint4 *dst = reinterpret_cast<uint4 *>(orow + c * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
          }
        }
      } else {
        const float scale = (row_scale != nullptr && row_ok) ? __bfloat162float(row_scale[row]) : 1.0f;
#pragma unroll 1
        for (int c = 0; c < kOutTileCols / 32; ++c) {
          uint32_t a[32];
          tc_ld32(taddr + c * 32, a);
          tc_wait_ld();
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float y0 = round_bf16(__uint_as_float(a[2 * i]));
            float y1 = round_bf16(__uint_as_float(a[2 * i + 1]));
            if (row_scale != nullptr) { y0 *= scale; y1 *= scale; }
            packed[i] = pack_bf16x2(y0, y1);
          }
          if (row_ok && n_tile * kOutTileCols + c * 32 < n_out_cols) {
            uint4 *dst = reinterpret_cast<uint4 *>(orow + c * 32);
#pragma unroll
            for (int q = 0; q < 4; ++q)
              dst[q] = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && status) atomicExch(status, 1);
    // let copies and MMAs that are still in flight land before the shared
    // memory and TMEM go back to the SM
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
                 : "memory");
  }
}

// ---- host side ------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
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

// bf16 tensor [d2][d1][d0] (d0 contiguous), box {64, box1, 1}, 128-byte swizzle.
int32_t make_map(CUtensorMap *tm, const void *base, uint64_t d0, uint64_t d1, uint64_t d2,
                 uint32_t box1, const char *what) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(SB_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {(cuuint32_t)kBlockK, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const cuuint32_t rank = d2 > 0 ? 3 : 2;
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void *>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(SB_E_CUDA, "cuTensorMapEncodeTiled(%s) failed with CUresult %d (dims %llu x %llu x %llu)",
                what, (int)r, (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2);
  return SB_OK;
}

template <int MODE>
int32_t launch_pass(const CUtensorMap &tm_a, const CUtensorMap &tm_b, const int32_t *tile_table,
                    int dense_rows, const int32_t *slot_of_expert, const void *row_scale, void *out,
                    int ld_out, int n_out_cols, int num_kb, int up_row_offset, int n_slots,
                    int32_t *status, int grid, cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<MODE>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  });
  if (attr_err != cudaSuccess) {
    // per-device attribute: retry for other devices of the process
    SB_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
  }
  kern<<<grid, kThreads, kSmemBytes, stream>>>(tm_a, tm_b, tile_table, dense_rows, slot_of_expert,
                                              static_cast<const __nv_bfloat16 *>(row_scale),
                                              static_cast<__nv_bfloat16 *>(out), ld_out, n_out_cols,
                                              num_kb, up_row_offset, n_slots, status);
  SB_LAUNCH_CHECK();
  return SB_OK;
}

}  // namespace

int32_t launch_grouped_swiglu(const void *rows, const int32_t *tile_table, int dense_rows,
                              const void *w13, const void *w2, const int32_t *slot_of_expert,
                              const void *row_scale, int R_cap, int H, int I, int S, void *hbuf,
                              void *out, int32_t *status, cudaStream_t stream) {
  if (H < kBlockK || I < kBlockK || H % kBlockK != 0 || I % kBlockK != 0)
    return fail(SB_E_UNSUPPORTED, "sb_grouped_swiglu: H and I must be multiples of %d (H=%d I=%d)",
                kBlockK, H, I);
  if (R_cap <= 0 || S < 1) return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: R_cap=%d S=%d", R_cap, S);
  if (tile_table == nullptr && (dense_rows < 0 || dense_rows > R_cap))
    return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: dense_rows=%d outside [0,%d]", dense_rows, R_cap);
  if (tile_table == nullptr && dense_rows == 0) return SB_OK;
  if (!rows || !w13 || !w2 || !hbuf || !out)
    return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: null pointer");
  if (!aligned(rows, 128) || !aligned(w13, 128) || !aligned(w2, 128) || !aligned(hbuf, 128) ||
      !aligned(out, 16))
    return fail(SB_E_INVALID_ARG, "sb_grouped_swiglu: operands must be 128-byte aligned");

  CUtensorMap tm_x, tm_w13, tm_h, tm_w2;
  int32_t rc;
  if ((rc = make_map(&tm_x, rows, (uint64_t)H, (uint64_t)R_cap, 0, kBlockM, "rows")) != SB_OK) return rc;
  if ((rc = make_map(&tm_w13, w13, (uint64_t)H, (uint64_t)2 * I, (uint64_t)S, kBlockN / 2, "w13")) != SB_OK) return rc;
  if ((rc = make_map(&tm_h, hbuf, (uint64_t)I, (uint64_t)R_cap, 0, kBlockM, "hbuf")) != SB_OK) return rc;
  if ((rc = make_map(&tm_w2, w2, (uint64_t)I, (uint64_t)H, (uint64_t)S, kBlockN, "w2")) != SB_OK) return rc;

  const int grid = sb_device_sm_count();
  if (grid <= 0) return fail(SB_E_CUDA, "sb_grouped_swiglu: no CUDA device");
  rc = launch_pass<kModeSwiglu>(tm_x, tm_w13, tile_table, dense_rows, slot_of_expert, nullptr, hbuf,
                                I, I, H / kBlockK, I, S, status, grid, stream);
  if (rc != SB_OK) return rc;
  return launch_pass<kModeScale>(tm_h, tm_w2, tile_table, dense_rows, slot_of_expert, row_scale, out,
                                 H, H, I / kBlockK, 0, S, status, grid, stream);
}

}  // namespace sb
